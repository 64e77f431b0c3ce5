// Dequantising product y = x . dequant(W)^T for GGUF Q4_0 / Q8_0 weights at decode sizes: what the reference does in
// three passes -- gguf::dequant_q4_0 / dequant_q8_0 (src/gguf.rs:286-326), the transposition of load_transposed_weight
// (src/models/llama/model.rs:243-257) and Tensor::matmul (src/tensor.rs:1342-1354) -- in one pass over the block stream.
//
// Arithmetic (exact integer sums per 32-element block on the int8 tensor-core path):
//   * the quants go to the MMA as they are: Q8_0 bytes as s8, Q4_0 nibbles as u8 after one shift and two logic ops per
//     eight of them (the "- 8" of the format is not applied to the weights, see below);
//   * each f32 activation becomes a 23-bit integer xi = round(x * 2^s), |xi| <= 2^22 (s per activation row and per
//     256-element slice of K, from the slice's largest element), written in three balanced base-256 digits
//     xi = d2 * 65536 + d1 * 256 + d0, -128 <= d <= 127 (the bytes of xi + 0x808080 with their top bits flipped): three
//     s8 planes, built ONCE per CTA and K chunk into shared memory by all warps together;
//   * one m16n8k32 MMA per digit plane (16 weight rows x 32 k x 8 activation rows) gives the exact sums of a block; the
//     three are joined in integer arithmetic ((c2 * 256 + c1) * 256 + c0, the last step in f32 for Q8_0 where it would
//     not fit) and the block's f16 scale is applied to the one result.  Q4_0's offset, sum((q - 8) xi) =
//     sum(q xi) - 8 sum(xi), enters as the accumulator input of the digit-0 MMA;
//   * per slice the sums are multiplied by 2^-s and added to the tile's f32 accumulators.
//   * one or two activation rows: the three digits of a row travel as three COLUMNS of one B operand (column 3 m + l), so a
//     block is ONE MMA; the per-digit sums are scaled and accumulated in f32 as they are and joined (x 1, 256, 65536) once
//     per tile.  (12.0 / 13.7 us against 15.0 / 15.8 us for Q4_0 / Q8_0 at N 14336, K 4096, one row.)
// Against the reference's sequential f32 loop this differs in summation order and in the 2^-22 (of the slice maximum)
// rounding of the activations: tolerance 1e-5 of max|y|.  A slice holding a non-finite activation makes that activation
// row's outputs NaN (the reference gives inf or NaN there).
//
// Data flow: one persistent CTA of 16 warps per SM.  A tile is 16 weight rows; K is walked in chunks whose digit planes
// fill 48 KB: 64 / rows slices, i.e. all of K up to 16384 for one activation row and 2048 elements for eight; inside a
// chunk a tile's slices are shared by kw = 1, 2, 4 or 8 warps.
// A warp streams its slices through a private ring in shared memory.  The upload lays the weight out so that everything
// one fill needs -- the quants of a tile's 16 rows for one slice and their 16 x 8 f16 scales -- is ONE contiguous piece
// of 2304 / 4352 bytes: a fill is a single bulk asynchronous copy with completion on an mbarrier (with one copy per row
// and one per row of scales, 32 small copies per fill, the kernel ran at the copy unit's rate: the same time for Q4_0 as
// for Q8_0).  No block-wide barrier runs inside a chunk.  With kw > 1 the f32 partial sums meet in shared memory behind
// a named barrier of those kw warps (fixed order: deterministic).  Chunks after the first add onto y (the same lane owns an
// output in every chunk).  Weights never depend on the preceding kernel, so the first fills are requested before
// griddepcontrol.wait.  Every mbarrier wait is bounded: on expiry PG_ERR_DEVICE_TIMEOUT goes to the context's status
// word and the kernel leaves through its remaining barriers.
//
// Layout of a fill (made at upload, csrc/pg_gguf.cu: repack_kernel): row r of the tile at r * SEG as 16-byte pieces;
// piece p = (block group) * 4 + t holds, for lane t of a fragment, Q4_0: word t (elements 8t..8t+7) of the group's four
// blocks; Q8_0: bytes 8t..8t+7 of the group's two blocks; it is stored at position p ^ ((r & 1) << 2), which makes the
// 128-bit reads of a quarter warp (two rows, four pieces each) free of bank conflicts without padding.  The scales
// follow at 16 * SEG + r * 16.
#include <cuda_fp16.h>

#include <algorithm>

#include "pg_internal.cuh"

namespace {

constexpr int GS_SLICE = 8;                       // blocks per slice (256 elements): the unit of activation scaling and of a ring fill
// A K chunk is as many slices as fill the digit-plane area for the activation rows at hand: 64 / rows slices (a power
// of two), i.e. all of K = 16384 for one row, 2048 elements for eight rows.
constexpr int GS_MAX_SLICES = 64;
// (A CTA of 12 warps with 96 KB of planes, which makes K = 4096 one chunk for eight rows too, was measured: no faster at
// eight rows -- 22.7 / 23.7 us against 23.2 / 23.0 us for Q4_0 / Q8_0 at N 14336 -- and slower at K 14336; the chunk
// boundaries are not what the eight-row case pays for.)
constexpr int GS_US_BYTES = GS_MAX_SLICES * 8 * 4 * 2;   // [slice][8] 2^-s, then [slice][8] NaN-or-zero markers

template <int TYPE, int W, bool SMALL>
struct GsCfg {
    static constexpr int WARPS = W, THREADS = W * 32;
    static constexpr int PLANES_BYTES = 48 * 1024;                           // [block][plane][row][t][8 B]: rows * blocks <= 512
    static constexpr int ROW_SLICES = PLANES_BYTES / 768;                    // rows * slices of a chunk
    // Q4_0: [block][row] -8 * sum(xi); SMALL: [block][4 * rows] -8 * sum(digit) per (row, digit) column
    static constexpr int OFF_BYTES = (TYPE == PG_GGUF_Q4_0) ? (SMALL ? PLANES_BYTES / 6 : PLANES_BYTES / 24) : 0;
    static constexpr int QB = (TYPE == PG_GGUF_Q4_0) ? 16 : 32;            // quant bytes per block
    static constexpr int SEG = GS_SLICE * QB;                                // quant bytes per row and fill
    static constexpr int SCALE_OFF = 16 * SEG;                               // [16 rows][16 B]
    static constexpr int SLOT_BYTES = SCALE_OFF + 16 * 16;                   // = one fill, as it lies in global memory
    static constexpr int SLOTS = (TYPE == PG_GGUF_Q4_0) ? 4 : 2;
    static constexpr int RING_BYTES = WARPS * SLOTS * SLOT_BYTES;
    static constexpr int RED_BYTES = WARPS * 2 * 512;                        // kw > 1: [warp][tile parity][lane] 16 B of partial sums
    static constexpr int BAR_BYTES = WARPS * SLOTS * 8 + 16;
    static constexpr int SMEM = PLANES_BYTES + OFF_BYTES + GS_US_BYTES + RING_BYTES + RED_BYTES + BAR_BYTES;
};

__device__ __forceinline__ void gs_mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void gs_mbar_expect(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool gs_mbar_try(uint32_t bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}
__device__ __forceinline__ bool gs_mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int32_t *status, unsigned long long limit_ns)
{
    unsigned long long t0 = 0;
    for (uint32_t it = 1;; ++it) {
        if (gs_mbar_try(bar, parity)) return true;
        if ((it & 0xff) == 0) {
            if (*abort_flag) return false;
            const unsigned long long now = pg_globaltimer_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > limit_ns) {
                *abort_flag = 1;
                atomicExch(status, (int32_t)PG_ERR_DEVICE_TIMEOUT);
                return false;
            }
        }
    }
}
__device__ __forceinline__ void gs_bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}
// Shared-memory reads are ordinary loads (offsets into the dynamic shared array), and the MMAs below are not `volatile`:
// the compiler may then start the loads and MMAs of the next blocks while a block's results are still being converted.
// (With `asm volatile` on both, every block's chain load -> MMA -> convert -> scale ran strictly after the previous
// block's, and the kernel took the same time for Q4_0 as for Q8_0.)  The mbarrier wait, the bulk copies and the named
// barrier are volatile with a memory clobber, which keeps the loads on the right side of them.
extern __shared__ __align__(128) unsigned char gs_smem[];
__device__ __forceinline__ uint4 gs_lds128(uint32_t off) { return *reinterpret_cast<const uint4 *>(gs_smem + off); }
__device__ __forceinline__ uint2 gs_lds64(uint32_t off) { return *reinterpret_cast<const uint2 *>(gs_smem + off); }
// D = A (16 weight rows x 32 k, u8 nibbles or s8 bytes) x B (32 k x 8 activation rows, s8 digits) + C
template <int TYPE>
__device__ __forceinline__ void gs_mma(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1, int c0,
                                       int c1)
{
    if (TYPE == PG_GGUF_Q4_0)
        asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%10,%11};"
                     : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c0), "r"(c1));
    else
        asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%10,%11};"
                     : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c0), "r"(c1));
}

// Digit planes of one K chunk for activation rows m0..m0+rows-1, built by the whole CTA: warp p handles (row p % rows, slice p / rows);
// its lane i holds elements 8i..8i+7 of the slice = elements 8t..8t+7 (t = i % 4) of block i / 4: exactly what fragment
// lane (row, t) of that block needs.  B operand order inside a block (the order in which the weight side presents k):
//   Q8_0: b0 = elements 8t+0..3, b1 = elements 8t+4..7;  Q4_0: b0 = elements 8t+{0,2,4,6}, b1 = elements 8t+{1,3,5,7}.
// SMALL (one or two activation rows): the three digits of a row are three COLUMNS of one B operand (column 3 m + l), so a
// block needs one MMA instead of three: planes [block][3 * rows columns][t][8 B], offsets [block][4 * rows] per column.
template <int TYPE, int W, int ROWS>
__device__ __forceinline__ void gs_build_planes(const float *__restrict__ x, int M, int m0, int rows_arg, int cslices, int nblk_row, int blk0,
                                                unsigned char *planes, int *off, float *us, float *ps)
{
    constexpr bool SMALL = ROWS == 1 || ROWS == 2;
    const int rows = ROWS ? ROWS : rows_arg;          // a compile-time constant folds into the index arithmetic below
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // four (row, slice) pairs per pass, their loads issued together: one pair per pass costs a memory latency per pair
    constexpr int PF = 4;
    const int total = rows * cslices;
    const int t = lane & 3;
#pragma unroll 1
    for (int p0 = warp; p0 < total; p0 += W * PF) {
        float4 la[PF], lb[PF];
#pragma unroll
        for (int i = 0; i < PF; i++) {
            const int p = p0 + i * W;
            la[i] = lb[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (p < total) {
                const int s = p / rows, m = p - s * rows;
                const int jb = s * GS_SLICE + (lane >> 2);
                if ((m0 + m < M) && (blk0 + jb < nblk_row)) {
                    const float4 *src = reinterpret_cast<const float4 *>(x + (int64_t)(m0 + m) * nblk_row * 32 + (int64_t)(blk0 + jb) * 32 + t * 8);
                    la[i] = pg_ld_fresh(src);
                    lb[i] = pg_ld_fresh(src + 1);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < PF; i++) {
        const int p = p0 + i * W;
        if (p >= total) break;
        const int s = p / rows, m = p - s * rows;
        const int jb = s * GS_SLICE + (lane >> 2);                     // block inside the chunk; t: quarter of the block
        const float v[8] = {la[i].x, la[i].y, la[i].z, la[i].w, lb[i].x, lb[i].y, lb[i].z, lb[i].w};
        float amax = 0.0f, poison = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            amax = fmaxf(amax, fabsf(v[j]));
            poison += v[j] - v[j];                 // 0, or NaN for a non-finite element
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            poison += __shfl_xor_sync(0xffffffffu, poison, o);
        }
        int e = 0;
        if (amax > 0.0f && amax < INFINITY) e = max(-100, min(100, ilogbf(amax)));
        const float sc = scalbnf(1.0f, 21 - e);    // |x| * sc < 2^22 on the slice
        uint32_t bz[8];
        int sum = 0;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int xi = __float2int_rn(v[j] * sc);
            sum += xi;
            bz[j] = (uint32_t)(xi + 0x00808080);   // bytes = the balanced digits + 128
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        uint32_t h0[4], h1[4];
        if (TYPE == PG_GGUF_Q4_0) {
            h0[0] = bz[0]; h0[1] = bz[2]; h0[2] = bz[4]; h0[3] = bz[6];
            h1[0] = bz[1]; h1[1] = bz[3]; h1[2] = bz[5]; h1[3] = bz[7];
        } else {
            h0[0] = bz[0]; h0[1] = bz[1]; h0[2] = bz[2]; h0[3] = bz[3];
            h1[0] = bz[4]; h1[1] = bz[5]; h1[2] = bz[6]; h1[3] = bz[7];
        }
#pragma unroll
        for (int l = 0; l < 3; l++) {
            // byte l of four elements -> one register, top bits flipped (digit + 128 -> digit as s8)
            const uint32_t sel = l == 0 ? 0x0040u : (l == 1 ? 0x0051u : 0x0062u);
            const uint32_t b0 = __byte_perm(__byte_perm(h0[0], h0[1], sel), __byte_perm(h0[2], h0[3], sel), 0x5410) ^ 0x80808080u;
            const uint32_t b1 = __byte_perm(__byte_perm(h1[0], h1[1], sel), __byte_perm(h1[2], h1[3], sel), 0x5410) ^ 0x80808080u;
            if (SMALL) {
                *reinterpret_cast<uint2 *>(planes + ((size_t)(jb * 3 * rows + m * 3 + l) * 4 + t) * 8) = make_uint2(b0, b1);
                if (TYPE == PG_GGUF_Q4_0) {
                    int ds = __dp4a((int)b0, 0x01010101, __dp4a((int)b1, 0x01010101, 0));   // sum of this lane's eight digits
                    ds += __shfl_xor_sync(0xffffffffu, ds, 1);
                    ds += __shfl_xor_sync(0xffffffffu, ds, 2);
                    if (t == 0) off[jb * 4 * rows + m * 3 + l] = -8 * ds;
                }
            } else {
                *reinterpret_cast<uint2 *>(planes + ((size_t)(jb * 3 + l) * (rows * 4) + (m * 4 + t)) * 8) = make_uint2(b0, b1);
            }
        }
        if (!SMALL && TYPE == PG_GGUF_Q4_0 && t == 0) off[jb * rows + m] = -8 * sum;
        if (lane == 0) {
            us[s * 8 + m] = scalbnf(1.0f, e - 21);
            ps[s * 8 + m] = poison;
        }
        }
    }
}

// Shared memory: planes | Q4_0: offsets | us, ps | rings [warp][slot] | partial sums | mbarriers [warp][slot] | abort flag
// Warp w: tile slot w / kw, K part w % kw (8 / kw slices of every chunk).  CTA b, slot s: tiles b + grid * (s + (16 / kw) * j).
// ROWS: activation rows of this launch when it is 1, 2 or 8 (constants in the index arithmetic of the inner loop); 0 = 3 to 7
// rows, taken from the argument.
template <int TYPE, int W, int ROWS>
__global__ void __launch_bounds__(W * 32, 1)
    gguf_stream_kernel(const float *__restrict__ x, const uint8_t *__restrict__ qs, int64_t N, int nblk_row, int M, int m0, int rows_arg,
                       int cslices, float *__restrict__ y, int kw, int32_t *status, unsigned long long limit_ns)
{
    constexpr bool SMALL = ROWS == 1 || ROWS == 2;
    const int rows = ROWS ? ROWS : rows_arg;
    using C = GsCfg<TYPE, W, SMALL>;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    unsigned char *planes = gs_smem;
    int *off = reinterpret_cast<int *>(gs_smem + C::PLANES_BYTES);
    float *us = reinterpret_cast<float *>(gs_smem + C::PLANES_BYTES + C::OFF_BYTES);
    float *ps = us + GS_MAX_SLICES * 8;
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(gs_smem);
    // (loads take offsets into the shared array; bulk copies and mbarriers take shared-space addresses = sbase + offset)
    const uint32_t planes_s = 0, off_s = C::PLANES_BYTES;
    const uint32_t us_s = off_s + C::OFF_BYTES, ps_s = us_s + GS_MAX_SLICES * 8 * 4;
    const uint32_t ring0 = us_s + GS_US_BYTES;
    const uint32_t ring = ring0 + (uint32_t)warp * (C::SLOTS * C::SLOT_BYTES);
    const uint32_t red = ring0 + C::RING_BYTES + (uint32_t)warp * 1024;
    const uint32_t bars = sbase + ring0 + C::RING_BYTES + C::RED_BYTES;
    const uint32_t my_bar = bars + (uint32_t)warp * (C::SLOTS * 8);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(gs_smem + ring0 + C::RING_BYTES + C::RED_BYTES + W * C::SLOTS * 8);
    if (threadIdx.x == 0) {
        for (int i = 0; i < W * C::SLOTS; i++) gs_mbar_init(bars + 8 * i, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    const int groups = W / kw, slot_idx = warp / kw, kpart = warp - slot_idx * kw;
    const int cblocks = cslices * GS_SLICE;                 // cslices: slices per chunk
    const int64_t tiles = (N + 15) >> 4;
    const int64_t first = blockIdx.x + (int64_t)gridDim.x * slot_idx, tstep = (int64_t)gridDim.x * groups;
    const int my_tiles = first < tiles ? (int)((tiles - first + tstep - 1) / tstep) : 0;
    const int nchunks = (nblk_row + cblocks - 1) / cblocks;
    const int64_t nslices = nblk_row >> 3;
    uint32_t fills = 0;                                     // ring fills consumed so far (= issued, at chunk boundaries)
    bool ok = true;
    // SMALL: B column of this lane (clamped to an existing one), first of its two offset columns, rows of its two C columns
    const int ncols = 3 * rows;
    const int bcol = g < ncols ? g : 0, ocol = 2 * t < 4 * rows ? 2 * t : 0;
    const int ma = min((2 * t) / 3, rows - 1), mb = min((2 * t + 1) / 3, rows - 1);

    for (int chunk = 0; chunk < nchunks; chunk++) {
        const int blk0 = chunk * cblocks;
        const int cs = min(cslices, (nblk_row - blk0) / GS_SLICE);   // slices this chunk has (K is a multiple of 256)
        const int spp = (cs + kw - 1) / kw;                          // slices of this chunk per warp of a tile
        const int s_lo = kpart * spp, nsl = max(0, min(spp, cs - s_lo));      // this warp's slices of the chunk
        const int total = my_tiles * nsl;
        // fill q of this chunk: tile j = q / nsl, slice s_lo + q % nsl
        auto issue = [&](int q) {
            const int j = q / nsl, s = s_lo + (q - j * nsl);
            const uint32_t f = fills + (uint32_t)q;
            const uint32_t slot = ring + (f % C::SLOTS) * C::SLOT_BYTES, bar = my_bar + (f % C::SLOTS) * 8;
            if (lane == 0) {
                gs_mbar_expect(bar, C::SLOT_BYTES);
                const int64_t tile = first + (int64_t)j * tstep;   // < tiles; rows past N inside it are zero
                gs_bulk_load(sbase + slot, qs + (tile * nslices + (blk0 >> 3) + s) * (int64_t)C::SLOT_BYTES, C::SLOT_BYTES, bar);
            }
        };
        for (int q = 0; q < C::SLOTS; q++)
            if (q < total) issue(q);
        if (chunk == 0) asm volatile("griddepcontrol.wait;" ::: "memory");   // the activations come from the preceding kernel
        if (chunk > 0) __syncthreads();                     // everybody is done with the previous chunk's planes
        gs_build_planes<TYPE, W, ROWS>(x, M, m0, rows, cslices, nblk_row, blk0, planes, off, us, ps);
        __syncthreads();

        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        int q = 0;
        for (int j = 0; j < my_tiles; j++) {
            for (int si = 0; si < nsl; si++, q++) {
                const uint32_t f = fills + (uint32_t)q;
                const uint32_t slot = ring + (f % C::SLOTS) * C::SLOT_BYTES;
                ok = ok && gs_mbar_wait(my_bar + (f % C::SLOTS) * 8, (f / C::SLOTS) & 1u, abort_flag, status, limit_ns);
                if (ok) {
                    const int s = s_lo + si;
                    const uint4 sc0 = gs_lds128(slot + C::SCALE_OFF + g * 16), sc1 = gs_lds128(slot + C::SCALE_OFF + (g + 8) * 16);
                    const uint32_t scw0[4] = {sc0.x, sc0.y, sc0.z, sc0.w}, scw1[4] = {sc1.x, sc1.y, sc1.z, sc1.w};
                    float as[4] = {0.f, 0.f, 0.f, 0.f};
                    constexpr int BPL = (TYPE == PG_GGUF_Q4_0) ? 4 : 2;     // blocks per 128-bit load of a row
#pragma unroll
                    for (int b4 = 0; b4 < GS_SLICE / BPL; b4++) {
                        const uint32_t piece = (uint32_t)(((b4 * 4 + t) ^ ((g & 1) << 2)) * 16);
                        const uint4 qa = gs_lds128(slot + (uint32_t)g * C::SEG + piece);
                        const uint4 qb = gs_lds128(slot + (uint32_t)(g + 8) * C::SEG + piece);
                        const uint32_t wa[4] = {qa.x, qa.y, qa.z, qa.w}, wb[4] = {qb.x, qb.y, qb.z, qb.w};
#pragma unroll
                        for (int bi = 0; bi < BPL; bi++) {
                            const int jb = b4 * BPL + bi;                   // block inside the slice
                            uint32_t r0lo, r0hi, r1lo, r1hi;                // k-slots 4t.., 16+4t.. of rows g and g+8
                            if (TYPE == PG_GGUF_Q4_0) {
                                r0lo = wa[bi] & 0x0F0F0F0Fu;
                                r0hi = (wa[bi] >> 4) & 0x0F0F0F0Fu;
                                r1lo = wb[bi] & 0x0F0F0F0Fu;
                                r1hi = (wb[bi] >> 4) & 0x0F0F0F0Fu;
                            } else {
                                r0lo = wa[2 * bi];
                                r0hi = wa[2 * bi + 1];
                                r1lo = wb[2 * bi];
                                r1hi = wb[2 * bi + 1];
                            }
                            const uint32_t p0 = scw0[jb >> 1], p1 = scw1[jb >> 1];
                            const __half2 h0 = *reinterpret_cast<const __half2 *>(&p0), h1 = *reinterpret_cast<const __half2 *>(&p1);
                            const float d0 = (jb & 1) ? __high2float(h0) : __low2float(h0);
                            const float d1 = (jb & 1) ? __high2float(h1) : __low2float(h1);
                            if (SMALL) {
                                // B operand: column g = digit g % 3 of activation row g / 3 (columns past 3 * rows: any data)
                                const uint32_t pb = planes_s + (uint32_t)((s * GS_SLICE + jb) * ncols + bcol) * 32 + t * 8;
                                const uint2 xd = gs_lds64(pb);
                                uint2 o = make_uint2(0u, 0u);
                                if (TYPE == PG_GGUF_Q4_0) o = gs_lds64(off_s + (uint32_t)((s * GS_SLICE + jb) * 4 * rows + ocol) * 4);
                                int c[4];
                                gs_mma<TYPE>(c, r0lo, r1lo, r0hi, r1hi, xd.x, xd.y, (int)o.x, (int)o.y);
#pragma unroll
                                for (int v = 0; v < 4; v++) as[v] = fmaf(v < 2 ? d0 : d1, __int2float_rn(c[v]), as[v]);
                            } else {
                                // B operand: this lane's activation row is g; rows that do not exist contribute zeros
                                const uint32_t pstride = (uint32_t)rows * 32;
                                const uint32_t pb = planes_s + (uint32_t)((s * GS_SLICE + jb) * 3) * pstride + lane * 8;
                                uint2 x0 = make_uint2(0u, 0u), x1 = x0, x2 = x0;
                                if (g < rows) {
                                    x0 = gs_lds64(pb);
                                    x1 = gs_lds64(pb + pstride);
                                    x2 = gs_lds64(pb + 2 * pstride);
                                }
                                int o0 = 0, o1 = 0;
                                if (TYPE == PG_GGUF_Q4_0) {
                                    const uint32_t ob = off_s + (uint32_t)((s * GS_SLICE + jb) * rows + 2 * t) * 4;
                                    if (2 * t < rows) o0 = *reinterpret_cast<const int *>(gs_smem + ob);
                                    if (2 * t + 1 < rows) o1 = *reinterpret_cast<const int *>(gs_smem + ob + 4);
                                }
                                int c0[4], c1[4], c2[4];
                                gs_mma<TYPE>(c0, r0lo, r1lo, r0hi, r1hi, x0.x, x0.y, o0, o1);
                                gs_mma<TYPE>(c1, r0lo, r1lo, r0hi, r1hi, x1.x, x1.y, 0, 0);
                                gs_mma<TYPE>(c2, r0lo, r1lo, r0hi, r1hi, x2.x, x2.y, 0, 0);
#pragma unroll
                                for (int v = 0; v < 4; v++) {
                                    const int hi = c2[v] * 256 + c1[v];
                                    float cf;
                                    if (TYPE == PG_GGUF_Q4_0)
                                        cf = __int2float_rn((int)((uint32_t)hi * 256u + (uint32_t)c0[v]));   // |sum((q - 8) xi)| <= 2^30
                                    else
                                        cf = fmaf(__int2float_rn(hi), 256.0f, __int2float_rn(c0[v]));
                                    as[v] = fmaf(v < 2 ? d0 : d1, cf, as[v]);
                                }
                            }
                        }
                    }
                    // the slice's sums back on the activations' scale; NaN for a row whose slice held a non-finite value
                    if (SMALL) {
                        // this lane's columns 2t, 2t+1 belong to activation rows ma, mb
                        const float ua = *reinterpret_cast<const float *>(gs_smem + us_s + (uint32_t)(s * 8 + ma) * 4);
                        const float ub = *reinterpret_cast<const float *>(gs_smem + us_s + (uint32_t)(s * 8 + mb) * 4);
                        const float za = *reinterpret_cast<const float *>(gs_smem + ps_s + (uint32_t)(s * 8 + ma) * 4);
                        const float zb = *reinterpret_cast<const float *>(gs_smem + ps_s + (uint32_t)(s * 8 + mb) * 4);
                        acc[0] += as[0] * ua + za;
                        acc[1] += as[1] * ub + zb;
                        acc[2] += as[2] * ua + za;
                        acc[3] += as[3] * ub + zb;
                    } else {
                        const uint2 u = gs_lds64(us_s + (uint32_t)(s * 8 + 2 * t) * 4), pz = gs_lds64(ps_s + (uint32_t)(s * 8 + 2 * t) * 4);
                        acc[0] += as[0] * __uint_as_float(u.x) + __uint_as_float(pz.x);
                        acc[1] += as[1] * __uint_as_float(u.y) + __uint_as_float(pz.y);
                        acc[2] += as[2] * __uint_as_float(u.x) + __uint_as_float(pz.x);
                        acc[3] += as[3] * __uint_as_float(u.y) + __uint_as_float(pz.y);
                    }
                    __syncwarp();                           // every lane has read the slot
                    if (q + C::SLOTS < total) issue(q + C::SLOTS);
                }
            }
            if (SMALL) {
                // join the digits: row 0 = columns 0, 1, 2 (lane t = 0: acc[0], acc[1]; t = 1: acc[0]), row 1 = columns 3, 4, 5
                // (t = 1: acc[1]; t = 2: acc[0], acc[1]); the results go where the store below expects rows 0 and 1: lane t = 0
                const int q4 = lane & ~3;
                float r0[2], r1[2];
#pragma unroll
                for (int h = 0; h < 2; h++) {               // weight rows g and g + 8
                    const float a0 = acc[2 * h], a1 = acc[2 * h + 1];
                    const float t1a0 = __shfl_sync(0xffffffffu, a0, q4 + 1), t1a1 = __shfl_sync(0xffffffffu, a1, q4 + 1);
                    const float t2a0 = __shfl_sync(0xffffffffu, a0, q4 + 2), t2a1 = __shfl_sync(0xffffffffu, a1, q4 + 2);
                    r0[h] = fmaf(t1a0, 65536.0f, fmaf(a1, 256.0f, a0));
                    r1[h] = fmaf(t2a1, 65536.0f, fmaf(t2a0, 256.0f, t1a1));
                }
                acc[0] = r0[0];
                acc[1] = r1[0];
                acc[2] = r0[1];
                acc[3] = r1[1];
            }
            // the kw warps of the tile add up in the first one (fixed order); two buffers by tile parity, so that one barrier
            // per tile is enough
            if (kw > 1) {
                const uint32_t cell = (uint32_t)(j & 1) * 512 + lane * 16;
                if (kpart != 0)
                    *reinterpret_cast<float4 *>(gs_smem + red + cell) = make_float4(acc[0], acc[1], acc[2], acc[3]);
                asm volatile("bar.sync %0, %1;" ::"r"(1 + slot_idx), "r"(kw * 32) : "memory");
                if (kpart == 0) {
                    for (int p = 1; p < kw; p++) {
                        const uint4 o = gs_lds128(red + (uint32_t)p * 1024 + cell);
                        acc[0] += __uint_as_float(o.x);
                        acc[1] += __uint_as_float(o.y);
                        acc[2] += __uint_as_float(o.z);
                        acc[3] += __uint_as_float(o.w);
                    }
                }
            }
            if (kpart == 0 && ok) {
                // C fragment: acc[0], acc[1] -> (weight row g, activation rows 2t, 2t+1); acc[2], acc[3] -> weight row g + 8
                const int64_t n0 = (first + (int64_t)j * tstep) * 16 + g;
#pragma unroll
                for (int v = 0; v < 4; v++) {
                    const int64_t n = n0 + (v >> 1) * 8;
                    const int m = m0 + 2 * t + (v & 1);
                    if (n < N && m < M) {
                        float *dst = y + (int64_t)m * N + n;
                        *dst = (chunk > 0) ? (*dst + acc[v]) : acc[v];   // the same lane wrote *dst in the chunk before
                    }
                }
            }
            acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
        }
        fills += (uint32_t)total;
    }
}

template <int TYPE, int W, int ROWS>
int32_t gs_launch(pg_ctx *ctx, const float *d_x, int M, int m0, int rows, const pg_gguf_weight *w, float *d_y)
{
    using C = GsCfg<TYPE, W, ROWS == 1 || ROWS == 2>;
    static_assert(C::SMEM <= 227 * 1024, "shared memory budget");
    auto kern = gguf_stream_kernel<TYPE, W, ROWS>;
    static std::atomic<uint64_t> smem_set{0};
    PG_CUDA(pg_max_smem_once(kern, C::SMEM, ctx->device, smem_set));
    const int nblk = (int)(w->k / 32);
    const int64_t tiles = (w->n + 15) / 16;
    // warps per tile: as few as still give about three quarters of the GPU's warps a part of a tile
    int kw = 1;
    while (kw < 8 && tiles * kw * 4 < (int64_t)ctx->sm_count * W * 3) kw *= 2;
    // tiles go round the CTAs first (tile = CTA + grid * group), so with every SM in the grid a CTA has at most one busy group
    // more than another: 896 tiles on 148 SMs are 6 or 7 busy groups of 8 per CTA, not 8 on 112 SMs and 36 SMs idle
    // (this kernel is bound by instruction issue: 15.0 against 15.9 us at N 14336, K 4096, one row)
    const int grid = (int)std::min<int64_t>(ctx->sm_count, tiles);
    int cslices = 8;                                        // slices per chunk: what the plane area holds for `rows` rows
    while (cslices * 2 * rows <= C::ROW_SLICES && cslices < GS_MAX_SLICES) cslices *= 2;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(W * 32);
    cfg.dynamicSmemBytes = C::SMEM;
    cfg.stream = ctx->stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    PG_CUDA(cudaLaunchKernelEx(&cfg, kern, d_x, (const uint8_t *)w->d_qs, w->n, nblk, M, m0, rows, cslices, d_y, kw, ctx->d_status,
                               ctx->wait_limit_ns));
    PG_LAUNCHED();
    return PG_OK;
}

template <int TYPE>
int32_t gs_run(pg_ctx *ctx, const float *d_x, int64_t m, const pg_gguf_weight *w, float *d_y)
{
    const int M = (int)m;
    for (int m0 = 0; m0 < M; m0 += 8) {
        const int rows = std::min(8, M - m0);
        const int32_t rc = rows == 1   ? gs_launch<TYPE, 16, 1>(ctx, d_x, M, m0, rows, w, d_y)
                           : rows == 2 ? gs_launch<TYPE, 16, 2>(ctx, d_x, M, m0, rows, w, d_y)
                           // (eight rows as a constant: 20.9 against 21.7 us for Q8_0, but 21.9 against 21.2 us for Q4_0, whose
                           // inner loop then spills)
                           : (rows == 8 && TYPE == PG_GGUF_Q8_0) ? gs_launch<TYPE, 16, 8>(ctx, d_x, M, m0, rows, w, d_y)
                                       : gs_launch<TYPE, 16, 0>(ctx, d_x, M, m0, rows, w, d_y);
        if (rc != PG_OK) return rc;
    }
    return PG_OK;
}

}  // namespace

bool pgk_matmul_gguf_stream_supports(const pg_gguf_weight *w, int64_t m)
{
    return w->tiled && m >= 1 && w->n >= 1;
}

int32_t pgk_matmul_gguf_stream(pg_ctx *ctx, const float *d_x, int64_t m, const pg_gguf_weight *w, float *d_y)
{
    if (w->type == PG_GGUF_Q4_0) return gs_run<PG_GGUF_Q4_0>(ctx, d_x, m, w, d_y);
    return gs_run<PG_GGUF_Q8_0>(ctx, d_x, m, w, d_y);
}
