// Dequantising product y = x . dequant(W)^T for GGUF Q4_0 / Q8_0 weights, decode sizes, on the
// tensor cores.  It replaces, without ever writing the f32 weight, what the reference does in three
// passes: gguf::dequant_q4_0 / dequant_q8_0 (src/gguf.rs:286-326), the transposition of
// load_transposed_weight (src/models/llama/model.rs:243-257) and Tensor::matmul
// (src/tensor.rs:1342-1354).
//
// Why tensor cores for a bandwidth-bound op: with f32 activations a CUDA-core kernel needs one
// FMA per weight and activation row plus the nibble->float conversions, which caps it far below
// the HBM rate already at M = 8.  Here
//   * the quants go to the MMA as exact fp16 integers, built with two logic ops per pair from the
//     packed nibbles/bytes (exponent-bias trick: 0x6400 | u is the half 1024 + u);
//   * each f32 activation is split into two fp16 parts, x * 2^s = hi + lo (s a power of two, per
//     activation row and per 256-element slice of K, that brings the slice's largest element into
//     [8,16), so that lo keeps an absolute precision of 2^-25 on that scale); every product
//     quant x part is exact and the sums accumulate in f32 inside the MMA;
//   * per 32-element block the partial sum is multiplied by the block's f16 scale: y += d * sum.
// The result differs from the reference's strictly sequential f32 loop only in summation order
// and in the 2^-28 relative truncation of the activations (documented tolerance: 1e-5 of max|y|;
// measured a few 1e-6, which is also the sequential f32 loop's own distance from an f64 sum).
//
// Data flow, per CTA of 16 warps (one CTA per SM, persistent over tiles of 16*R weight rows), ONE
// launch per eight activation rows whatever K is:
//   * K is walked in chunks of 128 blocks (4096 elements).  Inside a chunk warp w owns a fixed
//     slice of eight 32-element blocks and builds the activation fragments of that slice itself,
//     straight from the f32 activations (slice maximum, power-of-two scale, hi/lo split), and
//     keeps them in registers for all the CTA's tiles: activations cost no memory traffic in the
//     main loop whatever M is, and no separate preparation kernel runs;
//   * the quants stream through a lane-private cp.async FIFO in shared memory (128-bit copies,
//     L2 only), several entries deep, so HBM requests stay in flight across tile boundaries.  The
//     upload interleaves each 64-byte group of quants so that the 16 bytes a lane needs for the
//     group's blocks are contiguous: a lane copies exactly what it will read back;
//   * per tile the 16 warps' partial sums meet in shared memory (fixed order: deterministic);
//     chunks after the first add onto y (the same CTA owns a tile in every chunk).
#include <cuda_fp16.h>

#include "pg_internal.cuh"

namespace {

constexpr int G_WARPS = 16;
constexpr int G_THREADS = G_WARPS * 32;
constexpr int G_SLICE = 8;                      // blocks of K per warp
constexpr int G_CHUNK = G_WARPS * G_SLICE;      // 128 blocks = 4096 elements per launch
// One FIFO entry of a warp: 16 B of quants per lane for rows g and g+8 (lane-private), then, filled
// only by the first step of a row group, the 16 B of block scales (eight f16) of each of the 16 rows.
constexpr int G_QAREA = 2 * 32 * 16;
constexpr int G_WSLOT = G_QAREA + 16 * 16;      // 1280 B per warp and entry
constexpr int G_SLOT_BYTES = G_WARPS * G_WSLOT;  // one entry for the whole CTA

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, uint32_t n)
{
    asm volatile("cp.async.cg.shared.global.L2::128B [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait()
{
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t a)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t sub_f16x2(uint32_t a, uint32_t b)
{
    uint32_t d;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t lop_and_or(uint32_t a, uint32_t mask, uint32_t magic)
{
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(mask), "r"(magic));  // (a & mask) | magic
    return d;
}
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// the eight quants of one block that lane t owns, as four fp16 pairs
template <int TYPE>
__device__ __forceinline__ void unpack(uint32_t w0, uint32_t w1, uint32_t (&a)[4])
{
    if (TYPE == PG_GGUF_Q4_0) {
        // w0 = word t of the block: nibbles e0..e7 from bit 0 up.  Pairs (e0,e4) (e1,e5)*16 (e2,e6) (e3,e7)*16.
        const uint32_t w8 = w0 >> 8;
        a[0] = sub_f16x2(lop_and_or(w0, 0x000F000Fu, 0x64006400u), 0x64086408u);
        a[1] = sub_f16x2(lop_and_or(w0, 0x00F000F0u, 0x64006400u), 0x64806480u);
        a[2] = sub_f16x2(lop_and_or(w8, 0x000F000Fu, 0x64006400u), 0x64086408u);
        a[3] = sub_f16x2(lop_and_or(w8, 0x00F000F0u, 0x64006400u), 0x64806480u);
    } else {
        // w0, w1 = bytes 8t..8t+7 of the block; q + 128 as unsigned bytes, then 0x6400 | u = 1024 + u
        const uint32_t u0 = w0 ^ 0x80808080u, u1 = w1 ^ 0x80808080u;
        a[0] = sub_f16x2(__byte_perm(u0, 0x64646464u, 0x4140), 0x64806480u);
        a[1] = sub_f16x2(__byte_perm(u0, 0x64646464u, 0x4342), 0x64806480u);
        a[2] = sub_f16x2(__byte_perm(u1, 0x64646464u, 0x4140), 0x64806480u);
        a[3] = sub_f16x2(__byte_perm(u1, 0x64646464u, 0x4342), 0x64806480u);
    }
}

// ---- activation fragments -------------------------------------------------------------------
// B operand of one 32-element block b, part p (0 = hi, 1 = lo): 32 lanes x 16 bytes, lane = (row % 8) * 4 + t
// holding the eight elements 8t..8t+7 of the block in the order the weight unpacking produces them:
//   Q8_0: e0 e1 e2 e3 e4 e5 e6 e7
//   Q4_0: e0 e4 e1' e5' e2 e6 e3' e7'   (' = divided by 16: the high nibbles are unpacked as 16*q)
template <int TYPE>
__device__ __forceinline__ void make_fragment(const float (&v)[8], uint4 &hi4, uint4 &lo4)
{
    float o[8];
    if (TYPE == PG_GGUF_Q4_0) {
        const float h = 0.0625f;
        o[0] = v[0]; o[1] = v[4]; o[2] = v[1] * h; o[3] = v[5] * h;
        o[4] = v[2]; o[5] = v[6]; o[6] = v[3] * h; o[7] = v[7] * h;
    } else {
#pragma unroll
        for (int j = 0; j < 8; j++) o[j] = v[j];
    }
    uint32_t hi[4], lo[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const __half h0 = __float2half_rn(o[2 * j]), h1 = __float2half_rn(o[2 * j + 1]);
        const __half l0 = __float2half_rn(o[2 * j] - __half2float(h0));
        const __half l1 = __float2half_rn(o[2 * j + 1] - __half2float(h1));
        hi[j] = (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h1) << 16);
        lo[j] = (uint32_t)__half_as_ushort(l0) | ((uint32_t)__half_as_ushort(l1) << 16);
    }
    hi4 = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    lo4 = make_uint4(lo[0], lo[1], lo[2], lo[3]);
}

// ---- the product -----------------------------------------------------------------------------
// BPS = blocks per 64-byte step of a row's quants: 4 for Q4_0 (16 B per block), 2 for Q8_0 (32 B).
// Interleaved quant layout (made at upload): inside each 64-byte group, the 16-byte chunk t holds
//   Q4_0: word t (nibbles 8t..8t+7) of the group's blocks 0,1,2,3
//   Q8_0: bytes 8t..8t+7 of block 0, then of block 1.
template <int TYPE, int R, int D>
__global__ void __launch_bounds__(G_THREADS, 1)
    gguf_mma_kernel(const float *__restrict__ x, const uint8_t *__restrict__ qs, const uint16_t *__restrict__ dd, int64_t N,
                    int nblk_row, int M, int m0, float *__restrict__ y)
{
    constexpr int BPS = (TYPE == PG_GGUF_Q4_0) ? 4 : 2;
    constexpr int STEPS = G_SLICE / BPS;          // steps per warp per row group
    constexpr int QB = (TYPE == PG_GGUF_Q4_0) ? 16 : 32;  // bytes of quants per block
    constexpr int TROWS = 16 * R;
    extern __shared__ uint4 smem_g[];
    // [D] entries of G_SLOT_BYTES, then float red[2][WARPS][R][8][16]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t wbase = (uint32_t)__cvta_generic_to_shared(smem_g) + warp * G_WSLOT;
    float *red = reinterpret_cast<float *>(reinterpret_cast<char *>(smem_g) + (size_t)D * G_SLOT_BYTES);
    const int wblk = warp * G_SLICE;              // first block of this warp's slice inside a chunk
    const int64_t tiles = (N + TROWS - 1) / TROWS;
    const int my_tiles = (tiles > blockIdx.x) ? (int)((tiles - blockIdx.x + gridDim.x - 1) / gridDim.x) : 0;
    const int nchunks = (nblk_row + G_CHUNK - 1) / G_CHUNK;

    // Issue side of the FIFO: walks (chunk, tile, row group, step) in the order the consumer does.  Each lane
    // copies its own 16 bytes of rows g and g+8; the first step of a row group also brings the block
    // scales of the warp's K slice for those rows (lanes t = 0, 1 copy them for g and g+8).
    // State: the block index of the start of rows g and g+8 of the current row group (rb0, rb1; -1 past the
    // edge of the matrix or of this CTA's work) and the first block of the current step inside the row (ib).
    int i_chunk = 0, i_tile = 0, i_step = 0, i_rg = 0, i_slot = 0;
    int64_t rb0 = -1, rb1 = -1;
    int ib = wblk;
    auto place = [&]() {   // row starts for (i_tile, i_rg); called when either changes
        const int64_t row = (blockIdx.x + (int64_t)i_tile * gridDim.x) * TROWS + i_rg * 16 + g;
        const bool live = (i_chunk < nchunks) && (i_tile < my_tiles);
        rb0 = (live && row < N) ? row * nblk_row : -1;
        rb1 = (live && row + 8 < N) ? (row + 8) * nblk_row : -1;
    };
    place();
    auto issue = [&]() {
        const uint32_t slot = wbase + (uint32_t)i_slot * G_SLOT_BYTES;
        const bool kok = ib < nblk_row;
        {
            const bool ok = kok && rb0 >= 0;
            const int64_t blk = ok ? rb0 + ib : 0;
            cp_async16(slot + lane * 16, qs + blk * QB + t * 16, ok ? 16u : 0u);
            if (i_step == 0 && t == 0) cp_async16(slot + G_QAREA + g * 16, dd + blk, ok ? 16u : 0u);
        }
        {
            const bool ok = kok && rb1 >= 0;
            const int64_t blk = ok ? rb1 + ib : 0;
            cp_async16(slot + (32 + lane) * 16, qs + blk * QB + t * 16, ok ? 16u : 0u);
            if (i_step == 0 && t == 1) cp_async16(slot + G_QAREA + (8 + g) * 16, dd + blk, ok ? 16u : 0u);
        }
        cp_commit();
        if (++i_slot == D) i_slot = 0;
        ib += BPS;
        if (++i_step == STEPS) {
            i_step = 0;
            ib -= STEPS * BPS;
            if (++i_rg == R) {
                i_rg = 0;
                if (++i_tile >= my_tiles) {
                    i_tile = 0;
                    ++i_chunk;
                    ib += G_CHUNK;
                }
            }
            place();
        }
    };
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (my_tiles > 0) {
#pragma unroll
        for (int i = 0; i < D - 1; i++) issue();
    }
    // the activations come from the preceding kernel
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (my_tiles == 0) return;

    const int xrow = m0 + g;                       // as B-operand owner this lane holds activation row g, elements 8t..8t+7
    const bool live = xrow < M;
    const float *xr = x + (int64_t)(live ? xrow : 0) * nblk_row * 32 + t * 8;
    int c_slot = 0, ti_all = 0;
    for (int chunk = 0; chunk < nchunks; chunk++) {
        const int blk0 = chunk * G_CHUNK;
        // ---- this warp's activation fragments for the chunk: slice maximum, power-of-two scale, hi/lo split
        float amax = 0.0f;
#pragma unroll
        for (int j = 0; j < G_SLICE; j++) {
            const int b = blk0 + wblk + j;
            if (live && b < nblk_row) {
                const float4 p = pg_ld_fresh(reinterpret_cast<const float4 *>(xr + (int64_t)b * 32));
                const float4 q = pg_ld_fresh(reinterpret_cast<const float4 *>(xr + (int64_t)b * 32) + 1);
                amax = fmaxf(amax, fmaxf(fmaxf(fmaxf(fabsf(p.x), fabsf(p.y)), fmaxf(fabsf(p.z), fabsf(p.w))),
                                         fmaxf(fmaxf(fabsf(q.x), fabsf(q.y)), fmaxf(fabsf(q.z), fabsf(q.w)))));
            }
        }
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        int e = 0;
        if (amax > 0.0f && amax < INFINITY) e = max(-100, min(100, ilogbf(amax)));
        const float sc = scalbnf(1.0f, 3 - e);    // |x| * sc < 16 on the slice
        const float unscale = scalbnf(1.0f, e - 3);
        uint4 xh[G_SLICE], xl[G_SLICE];
#pragma unroll
        for (int j = 0; j < G_SLICE; j++) {
            const int b = blk0 + wblk + j;
            float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (live && b < nblk_row) {
                const float4 p = pg_ld_fresh(reinterpret_cast<const float4 *>(xr + (int64_t)b * 32));
                const float4 q = pg_ld_fresh(reinterpret_cast<const float4 *>(xr + (int64_t)b * 32) + 1);
                v[0] = p.x * sc; v[1] = p.y * sc; v[2] = p.z * sc; v[3] = p.w * sc;
                v[4] = q.x * sc; v[5] = q.y * sc; v[6] = q.z * sc; v[7] = q.w * sc;
            }
            make_fragment<TYPE>(v, xh[j], xl[j]);
        }
        // as accumulator owner this lane holds activation rows 2t and 2t+1: their scales live in lanes 8t and 8t+4
        const float us0 = __shfl_sync(0xffffffffu, unscale, 8 * t), us1 = __shfl_sync(0xffffffffu, unscale, 8 * t + 4);

        for (int ti = 0; ti < my_tiles; ti++, ti_all++) {
            float *mine = red + ((size_t)(ti_all & 1) * G_WARPS + warp) * (R * 128);
#pragma unroll
            for (int rg = 0; rg < R; rg++) {
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                uint4 sc0, sc1;  // eight f16 block scales of rows g and g+8 (this warp's K slice)
#pragma unroll
                for (int step = 0; step < STEPS; step++) {
                    issue();
                    cp_wait<D - 1>();
                    const uint32_t slot = wbase + (uint32_t)c_slot * G_SLOT_BYTES;
                    if (++c_slot == D) c_slot = 0;
                    if (step == 0) {
                        __syncwarp();  // the scales were copied by other lanes of the group
                        sc0 = lds128(slot + G_QAREA + g * 16);
                        sc1 = lds128(slot + G_QAREA + (8 + g) * 16);
                    }
                    const uint4 qa = lds128(slot + lane * 16), qb = lds128(slot + (32 + lane) * 16);  // rows g, g+8
                    const uint32_t wa[4] = {qa.x, qa.y, qa.z, qa.w}, wb[4] = {qb.x, qb.y, qb.z, qb.w};
#pragma unroll
                    for (int bi = 0; bi < BPS; bi++) {
                        const int j = step * BPS + bi;  // block inside the warp's slice
                        uint32_t a0[4], a1[4];          // rows g and g+8
                        if (TYPE == PG_GGUF_Q4_0) {
                            unpack<TYPE>(wa[bi], 0u, a0);
                            unpack<TYPE>(wb[bi], 0u, a1);
                        } else {
                            unpack<TYPE>(wa[2 * bi], wa[2 * bi + 1], a0);
                            unpack<TYPE>(wb[2 * bi], wb[2 * bi + 1], a1);
                        }
                        float c[4] = {0.f, 0.f, 0.f, 0.f};
                        mma_f16(c, a0[0], a1[0], a0[1], a1[1], xh[j].x, xh[j].y);
                        mma_f16(c, a0[2], a1[2], a0[3], a1[3], xh[j].z, xh[j].w);
                        mma_f16(c, a0[0], a1[0], a0[1], a1[1], xl[j].x, xl[j].y);
                        mma_f16(c, a0[2], a1[2], a0[3], a1[3], xl[j].z, xl[j].w);
                        // f16 scale of block j of the slice, rows g and g+8
                        const uint32_t p0 = (j < 2) ? sc0.x : (j < 4) ? sc0.y : (j < 6) ? sc0.z : sc0.w;
                        const uint32_t p1 = (j < 2) ? sc1.x : (j < 4) ? sc1.y : (j < 6) ? sc1.z : sc1.w;
                        const __half2 h0 = *reinterpret_cast<const __half2 *>(&p0), h1 = *reinterpret_cast<const __half2 *>(&p1);
                        const float d0 = (j & 1) ? __high2float(h0) : __low2float(h0);
                        const float d1 = (j & 1) ? __high2float(h1) : __low2float(h1);
                        acc[0] = fmaf(d0, c[0], acc[0]);
                        acc[1] = fmaf(d0, c[1], acc[1]);
                        acc[2] = fmaf(d1, c[2], acc[2]);
                        acc[3] = fmaf(d1, c[3], acc[3]);
                    }
                }
                // partial sums of this warp's K slice (scaling undone) -> shared memory, [buf][warp][rg][m 0..7][row 0..15]
                mine[rg * 128 + (2 * t) * 16 + g] = acc[0] * us0;
                mine[rg * 128 + (2 * t + 1) * 16 + g] = acc[1] * us1;
                mine[rg * 128 + (2 * t) * 16 + g + 8] = acc[2] * us0;
                mine[rg * 128 + (2 * t + 1) * 16 + g + 8] = acc[3] * us1;
            }
            __syncthreads();
            const int64_t tile = blockIdx.x + (int64_t)ti * gridDim.x;
            for (int idx = threadIdx.x; idx < 8 * TROWS; idx += G_THREADS) {
                const int mm = idx / TROWS, nn = idx - mm * TROWS;     // consecutive threads -> consecutive n
                const int rg = nn >> 4, row = nn & 15;
                const int64_t n = tile * TROWS + nn;
                if (m0 + mm >= M || n >= N) continue;
                const float *src = red + (size_t)(ti_all & 1) * G_WARPS * (R * 128) + rg * 128 + mm * 16 + row;
                float sum = 0.0f;
#pragma unroll
                for (int w = 0; w < G_WARPS; w++) sum += src[(size_t)w * (R * 128)];
                float *dst = y + (int64_t)(m0 + mm) * N + n;
                *dst = (chunk > 0) ? (*dst + sum) : sum;   // the same thread wrote *dst in the chunk before
            }
        }
    }
    cp_wait<0>();
}

template <int TYPE, int R, int D>
int32_t run(pg_ctx *ctx, const float *d_x, int64_t m, const pg_gguf_weight *w, float *d_y)
{
    const int K = (int)w->k, nblk = K / 32, M = (int)m;
    const size_t smem = (size_t)D * G_SLOT_BYTES + 2 * G_WARPS * R * 128 * sizeof(float);
    auto kern = gguf_mma_kernel<TYPE, R, D>;
    static std::atomic<uint64_t> smem_set{0};
    PG_CUDA(pg_max_smem_once(kern, (int)smem, ctx->device, smem_set));
    const int64_t tiles = (w->n + 16 * R - 1) / (16 * R);
    const int grid = (int)(tiles < ctx->sm_count ? tiles : ctx->sm_count);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    for (int m0 = 0; m0 < M; m0 += 8) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(G_THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = ctx->stream;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        PG_CUDA(cudaLaunchKernelEx(&cfg, kern, d_x, (const uint8_t *)w->d_qs, (const uint16_t *)w->d_d, w->n, nblk, M, m0, d_y));
        PG_LAUNCHED();
    }
    return PG_OK;
}

}  // namespace

static int g_gguf_rows = 0;  // tuning: row groups per tile, 0 = heuristic
extern "C" PG_API void pg_tune_gguf_rows(int r) { g_gguf_rows = r; }

bool pgk_matmul_gguf_mma_supports(const pg_gguf_weight *w, int64_t m)
{
    return w->interleaved && m >= 1 && m <= 64 && w->n >= 1;
}

int32_t pgk_matmul_gguf_mma(pg_ctx *ctx, const float *d_x, int64_t m, const pg_gguf_weight *w, float *d_y)
{
    // One 16-row group per tile when that is what it takes to give every SM several tiles.
    const bool fine = g_gguf_rows ? (g_gguf_rows == 1) : (w->n < 64ll * 32 * ctx->sm_count);
    if (w->type == PG_GGUF_Q4_0)
        return fine ? run<PG_GGUF_Q4_0, 1, 8>(ctx, d_x, m, w, d_y) : run<PG_GGUF_Q4_0, 2, 6>(ctx, d_x, m, w, d_y);
    return fine ? run<PG_GGUF_Q8_0, 1, 8>(ctx, d_x, m, w, d_y) : run<PG_GGUF_Q8_0, 2, 6>(ctx, d_x, m, w, d_y);
}
