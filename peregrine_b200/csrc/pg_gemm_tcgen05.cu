// Prefill-size W8A8 product: the integer GEMM of src/quant.rs:154-166 /
// simd_kernels::gemm_i8_sdot (src/simd_kernels.rs:1087-1214) on the 5th-generation tensor
// cores.
//
//   A = quantised activations [M,K] i8 (K-major), B = data_i8_t [N,K] i8 (K-major): both are
//   exactly the layouts the reference keeps, so no repacking is needed.
//   D[128 x BN] s32 accumulates in tensor memory (TMEM), two accumulators so that the epilogue
//   of one tile overlaps the main loop of the next.
//
// One persistent CTA per SM, warp-specialised:
//   warp 0   producer   TMA (cp.async.bulk.tensor, 128B swizzle) of a 128 x 128B tile of A and a
//                       BN x 128B tile of B into a ring of shared-memory stages
//   warp 1   MMA        one elected lane issues tcgen05.mma.cta_group::1.kind::i8 (M=128, N=BN,
//                       K=32 per instruction, four per stage); tcgen05.commit releases stages
//                       and publishes finished accumulators
//   warps 2-5 epilogue  tcgen05.ld of their TMEM lane quarter, then
//                       `acc as f32 * a_scale[m] * w_scale[n]` as two rounded products, stored
//                       straight to global memory (and the raw s32 sums when asked for)
//
// Integer accumulation is exact, so the result is bit-identical to the scalar loop whatever the
// tiling.  Rows/columns/K past the matrix edge are zero-filled by TMA and masked on store.
//
// Every mbarrier wait is bounded: a wait that sees no progress for about a second records
// PG_ERR_DEVICE_TIMEOUT in the context's status word, raises a CTA-wide abort flag that all
// other waits poll, and the CTA leaves through the normal teardown (TMEM is freed).
#include <cuda.h>

#include "pg_internal.cuh"
#include "pg_tc_epilogue.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 128;  // bytes of K per stage = one 128-byte swizzle span
constexpr int UMMA_K = 32;
constexpr int NUM_THREADS = 192;
constexpr unsigned long long WAIT_LIMIT_NS = 1000ull * 1000ull * 1000ull;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long globaltimer()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity)
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

// Bounded wait.  Returns false when the CTA is aborting (this wait or another one gave up).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int32_t *status)
{
    unsigned long long t0 = 0;
    for (uint32_t it = 1;; ++it) {
        if (mbar_try(bar, parity)) return true;
        if ((it & 0xff) == 0) {
            if (*abort_flag) return false;
            const unsigned long long now = globaltimer();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > WAIT_LIMIT_NS) {
                *abort_flag = 1;
                atomicExch(status, (int32_t)PG_ERR_DEVICE_TIMEOUT);
                return false;
            }
        }
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *tmap, uint32_t bar, int x, int y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
        "l"(tmap), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(d_tmem), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
          "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// K-major operand tile in shared memory, 128-byte swizzle: rows are 128 B apart, groups of
// eight rows 1024 B apart (stride byte offset), leading byte offset unused by swizzled K-major
// layouts (encoded 1), descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// kind::i8 instruction descriptor: D = s32 (2 at bit 4), A and B = signed 8-bit (1 at bits 7 and
// 10), both K-major (bits 15, 16 clear), N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n)
{
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// AR: rows of A one copy brings (32 or 64 where M is that small, else 128).  The MMA always reads a 128-row A tile; with
// AR < 128 the rows behind the copied ones are whatever follows in shared memory (the stage's B tile, the next stage):
// they only feed accumulator rows >= M, which the epilogue never stores.  What the smaller A tile buys is a deeper ring
// in the same shared memory, and the ring's depth is what bounds this kernel at small M.
__host__ __device__ constexpr int ring_stages(int bn, int ar)
{
    const int stage = ar * BK + bn * BK;
    const int room = 232448 - (1024 + 256 + 4 * PG_EPI_WARP_BYTES);
    const int fit = room / stage;
    return fit > 12 ? 12 : fit;   // the barrier block holds 2 * 12 + 4 barriers
}

template <int BN, int AR>
struct Cfg {
    static constexpr int STAGE_A = AR * BK;
    static constexpr int STAGE_B = BN * BK;
    static constexpr int STAGE = STAGE_A + STAGE_B;
    static constexpr int STAGES = ring_stages(BN, AR);
    static constexpr int TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;  // power of two >= 32
    static constexpr size_t SMEM = (size_t)STAGES * STAGE + 1024 /*alignment slack*/ + 256 /*barriers*/ + 4 * PG_EPI_WARP_BYTES;
};

template <int BN, int AR>
__global__ void __launch_bounds__(NUM_THREADS, 1)
    gemm_i8_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                           const float *__restrict__ a_scales, const float *__restrict__ w_scales, int M, int N, int K,
                           float *__restrict__ y, int32_t *__restrict__ acc_out, int32_t *status, int splits, int32_t *__restrict__ ws,
                           unsigned int *__restrict__ tickets)
{
    using C = Cfg<BN, AR>;
    constexpr int STAGES = C::STAGES;
    // Programmatic dependent launch: the next kernel may start its prologue now, and this one started while its
    // predecessor (the activation quantiser) was still running.  What the predecessor wrote -- the activations and their
    // scales -- is touched only behind griddepcontrol.wait; the weights are requested before it.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (base - raw_addr);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (size_t)STAGES * C::STAGE);
    // full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]
    const uint32_t bar_full = smem_u32(bars);
    const uint32_t bar_empty = bar_full + 8 * STAGES;
    const uint32_t bar_tfull = bar_empty + 8 * STAGES;
    const uint32_t bar_tempty = bar_tfull + 16;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (M + BM - 1) / BM;
    const int tiles_n = (N + BN - 1) / BN;
    const int kblocks = (K + BK - 1) / BK;
    // Split K (splits > 1, one row of tiles): a unit is (tile, part of the k-blocks); every part writes its s32 sums to a
    // slab of its own in the workspace (plain 128-bit stores), and whichever part of a tile arrives last (a ticket per tile
    // and accumulator-lane quarter) adds the slabs up, applies the scales and writes y.  Nobody waits for anybody, and
    // integer sums are exact in any order.  (Adding the parts with red.global.add.s32 into one zeroed matrix was the first
    // form: 15 to 60 us slower, four-byte reductions run at about 35 G/s.)
    const int total_tiles = tiles_m * tiles_n * splits;   // units
    const int kpb = (kblocks + splits - 1) / splits;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(bar_tfull + 8 * i, 1);
            mbar_init(bar_tempty + 8 * i, 4);  // one arrival per epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- producer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            // the weight tiles of the first stages of this CTA's first tile, before the predecessor has finished
            int early = 0;
            if ((int)blockIdx.x < total_tiles) {
                const int u = (int)blockIdx.x, tile = u / splits, kb0 = (u - tile * splits) * kpb;
                const int n0 = (tile / tiles_m) * BN;
                const int mine = min(kblocks, kb0 + kpb) - kb0;
                early = mine < STAGES ? mine : STAGES;
                for (int i = 0; i < early; i++) {
                    mbar_arrive_expect_tx(bar_full + 8 * i, C::STAGE);
                    tma_load_2d(base + i * C::STAGE + C::STAGE_A, &tmap_b, bar_full + 8 * i, (kb0 + i) * BK, n0);
                }
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int u = blockIdx.x; ok && u < total_tiles; u += gridDim.x) {
                const int t = u / splits, kb0 = (u - t * splits) * kpb, kb1 = min(kblocks, kb0 + kpb);
                const int m0 = (t % tiles_m) * BM;
                const int n0 = (t / tiles_m) * BN;
                for (int kb = kb0; kb < kb1; kb++) {
                    if (!(ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, status))) break;
                    const uint32_t sa = base + stage * C::STAGE;
                    if (early > 0) {
                        early--;                            // announced and half filled above
                    } else {
                        mbar_arrive_expect_tx(bar_full + 8 * stage, C::STAGE);
                        tma_load_2d(sa + C::STAGE_A, &tmap_b, bar_full + 8 * stage, kb * BK, n0);
                    }
                    tma_load_2d(sa, &tmap_a, bar_full + 8 * stage, kb * BK, m0);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
            if (!ok) {
                // give copies that are still in flight a bounded time to land before the CTA exits
                const unsigned long long t0 = globaltimer();
                while (globaltimer() - t0 < 2000000ull) {
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BM, BN);
            uint32_t stage = 0, phase = 0;
            uint32_t acc = 0, acc_phase = 0;
            bool ok = true;
            for (int u = blockIdx.x; ok && u < total_tiles; u += gridDim.x) {
                const int kb0 = (u % splits) * kpb, kb1 = min(kblocks, kb0 + kpb);
                if (!(ok = mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag, status))) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = kb0; kb < kb1; kb++) {
                    if (!(ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag, status))) break;
                    tc_fence_after();
                    const uint32_t sa = base + stage * C::STAGE;
                    const uint64_t da = make_smem_desc(sa);
                    const uint64_t db = make_smem_desc(sa + C::STAGE_A);
#pragma unroll
                    for (int j = 0; j < BK / UMMA_K; j++) {
                        // +32 bytes of K inside the swizzle span = +2 in the 16-byte address field
                        umma_i8(d_tmem, da + (uint64_t)(j * (UMMA_K >> 4)), db + (uint64_t)(j * (UMMA_K >> 4)), idesc,
                                (kb != kb0 || j != 0) ? 1u : 0u);
                    }
                    umma_commit(bar_empty + 8 * stage);  // stage reusable once these MMAs have read it
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                umma_commit(bar_tfull + 8 * acc);  // accumulator complete
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1;
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const int q = warp & 3;  // TMEM lane quarter this warp may read
        asm volatile("griddepcontrol.wait;" ::: "memory");   // a_scales come from the predecessor; y may still be read by it
        uint32_t acc = 0, acc_phase = 0;
        const bool vec_ok = ((N & 3) == 0) && (((uintptr_t)y & 15) == 0) && (((uintptr_t)acc_out & 15) == 0) &&
                            (((uintptr_t)w_scales & 15) == 0);
        bool ok = true;
        for (int u = blockIdx.x; ok && u < total_tiles; u += gridDim.x) {
            const int t = u / splits;
            const int m0 = (t % tiles_m) * BM;
            const int n0 = (t / tiles_m) * BN;
            ok = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, status);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int row_base = m0 + q * 32;
            const int row = row_base + lane;
            const float as = (row < M && y) ? a_scales[row] : 0.0f;
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
            const uint32_t stage_buf = base + (uint32_t)((size_t)STAGES * C::STAGE) + 256u + (uint32_t)q * PG_EPI_WARP_BYTES;
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t v[32];
                tmem_ld32(taddr + c, v);
                if (row_base >= M || n0 + c >= N) continue;   // uniform over the warp
                const int64_t off0 = (int64_t)row_base * N + n0 + c;
                if (splits > 1) {
                    // (the host takes this path only when the vector conditions hold)
                    pg_store_block_32x32(reinterpret_cast<uint32_t *>(ws + (int64_t)(u - t * splits) * M * N + off0), N, M - row_base,
                                         N - (n0 + c), stage_buf, lane, v);
                } else if (vec_ok) {
                    // coalesced: the warp exchanges the block through shared memory and writes whole row segments
                    if (acc_out) pg_store_block_32x32(reinterpret_cast<uint32_t *>(acc_out + off0), N, M - row_base, N - (n0 + c), stage_buf, lane, v);
                    if (y) {
                        uint32_t o[32];
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            float4 ws = make_float4(0.f, 0.f, 0.f, 0.f);
                            if (n0 + c + j < N) ws = __ldg(reinterpret_cast<const float4 *>(w_scales + n0 + c + j));
                            o[j] = __float_as_uint(__fmul_rn(__fmul_rn(__int2float_rn((int)v[j]), as), ws.x));
                            o[j + 1] = __float_as_uint(__fmul_rn(__fmul_rn(__int2float_rn((int)v[j + 1]), as), ws.y));
                            o[j + 2] = __float_as_uint(__fmul_rn(__fmul_rn(__int2float_rn((int)v[j + 2]), as), ws.z));
                            o[j + 3] = __float_as_uint(__fmul_rn(__fmul_rn(__int2float_rn((int)v[j + 3]), as), ws.w));
                        }
                        pg_store_block_32x32(reinterpret_cast<uint32_t *>(y + off0), N, M - row_base, N - (n0 + c), stage_buf, lane, o);
                    }
                } else if (row < M) {
                    const int64_t off = off0 + (int64_t)lane * N;
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        if (n0 + c + j < N) {
                            if (acc_out) acc_out[off + j] = (int)v[j];
                            if (y) y[off + j] = __fmul_rn(__fmul_rn(__int2float_rn((int)v[j]), as), __ldg(w_scales + n0 + c + j));
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1;
            }
            if (splits > 1 && row_base < M) {
                // this warp's rows of the tile: last part in -> finish them
                __syncwarp();
                unsigned int old = 0;
                if (lane == 0) {
                    __threadfence();                        // the warp's slab stores (ordered before this lane by the warp barrier) first
                    old = atomicAdd(tickets + t * 4 + q, 1u);
                }
                old = __shfl_sync(0xffffffffu, old, 0);
                if (old == (unsigned int)(splits - 1)) {
                    __threadfence();
                    // lane: four columns (c4) of rows r4, r4 + 4, ... of each 32 x 32 block; the slabs are read sixteen 128-bit
                    // loads at a time (two parts x eight rows) before anything is added or stored: one load after the
                    // other, a tile's 128 loads per lane cost 20 us
                    const int c4 = (lane & 7) * 4, r4 = lane >> 3;
                    float ar[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const int r = row_base + i * 4 + r4;
                        ar[i] = (r < M && y) ? a_scales[r] : 0.0f;
                    }
                    const int64_t slab = (int64_t)M * N;
                    for (int c = 0; c < BN && n0 + c < N; c += 32) {
                        const int col = n0 + c + c4;
                        if (col >= N) continue;
                        const float4 wsc = __ldg(reinterpret_cast<const float4 *>(w_scales + col));
                        int4 sum[8];
#pragma unroll
                        for (int i = 0; i < 8; i++) sum[i] = make_int4(0, 0, 0, 0);
                        for (int p = 0; p < splits; p += 2) {
                            int4 part[16];
#pragma unroll
                            for (int h = 0; h < 2; h++)
#pragma unroll
                                for (int i = 0; i < 8; i++) {
                                    const int r = row_base + i * 4 + r4;
                                    part[h * 8 + i] = (r < M && p + h < splits)
                                                          ? __ldcg(reinterpret_cast<const int4 *>(ws + (int64_t)(p + h) * slab + (int64_t)r * N + col))
                                                          : make_int4(0, 0, 0, 0);
                                }
#pragma unroll
                            for (int h = 0; h < 2; h++)
#pragma unroll
                                for (int i = 0; i < 8; i++) {
                                    sum[i].x += part[h * 8 + i].x;
                                    sum[i].y += part[h * 8 + i].y;
                                    sum[i].z += part[h * 8 + i].z;
                                    sum[i].w += part[h * 8 + i].w;
                                }
                        }
#pragma unroll
                        for (int i = 0; i < 8; i++) {
                            const int r = row_base + i * 4 + r4;
                            if (r >= M) continue;
                            if (acc_out) *reinterpret_cast<int4 *>(acc_out + (int64_t)r * N + col) = sum[i];
                            if (y) {
                                float4 o;
                                o.x = __fmul_rn(__fmul_rn(__int2float_rn(sum[i].x), ar[i]), wsc.x);
                                o.y = __fmul_rn(__fmul_rn(__int2float_rn(sum[i].y), ar[i]), wsc.y);
                                o.z = __fmul_rn(__fmul_rn(__int2float_rn(sum[i].z), ar[i]), wsc.z);
                                o.w = __fmul_rn(__fmul_rn(__int2float_rn(sum[i].w), ar[i]), wsc.w);
                                *reinterpret_cast<float4 *>(y + (int64_t)r * N + col) = o;
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) tickets[t * 4 + q] = 0;
                }
            }
        }
    }

    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ---------------------------------------------------------------- host side ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode()
{
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// [rows, K] i8 row-major; box = 128 bytes of K x box_rows rows; 128-byte swizzle; OOB reads give 0.
int32_t encode_kmajor(CUtensorMap *map, const void *ptr, int64_t rows, int64_t k, int box_rows)
{
    EncodeTiledFn enc = get_encode();
    if (!enc) PG_FAIL(PG_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)k};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) PG_FAIL(PG_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d (rows=%lld k=%lld)", (int)r, (long long)rows, (long long)k);
    return PG_OK;
}

// tickets (one per tile and accumulator-lane quarter, zero between calls) | s32 sums [parts][M, N]
constexpr size_t SPLIT_TICKET_BYTES = 64 * 1024;
constexpr size_t SPLIT_MAX_BYTES = 64u << 20;

template <int BN, int AR>
int32_t launch(pg_ctx *ctx, const int8_t *d_a, const float *d_as, int M, int K, pg_qtensor *w, float *d_y, int32_t *d_acc, int splits)
{
    using C = Cfg<BN, AR>;
    const int N = (int)w->cols;
    CUtensorMap ta;
    int32_t rc = encode_kmajor(&ta, d_a, M, K, AR);
    if (rc) return rc;
    if (w->tmap_b_box_rows != BN) {
        rc = encode_kmajor(reinterpret_cast<CUtensorMap *>(w->tmap_b), w->d_data_i8_t, N, K, BN);
        if (rc) return rc;
        w->tmap_b_box_rows = BN;
    }
    auto kern = gemm_i8_tcgen05_kernel<BN, AR>;
    static std::atomic<uint64_t> smem_set{0};
    PG_CUDA(pg_max_smem_once(kern, (int)C::SMEM, ctx->device, smem_set));
    const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * splits;
    const int grid = tiles < ctx->sm_count ? tiles : ctx->sm_count;
    int32_t *ws = nullptr;
    unsigned int *tickets = nullptr;
    if (splits > 1) {
        tickets = reinterpret_cast<unsigned int *>(ctx->splitk);
        ws = reinterpret_cast<int32_t *>(reinterpret_cast<unsigned char *>(ctx->splitk) + SPLIT_TICKET_BYTES);
    }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = C::SMEM;
    cfg.stream = ctx->stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    PG_CUDA(cudaLaunchKernelEx(&cfg, kern, ta, *reinterpret_cast<CUtensorMap *>(w->tmap_b), d_as, (const float *)w->d_scales, M, N, K,
                               d_y, d_acc, ctx->d_status, splits, ws, tickets));
    PG_LAUNCHED();
    return PG_OK;
}

int g_force_bn = 0;
int g_pair_mode = 0;  // 0 = heuristic, 1 = never use CTA pairs, 2 = always
int g_split_mode = 0; // 0 = heuristic, 1 = never split K, 2/4/8 = that many parts

}  // namespace

extern "C" PG_API void pg_tune_tcgen05_bn(int bn) { g_force_bn = bn; }
extern "C" PG_API void pg_tune_tcgen05_pair(int mode) { g_pair_mode = mode; }
extern "C" PG_API void pg_tune_tcgen05_split(int mode) { g_split_mode = mode; }

bool pgk_gemm_i8_tcgen05_supports(int64_t m, int64_t k, int64_t n)
{
    return m >= 1 && n >= 1 && k >= 16 && (k % 16 == 0) && m < (1ll << 31) && n < (1ll << 31) && k < (1ll << 31) &&
           m * n < (1ll << 40);
}

int32_t pgk_gemm_i8_tcgen05(pg_ctx *ctx, const int8_t *d_a, const float *d_as, int64_t m, int64_t k, pg_qtensor *w, float *d_y,
                            int32_t *d_acc)
{
    const int64_t n = w->cols;
    if (!pgk_gemm_i8_tcgen05_supports(m, k, n) || ((uintptr_t)d_a & 15) || ((uintptr_t)w->d_data_i8_t & 15))
        PG_FAIL(PG_ERR_UNSUPPORTED, "gemm_i8 tcgen05 kernel needs K%%16==0 and 16-byte aligned operands (K=%lld)", (long long)k);
    // CTA pairs (256 x 256 tiles) as soon as those tiles can occupy half of the SM pairs: measured
    // faster than one CTA per tile from M = 512 upwards (2896 vs 2658 TOPS at M 8192, N 14336)
    const int64_t pair_tiles = ((m + 255) / 256) * ((n + 255) / 256);
    // (not for a single row of tiles: at M <= 128 the ring's latency decides, see below: 23.0 us for pairs against
    // 18.5 us for one CTA per 128-column tile at M 64, N 14336)
    const bool pair = g_pair_mode == 2 || (g_pair_mode == 0 && !g_force_bn && m > BM && pair_tiles >= ctx->sm_count / 4);
    if (pair) return pgk_gemm_i8_tcgen05_2cta(ctx, d_a, d_as, m, k, w, d_y, d_acc);
    // Largest N tile that still gives every SM a tile.
    const int64_t tiles_m = (m + BM - 1) / BM;
    int bn = 64;
    if (tiles_m * ((n + 127) / 128) >= ctx->sm_count) bn = 128;
    if (tiles_m * ((n + 255) / 256) >= ctx->sm_count) bn = 256;
    // One row of tiles (M <= 128): the MMAs are not what bounds the kernel then.  Measured at M = 64, a k-block (128
    // bytes per column) takes a CTA 280 / 325 / 480 / 680 ns at 32 / 64 / 128 / 256 columns, whatever K and N are:
    // about 1.8 ns x (128 + columns).  Take the tile width with the smallest waves x time-per-k-block (N 14336: one
    // wave of 128-column tiles, 18.5 us, against 23.8 us for two waves of 64-column tiles; N 4096: 32-column tiles;
    // N 6144: 64-column tiles), and the smallest A tile that holds M rows (a deeper ring: 102 -> 92 us at N 128256,
    // 22.7 -> 18.6 us at M 17, N 14336; no change at M 64, N 14336).
    const int ar = m <= 32 ? 32 : (m <= 64 ? 64 : BM);
    int splits = 1;
    if (tiles_m == 1) {
        // also over parts of K when the tiles alone leave SMs idle and K is long.  Model (nanoseconds, fitted to
        // measurements at M 64): a unit costs its k-blocks x the larger of 250 (copy issue, barrier round trip, commit)
        // and the fill time above; the whole cannot beat the weights at 5.3 TB/s; the parts of a tile meeting in L2 cost
        // 3000 + 1750 per part (the last part reads the others' sums back: K 14336, N 4096, 128-column tiles: 34.4 us
        // whole, 25.7 us in two parts, 24.1 us in four, of which 13.9 us are the main loop; K 4096, N 4096: 12.9 us
        // whole, 14.6 / 16.8 us in two / four parts, so short K stays whole).
        const int64_t kblocks = (k + BK - 1) / BK;
        const bool can_split = g_split_mode != 1 && (n % 4 == 0) && (((uintptr_t)d_y | (uintptr_t)d_acc | (uintptr_t)w->d_scales) & 15) == 0 &&
                               ((n + 31) / 32) * 4 * sizeof(unsigned int) <= SPLIT_TICKET_BYTES && n <= 32768;
        double best = 0.0;
        for (int cand = 32; cand <= 256; cand *= 2) {
            for (int sp = 1; sp <= (can_split ? 8 : 1); sp *= 2) {
                const int64_t kpb = (kblocks + sp - 1) / sp;
                if (sp > 1 && (sp - 1) * kpb >= kblocks) continue;      // a part without k-blocks
                if (sp > 1 && (size_t)sp * (size_t)m * (size_t)n * sizeof(int32_t) > SPLIT_MAX_BYTES) continue;
                const int64_t units = ((n + cand - 1) / cand) * sp;
                const int64_t waves = (units + ctx->sm_count - 1) / ctx->sm_count;
                const double per_kb = std::max(250.0, 1.8 * (ar + cand));
                const double cost = std::max((double)waves * (double)kpb * per_kb, (double)k * (double)n / 5300.0) + (sp > 1 ? 3000.0 + 1750.0 * sp : 0.0);
                if (best == 0.0 || cost < best) {
                    best = cost;
                    bn = cand;
                    splits = sp;
                }
            }
        }
        if (g_split_mode >= 2 && can_split) splits = g_split_mode;
        while (splits > 1 && (splits - 1) * ((kblocks + splits - 1) / splits) >= kblocks) splits /= 2;   // no part without k-blocks
        while (splits > 1 && (size_t)splits * (size_t)m * (size_t)n * sizeof(int32_t) > SPLIT_MAX_BYTES) splits /= 2;
        if (splits > 1) {
            const size_t need = SPLIT_TICKET_BYTES + (size_t)splits * (size_t)m * (size_t)n * sizeof(int32_t);
            if (need > ctx->splitk_bytes && (ctx->no_growth || ctx->capturing)) {
                splits = 1;     // a caller that may not allocate (pg_matmul_quantized_static), or a graph being recorded: whole K per tile
            } else {
                const int32_t rr = pg_splitk_reserve(ctx, need);
                if (rr != PG_OK) return rr;
            }
        }
    }
    if (g_force_bn) bn = g_force_bn;
#define PG_TC_LAUNCH(BN_, AR_) return launch<BN_, AR_>(ctx, d_a, d_as, (int)m, (int)k, w, d_y, d_acc, splits)
#define PG_TC_ROWS(BN_)                \
    do {                               \
        if (ar == 32) PG_TC_LAUNCH(BN_, 32); \
        if (ar == 64) PG_TC_LAUNCH(BN_, 64); \
        PG_TC_LAUNCH(BN_, 128);        \
    } while (0)
    if (bn == 256) PG_TC_ROWS(256);
    if (bn == 128) PG_TC_ROWS(128);
    if (bn == 32) PG_TC_ROWS(32);
    PG_TC_ROWS(64);
#undef PG_TC_ROWS
#undef PG_TC_LAUNCH
}
