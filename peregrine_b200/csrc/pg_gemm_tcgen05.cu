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
                           float *__restrict__ y, int32_t *__restrict__ acc_out, int32_t *status)
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
    const int total_tiles = tiles_m * tiles_n;
    const int kblocks = (K + BK - 1) / BK;

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
                const int n0 = ((int)blockIdx.x / tiles_m) * BN;
                early = kblocks < STAGES ? kblocks : STAGES;
                for (int kb = 0; kb < early; kb++) {
                    mbar_arrive_expect_tx(bar_full + 8 * kb, C::STAGE);
                    tma_load_2d(base + kb * C::STAGE + C::STAGE_A, &tmap_b, bar_full + 8 * kb, kb * BK, n0);
                }
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
                const int m0 = (t % tiles_m) * BM;
                const int n0 = (t / tiles_m) * BN;
                for (int kb = 0; kb < kblocks; kb++) {
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
            for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
                if (!(ok = mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag, status))) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < kblocks; kb++) {
                    if (!(ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag, status))) break;
                    tc_fence_after();
                    const uint32_t sa = base + stage * C::STAGE;
                    const uint64_t da = make_smem_desc(sa);
                    const uint64_t db = make_smem_desc(sa + C::STAGE_A);
#pragma unroll
                    for (int j = 0; j < BK / UMMA_K; j++) {
                        // +32 bytes of K inside the swizzle span = +2 in the 16-byte address field
                        umma_i8(d_tmem, da + (uint64_t)(j * (UMMA_K >> 4)), db + (uint64_t)(j * (UMMA_K >> 4)), idesc,
                                (kb | j) != 0 ? 1u : 0u);
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
        for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
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
                if (vec_ok) {
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

template <int BN, int AR>
int32_t launch(pg_ctx *ctx, const int8_t *d_a, const float *d_as, int M, int K, pg_qtensor *w, float *d_y, int32_t *d_acc)
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
    const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int grid = tiles < ctx->sm_count ? tiles : ctx->sm_count;
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
                               d_y, d_acc, ctx->d_status));
    PG_LAUNCHED();
    return PG_OK;
}

int g_force_bn = 0;
int g_pair_mode = 0;  // 0 = heuristic, 1 = never use CTA pairs, 2 = always

}  // namespace

extern "C" PG_API void pg_tune_tcgen05_bn(int bn) { g_force_bn = bn; }
extern "C" PG_API void pg_tune_tcgen05_pair(int mode) { g_pair_mode = mode; }

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
    if (tiles_m == 1) {
        double best = 0.0;
        for (int cand = 32; cand <= 256; cand *= 2) {
            const int64_t waves = ((n + cand - 1) / cand + ctx->sm_count - 1) / ctx->sm_count;
            const double cost = (double)waves * 1.8 * (128 + cand);
            if (best == 0.0 || cost < best) {
                best = cost;
                bn = cand;
            }
        }
    }
    if (g_force_bn) bn = g_force_bn;
#define PG_TC_LAUNCH(BN_, AR_) return launch<BN_, AR_>(ctx, d_a, d_as, (int)m, (int)k, w, d_y, d_acc)
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
