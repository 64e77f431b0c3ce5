// Prefill-size W8A8 product on CTA pairs: the integer GEMM of src/quant.rs:154-166 /
// simd_kernels::gemm_i8_sdot (src/simd_kernels.rs:1087-1214) with tcgen05.mma.cta_group::2.
//
// Two CTAs of a thread-block cluster (two SMs) compute one 256 x 256 tile together.  Each CTA
// stages its own 128 rows of A and ITS HALF (128 rows) of the B tile, and one thread of the leader
// CTA issues MMAs that read both CTAs' shared memory; each CTA's tensor memory receives its 128
// rows of the accumulator.  Compared with one CTA per 128 x 256 tile this moves a third fewer
// operand bytes from L2 per multiply-accumulate, which is what bounds the one-CTA kernel (its
// shared memory cannot hold more bytes in flight).  No multicast load is used: every CTA fetches
// what it stages itself, with plain tiled TMA loads that signal the leader's barrier.
//
// Roles per CTA: warp 0 producer (TMA), warp 1 MMA issuer (leader CTA only) and TMEM owner, warps
// 2-5 epilogue (tcgen05.ld -> `acc as f32 * a_scale[m] * w_scale[n]` -> global stores).  Barriers:
//   full[s]   in the leader: one arrival (leader's expect_tx) + the bytes of both CTAs' loads
//   empty[s]  in each CTA:   tcgen05.commit multicast to both CTAs when the stage's MMAs are done
//   tfull[a]  in each CTA:   tcgen05.commit multicast when accumulator a is complete
//   tempty[a] in the leader: the eight epilogue warps of both CTAs arrive (the peer's remotely)
// Every wait is bounded (about a second without progress -> PG_ERR_DEVICE_TIMEOUT in the status
// word, CTA-wide abort flag, normal teardown including the TMEM release).
#include <cuda.h>

#include "pg_internal.cuh"
#include "pg_tc_epilogue.cuh"

namespace {

constexpr int TM = 128;        // rows of A per CTA
constexpr int TNH = 128;       // rows of B per CTA (half of the 256-wide tile)
constexpr int TN = 256;
constexpr int BK = 128;        // bytes of K per stage = one 128-byte swizzle span
constexpr int UMMA_K = 32;
constexpr int STAGES = 6;
constexpr int STAGE_A = TM * BK, STAGE_B = TNH * BK, STAGE = STAGE_A + STAGE_B;   // 32 KiB
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;  // two 256-column accumulators
constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE + 1024 + 256 + 4 * PG_EPI_WARP_BYTES;
constexpr unsigned long long WAIT_LIMIT_NS = 1000ull * 1000ull * 1000ull;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long globaltimer()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t cta)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta));
    return r;
}
__device__ __forceinline__ void cluster_sync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
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
// tiled TMA load of this CTA's tile; completion bytes go to `bar`, a shared::cluster address that
// may belong to the peer CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *tmap, uint32_t bar, int x, int y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
        "l"(tmap), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_i8_pair(uint32_t d_tmem, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
        ::"r"(d_tmem), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
// arrives on the barrier at this shared-memory offset in both CTAs of the pair
__device__ __forceinline__ void umma_commit_pair(uint32_t bar)
{
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                 "h"(mask)
                 : "memory");
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
// K-major, 128-byte swizzle, 8-row groups 1024 B apart, descriptor version 1 (same as the one-CTA kernel)
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
// kind::i8: D = s32, A/B = s8, K-major, N >> 3 at bit 17, M >> 4 at bit 24 (M = 256 over the pair)
constexpr uint32_t IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);

__global__ void __launch_bounds__(NUM_THREADS, 1)
    gemm_i8_tcgen05_2cta_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                                const float *__restrict__ a_scales, const float *__restrict__ w_scales, int M, int N, int K,
                                float *__restrict__ y, int32_t *__restrict__ acc_out, int32_t *status)
{
    // programmatic dependent launch: see gemm_i8_tcgen05_kernel; the predecessor's output (activations, their scales) is
    // touched only behind griddepcontrol.wait
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (base - raw_addr);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (size_t)STAGES * STAGE);
    const uint32_t bar_full = smem_u32(bars);
    const uint32_t bar_empty = bar_full + 8 * STAGES;
    const uint32_t bar_tfull = bar_empty + 8 * STAGES;
    const uint32_t bar_tempty = bar_tfull + 16;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const int tiles_m = (M + 2 * TM - 1) / (2 * TM);
    const int tiles_n = (N + TN - 1) / TN;
    const int total_tiles = tiles_m * tiles_n;
    const int kblocks = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(bar_tfull + 8 * i, 1);
            mbar_init(bar_tempty + 8 * i, 8);  // four epilogue warps in each of the two CTAs
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    cluster_sync();  // both CTAs' barriers exist before anyone signals across the pair
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- producer (both CTAs)
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            // this CTA's half of the weight tiles of the first stages of the first tile, before the predecessor has finished
            // (a stage's barrier may get the bytes of the other CTA before the leader has announced them: the transaction
            // count is signed inside a phase, and the phase cannot complete before the leader's arrival)
            int early = 0;
            if (pair < total_tiles) {
                const int n0 = (pair / tiles_m) * TN + (int)rank * TNH;
                early = kblocks < STAGES ? kblocks : STAGES;
                for (int kb = 0; kb < early; kb++) {
                    if (leader) mbar_arrive_expect_tx(bar_full + 8 * kb, 2 * STAGE);
                    tma_load_2d_pair(base + kb * STAGE + STAGE_A, &tmap_b, mapa(bar_full + 8 * kb, 0), kb * BK, n0);
                }
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int t = pair; ok && t < total_tiles; t += npairs) {
                const int m0 = (t % tiles_m) * (2 * TM) + (int)rank * TM;
                const int n0 = (t / tiles_m) * TN + (int)rank * TNH;
                for (int kb = 0; kb < kblocks; kb++) {
                    if (!(ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, status))) break;
                    const uint32_t sa = base + stage * STAGE;
                    const uint32_t full_leader = mapa(bar_full + 8 * stage, 0);
                    if (early > 0) {
                        early--;                            // announced and half filled above
                    } else {
                        if (leader) mbar_arrive_expect_tx(bar_full + 8 * stage, 2 * STAGE);  // the bytes of both CTAs
                        tma_load_2d_pair(sa + STAGE_A, &tmap_b, full_leader, kb * BK, n0);
                    }
                    tma_load_2d_pair(sa, &tmap_a, full_leader, kb * BK, m0);
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
        // ---------------------------------------------------------------- MMA issuer (leader only)
        if (leader && lane == 0) {
            uint32_t stage = 0, phase = 0;
            uint32_t acc = 0, acc_phase = 0;
            bool ok = true;
            for (int t = pair; ok && t < total_tiles; t += npairs) {
                if (!(ok = mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag, status))) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * TN;
                for (int kb = 0; kb < kblocks; kb++) {
                    if (!(ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag, status))) break;
                    tc_fence_after();
                    const uint32_t sa = base + stage * STAGE;
                    const uint64_t da = make_smem_desc(sa);
                    const uint64_t db = make_smem_desc(sa + STAGE_A);
#pragma unroll
                    for (int j = 0; j < BK / UMMA_K; j++)
                        umma_i8_pair(d_tmem, da + (uint64_t)(j * (UMMA_K >> 4)), db + (uint64_t)(j * (UMMA_K >> 4)), IDESC,
                                     (kb | j) != 0 ? 1u : 0u);
                    umma_commit_pair(bar_empty + 8 * stage);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                umma_commit_pair(bar_tfull + 8 * acc);
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1;
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue (both CTAs)
        const int q = warp & 3;
        asm volatile("griddepcontrol.wait;" ::: "memory");   // a_scales come from the predecessor; y may still be read by it
        uint32_t acc = 0, acc_phase = 0;
        const bool vec_ok = ((N & 3) == 0) && (((uintptr_t)y & 15) == 0) && (((uintptr_t)acc_out & 15) == 0) &&
                            (((uintptr_t)w_scales & 15) == 0);
        bool ok = true;
        for (int t = pair; ok && t < total_tiles; t += npairs) {
            const int m0 = (t % tiles_m) * (2 * TM) + (int)rank * TM;
            const int n0 = (t / tiles_m) * TN;
            ok = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, status);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int row_base = m0 + q * 32;
            const int row = row_base + lane;
            const float as = (row < M && y) ? a_scales[row] : 0.0f;
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * TN;
            const uint32_t stage_buf = base + (uint32_t)((size_t)STAGES * STAGE) + 256u + (uint32_t)q * PG_EPI_WARP_BYTES;
#pragma unroll 1
            for (int c = 0; c < TN; c += 32) {
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
            if (lane == 0) mbar_arrive_cluster(mapa(bar_tempty + 8 * acc, 0));  // the leader's barrier
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1;
            }
        }
    }

    // neither CTA may leave while the other can still touch its shared memory, barriers or TMEM;
    // the single-lane roles rejoin their warps first (the cluster barrier is warp-aligned)
    __syncwarp();
    tc_fence_before();
    cluster_sync();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int32_t encode_kmajor(CUtensorMap *map, const void *ptr, int64_t rows, int64_t k, int box_rows)
{
    static EncodeTiledFn enc = nullptr;
    if (!enc) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
            enc = (EncodeTiledFn)p;
    }
    if (!enc) PG_FAIL(PG_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)k};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) PG_FAIL(PG_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return PG_OK;
}

}  // namespace

int32_t pgk_gemm_i8_tcgen05_2cta(pg_ctx *ctx, const int8_t *d_a, const float *d_as, int64_t m, int64_t k, pg_qtensor *w,
                                 float *d_y, int32_t *d_acc)
{
    const int M = (int)m, K = (int)k, N = (int)w->cols;
    CUtensorMap ta;
    int32_t rc = encode_kmajor(&ta, d_a, M, K, TM);
    if (rc) return rc;
    if (w->tmap_b_box_rows != TNH) {
        rc = encode_kmajor(reinterpret_cast<CUtensorMap *>(w->tmap_b), w->d_data_i8_t, N, K, TNH);
        if (rc) return rc;
        w->tmap_b_box_rows = TNH;
    }
    static std::atomic<uint64_t> smem_set{0};
    PG_CUDA(pg_max_smem_once(gemm_i8_tcgen05_2cta_kernel, (int)SMEM_BYTES, ctx->device, smem_set));
    const int tiles = ((M + 2 * TM - 1) / (2 * TM)) * ((N + TN - 1) / TN);
    const int max_pairs = ctx->sm_count / 2;
    const int pairs = tiles < max_pairs ? tiles : max_pairs;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    PG_CUDA(cudaLaunchKernelEx(&cfg, gemm_i8_tcgen05_2cta_kernel, ta, *reinterpret_cast<CUtensorMap *>(w->tmap_b), d_as,
                               (const float *)w->d_scales, M, N, K, d_y, d_acc, ctx->d_status));
    PG_LAUNCHED();
    return PG_OK;
}
