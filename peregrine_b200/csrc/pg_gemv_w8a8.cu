// Decode-size W8A8 product (M <= 64): the integer GEMM of src/quant.rs:154-166 /
// simd_kernels::gemm_i8_sdot (src/simd_kernels.rs:1087-1214) for a handful of rows.
//
// The op is bound by reading data_i8_t [N,K] once from HBM, so the kernel is built around
// keeping that stream full:
//   * a CTA owns 8*NG output columns (= 8*NG contiguous rows of data_i8_t) and all K; its
//     warps take interleaved 64-byte slices of K, so the CTA reads contiguous spans;
//   * every lane moves its weights with 128-bit asynchronous copies (cp.async, L2 only) into a
//     private FIFO in shared memory, D k-steps deep.  Bytes in flight are therefore set by the
//     FIFO depth, not by registers or by how many warps are resident, and a lane only ever reads
//     back what it copied itself, so no barrier is needed inside the loop;
//   * the activations (<= 64 x K bytes, shared by every CTA) come through L1 with the same
//     128-bit pattern, issued before the wait on the FIFO so that their latency is hidden by it;
//   * the dot products run on the warp-level int8 MMA m16n8k32 (exact s32 accumulation).
//     A dot product is invariant under a permutation of K applied to both operands, so a
//     lane's 16 contiguous K-bytes feed two consecutive MMAs directly, without shuffles;
//   * the warps' partial sums meet in shared memory (integer adds: exact in any order) and
//     the epilogue applies `acc as f32 * a_scale[m] * w_scale[n]` as two rounded products.
//
// The kernel is launched with programmatic stream serialisation: the weight prefetch does not
// depend on the preceding kernel (the activation quantiser), so it is issued before
// griddepcontrol.wait and overlaps the predecessor's tail.
#include "pg_internal.cuh"

namespace {

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, uint32_t src_bytes)
{
    asm volatile("cp.async.cg.shared.global.L2::128B [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait()
{
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ uint4 ld_cached_v4(const void *p)
{
    uint4 v;
    // Written by the preceding kernel (the quantiser) and re-read by every CTA of an SM: an ordinary coherent load
    // that allocates in L1 (griddepcontrol.wait makes the predecessor's stores visible to these), never the
    // non-coherent path, whose lines may predate the predecessor's stores.
    asm volatile("ld.global.ca.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_s8_16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                             uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void st_cluster_s32(uint32_t local_addr, uint32_t cta, int32_t v)
{
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(cta));
    asm volatile("st.shared::cluster.s32 [%0], %1;" ::"r"(remote), "r"(v) : "memory");
}
__device__ __forceinline__ void cluster_sync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// MB: 16-row blocks of activations; NG: 8-column groups per CTA; WARPS: K split inside the CTA;
// D: FIFO depth in k-steps; HI: rows 8..15 of a block exist (false when M <= 8, which halves the
// activation loads); S: K split across the S CTAs of a thread-block cluster, whose partial sums
// are added through distributed shared memory (used when N alone gives too few CTAs to balance
// the SMs).
template <int MB, int NG, int WARPS, int D, bool HI, int S>
__global__ void __launch_bounds__(WARPS * 32)
    gemv_w8a8_kernel(const int8_t *__restrict__ a, const float *__restrict__ a_scales, int M, int K,
                     const int8_t *__restrict__ bt, const float *__restrict__ w_scales, int64_t N, float *__restrict__ y,
                     int32_t *__restrict__ acc_out)
{
    constexpr int NT = NG * 8;
    constexpr int ROWS = MB * 16;
    constexpr int THREADS = WARPS * 32;
    // [D][NG][THREADS] uint4, reused as int32 [WARPS][ROWS][NT] for the reduction; then, never
    // aliased with the FIFO, int32 [S-1][ROWS][NT] that the other CTAs of the cluster write into
    extern __shared__ uint4 fifo[];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr uint32_t FIFO_BYTES = (uint32_t)D * NG * THREADS * 16;
    constexpr uint32_t RED_BYTES = (uint32_t)WARPS * ROWS * NT * 4;
    constexpr uint32_t XBUF_OFF = FIFO_BYTES > RED_BYTES ? FIFO_BYTES : RED_BYTES;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = lane >> 2, t = lane & 3;
    const uint32_t slice = (S > 1) ? cluster_ctarank() : 0u;
    const int64_t n0 = (int64_t)(blockIdx.x / S) * NT;
    const uint32_t fifo_base = (uint32_t)__cvta_generic_to_shared(fifo) + threadIdx.x * 16;

    int acc[MB][NG][4];
#pragma unroll
    for (int mb = 0; mb < MB; mb++)
#pragma unroll
        for (int g = 0; g < NG; g++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc[mb][g][i] = 0;

    const int8_t *wp[NG];
    bool wok[NG];
#pragma unroll
    for (int g = 0; g < NG; g++) {
        const int64_t n = n0 + g * 8 + r;
        wok[g] = n < N;
        wp[g] = bt + (wok[g] ? n : 0) * (int64_t)K + t * 16;
    }
    const int ksteps_all = (K + 63) >> 6;
    const int per_slice = (ksteps_all + S - 1) / S;
    const int ks0 = (int)slice * per_slice;
    const int ksteps = max(0, min(ksteps_all - ks0, per_slice));  // k-steps of this CTA: [ks0, ks0 + ksteps)
    const int my_steps = (ksteps > warp) ? (ksteps - warp + WARPS - 1) / WARPS : 0;

    // copies k-step `i` of this warp (or zero-fills its slot) and closes one cp.async group
    auto issue = [&](int i) {
        const int kb = (ks0 + warp + i * WARPS) << 6;
        const bool kok = (i < my_steps) && (kb + t * 16 < K);
        const uint32_t slot = fifo_base + (uint32_t)(i % D) * (NG * THREADS * 16);
#pragma unroll
        for (int g = 0; g < NG; g++) {
            const bool ok = kok && wok[g];
            cp_async16(slot + g * (THREADS * 16), ok ? (const void *)(wp[g] + kb) : (const void *)bt, ok ? 16u : 0u);
        }
        cp_async_commit();
    };
#pragma unroll
    for (int i = 0; i < D - 1; i++) issue(i);

    // Everything above reads only the weights.  The activations come from the preceding kernel.
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const int8_t *alo[MB], *ahi[MB];
    bool oklo[MB], okhi[MB];
#pragma unroll
    for (int mb = 0; mb < MB; mb++) {
        const int m = mb * 16 + r;
        oklo[mb] = m < M;
        okhi[mb] = HI && (m + 8 < M);
        alo[mb] = a + (int64_t)(oklo[mb] ? m : 0) * K + t * 16;
        ahi[mb] = a + (int64_t)(okhi[mb] ? m + 8 : 0) * K + t * 16;
    }
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    for (int i = 0; i < my_steps; i++) {
        issue(i + D - 1);
        const int kb = (ks0 + warp + i * WARPS) << 6;
        const bool kok = kb + t * 16 < K;
        uint4 xl[MB], xh[MB];
#pragma unroll
        for (int mb = 0; mb < MB; mb++) {
            xl[mb] = (kok && oklo[mb]) ? ld_cached_v4(alo[mb] + kb) : zero;
            xh[mb] = (HI && kok && okhi[mb]) ? ld_cached_v4(ahi[mb] + kb) : zero;
        }
        cp_async_wait<D - 1>();
        const uint32_t slot = fifo_base + (uint32_t)(i % D) * (NG * THREADS * 16);
#pragma unroll
        for (int g = 0; g < NG; g++) {
            const uint4 w = lds128(slot + g * (THREADS * 16));
#pragma unroll
            for (int mb = 0; mb < MB; mb++) {
                mma_s8_16832(acc[mb][g], xl[mb].x, xh[mb].x, xl[mb].y, xh[mb].y, w.x, w.y);
                mma_s8_16832(acc[mb][g], xl[mb].z, xh[mb].z, xl[mb].w, xh[mb].w, w.z, w.w);
            }
        }
    }
    cp_async_wait<0>();
    // the activation scales were written by the preceding kernel: one L2 load each, not one per output
    __shared__ float as_s[MB * 16];
    if (threadIdx.x < ROWS) as_s[threadIdx.x] = ((int)threadIdx.x < M) ? pg_ld_fresh(a_scales + threadIdx.x) : 0.0f;
    __syncthreads();  // every lane is done with its FIFO: the memory becomes the reduction buffer

    // C fragment: c0,c1 -> (row r, cols 2t, 2t+1); c2,c3 -> (row r+8, same cols)
    int32_t *red = reinterpret_cast<int32_t *>(fifo);
    int32_t *mine = red + warp * (ROWS * NT);
#pragma unroll
    for (int mb = 0; mb < MB; mb++) {
#pragma unroll
        for (int g = 0; g < NG; g++) {
            const int col = g * 8 + 2 * t;
            mine[(mb * 16 + r) * NT + col] = acc[mb][g][0];
            mine[(mb * 16 + r) * NT + col + 1] = acc[mb][g][1];
            mine[(mb * 16 + r + 8) * NT + col] = acc[mb][g][2];
            mine[(mb * 16 + r + 8) * NT + col + 1] = acc[mb][g][3];
        }
    }
    __syncthreads();
    if (S > 1) {
        // the other CTAs of the cluster hand their partial sums to CTA 0
        if (slice != 0) {
            const uint32_t xbuf = (uint32_t)__cvta_generic_to_shared(fifo) + XBUF_OFF + (slice - 1) * (ROWS * NT * 4);
            for (int idx = threadIdx.x; idx < ROWS * NT; idx += THREADS) {
                int32_t sum = 0;
#pragma unroll
                for (int wv = 0; wv < WARPS; wv++) sum += red[wv * (ROWS * NT) + idx];
                st_cluster_s32(xbuf + idx * 4, 0u, sum);
            }
        }
        cluster_sync();
        if (slice != 0) return;
    }
    const int32_t *xsum = reinterpret_cast<const int32_t *>(reinterpret_cast<const char *>(fifo) + XBUF_OFF);
    for (int idx = threadIdx.x; idx < ROWS * NT; idx += THREADS) {
        const int m = idx / NT;
        const int64_t n = n0 + (idx % NT);
        if (m >= M || n >= N) continue;
        int32_t sum = 0;
#pragma unroll
        for (int wv = 0; wv < WARPS; wv++) sum += red[wv * (ROWS * NT) + idx];
#pragma unroll
        for (int j = 0; j < S - 1; j++) sum += xsum[j * (ROWS * NT) + idx];
        if (acc_out) acc_out[(int64_t)m * N + n] = sum;
        if (y) y[(int64_t)m * N + n] = __fmul_rn(__fmul_rn(__int2float_rn(sum), as_s[m]), __ldg(w_scales + n));
    }
}

int g_carveout_pct = -1;  // tuning: preferred shared-memory carve-out in percent, -1 = driver's choice

template <int MB, int NG, int WARPS, int D, bool HI, int S>
int32_t launch(pg_ctx *ctx, const int8_t *a, const float *as, int M, int K, const int8_t *bt, const float *ws, int64_t N,
               float *y, int32_t *acc)
{
    constexpr int NT = NG * 8;
    constexpr size_t fifo_bytes = (size_t)D * NG * WARPS * 32 * 16;
    constexpr size_t red_bytes = (size_t)WARPS * MB * 16 * NT * sizeof(int32_t);
    constexpr size_t smem = (fifo_bytes > red_bytes ? fifo_bytes : red_bytes) + (size_t)(S - 1) * MB * 16 * NT * sizeof(int32_t);
    auto kern = gemv_w8a8_kernel<MB, NG, WARPS, D, HI, S>;
    static std::atomic<uint64_t> smem_set{0};
    if (smem > 48 * 1024) PG_CUDA(pg_max_smem_once(kern, (int)smem, ctx->device, smem_set));
    if (g_carveout_pct >= 0) PG_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, g_carveout_pct));
    const int64_t blocks = ((N + NT - 1) / NT) * S;
    PG_REQUIRE(blocks <= 0x7fffffff, "gemm_i8 stream: N too large");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = S;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (S > 1) ? 2 : 1;
    PG_CUDA(cudaLaunchKernelEx(&cfg, kern, a, as, M, K, bt, ws, N, y, acc));
    PG_LAUNCHED();
    return PG_OK;
}

int g_force_ng = 0;     // tuning overrides, 0 = heuristic
int g_force_depth = 0;
int g_force_split = 0;

}  // namespace

extern "C" PG_API void pg_tune_stream_ng(int ng) { g_force_ng = ng; }
extern "C" PG_API void pg_tune_stream_depth(int depth) { g_force_depth = depth; }
extern "C" PG_API void pg_tune_stream_carveout(int pct) { g_carveout_pct = pct; }
extern "C" PG_API void pg_tune_stream_split(int split) { g_force_split = split; }

bool pgk_gemm_i8_stream_supports(int64_t m, int64_t k, int64_t n)
{
    return m >= 1 && m <= 64 && n >= 1 && k >= 16 && (k % 16 == 0) && k <= (1 << 30);
}

int32_t pgk_gemm_i8_stream(pg_ctx *ctx, const int8_t *d_a, const float *d_as, int64_t m, int64_t k, const int8_t *d_bt,
                           const float *d_ws, int64_t n, float *d_y, int32_t *d_acc)
{
    if (!pgk_gemm_i8_stream_supports(m, k, n) || ((uintptr_t)d_a & 15) || ((uintptr_t)d_bt & 15))
        PG_FAIL(PG_ERR_UNSUPPORTED, "gemm_i8 stream kernel needs 1<=M<=64, K%%16==0 and 16-byte aligned operands (M=%lld K=%lld)",
                (long long)m, (long long)k);
    const int M = (int)m, K = (int)k;
    // Measured on B200 over the Llama-3-8B projection shapes: 16 columns per CTA and a FIFO of four
    // k-steps are best throughout; when N alone gives fewer than four CTAs per SM, K is also split
    // over a cluster of two CTAs.
    int ng = 2;
    if (g_force_ng) ng = g_force_ng;
    const int64_t tiles = (n + 8 * ng - 1) / (8 * ng);
    int split = (tiles < 4 * (int64_t)ctx->sm_count && k >= 2048) ? 2 : 1;
    if (g_force_split) split = g_force_split;
    int depth = 4;
    if (g_force_depth) depth = g_force_depth;
#define PG_GEMV_CASE(MB, NG, D, HI)                                                                               \
    do {                                                                                                          \
        if (split == 1) return launch<MB, NG, 8, D, HI, 1>(ctx, d_a, d_as, M, K, d_bt, d_ws, n, d_y, d_acc);      \
        if (split == 2) return launch<MB, NG, 8, D, HI, 2>(ctx, d_a, d_as, M, K, d_bt, d_ws, n, d_y, d_acc);      \
        return launch<MB, NG, 8, D, HI, 4>(ctx, d_a, d_as, M, K, d_bt, d_ws, n, d_y, d_acc);                      \
    } while (0)
#define PG_GEMV_DEPTHS(MB, NG, HI)                         \
    do {                                                   \
        if (depth <= 4) PG_GEMV_CASE(MB, NG, 4, HI);       \
        PG_GEMV_CASE(MB, NG, 8, HI);                       \
    } while (0)
    if (M <= 8) {
        if (ng == 1) PG_GEMV_DEPTHS(1, 1, false);
        if (ng == 2) PG_GEMV_DEPTHS(1, 2, false);
        PG_GEMV_CASE(1, 4, 4, false);
    } else if (M <= 16) {
        if (ng == 1) PG_GEMV_DEPTHS(1, 1, true);
        if (ng == 2) PG_GEMV_DEPTHS(1, 2, true);
        PG_GEMV_CASE(1, 4, 4, true);
    } else if (M <= 32) {
        if (ng == 1) PG_GEMV_CASE(2, 1, 4, true);
        PG_GEMV_CASE(2, 2, 4, true);
    } else if (M <= 48) {
        PG_GEMV_CASE(3, 1, 4, true);
    } else {
        PG_GEMV_CASE(4, 1, 4, true);
    }
#undef PG_GEMV_DEPTHS
#undef PG_GEMV_CASE
}
