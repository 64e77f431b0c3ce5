// Decode-size W8A8 product (M <= 64): the integer GEMM of src/quant.rs:154-166 /
// simd_kernels::gemm_i8_sdot (src/simd_kernels.rs:1087-1214) for a handful of rows.
//
// The op is bound by reading data_i8_t [N,K] once from HBM, so the kernel is built around
// that stream:
//   * a CTA owns 8*NG output columns (= 8*NG contiguous rows of data_i8_t) and all K; its
//     warps take interleaved 64-byte slices of K, so the CTA reads contiguous spans;
//   * every lane issues 128-bit, sector-aligned, L1-bypassing loads of the weights, U steps
//     deep, before any arithmetic of those steps;
//   * the activations (<= 64 x K bytes, shared by every CTA) come through L1 with the same
//     128-bit pattern;
//   * the dot products run on the warp-level int8 MMA m16n8k32 (exact s32 accumulation).
//     A dot product is invariant under a permutation of K applied to both operands, so a
//     lane's 16 contiguous K-bytes feed two consecutive MMAs directly, without shuffles;
//   * the warps' partial sums meet in shared memory (integer adds: exact in any order) and
//     the epilogue applies `acc as f32 * a_scale[m] * w_scale[n]` as two rounded products.
#include "pg_internal.cuh"

namespace {

__device__ __forceinline__ uint4 ld_stream_v4(const void *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ uint4 ld_cached_v4(const void *p)
{
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
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

// MB: 16-row blocks of activations; NG: 8-column groups per CTA; WARPS: K split; U: steps in flight;
// HI: rows 8..15 of a block exist (false when M <= 8, which halves the activation loads).
template <int MB, int NG, int WARPS, int U, bool HI>
__global__ void __launch_bounds__(WARPS * 32)
    gemv_w8a8_kernel(const int8_t *__restrict__ a, const float *__restrict__ a_scales, int M, int K,
                     const int8_t *__restrict__ bt, const float *__restrict__ w_scales, int64_t N, float *__restrict__ y,
                     int32_t *__restrict__ acc_out)
{
    constexpr int NT = NG * 8;
    constexpr int ROWS = MB * 16;
    extern __shared__ int32_t red[];  // [WARPS][ROWS][NT]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = lane >> 2, t = lane & 3;
    const int64_t n0 = (int64_t)blockIdx.x * NT;

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

    const int ksteps = (K + 63) >> 6;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    for (int s0 = warp; s0 < ksteps; s0 += WARPS * U) {
        uint4 w[U][NG], xl[U][MB], xh[U][MB];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int s = s0 + u * WARPS;
            const int kb = s << 6;
            const bool kok = (s < ksteps) && (kb + t * 16 < K);
#pragma unroll
            for (int g = 0; g < NG; g++) w[u][g] = (kok && wok[g]) ? ld_stream_v4(wp[g] + kb) : zero;
#pragma unroll
            for (int mb = 0; mb < MB; mb++) {
                xl[u][mb] = (kok && oklo[mb]) ? ld_cached_v4(alo[mb] + kb) : zero;
                xh[u][mb] = (HI && kok && okhi[mb]) ? ld_cached_v4(ahi[mb] + kb) : zero;
            }
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
#pragma unroll
            for (int mb = 0; mb < MB; mb++) {
#pragma unroll
                for (int g = 0; g < NG; g++) {
                    mma_s8_16832(acc[mb][g], xl[u][mb].x, xh[u][mb].x, xl[u][mb].y, xh[u][mb].y, w[u][g].x, w[u][g].y);
                    mma_s8_16832(acc[mb][g], xl[u][mb].z, xh[u][mb].z, xl[u][mb].w, xh[u][mb].w, w[u][g].z, w[u][g].w);
                }
            }
        }
    }

    // C fragment: c0,c1 -> (row r, cols 2t, 2t+1); c2,c3 -> (row r+8, same cols)
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
    for (int idx = threadIdx.x; idx < ROWS * NT; idx += WARPS * 32) {
        const int m = idx / NT;
        const int64_t n = n0 + (idx % NT);
        if (m >= M || n >= N) continue;
        int32_t sum = 0;
#pragma unroll
        for (int wv = 0; wv < WARPS; wv++) sum += red[wv * (ROWS * NT) + idx];
        if (acc_out) acc_out[(int64_t)m * N + n] = sum;
        if (y) y[(int64_t)m * N + n] = __fmul_rn(__fmul_rn(__int2float_rn(sum), a_scales[m]), __ldg(w_scales + n));
    }
}

template <int MB, int NG, int WARPS, int U, bool HI>
int32_t launch(pg_ctx *ctx, const int8_t *a, const float *as, int M, int K, const int8_t *bt, const float *ws, int64_t N,
               float *y, int32_t *acc)
{
    constexpr int NT = NG * 8;
    const size_t smem = (size_t)WARPS * MB * 16 * NT * sizeof(int32_t);
    auto kern = gemv_w8a8_kernel<MB, NG, WARPS, U, HI>;
    if (smem > 48 * 1024) PG_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int64_t blocks = (N + NT - 1) / NT;
    PG_REQUIRE(blocks <= 0x7fffffff, "gemm_i8 stream: N too large");
    kern<<<(unsigned)blocks, WARPS * 32, smem, ctx->stream>>>(a, as, M, K, bt, ws, N, y, acc);
    PG_LAUNCHED();
    return PG_OK;
}

int g_force_ng = 0;  // tuning override, 0 = heuristic

}  // namespace

extern "C" PG_API void pg_tune_stream_ng(int ng) { g_force_ng = ng; }

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
    // Columns per CTA: small enough that every SM gets several CTAs, large enough that the
    // activations are not re-read from L2 more often than needed when they outgrow L1.
    int ng = 1;
    const int64_t act_bytes = m * k;
    if (n >= 8 * 8 * (int64_t)ctx->sm_count || act_bytes > 128 * 1024) ng = 2;
    if (n >= 32 * 8 * (int64_t)ctx->sm_count) ng = 4;
    if (g_force_ng) ng = g_force_ng;
#define PG_GEMV_CASE(MB, NG, U, HI) return launch<MB, NG, 8, U, HI>(ctx, d_a, d_as, M, K, d_bt, d_ws, n, d_y, d_acc)
    if (M <= 8) {
        if (ng == 1) PG_GEMV_CASE(1, 1, 4, false);
        if (ng == 2) PG_GEMV_CASE(1, 2, 4, false);
        PG_GEMV_CASE(1, 4, 2, false);
    } else if (M <= 16) {
        if (ng == 1) PG_GEMV_CASE(1, 1, 4, true);
        if (ng == 2) PG_GEMV_CASE(1, 2, 4, true);
        PG_GEMV_CASE(1, 4, 2, true);
    } else if (M <= 32) {
        if (ng == 1) PG_GEMV_CASE(2, 1, 2, true);
        PG_GEMV_CASE(2, 2, 2, true);
    } else if (M <= 48) {
        PG_GEMV_CASE(3, 1, 2, true);
    } else {
        PG_GEMV_CASE(4, 1, 2, true);
    }
#undef PG_GEMV_CASE
}
