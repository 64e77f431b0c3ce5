// The dequantising product of the reference's GPU seam: quant::matmul_quantized_gpu (src/quant.rs:195-218) dispatches
// matmul_dequant_i8 / matmul_dequant_simd_i8 (src/metal/shaders.rs:2329-2465, selector src/metal/context.rs:2226-2306),
// which keep the activations in f32 and dequantise the int8 weights on the way into the tile:
//
//     C[m, n] = sum_k A[m, k] * (float(W_i8[k, n]) * w_scale[n])          f32 throughout ("W8A32")
//
// -- a different product from the CPU path's W8A8 (no activation quantiser, no integer sums).  Both Metal kernels walk k
// upwards tile by tile, so their sum is the ascending-k f32 sum up to the association inside a tile.
//
//   w8a32_sequential_kernel   one thread per output, ascending k, separately rounded multiply and add: the order of the
//                             16 x 16 kernel's inner loops; bit-exact against the CPU restatement; the checker
//   w8a32_stream_kernel       the bandwidth-bound form for decode sizes: a warp owns an output column, its lanes take
//                             16-byte pieces of the column's int8 row of data_i8_t [N, K] (one pass over the weights
//                             for up to 8 activation rows), per-element dequantisation exactly as above, partial sums
//                             added across lanes at the end (f32 sums in another order: checked to 1e-5 of max|C|)
#include "pg_internal.cuh"

namespace {

__global__ void __launch_bounds__(256) w8a32_sequential_kernel(const float *__restrict__ a, const int8_t *__restrict__ wt,
                                                               const float *__restrict__ ws, int64_t M, int64_t N, int64_t K,
                                                               float *__restrict__ c)
{
    const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (idx >= M * N) return;
    const int64_t m = idx / N, n = idx - m * N;
    const float s = ws[n];
    const int8_t *w = wt + n * K;
    const float *x = a + m * K;
    float sum = 0.0f;
    for (int64_t k = 0; k < K; k++) sum = __fadd_rn(sum, __fmul_rn(x[k], __fmul_rn((float)w[k], s)));
    c[idx] = sum;
}

constexpr int WS_ROWS = 8;   // activation rows per pass over the weights

// grid-stride over columns, one warp per column; K % 16 == 0, 16-byte aligned rows
__global__ void __launch_bounds__(256) w8a32_stream_kernel(const float *__restrict__ a, const int8_t *__restrict__ wt,
                                                           const float *__restrict__ ws, int M, int64_t N, int K, int m0,
                                                           float *__restrict__ c)
{
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * 256 + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * 256) >> 5;
    const int rows = min(WS_ROWS, M - m0);
    for (int64_t n = warp; n < N; n += nwarps) {
        const float s = __ldg(ws + n);
        const uint4 *w = reinterpret_cast<const uint4 *>(wt + n * K);
        float acc[WS_ROWS];
#pragma unroll
        for (int r = 0; r < WS_ROWS; r++) acc[r] = 0.0f;
        for (int kc = lane; kc < (K >> 4); kc += 32) {
            const uint4 q = __ldcs(w + kc);                       // weights are read once: streaming load
            const uint32_t words[4] = {q.x, q.y, q.z, q.w};
            float wv[16];
#pragma unroll
            for (int j = 0; j < 16; j++) wv[j] = __fmul_rn((float)(int8_t)(words[j >> 2] >> (8 * (j & 3))), s);
#pragma unroll
            for (int r = 0; r < WS_ROWS; r++) {
                if (r < rows) {
                    const float4 *x = reinterpret_cast<const float4 *>(a + (int64_t)(m0 + r) * K) + kc * 4;
#pragma unroll
                    for (int j4 = 0; j4 < 4; j4++) {
                        const float4 xv = __ldg(x + j4);
                        acc[r] = fmaf(xv.x, wv[4 * j4], acc[r]);
                        acc[r] = fmaf(xv.y, wv[4 * j4 + 1], acc[r]);
                        acc[r] = fmaf(xv.z, wv[4 * j4 + 2], acc[r]);
                        acc[r] = fmaf(xv.w, wv[4 * j4 + 3], acc[r]);
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < WS_ROWS; r++) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], o);
            if (lane == 0 && r < rows) c[(int64_t)(m0 + r) * N + n] = acc[r];
        }
    }
}

}  // namespace

extern "C" PG_API int32_t pg_matmul_dequant_w8a32(pg_ctx *ctx, const float *d_x, int64_t m, int64_t k, const pg_qtensor *w, float *d_y,
                                                  int32_t sequential)
{
    PG_ENTER(ctx);
    PG_REQUIRE(w != nullptr, "matmul_dequant_w8a32: weights not on GPU");      // expect("weights not on GPU"), src/quant.rs:208-209
    PG_REQUIRE(m >= 0 && k >= 0, "matmul_dequant_w8a32: negative shape");
    PG_REQUIRE(w->rows == k, "matmul_dequant_w8a32: w.rows (%lld) != k (%lld)", (long long)w->rows, (long long)k);
    const int64_t n = w->cols;
    if (m * n == 0) return PG_OK;
    PG_REQUIRE(d_y && (k == 0 || d_x), "matmul_dequant_w8a32: null pointer");
    PG_REQUIRE(m * n < (1ll << 40) && m <= 0x7fffffff && k <= 0x7fffffff, "matmul_dequant_w8a32: shape too large");
    const bool fast = !sequential && k > 0 && (k % 16 == 0) && (((uintptr_t)w->d_data_i8_t | (uintptr_t)d_x) & 15) == 0;
    if (!fast) {
        const int64_t blocks = (m * n + 255) / 256;
        PG_REQUIRE(blocks <= 0x7fffffff, "matmul_dequant_w8a32: shape too large");
        w8a32_sequential_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(d_x, w->d_data_i8_t, w->d_scales, m, n, k, d_y);
        PG_LAUNCHED();
        return PG_OK;
    }
    int64_t blocks = (n + 7) / 8;
    if (blocks > 8ll * ctx->sm_count) blocks = 8ll * ctx->sm_count;
    for (int64_t m0 = 0; m0 < m; m0 += WS_ROWS) {
        w8a32_stream_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(d_x, w->d_data_i8_t, w->d_scales, (int)m, n, (int)k, (int)m0, d_y);
        PG_LAUNCHED();
    }
    return PG_OK;
}
