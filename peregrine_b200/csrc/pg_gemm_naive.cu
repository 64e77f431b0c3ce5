// The on-device checker for the integer GEMM: one thread per output element, the plain
// sum of src/quant.rs:157-165 (i32 accumulate, then `acc as f32 * a_scale * w_scale`).
// It is slow by design and shares nothing with the fast kernels, so it can check them
// on shapes that are too large to sweep on the CPU.  It also serves any shape the fast
// kernels reject (K not a multiple of 16, misaligned pointers).
#include "pg_internal.cuh"

namespace {

__global__ void __launch_bounds__(256) gemm_i8_naive_kernel(const int8_t *__restrict__ a, const float *__restrict__ a_scales,
                                                             int64_t m, int64_t k, const int8_t *__restrict__ bt,
                                                             const float *__restrict__ w_scales, int64_t n,
                                                             float *__restrict__ y, int32_t *__restrict__ acc_out, int vec4)
{
    const int64_t ni = (int64_t)blockIdx.x * 256 + threadIdx.x;
    const int64_t mi = blockIdx.y;
    if (ni >= n || mi >= m) return;
    const int8_t *ar = a + mi * k;
    const int8_t *br = bt + ni * k;
    int32_t acc = 0;
    int64_t p = 0;
    if (vec4) {
        const int *a4 = reinterpret_cast<const int *>(ar);
        const int *b4 = reinterpret_cast<const int *>(br);
        for (; p + 4 <= k; p += 4) acc = __dp4a(a4[p >> 2], b4[p >> 2], acc);
    }
    for (; p < k; p++) acc += (int32_t)ar[p] * (int32_t)br[p];
    if (acc_out) acc_out[mi * n + ni] = acc;
    if (y) y[mi * n + ni] = __fmul_rn(__fmul_rn(__int2float_rn(acc), a_scales[mi]), w_scales[ni]);
}

}  // namespace

int32_t pgk_gemm_i8_naive(pg_ctx *ctx, const int8_t *d_a, const float *d_as, int64_t m, int64_t k, const int8_t *d_bt,
                          const float *d_ws, int64_t n, float *d_y, int32_t *d_acc)
{
    if (m == 0 || n == 0) return PG_OK;
    const int vec4 = (k % 4 == 0) && (((uintptr_t)d_a & 3) == 0) && (((uintptr_t)d_bt & 3) == 0);
    for (int64_t m0 = 0; m0 < m; m0 += 65535) {
        const int64_t mc = (m - m0 < 65535) ? (m - m0) : 65535;
        dim3 g((unsigned)((n + 255) / 256), (unsigned)mc);
        gemm_i8_naive_kernel<<<g, 256, 0, ctx->stream>>>(d_a + m0 * k, d_as ? d_as + m0 : nullptr, mc, k, d_bt, d_ws, n,
                                                         d_y ? d_y + m0 * n : nullptr, d_acc ? d_acc + m0 * n : nullptr, vec4);
        PG_LAUNCHED();
    }
    return PG_OK;
}
