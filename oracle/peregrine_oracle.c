/*
 * CPU oracle for the quantized-inference path of etam103/peregrine.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker that the CUDA kernels are
 * compared against and the CPU baseline that the benchmark times.  Nothing in
 * the shipped library links, loads or calls it.
 *
 * It restates, in plain C, the scalar (non-aarch64) branch of the reference's
 * Rust code, which is the branch an x86-64 host compiles:
 *
 *   src/quant.rs:27-75     quantize_weights
 *   src/quant.rs:97-109    quantize_activations (scalar branch)
 *   src/quant.rs:115-123   dequantize
 *   src/quant.rs:154-166   matmul_quantized (scalar i32 GEMM + two-scale epilogue)
 *   src/gguf.rs:286-302    dequant_q8_0
 *   src/gguf.rs:307-326    dequant_q4_0
 *   src/gguf.rs:331-351    dequant_q4_1
 *   src/gguf.rs:354-382    f16_to_f32
 *   src/tensor.rs:1342-1354  Tensor::matmul, naive branch (f32, ascending p)
 *   src/metal/shaders.rs:2329-2379  matmul_dequant_i8 arithmetic (W8A32)
 *
 * Parity pin: the reference is Rust and no Rust toolchain exists on the build
 * or GPU machines, so the reference itself cannot be run beside this file.  The
 * restatement is pinned against every known-answer test the reference holds
 * for this path (f16 KATs, Q8_0/Q4_0/Q4_1 single-block KATs, the closed-form
 * quant round-trip and int8-vs-f32 matmul tests); tests/test_oracle_kats.py
 * re-runs them.  No reference test pins i8 values or i32 accumulators bit for
 * bit, so those are pinned only by this restatement of the source.
 *
 * Build rules that matter for bit-exactness: -ffp-contract=off, no -ffast-math,
 * float arithmetic only (no double intermediates).
 *
 * Rust semantics reproduced explicitly:
 *   f32::max(a, b)      returns the non-NaN operand       -> fmaxf
 *   f32::round          half away from zero               -> roundf
 *   f32::clamp(lo, hi)  keeps NaN                         -> comparisons, not fmin/fmax
 *   `as i8` on f32      saturating, NaN -> 0              -> f32_as_i8()
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#if defined(_OPENMP)
#include <omp.h>
#define PGO_PARALLEL_FOR _Pragma("omp parallel for schedule(static)")
#else
#define PGO_PARALLEL_FOR
#endif

#define PGO_EXPORT __attribute__((visibility("default")))

/* Rust `(v.round().clamp(-127.0, 127.0)) as i8` */
static inline int8_t f32_round_clamp_as_i8(float v)
{
    float r = roundf(v);
    if (r < -127.0f) r = -127.0f;      /* NaN compares false twice and survives */
    else if (r > 127.0f) r = 127.0f;
    if (r != r) return 0;              /* Rust float->int cast maps NaN to 0 */
    return (int8_t)r;
}

PGO_EXPORT int pgo_num_threads(void)
{
#if defined(_OPENMP)
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* src/gguf.rs:354-382 */
PGO_EXPORT float pgo_f16_to_f32(uint16_t bits)
{
    uint32_t sign = (bits >> 15) & 1u;
    uint32_t exp = (bits >> 10) & 0x1Fu;
    uint32_t mant = bits & 0x3FFu;
    uint32_t out;
    if (exp == 0) {
        if (mant == 0) {
            out = sign << 31;
        } else {
            uint32_t m = mant;
            int32_t e = 0;
            while ((m & 0x400u) == 0) { m <<= 1; e -= 1; }
            m &= 0x3FFu;
            uint32_t f32_exp = (uint32_t)(127 - 15 + 1 + e);
            out = (sign << 31) | (f32_exp << 23) | (m << 13);
        }
    } else if (exp == 31) {
        out = (sign << 31) | (0xFFu << 23) | (mant << 13);
    } else {
        out = (sign << 31) | ((exp + 127 - 15) << 23) | (mant << 13);
    }
    float f;
    memcpy(&f, &out, 4);
    return f;
}

/* Bit pattern of the above for a whole array: a float returned by value can
 * have a signalling-NaN payload quieted on its way through the caller. */
PGO_EXPORT void pgo_f16_to_f32_bits(const uint16_t *bits, size_t count, uint32_t *out)
{
    for (size_t i = 0; i < count; i++) {
        float f = pgo_f16_to_f32(bits[i]);
        memcpy(&out[i], &f, 4);
    }
}

/* src/quant.rs:27-75.  w is [rows=K, cols=N] row-major.
 * out_i8 [K,N], out_i8_t [N,K], out_scales [N]. */
PGO_EXPORT void pgo_quantize_weights(const float *w, size_t rows, size_t cols,
                                     int8_t *out_i8, int8_t *out_i8_t, float *out_scales)
{
    /* quant.rs:31-39: strict '>' from 0.0, so NaN never becomes the maximum */
    for (size_t n = 0; n < cols; n++) out_scales[n] = 0.0f;
    for (size_t m = 0; m < rows; m++) {
        for (size_t n = 0; n < cols; n++) {
            float v = fabsf(w[m * cols + n]);
            if (v > out_scales[n]) out_scales[n] = v;
        }
    }
    /* quant.rs:42-45 */
    for (size_t n = 0; n < cols; n++) {
        float amax = out_scales[n];
        out_scales[n] = (amax == 0.0f) ? 1.0f : amax / 127.0f;
    }
    /* quant.rs:48-54: true division, then round/clamp/cast */
    PGO_PARALLEL_FOR
    for (size_t m = 0; m < rows; m++) {
        for (size_t n = 0; n < cols; n++) {
            float v = w[m * cols + n] / out_scales[n];
            out_i8[m * cols + n] = f32_round_clamp_as_i8(v);
        }
    }
    /* quant.rs:57-62 */
    if (out_i8_t) {
        PGO_PARALLEL_FOR
        for (size_t n = 0; n < cols; n++)
            for (size_t k = 0; k < rows; k++)
                out_i8_t[n * rows + k] = out_i8[k * cols + n];
    }
}

/* src/quant.rs:97-109.  x is [rows=M, cols=K]. */
PGO_EXPORT void pgo_quantize_activations(const float *x, size_t rows, size_t cols,
                                         int8_t *out_i8, float *out_scales)
{
    PGO_PARALLEL_FOR
    for (size_t m = 0; m < rows; m++) {
        const float *row = x + m * cols;
        float amax = 0.0f;
        for (size_t k = 0; k < cols; k++) amax = fmaxf(amax, fabsf(row[k]));
        float scale = (amax == 0.0f) ? 1.0f : amax / 127.0f;
        out_scales[m] = scale;
        float inv_scale = 1.0f / scale;
        for (size_t k = 0; k < cols; k++)
            out_i8[m * cols + k] = f32_round_clamp_as_i8(row[k] * inv_scale);
    }
}

/* src/quant.rs:115-123 */
PGO_EXPORT void pgo_dequantize(const int8_t *data_i8, const float *scales,
                               size_t rows, size_t cols, float *out)
{
    for (size_t m = 0; m < rows; m++)
        for (size_t n = 0; n < cols; n++)
            out[m * cols + n] = (float)data_i8[m * cols + n] * scales[n];
}

/* src/quant.rs:154-166 on already-quantised operands.
 * a_i8 [M,K], b_t [N,K]; out [M,N]; acc_out [M,N] optional (the i32 sums). */
PGO_EXPORT void pgo_gemm_i8(const int8_t *a_i8, const float *a_scales,
                            const int8_t *b_t, const float *w_scales,
                            size_t m, size_t n, size_t k, float *out, int32_t *acc_out)
{
    PGO_PARALLEL_FOR
    for (size_t mn = 0; mn < m * n; mn++) {
        size_t mi = mn / n, ni = mn % n;
        const int8_t *ar = a_i8 + mi * k;
        const int8_t *br = b_t + ni * k;
        int32_t acc = 0;
        for (size_t ki = 0; ki < k; ki++) acc += (int32_t)ar[ki] * (int32_t)br[ki];
        if (acc_out) acc_out[mn] = acc;
        if (out) {
            float t = (float)acc * a_scales[mi];   /* left-associated: two rounded products */
            out[mn] = t * w_scales[ni];
        }
    }
}

/* Selected accumulators only: idx[i] = m*N+n.  For shapes too large to sweep. */
PGO_EXPORT void pgo_gemm_i8_sampled(const int8_t *a_i8, const int8_t *b_t,
                                    size_t n, size_t k, const int64_t *idx, size_t count,
                                    int32_t *acc_out)
{
    PGO_PARALLEL_FOR
    for (size_t i = 0; i < count; i++) {
        size_t mi = (size_t)idx[i] / n, ni = (size_t)idx[i] % n;
        const int8_t *ar = a_i8 + mi * k;
        const int8_t *br = b_t + ni * k;
        int32_t acc = 0;
        for (size_t ki = 0; ki < k; ki++) acc += (int32_t)ar[ki] * (int32_t)br[ki];
        acc_out[i] = acc;
    }
}

/* src/quant.rs:129-169: quantise A, then the GEMM above.
 * a_i8_out [M,K] / a_scales_out [M] are caller scratch and hold the
 * intermediate quantised activations on return. */
PGO_EXPORT void pgo_matmul_quantized(const float *a, size_t m, size_t k,
                                     const int8_t *w_i8_t, const float *w_scales, size_t n,
                                     float *out, int32_t *acc_out,
                                     int8_t *a_i8_out, float *a_scales_out)
{
    pgo_quantize_activations(a, m, k, a_i8_out, a_scales_out);
    pgo_gemm_i8(a_i8_out, a_scales_out, w_i8_t, w_scales, m, n, k, out, acc_out);
}

/* src/gguf.rs:286-302.  Returns 0, or -1 where the reference asserts. */
PGO_EXPORT int pgo_dequant_q8_0(const uint8_t *data, size_t data_len, size_t num_elements, float *out)
{
    if (num_elements % 32 != 0) return -1;
    size_t nb = num_elements / 32;
    if (data_len < nb * 34) return -1;
    PGO_PARALLEL_FOR
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *p = data + b * 34;
        float scale = pgo_f16_to_f32((uint16_t)(p[0] | (p[1] << 8)));
        for (int i = 0; i < 32; i++) out[b * 32 + i] = (float)(int8_t)p[2 + i] * scale;
    }
    return 0;
}

/* src/gguf.rs:307-326: byte i holds element 2i (low nibble) and 2i+1 (high nibble). */
PGO_EXPORT int pgo_dequant_q4_0(const uint8_t *data, size_t data_len, size_t num_elements, float *out)
{
    if (num_elements % 32 != 0) return -1;
    size_t nb = num_elements / 32;
    if (data_len < nb * 18) return -1;
    PGO_PARALLEL_FOR
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *p = data + b * 18;
        float scale = pgo_f16_to_f32((uint16_t)(p[0] | (p[1] << 8)));
        for (int i = 0; i < 16; i++) {
            int32_t lo = (int32_t)(p[2 + i] & 0x0F) - 8;
            int32_t hi = (int32_t)((p[2 + i] >> 4) & 0x0F) - 8;
            out[b * 32 + 2 * i] = (float)lo * scale;
            out[b * 32 + 2 * i + 1] = (float)hi * scale;
        }
    }
    return 0;
}

/* src/gguf.rs:331-351: nibble * scale + min, product and sum rounded separately. */
PGO_EXPORT int pgo_dequant_q4_1(const uint8_t *data, size_t data_len, size_t num_elements, float *out)
{
    if (num_elements % 32 != 0) return -1;
    size_t nb = num_elements / 32;
    if (data_len < nb * 20) return -1;
    PGO_PARALLEL_FOR
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *p = data + b * 20;
        float scale = pgo_f16_to_f32((uint16_t)(p[0] | (p[1] << 8)));
        float min = pgo_f16_to_f32((uint16_t)(p[2] | (p[3] << 8)));
        for (int i = 0; i < 16; i++) {
            float lo = (float)(p[4 + i] & 0x0F);
            float hi = (float)((p[4 + i] >> 4) & 0x0F);
            out[b * 32 + 2 * i] = lo * scale + min;
            out[b * 32 + 2 * i + 1] = hi * scale + min;
        }
    }
    return 0;
}

/* src/tensor.rs:1342-1354: [M,K] x [K,N], sum from 0.0 in ascending p. */
PGO_EXPORT void pgo_matmul_f32(const float *a, const float *b, size_t m, size_t k, size_t n, float *out)
{
    PGO_PARALLEL_FOR
    for (size_t i = 0; i < m; i++) {
        for (size_t j = 0; j < n; j++) {
            float sum = 0.0f;
            for (size_t p = 0; p < k; p++) sum += a[i * k + p] * b[p * n + j];
            out[i * n + j] = sum;
        }
    }
}

/* What the Llama linears compute from a GGUF tensor today: the weight [N,K]
 * (GGUF [out,in]) is dequantised to f32 (gguf.rs:485-517), transposed to [K,N]
 * (models/llama/model.rs:243-257) and multiplied by Tensor::matmul.  Element
 * (m,n) is therefore sum_{p ascending} x[m,p] * wd[n,p]; the transposition only
 * moves data, so it is folded away here.  wd is the dequantised [N,K] weight. */
PGO_EXPORT void pgo_matmul_f32_wt(const float *x, const float *wd, size_t m, size_t k, size_t n, float *out)
{
    PGO_PARALLEL_FOR
    for (size_t j = 0; j < n; j++) {
        const float *wr = wd + j * k;
        for (size_t i = 0; i < m; i++) {
            const float *xr = x + i * k;
            float sum = 0.0f;
            for (size_t p = 0; p < k; p++) sum += xr[p] * wr[p];
            out[i * n + j] = sum;
        }
    }
}

/* The same product with f64 accumulation: arbiter for order-dependent f32 sums. */
PGO_EXPORT void pgo_matmul_f64acc_wt(const float *x, const float *wd, size_t m, size_t k, size_t n, double *out)
{
    PGO_PARALLEL_FOR
    for (size_t j = 0; j < n; j++) {
        const float *wr = wd + j * k;
        for (size_t i = 0; i < m; i++) {
            const float *xr = x + i * k;
            double sum = 0.0;
            for (size_t p = 0; p < k; p++) sum += (double)xr[p] * (double)wr[p];
            out[i * n + j] = sum;
        }
    }
}

/* Arithmetic of the reference's Metal kernel matmul_dequant_i8
 * (src/metal/shaders.rs:2329-2379): activations stay f32, each weight is
 * float(q) * scale[n], f32 accumulation in ascending k.  w_i8 is [K,N]. */
PGO_EXPORT void pgo_matmul_dequant_w8a32(const float *a, const int8_t *w_i8, const float *w_scales,
                                         size_t m, size_t n, size_t k, float *out)
{
    PGO_PARALLEL_FOR
    for (size_t i = 0; i < m; i++) {
        for (size_t j = 0; j < n; j++) {
            float sum = 0.0f;
            for (size_t p = 0; p < k; p++) {
                float wv = (float)w_i8[p * n + j] * w_scales[j];
                sum += a[i * k + p] * wv;
            }
            out[i * n + j] = sum;
        }
    }
}
