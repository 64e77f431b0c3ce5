/*
 * Block encoders for GGUF Q8_0 / Q4_0 / Q4_1 test data.
 *
 * TEST INFRASTRUCTURE ONLY, and NOT a restatement of the reference: the
 * reference ships decoders only (src/gguf.rs:286-351) and has no encoder.  The
 * single contract of these generators is that the reference decoder accepts
 * their bytes: 32-element blocks, little-endian f16 scale first, then the
 * quants; Q4_0/Q4_1 pack element 2i in the low nibble and 2i+1 in the high
 * nibble of byte i (the order src/gguf.rs:317-323 reads).  The oracle and the
 * CUDA kernels both consume the same bytes, so the choice of encoder cannot
 * affect parity.
 *
 *   Q8_0: d = f16(absmax/127), q = clamp(roundf(x / f32(d)), -127, 127)
 *   Q4_0: d = f16(absmax/7),   q = clamp(roundf(x / f32(d)), -8, 7) + 8
 *   Q4_1: d = f16((max-min)/15), m = f16(min), q = clamp(roundf((x - f32(m)) / f32(d)), 0, 15)
 *   d == 0 encodes every element as 0 (nibble 8 for Q4_0).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#define PGO_EXPORT __attribute__((visibility("default")))

float pgo_f16_to_f32(uint16_t bits);

/* f32 -> f16, round to nearest even, overflow to inf, subnormals kept */
PGO_EXPORT uint16_t pgo_f32_to_f16(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7FFFFFFFu;
    if (absx >= 0x7F800000u)                       /* inf / NaN */
        return (uint16_t)(sign | 0x7C00u | (absx > 0x7F800000u ? (0x200u | ((absx >> 13) & 0x3FFu)) : 0));
    if (absx >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);   /* rounds to >= 65520 -> inf */
    if (absx < 0x33000001u) return (uint16_t)sign;                /* <= 2^-25 rounds to 0 */
    int32_t e = (int32_t)(absx >> 23) - 127;
    uint32_t mant = (absx & 0x7FFFFFu) | 0x800000u;
    uint32_t shift, half;
    uint32_t out;
    if (e < -14) {                                 /* subnormal half */
        shift = (uint32_t)(13 + (-14 - e));
        out = mant >> shift;
    } else {
        shift = 13;
        out = ((uint32_t)(e + 15) << 10) + ((mant >> 13) & 0x3FFu);
    }
    half = 1u << (shift - 1);
    uint32_t rem = mant & ((1u << shift) - 1);
    if (rem > half || (rem == half && (out & 1u))) out += 1;      /* carries propagate into the exponent */
    return (uint16_t)(sign | out);
}

static inline float clampf(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }

PGO_EXPORT void pgo_encode_q8_0(const float *x, size_t num_elements, uint8_t *out)
{
    size_t nb = num_elements / 32;
    for (size_t b = 0; b < nb; b++) {
        const float *p = x + b * 32;
        uint8_t *o = out + b * 34;
        float amax = 0.0f;
        for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(p[i]));
        uint16_t dh = pgo_f32_to_f16(amax / 127.0f);
        float d = pgo_f16_to_f32(dh);
        o[0] = (uint8_t)(dh & 0xFF);
        o[1] = (uint8_t)(dh >> 8);
        for (int i = 0; i < 32; i++) {
            float q = (d == 0.0f) ? 0.0f : clampf(roundf(p[i] / d), -127.0f, 127.0f);
            o[2 + i] = (uint8_t)(int8_t)q;
        }
    }
}

PGO_EXPORT void pgo_encode_q4_0(const float *x, size_t num_elements, uint8_t *out)
{
    size_t nb = num_elements / 32;
    for (size_t b = 0; b < nb; b++) {
        const float *p = x + b * 32;
        uint8_t *o = out + b * 18;
        float amax = 0.0f;
        for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(p[i]));
        uint16_t dh = pgo_f32_to_f16(amax / 7.0f);
        float d = pgo_f16_to_f32(dh);
        o[0] = (uint8_t)(dh & 0xFF);
        o[1] = (uint8_t)(dh >> 8);
        for (int i = 0; i < 16; i++) {
            float q0 = (d == 0.0f) ? 0.0f : clampf(roundf(p[2 * i] / d), -8.0f, 7.0f);
            float q1 = (d == 0.0f) ? 0.0f : clampf(roundf(p[2 * i + 1] / d), -8.0f, 7.0f);
            o[2 + i] = (uint8_t)(((int)q0 + 8) | (((int)q1 + 8) << 4));
        }
    }
}

PGO_EXPORT void pgo_encode_q4_1(const float *x, size_t num_elements, uint8_t *out)
{
    size_t nb = num_elements / 32;
    for (size_t b = 0; b < nb; b++) {
        const float *p = x + b * 32;
        uint8_t *o = out + b * 20;
        float mn = p[0], mx = p[0];
        for (int i = 1; i < 32; i++) { mn = fminf(mn, p[i]); mx = fmaxf(mx, p[i]); }
        uint16_t dh = pgo_f32_to_f16((mx - mn) / 15.0f);
        uint16_t mh = pgo_f32_to_f16(mn);
        float d = pgo_f16_to_f32(dh), m = pgo_f16_to_f32(mh);
        o[0] = (uint8_t)(dh & 0xFF); o[1] = (uint8_t)(dh >> 8);
        o[2] = (uint8_t)(mh & 0xFF); o[3] = (uint8_t)(mh >> 8);
        for (int i = 0; i < 16; i++) {
            float q0 = (d == 0.0f) ? 0.0f : clampf(roundf((p[2 * i] - m) / d), 0.0f, 15.0f);
            float q1 = (d == 0.0f) ? 0.0f : clampf(roundf((p[2 * i + 1] - m) / d), 0.0f, 15.0f);
            o[4 + i] = (uint8_t)((int)q0 | ((int)q1 << 4));
        }
    }
}
