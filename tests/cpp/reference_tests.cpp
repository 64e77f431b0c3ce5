// The reference's own tests for the quantized path, re-written against the C++ mirror of its API
// (include/peregrine_b200.hpp).  Inputs, shapes and tolerances are the reference's:
//   src/quant.rs:225-291            roundtrip, int8-vs-f32 matmul
//   tests/quant_parity.rs:6-77      roundtrip max error, i8 vs f32 matmul
//   tests/quant_parity.rs:79-107    GPU result read back after an explicit sync (to_gpu / matmul_quantized_gpu)
//   src/gguf.rs:574-631, tests/gguf_parity.rs:7-76   f16 and block known answers
// Exit code 0 = all passed.  Needs a B200 (there is no CPU path).
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "peregrine_b200.hpp"

using namespace peregrine;

static int failures = 0;
#define EXPECT(cond, ...)                     \
    do {                                      \
        if (!(cond)) {                        \
            std::printf("FAIL %s:%d: ", __FILE__, __LINE__); \
            std::printf(__VA_ARGS__);         \
            std::printf("\n");                \
            ++failures;                       \
        }                                     \
    } while (0)

static std::vector<float> matmul_f32(const std::vector<float> &a, const std::vector<float> &w, int m, int k, int n)
{
    std::vector<float> out(m * n);
    for (int mi = 0; mi < m; mi++)
        for (int ni = 0; ni < n; ni++) {
            float sum = 0.0f;
            for (int ki = 0; ki < k; ki++) sum += a[mi * k + ki] * w[ki * n + ni];
            out[mi * n + ni] = sum;
        }
    return out;
}

static void roundtrip(const metal::GpuContext &g, int rows, int cols, const std::vector<float> &data, float eps)
{
    auto qt = quant::quantize_weights(g, data, rows, cols);
    auto rec = quant::dequantize(g, qt);
    for (int n = 0; n < cols; n++) {
        float amax = 0.0f;
        for (int m = 0; m < rows; m++) amax = std::fmax(amax, std::fabs(data[m * cols + n]));
        const float scale = amax == 0.0f ? 1.0f : amax / 127.0f;
        for (int m = 0; m < rows; m++) {
            const float err = std::fabs(data[m * cols + n] - rec[m * cols + n]);
            EXPECT(err <= scale + eps, "col %d row %d: err %g > scale %g", n, m, err, scale);
        }
    }
}

static void i8_vs_f32(const metal::GpuContext &g, int m, int k, int n, int mod, float rt, float at, bool via_gpu_buffer)
{
    std::vector<float> a(m * k), w(k * n);
    for (int i = 0; i < m * k; i++) a[i] = (float)((i * 7 + 3) % mod) / (float)mod - 0.5f;
    for (int i = 0; i < k * n; i++) w[i] = (float)((i * 13 + 7) % mod) / (float)mod - 0.5f;
    auto expected = matmul_f32(a, w, m, k, n);
    auto qt = quant::quantize_weights(g, w, k, n);
    std::vector<float> result;
    if (via_gpu_buffer) {
        qt.to_gpu(g);
        auto buf = quant::matmul_quantized_gpu(g, a, m, k, qt);
        g.sync();
        result = buf.read();
    } else {
        result = quant::matmul_quantized(g, a, m, k, qt);
    }
    for (int i = 0; i < m * n; i++) {
        const float diff = std::fabs(result[i] - expected[i]);
        const float rtol = diff / std::fmax(std::fabs(expected[i]), 1e-6f);
        EXPECT(rtol < rt || diff < at, "i=%d: got %g, expected %g", i, result[i], expected[i]);
    }
}

int main()
{
    metal::GpuContext g(0);
    {   // src/quant.rs:225-249
        const int rows = 32, cols = 64;
        std::vector<float> d(rows * cols);
        for (int i = 0; i < rows * cols; i++) d[i] = ((float)i - (float)(rows * cols / 2)) * 0.01f;
        roundtrip(g, rows, cols, d, 1e-6f);
    }
    {   // tests/quant_parity.rs:6-32
        const int rows = 64, cols = 128;
        std::vector<float> d(rows * cols);
        for (int i = 0; i < rows * cols; i++) d[i] = (float)((i * 17 + 5) % 400) / 100.0f - 2.0f;
        roundtrip(g, rows, cols, d, 1e-7f);
    }
    i8_vs_f32(g, 16, 64, 32, 100, 0.05f, 0.01f, false);   // src/quant.rs:252-291
    i8_vs_f32(g, 32, 128, 64, 200, 0.15f, 0.05f, false);  // tests/quant_parity.rs:35-77
    i8_vs_f32(g, 32, 128, 64, 200, 0.15f, 0.05f, true);   // tests/quant_parity.rs:79-107 (device buffer, explicit sync)

    // src/gguf.rs:574-585
    EXPECT(gguf::f16_to_f32(g, 0x0000) == 0.0f, "f16 0");
    EXPECT(gguf::f16_to_f32(g, 0x3C00) == 1.0f, "f16 1");
    EXPECT(gguf::f16_to_f32(g, 0xBC00) == -1.0f, "f16 -1");
    EXPECT(gguf::f16_to_f32(g, 0x3800) == 0.5f, "f16 0.5");
    EXPECT(gguf::f16_to_f32(g, 0x8000) == 0.0f && std::signbit(gguf::f16_to_f32(g, 0x8000)), "f16 -0");
    {   // src/gguf.rs:588-601 and tests/gguf_parity.rs:7-28
        std::vector<uint8_t> b(34, 0);
        b[1] = 0x3C;
        for (int i = 0; i < 32; i++) b[2 + i] = (uint8_t)i;
        auto r = gguf::dequant_q8_0(g, b, 32);
        for (int i = 0; i < 32; i++) EXPECT(std::fabs(r[i] - (float)i) < 1e-3f, "q8_0 idx %d", i);
        b[0] = 0x00; b[1] = 0x38;
        for (int i = 0; i < 32; i++) b[2 + i] = (uint8_t)(i + 1);
        r = gguf::dequant_q8_0(g, b, 32);
        for (int i = 0; i < 32; i++) EXPECT(std::fabs(r[i] - (i + 1.0f) * 0.5f) < 0.01f, "q8_0 roundtrip idx %d", i);
    }
    {   // src/gguf.rs:604-615 and tests/gguf_parity.rs:31-50
        std::vector<uint8_t> b(18, 0);
        b[1] = 0x3C; b[2] = 0x98;
        auto r = gguf::dequant_q4_0(g, b, 32);
        EXPECT(std::fabs(r[0]) < 1e-3f && std::fabs(r[1] - 1.0f) < 1e-3f, "q4_0 nibble order: %g %g", r[0], r[1]);
        b.assign(18, 0x88); b[0] = 0x00; b[1] = 0x40;
        r = gguf::dequant_q4_0(g, b, 32);
        for (int i = 0; i < 32; i++) EXPECT(std::fabs(r[i]) < 0.01f, "q4_0 symmetry idx %d", i);
    }
    {   // src/gguf.rs:618-631 and tests/gguf_parity.rs:53-76
        std::vector<uint8_t> b(20, 0);
        b[1] = 0x3C; b[4] = 0x53;
        auto r = gguf::dequant_q4_1(g, b, 32);
        EXPECT(std::fabs(r[0] - 3.0f) < 1e-3f && std::fabs(r[1] - 5.0f) < 1e-3f, "q4_1 simple");
        b.assign(20, 0); b[1] = 0x3C; b[3] = 0x49;
        r = gguf::dequant_q4_1(g, b, 32);
        for (int i = 0; i < 32; i++) EXPECT(std::fabs(r[i] - 10.0f) < 0.1f, "q4_1 min idx %d", i);
    }
    {   // the reference's assert!s become exceptions
        bool threw = false;
        try {
            gguf::dequant_q8_0(g, std::vector<uint8_t>(34, 0), 31);
        } catch (const Panic &) {
            threw = true;
        }
        EXPECT(threw, "num_elements %% 32 != 0 must be rejected");
        threw = false;
        try {
            auto qt = quant::quantize_weights(g, std::vector<float>(64 * 8, 0.5f), 64, 8);
            quant::matmul_quantized(g, std::vector<float>(2 * 32, 1.0f), 2, 32, qt);
        } catch (const Panic &) {
            threw = true;
        }
        EXPECT(threw, "w.rows != k must be rejected");
    }
    {   // Huffman-coded weights (src/huffman.rs): bit lengths 3, 3, 2, 1 for the values -118, -108, -98, -88 give the canonical
        // codes 110, 111, 10, 0; the 2 x 2 matrix [-88, -98; -118, -108] is the stream 0 10 110 111 = 0x5B 0x80
        huffman::HuffmanTensor ht;
        ht.bit_lengths.assign(256, 0);
        ht.bit_lengths[10] = 3; ht.bit_lengths[20] = 3; ht.bit_lengths[30] = 2; ht.bit_lengths[40] = 1;
        ht.streams = {{0x5B, 0x80}};
        ht.stream_lengths = {4};
        ht.scales = {0.5f, 0.25f};
        ht.rows = 2; ht.cols = 2;
        auto qt = ht.decode_to_quantized(g);
        const int8_t want[4] = {-88, -98, -118, -108}, want_t[4] = {-88, -118, -98, -108};
        for (int i = 0; i < 4; i++) EXPECT(qt.data_i8[i] == want[i] && qt.data_i8_t[i] == want_t[i], "huffman decode idx %d", i);
        // y = x . (q * scale): x = [1, 0] picks the first row
        auto y = huffman::matmul_huffman(g, {1.0f, 0.0f}, 1, 2, ht);
        EXPECT(std::fabs(y[0] - (-88.0f * 0.5f)) < 0.5f && std::fabs(y[1] - (-98.0f * 0.25f)) < 0.25f, "matmul_huffman: %g %g", y[0], y[1]);
        bool threw = false;
        ht.stream_lengths = {3};
        try {
            ht.to_gpu(g);
        } catch (const Panic &) {
            threw = true;
        }
        EXPECT(threw, "streams that do not hold rows * cols symbols must be rejected");
    }
    std::printf(failures ? "%d FAILURES\n" : "all reference tests passed\n", failures);
    return failures ? 1 : 0;
}
