// C++ host-side mirror of the reference's Rust API for the quantized path, on top of the C ABI
// (peregrine_b200.h).  Same names, argument order and error behaviour as
//
//   peregrine::quant   src/quant.rs:12-218     QuantizedTensor, quantize_weights,
//                                              quantize_activations, dequantize, matmul_quantized,
//                                              QuantizedTensor::to_gpu / from_gpu, matmul_quantized_gpu
//   peregrine::gguf    src/gguf.rs:286-401     dequant_q8_0 / q4_0 / q4_1, f16_to_f32,
//                                              load_tensor_q8_as_quantized
//   peregrine::metal   src/metal/context.rs    GpuContext (alloc / upload / sync), GpuBuffer<T>::read
//
// Where the reference panics (assert!, expect) these throw peregrine::Panic carrying the library's
// message.  Header-only; link with -lperegrine_b200.
#pragma once

#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "peregrine_b200.h"

namespace peregrine {

struct Panic : std::runtime_error {
    int32_t code;
    Panic(int32_t c, const std::string &m) : std::runtime_error(m), code(c) {}
};

inline void check(int32_t rc)
{
    if (rc != PG_OK) throw Panic(rc, pg_last_error());
}

namespace metal {

class GpuContext;

// GpuBuffer<T>: a typed device allocation; read() blocks and copies back.
template <typename T>
class GpuBuffer {
public:
    GpuBuffer(pg_ctx *ctx, size_t count) : ctx_(ctx), count_(count) { check(pg_mem_alloc(ctx, count * sizeof(T), &ptr_)); }
    GpuBuffer(const GpuBuffer &) = delete;
    GpuBuffer &operator=(const GpuBuffer &) = delete;
    GpuBuffer(GpuBuffer &&o) noexcept : ctx_(o.ctx_), ptr_(o.ptr_), count_(o.count_) { o.ptr_ = nullptr; }
    ~GpuBuffer()
    {
        if (ptr_) pg_mem_free(ctx_, ptr_);
    }
    T *ptr() const { return static_cast<T *>(ptr_); }
    size_t len() const { return count_; }
    std::vector<T> read() const
    {
        std::vector<T> out(count_);
        check(pg_mem_download(ctx_, out.data(), ptr_, count_ * sizeof(T)));
        return out;
    }

private:
    pg_ctx *ctx_;
    void *ptr_ = nullptr;
    size_t count_;
};

// One CUDA device + stream (the reference keeps one per thread).
class GpuContext {
public:
    explicit GpuContext(int device = 0, void *stream = nullptr) { check(pg_ctx_create(device, stream, &ctx_)); }
    GpuContext(const GpuContext &) = delete;
    GpuContext &operator=(const GpuContext &) = delete;
    ~GpuContext() { pg_ctx_destroy(ctx_); }
    pg_ctx *raw() const { return ctx_; }
    template <typename T>
    GpuBuffer<T> alloc(size_t count) const
    {
        return GpuBuffer<T>(ctx_, count);
    }
    template <typename T>
    GpuBuffer<T> upload(const std::vector<T> &host) const
    {
        GpuBuffer<T> b(ctx_, host.size());
        check(pg_mem_upload(ctx_, b.ptr(), host.data(), host.size() * sizeof(T)));
        check(pg_ctx_sync(ctx_));  // `host` may be a temporary
        return b;
    }
    void sync() const { check(pg_ctx_sync(ctx_)); }

private:
    pg_ctx *ctx_ = nullptr;
};

}  // namespace metal

namespace quant {

using metal::GpuBuffer;
using metal::GpuContext;

// src/quant.rs:12-23.  `gpu` plays the role of gpu_data_i8 / gpu_scales.
struct QuantizedTensor {
    std::vector<int8_t> data_i8;    // [rows, cols]
    std::vector<int8_t> data_i8_t;  // [cols, rows]
    std::vector<float> scales;      // [cols]
    size_t rows = 0, cols = 0;
    std::shared_ptr<pg_qtensor> gpu;

    // QuantizedTensor::to_gpu (idempotent) / from_gpu
    void to_gpu(const GpuContext &g)
    {
        if (gpu) return;
        pg_qtensor *h = nullptr;
        check(pg_qtensor_upload(g.raw(), data_i8.empty() ? nullptr : data_i8.data(), data_i8_t.data(), scales.data(), (int64_t)rows,
                                (int64_t)cols, 0, (int64_t)cols, &h));
        pg_ctx *ctx = g.raw();
        gpu = std::shared_ptr<pg_qtensor>(h, [ctx](pg_qtensor *p) { pg_qtensor_free(ctx, p); });
    }
    void from_gpu(const GpuContext &g)
    {
        if (!gpu) return;
        check(pg_qtensor_download(g.raw(), gpu.get(), data_i8.empty() ? nullptr : data_i8.data(), data_i8_t.data(), scales.data()));
    }
};

inline void require_len(size_t got, size_t want, const char *what)
{
    if (got != want) throw Panic(PG_ERR_INVALID, std::string(what) + ": data.len() != rows * cols");
}

// src/quant.rs:27-75
inline QuantizedTensor quantize_weights(const GpuContext &g, const std::vector<float> &data, size_t rows, size_t cols)
{
    require_len(data.size(), rows * cols, "quantize_weights");
    QuantizedTensor qt;
    qt.rows = rows;
    qt.cols = cols;
    qt.data_i8.resize(rows * cols);
    qt.data_i8_t.resize(rows * cols);
    qt.scales.resize(cols);
    check(pg_quantize_weights_host(g.raw(), data.data(), (int64_t)rows, (int64_t)cols, qt.data_i8.data(), qt.data_i8_t.data(),
                                   qt.scales.data()));
    return qt;
}

// src/quant.rs:79-112
inline std::pair<std::vector<int8_t>, std::vector<float>> quantize_activations(const GpuContext &g, const std::vector<float> &data,
                                                                              size_t rows, size_t cols)
{
    require_len(data.size(), rows * cols, "quantize_activations");
    std::vector<int8_t> q(rows * cols);
    std::vector<float> s(rows);
    check(pg_quantize_activations_host(g.raw(), data.data(), (int64_t)rows, (int64_t)cols, q.data(), s.data()));
    return {std::move(q), std::move(s)};
}

// src/quant.rs:115-123
inline std::vector<float> dequantize(const GpuContext &g, const QuantizedTensor &qt)
{
    auto d_q = g.upload(qt.data_i8);
    auto d_s = g.upload(qt.scales);
    auto d_o = g.alloc<float>(qt.rows * qt.cols);
    check(pg_dequantize(g.raw(), d_q.ptr(), d_s.ptr(), (int64_t)qt.rows, (int64_t)qt.cols, d_o.ptr()));
    return d_o.read();
}

// src/quant.rs:129-169: host slices in, host result out; weights are uploaded on first use.
inline std::vector<float> matmul_quantized(const GpuContext &g, const std::vector<float> &a_data, size_t m, size_t k, QuantizedTensor &w)
{
    if (w.rows != k) throw Panic(PG_ERR_INVALID, "matmul_quantized: w.rows != k");
    require_len(a_data.size(), m * k, "matmul_quantized");
    w.to_gpu(g);
    std::vector<float> out(m * w.cols);
    check(pg_matmul_quantized_host(g.raw(), a_data.data(), (int64_t)m, (int64_t)k, w.gpu.get(), out.data()));
    return out;
}

// src/quant.rs:195-218: uploads A, enqueues, returns the device buffer WITHOUT synchronising.
inline GpuBuffer<float> matmul_quantized_gpu(const GpuContext &g, const std::vector<float> &a_data, size_t m, size_t k,
                                             const QuantizedTensor &w)
{
    if (w.rows != k) throw Panic(PG_ERR_INVALID, "matmul_quantized_gpu: w.rows != k");
    require_len(a_data.size(), m * k, "matmul_quantized_gpu");
    if (!w.gpu) throw Panic(PG_ERR_INVALID, "weights not on GPU");
    auto a_buf = g.upload(a_data);
    auto out = g.alloc<float>(m * w.cols);
    check(pg_matmul_quantized(g.raw(), a_buf.ptr(), (int64_t)m, (int64_t)k, w.gpu.get(), out.ptr()));
    g.sync();  // a_buf is released on return; the reference's Metal buffer is reference-counted instead
    return out;
}

}  // namespace quant

namespace gguf {

using metal::GpuContext;

inline std::vector<float> dequant_blocks(const GpuContext &g, int32_t type, const std::vector<uint8_t> &data, size_t num_elements)
{
    std::vector<float> out(num_elements);
    check(pg_dequant_blocks_host(g.raw(), type, data.data(), data.size(), (int64_t)num_elements, out.data()));
    return out;
}
// src/gguf.rs:286-302, 307-326, 331-351
inline std::vector<float> dequant_q8_0(const GpuContext &g, const std::vector<uint8_t> &d, size_t n) { return dequant_blocks(g, PG_GGUF_Q8_0, d, n); }
inline std::vector<float> dequant_q4_0(const GpuContext &g, const std::vector<uint8_t> &d, size_t n) { return dequant_blocks(g, PG_GGUF_Q4_0, d, n); }
inline std::vector<float> dequant_q4_1(const GpuContext &g, const std::vector<uint8_t> &d, size_t n) { return dequant_blocks(g, PG_GGUF_Q4_1, d, n); }

// src/gguf.rs:354-382
inline float f16_to_f32(const GpuContext &g, uint16_t bits)
{
    auto d_in = g.upload(std::vector<uint16_t>{bits});
    auto d_out = g.alloc<float>(1);
    check(pg_f16_to_f32(g.raw(), d_in.ptr(), 1, d_out.ptr()));
    return d_out.read()[0];
}

// src/gguf.rs:386-401
inline quant::QuantizedTensor load_tensor_q8_as_quantized(const GpuContext &g, const std::vector<uint8_t> &data, size_t rows, size_t cols)
{
    pg_qtensor *h = nullptr;
    check(pg_qtensor_from_q8_0(g.raw(), data.data(), data.size(), (int64_t)rows, (int64_t)cols, &h));
    quant::QuantizedTensor qt;
    qt.rows = rows;
    qt.cols = cols;
    qt.data_i8.resize(rows * cols);
    qt.data_i8_t.resize(rows * cols);
    qt.scales.resize(cols);
    pg_ctx *ctx = g.raw();
    qt.gpu = std::shared_ptr<pg_qtensor>(h, [ctx](pg_qtensor *p) { pg_qtensor_free(ctx, p); });
    qt.from_gpu(g);
    return qt;
}

// A GGUF [out = N, in = K] weight kept in block form on the GPU; matmul gives y[M,N] = x[M,K] . dequant(W)^T
// (what load_tensor_f32 + load_transposed_weight + Tensor::matmul compute: src/gguf.rs:485-517,
// src/models/llama/model.rs:243-257, src/tensor.rs:1342-1354).
class GgufWeight {
public:
    GgufWeight(const GpuContext &g, int32_t type, const std::vector<uint8_t> &raw, size_t n, size_t k) : ctx_(g.raw()), n_(n), k_(k)
    {
        check(pg_gguf_upload(ctx_, type, raw.data(), raw.size(), (int64_t)n, (int64_t)k, 0, (int64_t)n, &w_));
    }
    GgufWeight(const GgufWeight &) = delete;
    GgufWeight &operator=(const GgufWeight &) = delete;
    ~GgufWeight() { pg_gguf_free(ctx_, w_); }
    std::vector<float> matmul(const std::vector<float> &x, size_t m) const
    {
        if (x.size() != m * k_) throw Panic(PG_ERR_INVALID, "matmul: x.len() != m * k");
        std::vector<float> y(m * n_);
        check(pg_matmul_gguf_host(ctx_, x.data(), (int64_t)m, w_, y.data()));
        return y;
    }

private:
    pg_ctx *ctx_;
    pg_gguf_weight *w_ = nullptr;
    size_t n_, k_;
};

}  // namespace gguf

namespace huffman {

using metal::GpuContext;

// src/huffman.rs:311-325, decoding side: the code book as HuffmanTable::to_bytes gives it (256 bit lengths), the
// bitstreams, the symbols per stream, the per-column scales.  (Building a code and encoding stay with the caller.)
struct HuffmanTensor {
    std::vector<uint8_t> bit_lengths;            // 256
    std::vector<std::vector<uint8_t>> streams;
    std::vector<size_t> stream_lengths;
    std::vector<float> scales;
    size_t rows = 0, cols = 0;

    // src/huffman.rs:430-437, with the decode on the device: the resident tensor
    quant::QuantizedTensor to_gpu(const GpuContext &g) const
    {
        if (bit_lengths.size() < 256) throw Panic(PG_ERR_INVALID, "codebook too short");
        if (streams.size() != stream_lengths.size()) throw Panic(PG_ERR_INVALID, "one length per stream");
        std::vector<uint8_t> packed;
        std::vector<uint64_t> sizes, lens;
        for (size_t i = 0; i < streams.size(); i++) {
            packed.insert(packed.end(), streams[i].begin(), streams[i].end());
            sizes.push_back(streams[i].size());
            lens.push_back(stream_lengths[i]);
        }
        pg_qtensor *h = nullptr;
        check(pg_qtensor_from_huffman(g.raw(), bit_lengths.data(), (int64_t)streams.size(), lens.data(), sizes.data(),
                                      packed.empty() ? nullptr : packed.data(), scales.data(), (int64_t)rows, (int64_t)cols, &h));
        quant::QuantizedTensor qt;
        qt.rows = rows;
        qt.cols = cols;
        qt.scales = scales;
        pg_ctx *ctx = g.raw();
        qt.gpu = std::shared_ptr<pg_qtensor>(h, [ctx](pg_qtensor *p) { pg_qtensor_free(ctx, p); });
        return qt;
    }
    // src/huffman.rs:374-404: all host fields filled in
    quant::QuantizedTensor decode_to_quantized(const GpuContext &g) const
    {
        quant::QuantizedTensor qt = to_gpu(g);
        qt.data_i8.resize(rows * cols);
        qt.data_i8_t.resize(rows * cols);
        if (rows * cols) qt.from_gpu(g);
        return qt;
    }
};

// src/huffman.rs:465-476
inline std::vector<float> matmul_huffman(const GpuContext &g, const std::vector<float> &a_data, size_t m, size_t k, const HuffmanTensor &ht)
{
    if (ht.rows != k) throw Panic(PG_ERR_INVALID, "matmul_huffman: ht.rows != k");
    quant::QuantizedTensor qt = ht.to_gpu(g);
    return quant::matmul_quantized(g, a_data, m, k, qt);
}

}  // namespace huffman
}  // namespace peregrine
