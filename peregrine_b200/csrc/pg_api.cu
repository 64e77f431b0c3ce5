// The extern "C" surface declared in include/peregrine_b200.h: argument checks (where the
// reference asserts), object lifetimes, host<->device staging for the *_host forms and the
// choice of kernel.  No arithmetic happens here.
#include <stdarg.h>
#include <string.h>

#include <new>

#include "pg_internal.cuh"

std::atomic<uint64_t> g_pg_launches{0};
static thread_local char g_err[512] = "";

void pg_set_error(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

// Grows one of the context's device blocks.  Work already enqueued may still use the old block, so the stream is
// drained first; a recorded graph may use it for as long as it lives, so with graphs alive the old block is parked
// (pg_ctx::retired) instead of freed.
static int32_t grow_block(pg_ctx *ctx, void **block, size_t *have, size_t bytes, const char *what, bool zeroed)
{
    if (bytes <= *have) return PG_OK;
    if (ctx->capturing)
        PG_FAIL(PG_ERR_INVALID, "%s memory would have to grow while a graph is being recorded; run the call once before recording", what);
    PG_CUDA(cudaStreamSynchronize(ctx->stream));
    if (*block) {
        if (ctx->live_graphs > 0)
            ctx->retired.push_back(*block);
        else
            PG_CUDA(cudaFree(*block));
    }
    *block = nullptr;
    *have = 0;
    size_t want = bytes + (bytes >> 2);
    want = (want + 255) & ~(size_t)255;
    PG_CUDA(cudaMalloc(block, want));
    if (zeroed) PG_CUDA(cudaMemsetAsync(*block, 0, want, ctx->stream));
    *have = want;
    return PG_OK;
}

int32_t pg_scratch_reserve(pg_ctx *ctx, size_t bytes) { return grow_block(ctx, &ctx->scratch, &ctx->scratch_bytes, bytes, "scratch", false); }
int32_t pg_staging_reserve(pg_ctx *ctx, size_t bytes) { return grow_block(ctx, &ctx->staging, &ctx->staging_bytes, bytes, "staging", false); }
int32_t pg_splitk_reserve(pg_ctx *ctx, size_t bytes) { return grow_block(ctx, &ctx->splitk, &ctx->splitk_bytes, bytes, "split-K workspace", true); }

int32_t pg_pinned_reserve(pg_ctx *ctx, size_t bytes)
{
    if (bytes <= ctx->h_pinned_bytes) return PG_OK;
    PG_CUDA(cudaStreamSynchronize(ctx->stream));
    if (ctx->h_pinned) PG_CUDA(cudaFreeHost(ctx->h_pinned));
    ctx->h_pinned = nullptr;
    ctx->h_pinned_bytes = 0;
    size_t want = bytes + (bytes >> 2);
    PG_CUDA(cudaMallocHost(&ctx->h_pinned, want));
    ctx->h_pinned_bytes = want;
    return PG_OK;
}

namespace {

inline size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

}  // namespace

extern "C" {

const char *pg_last_error(void) { return g_err; }
int32_t pg_version(void) { return 100; }
uint64_t pg_launch_count(void) { return g_pg_launches.load(); }

int32_t pg_ctx_create(int32_t device, void *stream, pg_ctx **out)
{
    PG_REQUIRE(out != nullptr, "pg_ctx_create: out is null");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        PG_FAIL(PG_ERR_UNSUPPORTED, "no CUDA device is visible (%s); this library has no CPU path",
                e == cudaSuccess ? "device count 0" : cudaGetErrorString(e));
    PG_REQUIRE(device >= 0 && device < count, "pg_ctx_create: device %d out of range (0..%d)", device, count - 1);
    cudaDeviceProp prop;
    PG_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        PG_FAIL(PG_ERR_UNSUPPORTED, "device %d is sm_%d%d; the kernels are built for sm_100a only", device, prop.major, prop.minor);
    DeviceGuard guard(device);
    if (!guard.ok) PG_FAIL(PG_ERR_CUDA, "cudaSetDevice(%d) failed", device);
    pg_ctx *ctx = new (std::nothrow) pg_ctx();
    if (!ctx) PG_FAIL(PG_ERR_NOMEM, "out of host memory");
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    if (stream) {
        ctx->stream = (cudaStream_t)stream;
    } else {
        cudaError_t se = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
        if (se != cudaSuccess) {
            delete ctx;
            PG_FAIL(PG_ERR_CUDA, "cudaStreamCreate failed: %s", cudaGetErrorString(se));
        }
        ctx->owns_stream = true;
    }
    cudaError_t me = cudaMalloc(&ctx->d_status, 16 * sizeof(int32_t));  // [0] status word; the rest is spare
    if (me == cudaSuccess) me = cudaMemset(ctx->d_status, 0, 16 * sizeof(int32_t));
    if (me != cudaSuccess) {
        if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
        delete ctx;
        PG_FAIL(PG_ERR_CUDA, "status word allocation failed: %s", cudaGetErrorString(me));
    }
    *out = ctx;
    return PG_OK;
}

int32_t pg_ctx_destroy(pg_ctx *ctx)
{
    if (!ctx) return PG_OK;
    DeviceGuard guard(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->staging) cudaFree(ctx->staging);
    if (ctx->splitk) cudaFree(ctx->splitk);
    for (void *p : ctx->retired) cudaFree(p);
    for (auto &h : ctx->host_calls)
        if (h.exec) cudaGraphExecDestroy(h.exec);
    if (ctx->d_status) cudaFree(ctx->d_status);
    if (ctx->h_pinned) cudaFreeHost(ctx->h_pinned);
    if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return PG_OK;
}

int32_t pg_ctx_sync(pg_ctx *ctx)
{
    PG_ENTER(ctx);
    PG_CUDA(cudaStreamSynchronize(ctx->stream));
    return PG_OK;
}

void *pg_ctx_stream(pg_ctx *ctx) { return ctx ? (void *)ctx->stream : nullptr; }

int32_t pg_ctx_device_status(pg_ctx *ctx, int32_t *status_out)
{
    PG_ENTER(ctx);
    int32_t v = 0;
    PG_CUDA(cudaMemcpyAsync(&v, ctx->d_status, sizeof(v), cudaMemcpyDeviceToHost, ctx->stream));
    PG_CUDA(cudaStreamSynchronize(ctx->stream));
    if (v != 0) {
        PG_CUDA(cudaMemsetAsync(ctx->d_status, 0, sizeof(v), ctx->stream));
        // a kernel that gave up may have left tickets of the split-K workspace taken: back to zero for the next call
        if (ctx->splitk) PG_CUDA(cudaMemsetAsync(ctx->splitk, 0, std::min(ctx->splitk_bytes, (size_t)64 * 1024), ctx->stream));
    }
    if (status_out) *status_out = v;
    return PG_OK;
}

int32_t pg_ctx_set_wait_limit_ns(pg_ctx *ctx, uint64_t ns)
{
    PG_REQUIRE(ctx != nullptr, "null context");
    PG_REQUIRE(ns >= 1000, "pg_ctx_set_wait_limit_ns: a limit below a microsecond would end waits that are about to succeed");
    ctx->wait_limit_ns = ns;
    return PG_OK;
}

uint64_t pg_ctx_scratch_bytes(const pg_ctx *ctx) { return ctx ? (uint64_t)(ctx->scratch_bytes + ctx->staging_bytes + ctx->splitk_bytes) : 0; }

int32_t pg_graph_begin(pg_ctx *ctx)
{
    PG_ENTER(ctx);
    PG_REQUIRE(!ctx->capturing, "pg_graph_begin: already recording");
    PG_CUDA(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    ctx->capturing = true;
    return PG_OK;
}

int32_t pg_graph_end(pg_ctx *ctx, pg_graph **out)
{
    PG_ENTER(ctx);
    PG_REQUIRE(out != nullptr, "pg_graph_end: out is null");
    *out = nullptr;
    PG_REQUIRE(ctx->capturing, "pg_graph_end: not recording");
    ctx->capturing = false;
    cudaGraph_t g = nullptr;
    // cudaStreamEndCapture ends the capture even when a recorded call had failed and invalidated it
    const cudaError_t ce = cudaStreamEndCapture(ctx->stream, &g);
    if (ce != cudaSuccess || !g) {
        cudaGetLastError();
        if (g) cudaGraphDestroy(g);
        PG_FAIL(PG_ERR_CUDA, "pg_graph_end: the recording was invalidated (%s); nothing was recorded", cudaGetErrorString(ce));
    }
    cudaGraphExec_t exec = nullptr;
    cudaError_t e = cudaGraphInstantiate(&exec, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) PG_FAIL(PG_ERR_CUDA, "cudaGraphInstantiate failed: %s", cudaGetErrorString(e));
    pg_graph *pgg = new (std::nothrow) pg_graph();
    if (!pgg) {
        cudaGraphExecDestroy(exec);
        PG_FAIL(PG_ERR_NOMEM, "out of host memory");
    }
    pgg->exec = exec;
    ctx->live_graphs++;
    *out = pgg;
    return PG_OK;
}

int32_t pg_graph_launch(pg_ctx *ctx, pg_graph *graph)
{
    PG_ENTER(ctx);
    PG_REQUIRE(graph && graph->exec, "pg_graph_launch: graph is null");
    PG_CUDA(cudaGraphLaunch(graph->exec, ctx->stream));
    return PG_OK;
}

int32_t pg_graph_free(pg_ctx *ctx, pg_graph *graph)
{
    if (!graph) return PG_OK;
    PG_ENTER(ctx);
    PG_CUDA(cudaStreamSynchronize(ctx->stream));
    if (graph->exec) cudaGraphExecDestroy(graph->exec);
    delete graph;
    if (ctx->live_graphs > 0 && --ctx->live_graphs == 0) {
        for (void *p : ctx->retired) cudaFree(p);
        ctx->retired.clear();
    }
    return PG_OK;
}

int32_t pg_mem_alloc(pg_ctx *ctx, size_t bytes, void **d_out)
{
    PG_ENTER(ctx);
    PG_REQUIRE(d_out != nullptr, "pg_mem_alloc: out is null");
    *d_out = nullptr;
    PG_CUDA(cudaMalloc(d_out, bytes ? bytes : 1));
    return PG_OK;
}

int32_t pg_mem_free(pg_ctx *ctx, void *d_ptr)
{
    PG_ENTER(ctx);
    if (d_ptr) {
        PG_CUDA(cudaStreamSynchronize(ctx->stream));
        PG_CUDA(cudaFree(d_ptr));
    }
    return PG_OK;
}

int32_t pg_mem_upload(pg_ctx *ctx, void *d_dst, const void *src, size_t bytes)
{
    PG_ENTER(ctx);
    if (bytes == 0) return PG_OK;
    PG_REQUIRE(d_dst && src, "pg_mem_upload: null pointer");
    PG_CUDA(cudaMemcpyAsync(d_dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return PG_OK;
}

int32_t pg_mem_download(pg_ctx *ctx, void *dst, const void *d_src, size_t bytes)
{
    PG_ENTER(ctx);
    if (bytes) {
        PG_REQUIRE(dst && d_src, "pg_mem_download: null pointer");
        PG_CUDA(cudaMemcpyAsync(dst, d_src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    }
    PG_CUDA(cudaStreamSynchronize(ctx->stream));
    return PG_OK;
}

// ------------------------------------------------------------ quantisers ----
int32_t pg_quantize_activations(pg_ctx *ctx, const float *d_x, int64_t rows, int64_t cols, int8_t *d_q, float *d_scales)
{
    PG_ENTER(ctx);
    PG_REQUIRE(rows >= 0 && cols >= 0, "quantize_activations: negative shape");
    PG_REQUIRE(rows == 0 || (d_scales && (cols == 0 || (d_x && d_q))), "quantize_activations: null pointer");
    return pgk_quantize_activations(ctx, d_x, rows, cols, d_q, d_scales);
}

int32_t pg_quantize_activations_host(pg_ctx *ctx, const float *x, int64_t rows, int64_t cols, int8_t *q, float *scales)
{
    PG_ENTER(ctx);
    PG_REQUIRE(rows >= 0 && cols >= 0, "quantize_activations: negative shape");
    if (rows == 0) return PG_OK;
    PG_REQUIRE(scales && (cols == 0 || (x && q)), "quantize_activations: null pointer");
    const size_t nx = align256((size_t)rows * cols * 4), nq = align256((size_t)rows * cols), ns = align256((size_t)rows * 4);
    int32_t rc = pg_staging_reserve(ctx, nx + nq + ns);
    if (rc) return rc;
    char *base = (char *)ctx->staging;
    float *d_x = (float *)base;
    int8_t *d_q = (int8_t *)(base + nx);
    float *d_s = (float *)(base + nx + nq);
    if (cols) PG_CUDA(cudaMemcpyAsync(d_x, x, (size_t)rows * cols * 4, cudaMemcpyHostToDevice, ctx->stream));
    rc = pgk_quantize_activations(ctx, d_x, rows, cols, d_q, d_s);
    if (rc) return rc;
    if (cols) PG_CUDA(cudaMemcpyAsync(q, d_q, (size_t)rows * cols, cudaMemcpyDeviceToHost, ctx->stream));
    PG_CUDA(cudaMemcpyAsync(scales, d_s, (size_t)rows * 4, cudaMemcpyDeviceToHost, ctx->stream));
    PG_CUDA(cudaStreamSynchronize(ctx->stream));
    return PG_OK;
}

int32_t pg_quantize_weights(pg_ctx *ctx, const float *d_w, int64_t rows, int64_t cols, int8_t *d_data_i8, int8_t *d_data_i8_t,
                            float *d_scales)
{
    PG_ENTER(ctx);
    PG_REQUIRE(rows >= 0 && cols >= 0, "quantize_weights: negative shape");
    PG_REQUIRE(cols == 0 || d_scales, "quantize_weights: scales is null");
    PG_REQUIRE(rows * cols == 0 || d_w, "quantize_weights: weights pointer is null");
    return pgk_quantize_weights(ctx, d_w, rows, cols, d_data_i8, d_data_i8_t, d_scales);
}

int32_t pg_quantize_weights_host(pg_ctx *ctx, const float *w, int64_t rows, int64_t cols, int8_t *data_i8, int8_t *data_i8_t,
                                 float *scales)
{
    PG_ENTER(ctx);
    PG_REQUIRE(rows >= 0 && cols >= 0, "quantize_weights: negative shape");
    if (cols == 0) return PG_OK;
    PG_REQUIRE(scales && (rows == 0 || w), "quantize_weights: null pointer");
    const size_t total = (size_t)rows * cols;
    void *d_w = nullptr, *d_q = nullptr, *d_qt = nullptr, *d_s = nullptr;
    int32_t rc = PG_OK;
    auto cleanup = [&]() {
        cudaFree(d_w);
        cudaFree(d_q);
        cudaFree(d_qt);
        cudaFree(d_s);
    };
#define PG_TRY(expr)                                                                  \
    do {                                                                              \
        cudaError_t _e = (expr);                                                      \
        if (_e != cudaSuccess) {                                                      \
            pg_set_error("%s failed: %s", #expr, cudaGetErrorString(_e));             \
            cleanup();                                                                \
            return _e == cudaErrorMemoryAllocation ? PG_ERR_NOMEM : PG_ERR_CUDA;      \
        }                                                                             \
    } while (0)
    PG_TRY(cudaMalloc(&d_w, total * 4 + 16));
    PG_TRY(cudaMalloc(&d_q, total + 16));
    PG_TRY(cudaMalloc(&d_qt, total + 16));
    PG_TRY(cudaMalloc(&d_s, (size_t)cols * 4));
    if (total) PG_TRY(cudaMemcpyAsync(d_w, w, total * 4, cudaMemcpyHostToDevice, ctx->stream));
    rc = pgk_quantize_weights(ctx, (const float *)d_w, rows, cols, (int8_t *)d_q, (int8_t *)d_qt, (float *)d_s);
    if (rc) {
        cleanup();
        return rc;
    }
    if (total && data_i8) PG_TRY(cudaMemcpyAsync(data_i8, d_q, total, cudaMemcpyDeviceToHost, ctx->stream));
    if (total && data_i8_t) PG_TRY(cudaMemcpyAsync(data_i8_t, d_qt, total, cudaMemcpyDeviceToHost, ctx->stream));
    PG_TRY(cudaMemcpyAsync(scales, d_s, (size_t)cols * 4, cudaMemcpyDeviceToHost, ctx->stream));
    PG_TRY(cudaStreamSynchronize(ctx->stream));
    cleanup();
    return PG_OK;
}

int32_t pg_dequantize(pg_ctx *ctx, const int8_t *d_data_i8, const float *d_scales, int64_t rows, int64_t cols, float *d_out)
{
    PG_ENTER(ctx);
    PG_REQUIRE(rows >= 0 && cols >= 0, "dequantize: negative shape");
    PG_REQUIRE(rows * cols == 0 || (d_data_i8 && d_scales && d_out), "dequantize: null pointer");
    return pgk_dequantize(ctx, d_data_i8, d_scales, rows, cols, d_out);
}

// ---------------------------------------------------------------- qtensor ----
int32_t pg_qtensor_upload(pg_ctx *ctx, const int8_t *data_i8, const int8_t *data_i8_t, const float *scales, int64_t rows,
                          int64_t cols, int64_t col_begin, int64_t col_end, pg_qtensor **out)
{
    PG_ENTER(ctx);
    PG_REQUIRE(out != nullptr, "qtensor_upload: out is null");
    *out = nullptr;
    PG_REQUIRE(rows >= 0 && cols >= 0, "qtensor_upload: negative shape");
    PG_REQUIRE(0 <= col_begin && col_begin <= col_end && col_end <= cols, "qtensor_upload: column range [%lld,%lld) outside [0,%lld)",
               (long long)col_begin, (long long)col_end, (long long)cols);
    PG_REQUIRE(data_i8_t && scales, "qtensor_upload: data_i8_t and scales are required");
    const int64_t nc = col_end - col_begin;
    pg_qtensor *t = new (std::nothrow) pg_qtensor();
    if (!t) PG_FAIL(PG_ERR_NOMEM, "out of host memory");
    t->rows = rows;
    t->cols = nc;
    t->owned = true;
    void *d_t = nullptr, *d_s = nullptr, *d_q = nullptr;
    auto fail = [&](cudaError_t e, const char *what) {
        pg_set_error("qtensor_upload: %s failed: %s", what, cudaGetErrorString(e));
        cudaFree(d_t);
        cudaFree(d_s);
        cudaFree(d_q);
        delete t;
        return e == cudaErrorMemoryAllocation ? PG_ERR_NOMEM : PG_ERR_CUDA;
    };
    cudaError_t e;
    const size_t tb = (size_t)nc * rows;
    // 1 KiB of slack after the weights lets tiled loads of the last rows stay inside the allocation
    if ((e = cudaMalloc(&d_t, tb + 1024)) != cudaSuccess) return fail(e, "cudaMalloc");
    if ((e = cudaMalloc(&d_s, (size_t)(nc ? nc : 1) * 4)) != cudaSuccess) return fail(e, "cudaMalloc");
    if (tb && (e = cudaMemcpyAsync(d_t, data_i8_t + col_begin * rows, tb, cudaMemcpyHostToDevice, ctx->stream)) != cudaSuccess)
        return fail(e, "upload of data_i8_t");
    if (nc && (e = cudaMemcpyAsync(d_s, scales + col_begin, (size_t)nc * 4, cudaMemcpyHostToDevice, ctx->stream)) != cudaSuccess)
        return fail(e, "upload of scales");
    if (data_i8) {
        if ((e = cudaMalloc(&d_q, tb + 16)) != cudaSuccess) return fail(e, "cudaMalloc");
        if (tb && (e = cudaMemcpy2DAsync(d_q, (size_t)nc, data_i8 + col_begin, (size_t)cols, (size_t)nc, (size_t)rows,
                                         cudaMemcpyHostToDevice, ctx->stream)) != cudaSuccess)
            return fail(e, "upload of data_i8");
    }
    if ((e = cudaStreamSynchronize(ctx->stream)) != cudaSuccess) return fail(e, "sync");
    t->d_data_i8_t = (const int8_t *)d_t;
    t->d_scales = (const float *)d_s;
    t->d_data_i8 = (const int8_t *)d_q;
    *out = t;
    return PG_OK;
}

int32_t pg_qtensor_wrap(pg_ctx *ctx, const int8_t *d_data_i8, const int8_t *d_data_i8_t, const float *d_scales, int64_t rows,
                        int64_t cols, pg_qtensor **out)
{
    PG_REQUIRE(ctx && out, "qtensor_wrap: null argument");
    *out = nullptr;
    PG_REQUIRE(rows >= 0 && cols >= 0, "qtensor_wrap: negative shape");
    PG_REQUIRE(rows * cols == 0 || (d_data_i8_t && d_scales), "qtensor_wrap: data_i8_t and scales are required");
    pg_qtensor *t = new (std::nothrow) pg_qtensor();
    if (!t) PG_FAIL(PG_ERR_NOMEM, "out of host memory");
    t->d_data_i8 = d_data_i8;
    t->d_data_i8_t = d_data_i8_t;
    t->d_scales = d_scales;
    t->rows = rows;
    t->cols = cols;
    t->owned = false;
    *out = t;
    return PG_OK;
}

int32_t pg_qtensor_from_f32(pg_ctx *ctx, const float *d_w, int64_t rows, int64_t cols, int32_t keep_data_i8, pg_qtensor **out)
{
    PG_ENTER(ctx);
    PG_REQUIRE(out != nullptr, "qtensor_from_f32: out is null");
    *out = nullptr;
    PG_REQUIRE(rows >= 0 && cols >= 0, "qtensor_from_f32: negative shape");
    PG_REQUIRE(rows * cols == 0 || d_w, "qtensor_from_f32: weights pointer is null");
    pg_qtensor *t = new (std::nothrow) pg_qtensor();
    if (!t) PG_FAIL(PG_ERR_NOMEM, "out of host memory");
    void *d_t = nullptr, *d_s = nullptr, *d_q = nullptr;
    const size_t tb = (size_t)rows * cols;
    cudaError_t e = cudaMalloc(&d_t, tb + 1024);
    if (e == cudaSuccess) e = cudaMalloc(&d_s, (size_t)(cols ? cols : 1) * 4);
    if (e == cudaSuccess && keep_data_i8) e = cudaMalloc(&d_q, tb + 16);
    int32_t rc = PG_OK;
    if (e != cudaSuccess) {
        pg_set_error("qtensor_from_f32: cudaMalloc failed: %s", cudaGetErrorString(e));
        rc = PG_ERR_NOMEM;
    } else {
        rc = pgk_quantize_weights(ctx, d_w, rows, cols, (int8_t *)d_q, (int8_t *)d_t, (float *)d_s);
    }
    if (rc != PG_OK) {
        cudaFree(d_t);
        cudaFree(d_s);
        cudaFree(d_q);
        delete t;
        return rc;
    }
    t->d_data_i8 = (const int8_t *)d_q;
    t->d_data_i8_t = (const int8_t *)d_t;
    t->d_scales = (const float *)d_s;
    t->rows = rows;
    t->cols = cols;
    t->owned = true;
    *out = t;
    return PG_OK;
}

int32_t pg_qtensor_download(pg_ctx *ctx, const pg_qtensor *t, int8_t *data_i8, int8_t *data_i8_t, float *scales)
{
    PG_ENTER(ctx);
    PG_REQUIRE(t != nullptr, "qtensor_download: tensor is null");
    const size_t tb = (size_t)t->rows * t->cols;
    if (data_i8) {
        PG_REQUIRE(t->d_data_i8 != nullptr, "qtensor_download: data_i8 is not on the GPU");
        if (tb) PG_CUDA(cudaMemcpyAsync(data_i8, t->d_data_i8, tb, cudaMemcpyDeviceToHost, ctx->stream));
    }
    if (data_i8_t && tb) PG_CUDA(cudaMemcpyAsync(data_i8_t, t->d_data_i8_t, tb, cudaMemcpyDeviceToHost, ctx->stream));
    if (scales && t->cols) PG_CUDA(cudaMemcpyAsync(scales, t->d_scales, (size_t)t->cols * 4, cudaMemcpyDeviceToHost, ctx->stream));
    PG_CUDA(cudaStreamSynchronize(ctx->stream));
    return PG_OK;
}

int32_t pg_qtensor_free(pg_ctx *ctx, pg_qtensor *t)
{
    if (!t) return PG_OK;
    PG_ENTER(ctx);
    for (size_t i = 0; i < ctx->host_calls.size();) {      // recorded host calls on these weights go with them
        if (ctx->host_calls[i].w == t) {
            if (ctx->host_calls[i].exec) cudaGraphExecDestroy(ctx->host_calls[i].exec);
            ctx->host_calls.erase(ctx->host_calls.begin() + i);
        } else {
            i++;
        }
    }
    if (t->owned) {
        PG_CUDA(cudaStreamSynchronize(ctx->stream));
        if (t->block) {
            cudaFree(t->block);
        } else {
            cudaFree((void *)t->d_data_i8);
            cudaFree((void *)t->d_data_i8_t);
            cudaFree((void *)t->d_scales);
        }
    }
    delete t;
    return PG_OK;
}

int64_t pg_qtensor_rows(const pg_qtensor *t) { return t ? t->rows : 0; }
int64_t pg_qtensor_cols(const pg_qtensor *t) { return t ? t->cols : 0; }
const int8_t *pg_qtensor_data_i8_t(const pg_qtensor *t) { return t ? t->d_data_i8_t : nullptr; }
const float *pg_qtensor_scales(const pg_qtensor *t) { return t ? t->d_scales : nullptr; }

// ---------------------------------------------------------- integer GEMM ----
static int32_t gemm_dispatch(pg_ctx *ctx, const int8_t *d_a, const float *d_as, int64_t m, int64_t k, const pg_qtensor *w,
                             float *d_y, int32_t *d_acc, int32_t algo)
{
    const int64_t n = w->cols;
    if (m == 0 || n == 0) return PG_OK;
    if (k == 0) {
        // empty sums: acc = 0, y = 0 * a_scale * w_scale = +0.0 (or NaN for a non-finite scale);
        // the naive kernel evaluates exactly that
        return pgk_gemm_i8_naive(ctx, d_a, d_as, m, k, w->d_data_i8_t, w->d_scales, n, d_y, d_acc);
    }
    const bool aligned = (((uintptr_t)d_a | (uintptr_t)w->d_data_i8_t) & 15) == 0;
    switch (algo) {
        case PG_ALGO_NAIVE:
            return pgk_gemm_i8_naive(ctx, d_a, d_as, m, k, w->d_data_i8_t, w->d_scales, n, d_y, d_acc);
        case PG_ALGO_STREAM:
            return pgk_gemm_i8_stream(ctx, d_a, d_as, m, k, w->d_data_i8_t, w->d_scales, n, d_y, d_acc);
        case PG_ALGO_TCGEN05:
            return pgk_gemm_i8_tcgen05(ctx, d_a, d_as, m, k, const_cast<pg_qtensor *>(w), d_y, d_acc);
        case PG_ALGO_WSTREAM:
            return pgk_gemm_i8_wstream(ctx, d_a, d_as, m, k, w->d_data_i8_t, w->d_scales, n, d_y, d_acc);
        case PG_ALGO_AUTO:
            if (aligned && pgk_gemm_i8_wstream_supports(m, k, n))
                return pgk_gemm_i8_wstream(ctx, d_a, d_as, m, k, w->d_data_i8_t, w->d_scales, n, d_y, d_acc);
            // 17 <= M <= 64: the per-lane FIFO kernel's time grows with M (it is MMA-issue bound there: 25 / 33 / 56 us
            // at M = 17 / 32 / 64 for K 4096, N 14336), the tcgen05 kernel's does not (16 us for any M <= 64).  On narrow
            // layers with short K the two are level up to M = 32 (10.8 / 11.3 us against 11.3 / 11.5 us at K = N = 4096);
            // with long K the tcgen05 kernel divides K over CTAs and wins (K 14336, N 4096: 22.6 against 30.8 us at M = 17).
            if (aligned && pgk_gemm_i8_stream_supports(m, k, n) &&
                !(pgk_gemm_i8_tcgen05_supports(m, k, n) && m > 16 && (m > 32 || n >= 40ll * ctx->sm_count || k >= 8192)))
                return pgk_gemm_i8_stream(ctx, d_a, d_as, m, k, w->d_data_i8_t, w->d_scales, n, d_y, d_acc);
            if (aligned && pgk_gemm_i8_tcgen05_supports(m, k, n))
                return pgk_gemm_i8_tcgen05(ctx, d_a, d_as, m, k, const_cast<pg_qtensor *>(w), d_y, d_acc);
            // shapes neither fast kernel takes (K not a multiple of 16, odd alignment)
            return pgk_gemm_i8_naive(ctx, d_a, d_as, m, k, w->d_data_i8_t, w->d_scales, n, d_y, d_acc);
    }
    PG_FAIL(PG_ERR_INVALID, "unknown algo %d", algo);
}

int32_t pg_gemm_i8(pg_ctx *ctx, const int8_t *d_a_i8, const float *d_a_scales, int64_t m, int64_t k, const pg_qtensor *w,
                   float *d_y, int32_t *d_acc, int32_t algo)
{
    PG_ENTER(ctx);
    PG_REQUIRE(w != nullptr, "gemm_i8: weights are null");
    PG_REQUIRE(m >= 0 && k >= 0, "gemm_i8: negative shape");
    PG_REQUIRE(w->rows == k, "gemm_i8: w.rows (%lld) != k (%lld)", (long long)w->rows, (long long)k);
    PG_REQUIRE(m * w->cols == 0 || ((d_y == nullptr || d_a_scales) && (d_y || d_acc)), "gemm_i8: null output or scales");
    PG_REQUIRE(m * k == 0 || d_a_i8, "gemm_i8: activations are null");
    return gemm_dispatch(ctx, d_a_i8, d_a_scales, m, k, w, d_y, d_acc, algo);
}

int32_t pg_matmul_quantized_ex(pg_ctx *ctx, const float *d_x, int64_t m, int64_t k, const pg_qtensor *w, float *d_y,
                               int32_t *d_acc, int8_t *d_a_i8, float *d_a_scales, int32_t algo)
{
    PG_ENTER(ctx);
    PG_REQUIRE(w != nullptr, "matmul_quantized: weights not on GPU");
    PG_REQUIRE(m >= 0 && k >= 0, "matmul_quantized: negative shape");
    PG_REQUIRE(w->rows == k, "matmul_quantized: w.rows (%lld) != k (%lld)", (long long)w->rows, (long long)k);
    PG_REQUIRE(m * k == 0 || d_x, "matmul_quantized: activations are null");
    PG_REQUIRE(m * w->cols == 0 || d_y || d_acc, "matmul_quantized: no output");
    if (m == 0) return PG_OK;
    int8_t *a_i8 = d_a_i8;
    float *a_s = d_a_scales;
    if (!a_i8 || !a_s) {
        const size_t nq = align256((size_t)m * k + 16), ns = align256((size_t)m * 4);
        int32_t rc = pg_scratch_reserve(ctx, nq + ns);
        if (rc) return rc;
        if (!a_i8) a_i8 = (int8_t *)ctx->scratch;
        if (!a_s) a_s = (float *)((char *)ctx->scratch + nq);
    }
    int32_t rc = pgk_quantize_activations(ctx, d_x, m, k, a_i8, a_s);
    if (rc) return rc;
    return gemm_dispatch(ctx, a_i8, a_s, m, k, w, d_y, d_acc, algo);
}

int32_t pg_matmul_quantized(pg_ctx *ctx, const float *d_x, int64_t m, int64_t k, const pg_qtensor *w, float *d_y)
{
    return pg_matmul_quantized_ex(ctx, d_x, m, k, w, d_y, nullptr, nullptr, nullptr, PG_ALGO_AUTO);
}

// Host buffers the GPU can address (page-locked: cudaHostAlloc, cudaHostRegister) need no copy engine for small
// payloads: a copy engine starts several microseconds after the kernel before it, a kernel does not.
//   x  the quantiser reads it across PCIe itself (128-bit loads, one pass), up to 1 MiB;
//   y  the product writes to device memory as always and a copy kernel behind it pushes the result to the host in
//      16-byte stores, up to 1 MiB.  (Letting the product write y to the host directly is slower beyond a few KiB: its
//      4-byte stores cross PCIe as tiny packets, 46 -> 115 us already at 16 x 4096 floats; kept behind the knob, off.)
// Measured over the nine decode cases of the benchmark, blocking call, sum: 382 us with copies both ways, 354 us with
// x read directly, 329 us with the push kernel as well.  Larger payloads and pageable memory keep the copy engines.
// pg_tune_host_direct(x_bytes, y_bytes) / pg_tune_host_push(y_bytes): 0 switches a path off, negative restores the default.
constexpr size_t HOST_DIRECT_X = 1 << 20, HOST_DIRECT_Y = 0, HOST_PUSH_Y = 1 << 20;
static size_t g_host_direct_x = HOST_DIRECT_X, g_host_direct_y = HOST_DIRECT_Y, g_host_push_y = HOST_PUSH_Y;
extern "C" PG_API void pg_tune_host_direct(int x_bytes, int y_bytes)
{
    g_host_direct_x = x_bytes < 0 ? HOST_DIRECT_X : (size_t)x_bytes;
    g_host_direct_y = y_bytes < 0 ? HOST_DIRECT_Y : (size_t)y_bytes;
}
extern "C" PG_API void pg_tune_host_push(int y_bytes) { g_host_push_y = y_bytes < 0 ? HOST_PUSH_Y : (size_t)y_bytes; }
static int g_host_graph = 1;
extern "C" PG_API void pg_tune_host_graph(int on) { g_host_graph = on; }

// The device's address of a page-locked host buffer, or null for ordinary (pageable) memory.
static void *device_view_of_host(const void *p)
{
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return a.type == cudaMemoryTypeHost ? a.devicePointer : nullptr;
}

int32_t pg_matmul_quantized_host(pg_ctx *ctx, const float *x, int64_t m, int64_t k, const pg_qtensor *w, float *y)
{
    PG_ENTER(ctx);
    PG_REQUIRE(w != nullptr, "matmul_quantized: weights not on GPU");
    PG_REQUIRE(m >= 0 && k >= 0, "matmul_quantized: negative shape");
    PG_REQUIRE(w->rows == k, "matmul_quantized: w.rows (%lld) != k (%lld)", (long long)w->rows, (long long)k);
    const int64_t n = w->cols;
    if (m * n == 0) return PG_OK;
    PG_REQUIRE((m * k == 0 || x) && y, "matmul_quantized: null pointer");
    const size_t nx = align256((size_t)m * k * 4 + 16), ny = align256((size_t)m * n * 4), nq = align256((size_t)m * k + 16),
                 ns = align256((size_t)m * 4);
    int32_t rc = pg_staging_reserve(ctx, nx + ny + nq + ns);
    if (rc) return rc;
    char *base = (char *)ctx->staging;
    float *d_x = (float *)base;
    float *d_y = (float *)(base + nx);
    int8_t *d_q = (int8_t *)(base + nx + ny);
    float *d_s = (float *)(base + nx + ny + nq);
    const size_t bx = (size_t)m * k * 4, by = (size_t)m * n * 4;
    const float *x_dev = (bx && bx <= g_host_direct_x && ((uintptr_t)x & 15) == 0) ? (const float *)device_view_of_host(x) : nullptr;
    float *y_view = (by <= std::max(g_host_direct_y, g_host_push_y) && ((uintptr_t)y & 15) == 0) ? (float *)device_view_of_host(y) : nullptr;
    float *y_dev = by <= g_host_direct_y ? y_view : nullptr;
    const bool push = !y_dev && y_view != nullptr;
    // the launches of one call (no copy engine involved when both buffers are reached by kernels)
    auto enqueue = [&]() -> int32_t {
        if (bx && !x_dev) PG_CUDA(cudaMemcpyAsync(d_x, x, bx, cudaMemcpyHostToDevice, ctx->stream));
        int32_t r = pgk_quantize_activations(ctx, x_dev ? x_dev : d_x, m, k, d_q, d_s);
        if (r) return r;
        r = gemm_dispatch(ctx, d_q, d_s, m, k, w, y_dev ? y_dev : d_y, nullptr, PG_ALGO_AUTO);
        if (r) return r;
        if (push) {
            r = pgk_copy_words(ctx, d_y, y_view, by);
            if (r) return r;
        } else if (!y_dev) {
            PG_CUDA(cudaMemcpyAsync(y, d_y, by, cudaMemcpyDeviceToHost, ctx->stream));
        }
        return PG_OK;
    };
    // Kernels only, nothing being recorded by the caller: a call seen before with these very buffers is replayed from a graph
    // of its own launches (recorded the second time it is seen, so that one-off calls pay nothing).  The key holds every
    // address and setting the launches were given.
    if (g_host_graph && !ctx->capturing && bx && x_dev && (push || y_dev)) {
        pg_ctx::HostCall key;
        key.x = x_dev; key.y = y_view; key.w = w; key.wt = w->d_data_i8_t; key.ws = w->d_scales; key.staging = ctx->staging;
        key.scratch = ctx->scratch; key.splitk = ctx->splitk; key.m = m; key.k = k; key.n = n; key.limit = ctx->wait_limit_ns;
        key.mode = (push ? 1 : 0) | (y_dev ? 2 : 0);
        pg_ctx::HostCall *hit = nullptr;
        for (auto &h : ctx->host_calls)
            if (h.x == key.x && h.y == key.y && h.w == key.w && h.wt == key.wt && h.ws == key.ws && h.staging == key.staging &&
                h.scratch == key.scratch && h.splitk == key.splitk && h.m == key.m && h.k == key.k && h.n == key.n && h.limit == key.limit &&
                h.mode == key.mode)
                hit = &h;
        if (hit && hit->exec) {
            hit->stamp = ++ctx->host_stamp;
            PG_CUDA(cudaGraphLaunch(hit->exec, ctx->stream));
            g_pg_launches.fetch_add(hit->kernels);
            PG_CUDA(cudaStreamSynchronize(ctx->stream));
            return PG_OK;
        }
        if (hit) {
            // second sighting: record, keep, replay
            const uint64_t before = g_pg_launches.load();
            cudaGraph_t graph = nullptr;
            cudaGraphExec_t exec = nullptr;
            bool ok = cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
            if (ok) {
                ctx->capturing = true;                      // nothing may grow while the launches are recorded
                const int32_t r = enqueue();
                ctx->capturing = false;
                ok = cudaStreamEndCapture(ctx->stream, &graph) == cudaSuccess && r == PG_OK && graph != nullptr;
            }
            const uint64_t kernels = g_pg_launches.load() - before;
            g_pg_launches.fetch_sub(kernels);               // recorded, not run
            if (ok) ok = cudaGraphInstantiate(&exec, graph, 0) == cudaSuccess;
            if (graph) cudaGraphDestroy(graph);
            if (ok) {
                hit->exec = exec;
                hit->kernels = kernels;
                hit->stamp = ++ctx->host_stamp;
                PG_CUDA(cudaGraphLaunch(exec, ctx->stream));
                g_pg_launches.fetch_add(kernels);
                PG_CUDA(cudaStreamSynchronize(ctx->stream));
                return PG_OK;
            }
            cudaGetLastError();                             // recording failed: forget it and run the call as it is
            hit->stamp = ++ctx->host_stamp;
        } else {
            if (ctx->host_calls.size() >= 64) {             // drop the entry used longest ago
                size_t old = 0;
                for (size_t i = 1; i < ctx->host_calls.size(); i++)
                    if (ctx->host_calls[i].stamp < ctx->host_calls[old].stamp) old = i;
                if (ctx->host_calls[old].exec) cudaGraphExecDestroy(ctx->host_calls[old].exec);
                ctx->host_calls.erase(ctx->host_calls.begin() + old);
            }
            key.stamp = ++ctx->host_stamp;
            ctx->host_calls.push_back(key);
        }
    }
    rc = enqueue();
    if (rc) return rc;
    PG_CUDA(cudaStreamSynchronize(ctx->stream));
    return PG_OK;
}

// ------------------------------------------------------------------- GGUF ----
static int block_size_of(int32_t type) { return type == PG_GGUF_Q8_0 ? 34 : type == PG_GGUF_Q4_0 ? 18 : type == PG_GGUF_Q4_1 ? 20 : 0; }

int32_t pg_dequant_blocks(pg_ctx *ctx, int32_t type, const uint8_t *d_raw, size_t raw_len, int64_t num_elements, float *d_out)
{
    PG_ENTER(ctx);
    const int bs = block_size_of(type);
    PG_REQUIRE(bs != 0, "dequant: unknown block type %d", type);
    PG_REQUIRE(num_elements >= 0 && num_elements % 32 == 0, "dequant: num_elements %% 32 != 0");
    const int64_t nb = num_elements / 32;
    PG_REQUIRE(raw_len >= (size_t)nb * bs, "dequant: data holds %zu bytes, %lld blocks need %lld", raw_len, (long long)nb,
               (long long)nb * bs);
    PG_REQUIRE(nb == 0 || (d_raw && d_out), "dequant: null pointer");
    return pgk_dequant_blocks(ctx, type, d_raw, nb, d_out);
}

int32_t pg_dequant_blocks_host(pg_ctx *ctx, int32_t type, const uint8_t *raw, size_t raw_len, int64_t num_elements, float *out)
{
    PG_ENTER(ctx);
    const int bs = block_size_of(type);
    PG_REQUIRE(bs != 0, "dequant: unknown block type %d", type);
    PG_REQUIRE(num_elements >= 0 && num_elements % 32 == 0, "dequant: num_elements %% 32 != 0");
    const int64_t nb = num_elements / 32;
    PG_REQUIRE(raw_len >= (size_t)nb * bs, "dequant: data holds %zu bytes, %lld blocks need %lld", raw_len, (long long)nb,
               (long long)nb * bs);
    if (nb == 0) return PG_OK;
    PG_REQUIRE(raw && out, "dequant: null pointer");
    void *d_raw = nullptr, *d_out = nullptr;
    cudaError_t e = cudaMalloc(&d_raw, (size_t)nb * bs);
    if (e == cudaSuccess) e = cudaMalloc(&d_out, (size_t)num_elements * 4);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_raw, raw, (size_t)nb * bs, cudaMemcpyHostToDevice, ctx->stream);
    int32_t rc = PG_OK;
    if (e == cudaSuccess) rc = pgk_dequant_blocks(ctx, type, (const uint8_t *)d_raw, nb, (float *)d_out);
    if (e == cudaSuccess && rc == PG_OK) e = cudaMemcpyAsync(out, d_out, (size_t)num_elements * 4, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    cudaFree(d_raw);
    cudaFree(d_out);
    if (e != cudaSuccess) PG_FAIL(e == cudaErrorMemoryAllocation ? PG_ERR_NOMEM : PG_ERR_CUDA, "dequant: %s", cudaGetErrorString(e));
    return rc;
}

int32_t pg_f16_to_f32(pg_ctx *ctx, const uint16_t *d_bits, int64_t count, float *d_out)
{
    PG_ENTER(ctx);
    PG_REQUIRE(count >= 0 && (count == 0 || (d_bits && d_out)), "f16_to_f32: bad arguments");
    return pgk_f16_to_f32(ctx, d_bits, count, d_out);
}

int32_t pg_gguf_upload(pg_ctx *ctx, int32_t type, const uint8_t *raw, size_t raw_len, int64_t n, int64_t k, int64_t row_begin,
                       int64_t row_end, pg_gguf_weight **out)
{
    PG_ENTER(ctx);
    PG_REQUIRE(out != nullptr, "gguf_upload: out is null");
    *out = nullptr;
    const int bs = block_size_of(type);
    PG_REQUIRE(bs != 0, "gguf_upload: unknown block type %d", type);
    PG_REQUIRE(n >= 0 && k >= 0 && k % 32 == 0, "gguf_upload: k (%lld) must be a multiple of 32", (long long)k);
    PG_REQUIRE(0 <= row_begin && row_begin <= row_end && row_end <= n, "gguf_upload: row range outside the tensor");
    const int64_t nblk = k / 32;
    PG_REQUIRE(raw_len >= (size_t)n * nblk * bs, "gguf_upload: data holds %zu bytes, need %lld", raw_len, (long long)(n * nblk * bs));
    const int64_t nr = row_end - row_begin;
    PG_REQUIRE(nr * nblk == 0 || raw, "gguf_upload: raw is null");
    pg_gguf_weight *w = new (std::nothrow) pg_gguf_weight();
    if (!w) PG_FAIL(PG_ERR_NOMEM, "out of host memory");
    w->type = type;
    w->n = nr;
    w->k = k;
    const size_t blocks = (size_t)nr * nblk;
    const size_t qbytes = pgk_gguf_qs_bytes(type, nr, k, nullptr);
    void *d_raw = nullptr;
    cudaError_t e = cudaMalloc((void **)&w->d_qs, qbytes + 64);
    if (e == cudaSuccess) e = cudaMalloc((void **)&w->d_d, blocks * 2 + 64);
    if (e == cudaSuccess && type == PG_GGUF_Q4_1) e = cudaMalloc((void **)&w->d_m, blocks * 2 + 64);
    if (e == cudaSuccess && blocks) e = cudaMalloc(&d_raw, blocks * bs);
    if (e == cudaSuccess && blocks)
        e = cudaMemcpyAsync(d_raw, raw + (size_t)row_begin * nblk * bs, blocks * bs, cudaMemcpyHostToDevice, ctx->stream);
    int32_t rc = PG_OK;
    if (e == cudaSuccess) rc = pgk_gguf_repack(ctx, type, (const uint8_t *)d_raw, nr, k, w);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    cudaFree(d_raw);
    if (e != cudaSuccess || rc != PG_OK) {
        if (e != cudaSuccess) pg_set_error("gguf_upload: %s", cudaGetErrorString(e));
        cudaFree(w->d_qs);
        cudaFree(w->d_d);
        cudaFree(w->d_m);
        delete w;
        return e == cudaErrorMemoryAllocation ? PG_ERR_NOMEM : (e != cudaSuccess ? PG_ERR_CUDA : rc);
    }
    *out = w;
    return PG_OK;
}

int32_t pg_gguf_free(pg_ctx *ctx, pg_gguf_weight *w)
{
    if (!w) return PG_OK;
    PG_ENTER(ctx);
    PG_CUDA(cudaStreamSynchronize(ctx->stream));
    cudaFree(w->d_qs);
    cudaFree(w->d_d);
    cudaFree(w->d_m);
    delete w;
    return PG_OK;
}

int64_t pg_gguf_rows(const pg_gguf_weight *w) { return w ? w->n : 0; }
int64_t pg_gguf_cols(const pg_gguf_weight *w) { return w ? w->k : 0; }

int32_t pg_matmul_gguf(pg_ctx *ctx, const float *d_x, int64_t m, const pg_gguf_weight *w, float *d_y)
{
    PG_ENTER(ctx);
    PG_REQUIRE(w != nullptr, "matmul_gguf: weight is null");
    PG_REQUIRE(m >= 0, "matmul_gguf: negative m");
    PG_REQUIRE(m * w->n == 0 || (d_y && (w->k == 0 || d_x)), "matmul_gguf: null pointer");
    return pgk_matmul_gguf(ctx, d_x, m, w, d_y);
}

int32_t pg_matmul_gguf_host(pg_ctx *ctx, const float *x, int64_t m, const pg_gguf_weight *w, float *y)
{
    PG_ENTER(ctx);
    PG_REQUIRE(w != nullptr, "matmul_gguf: weight is null");
    PG_REQUIRE(m >= 0, "matmul_gguf: negative m");
    if (m * w->n == 0) return PG_OK;
    PG_REQUIRE(y && (w->k == 0 || x), "matmul_gguf: null pointer");
    const size_t nx = align256((size_t)m * w->k * 4 + 16), ny = align256((size_t)m * w->n * 4);
    int32_t rc = pg_staging_reserve(ctx, nx + ny);
    if (rc) return rc;
    float *d_x = (float *)ctx->staging;
    float *d_y = (float *)((char *)ctx->staging + nx);
    if (m * w->k) PG_CUDA(cudaMemcpyAsync(d_x, x, (size_t)m * w->k * 4, cudaMemcpyHostToDevice, ctx->stream));
    rc = pgk_matmul_gguf(ctx, d_x, m, w, d_y);
    if (rc) return rc;
    PG_CUDA(cudaMemcpyAsync(y, d_y, (size_t)m * w->n * 4, cudaMemcpyDeviceToHost, ctx->stream));
    PG_CUDA(cudaStreamSynchronize(ctx->stream));
    return PG_OK;
}

int32_t pg_qtensor_from_q8_0(pg_ctx *ctx, const uint8_t *raw, size_t raw_len, int64_t rows, int64_t cols, pg_qtensor **out)
{
    PG_ENTER(ctx);
    PG_REQUIRE(out != nullptr, "qtensor_from_q8_0: out is null");
    *out = nullptr;
    PG_REQUIRE(rows >= 0 && cols >= 0 && cols % 32 == 0, "qtensor_from_q8_0: cols %% 32 != 0");
    const int64_t nb = rows * cols / 32;
    PG_REQUIRE(raw_len >= (size_t)nb * 34, "qtensor_from_q8_0: data too short");
    PG_REQUIRE(nb == 0 || raw, "qtensor_from_q8_0: raw is null");
    void *d_raw = nullptr, *d_f = nullptr;
    cudaError_t e = cudaMalloc(&d_raw, (size_t)nb * 34 + 16);
    if (e == cudaSuccess) e = cudaMalloc(&d_f, (size_t)nb * 32 * 4 + 16);
    if (e == cudaSuccess && nb) e = cudaMemcpyAsync(d_raw, raw, (size_t)nb * 34, cudaMemcpyHostToDevice, ctx->stream);
    int32_t rc = PG_OK;
    if (e == cudaSuccess) rc = pgk_dequant_blocks(ctx, PG_GGUF_Q8_0, (const uint8_t *)d_raw, nb, (float *)d_f);
    if (e == cudaSuccess && rc == PG_OK) rc = pg_qtensor_from_f32(ctx, (const float *)d_f, rows, cols, 1, out);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    cudaFree(d_raw);
    cudaFree(d_f);
    if (e != cudaSuccess) PG_FAIL(e == cudaErrorMemoryAllocation ? PG_ERR_NOMEM : PG_ERR_CUDA, "qtensor_from_q8_0: %s", cudaGetErrorString(e));
    return rc;
}

// A quantised tensor as the serial format stores it (src/serial.rs:127-222: i8 [rows, cols] row-major + f32 scales
// [cols]): uploaded once, the GEMM layout data_i8_t [cols, rows] rebuilt on the device.
int32_t pg_qtensor_from_i8(pg_ctx *ctx, const int8_t *data_i8, const float *scales, int64_t rows, int64_t cols, pg_qtensor **out)
{
    PG_ENTER(ctx);
    PG_REQUIRE(out != nullptr, "qtensor_from_i8: out is null");
    *out = nullptr;
    PG_REQUIRE(rows >= 0 && cols >= 0, "qtensor_from_i8: negative shape");
    PG_REQUIRE(rows * cols == 0 || data_i8, "qtensor_from_i8: data is null");
    PG_REQUIRE(cols == 0 || scales, "qtensor_from_i8: scales are null");
    pg_qtensor *t = new (std::nothrow) pg_qtensor();
    if (!t) PG_FAIL(PG_ERR_NOMEM, "out of host memory");
    t->rows = rows;
    t->cols = cols;
    t->owned = true;
    const size_t tb = (size_t)rows * cols;
    // one allocation: data_i8 | data_i8_t (+ 1 KiB of slack for tiled loads of the last rows) | scales
    void *d_q = nullptr, *d_t = nullptr, *d_s = nullptr;
    const size_t o_t = align256(tb + 16), o_s = o_t + align256(tb + 1024);
    cudaError_t e = cudaMalloc(&d_q, o_s + (size_t)(cols ? cols : 1) * 4);
    if (e == cudaSuccess) {
        d_t = (char *)d_q + o_t;
        d_s = (char *)d_q + o_s;
    }
    if (e == cudaSuccess && tb) e = cudaMemcpyAsync(d_q, data_i8, tb, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess && cols) e = cudaMemcpyAsync(d_s, scales, (size_t)cols * 4, cudaMemcpyHostToDevice, ctx->stream);
    int32_t rc = PG_OK;
    if (e == cudaSuccess) rc = pgk_transpose_i8(ctx, (const int8_t *)d_q, rows, cols, (int8_t *)d_t);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);   // the host arrays may go away after the call
    if (e != cudaSuccess || rc != PG_OK) {
        cudaFree(d_q);   // the one block
        delete t;
        if (e != cudaSuccess) PG_FAIL(e == cudaErrorMemoryAllocation ? PG_ERR_NOMEM : PG_ERR_CUDA, "qtensor_from_i8: %s", cudaGetErrorString(e));
        return rc;
    }
    t->d_data_i8 = (const int8_t *)d_q;
    t->d_data_i8_t = (const int8_t *)d_t;
    t->d_scales = (const float *)d_s;
    t->block = d_q;
    *out = t;
    return PG_OK;
}

// Checks the stream tables and decodes the bitstreams (host memory, back to back as the serial format holds them) into d_out.
static int32_t huffman_decode_to_device(pg_ctx *ctx, const uint8_t *bit_lengths, int64_t num_streams, const uint64_t *stream_symbols,
                                        const uint64_t *stream_bytes, const uint8_t *streams, uint64_t expect_symbols, int8_t *d_out)
{
    PG_REQUIRE(bit_lengths != nullptr, "huffman: the code book is null");
    PG_REQUIRE(num_streams >= 0 && (num_streams == 0 || (stream_symbols && stream_bytes)), "huffman: stream tables are null");
    uint64_t symbols = 0, bytes = 0;
    for (int64_t s = 0; s < num_streams; s++) {
        symbols += stream_symbols[s];
        bytes += stream_bytes[s];
    }
    // decode_to_quantized asserts that the streams hold rows * cols symbols (src/huffman.rs:384)
    PG_REQUIRE(symbols == expect_symbols, "huffman: the streams hold %llu symbols, %llu expected", (unsigned long long)symbols,
               (unsigned long long)expect_symbols);
    PG_REQUIRE(bytes == 0 || streams, "huffman: the bitstreams are null");
    if (symbols == 0) return PG_OK;
    return pgk_huffman_decode(ctx, bit_lengths, num_streams, stream_symbols, stream_bytes, streams, d_out);
}

int32_t pg_huffman_decode_host(pg_ctx *ctx, const uint8_t *bit_lengths, int64_t num_streams, const uint64_t *stream_symbols,
                               const uint64_t *stream_bytes, const uint8_t *streams, int8_t *out)
{
    PG_ENTER(ctx);
    uint64_t symbols = 0;
    for (int64_t s = 0; s < num_streams && stream_symbols; s++) symbols += stream_symbols[s];
    if (symbols == 0 && num_streams >= 0) return PG_OK;
    PG_REQUIRE(out != nullptr, "huffman_decode: out is null");
    int8_t *d_out = nullptr;
    cudaError_t e = cudaMalloc((void **)&d_out, symbols + 16);
    if (e != cudaSuccess) PG_FAIL(e == cudaErrorMemoryAllocation ? PG_ERR_NOMEM : PG_ERR_CUDA, "huffman_decode: %s", cudaGetErrorString(e));
    int32_t rc = huffman_decode_to_device(ctx, bit_lengths, num_streams, stream_symbols, stream_bytes, streams, symbols, d_out);
    if (rc == PG_OK) {
        e = cudaMemcpyAsync(out, d_out, symbols, cudaMemcpyDeviceToHost, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    }
    cudaFree(d_out);
    if (rc == PG_OK && e != cudaSuccess) PG_FAIL(PG_ERR_CUDA, "huffman_decode: %s", cudaGetErrorString(e));
    return rc;
}

int32_t pg_qtensor_from_huffman(pg_ctx *ctx, const uint8_t *bit_lengths, int64_t num_streams, const uint64_t *stream_symbols,
                                const uint64_t *stream_bytes, const uint8_t *streams, const float *scales, int64_t rows, int64_t cols,
                                pg_qtensor **out)
{
    PG_ENTER(ctx);
    PG_REQUIRE(out != nullptr, "qtensor_from_huffman: out is null");
    *out = nullptr;
    PG_REQUIRE(rows >= 0 && cols >= 0, "qtensor_from_huffman: negative shape");
    PG_REQUIRE(cols == 0 || scales, "qtensor_from_huffman: scales are null");
    pg_qtensor *t = new (std::nothrow) pg_qtensor();
    if (!t) PG_FAIL(PG_ERR_NOMEM, "out of host memory");
    t->rows = rows;
    t->cols = cols;
    t->owned = true;
    const size_t tb = (size_t)rows * cols;
    // one allocation: data_i8 | data_i8_t (+ 1 KiB of slack for tiled loads of the last rows) | scales
    void *d_q = nullptr, *d_t = nullptr, *d_s = nullptr;
    const size_t o_t = align256(tb + 16), o_s = o_t + align256(tb + 1024);
    cudaError_t e = cudaMalloc(&d_q, o_s + (size_t)(cols ? cols : 1) * 4);
    if (e == cudaSuccess) {
        d_t = (char *)d_q + o_t;
        d_s = (char *)d_q + o_s;
    }
    if (e == cudaSuccess && cols) e = cudaMemcpyAsync(d_s, scales, (size_t)cols * 4, cudaMemcpyHostToDevice, ctx->stream);
    int32_t rc = PG_OK;
    if (e == cudaSuccess) rc = huffman_decode_to_device(ctx, bit_lengths, num_streams, stream_symbols, stream_bytes, streams, tb, (int8_t *)d_q);
    if (e == cudaSuccess && rc == PG_OK) rc = pgk_transpose_i8(ctx, (const int8_t *)d_q, rows, cols, (int8_t *)d_t);
    if (e == cudaSuccess && rc == PG_OK) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess || rc != PG_OK) {
        cudaFree(d_q);   // the one block
        delete t;
        if (e != cudaSuccess) PG_FAIL(e == cudaErrorMemoryAllocation ? PG_ERR_NOMEM : PG_ERR_CUDA, "qtensor_from_huffman: %s", cudaGetErrorString(e));
        return rc;
    }
    t->d_data_i8 = (const int8_t *)d_q;
    t->d_data_i8_t = (const int8_t *)d_t;
    t->d_scales = (const float *)d_s;
    t->block = d_q;
    *out = t;
    return PG_OK;
}

int32_t pg_matmul_f32(pg_ctx *ctx, const float *d_a, const float *d_b, int64_t m, int64_t k, int64_t n, float *d_out)
{
    PG_ENTER(ctx);
    PG_REQUIRE(m >= 0 && k >= 0 && n >= 0, "matmul_f32: negative shape");
    PG_REQUIRE(m * n == 0 || (d_out && (k == 0 || (d_a && d_b))), "matmul_f32: null pointer");
    return pgk_matmul_f32(ctx, d_a, d_b, m, k, n, d_out);
}

}  // extern "C"
