// pg_matmul_quantized_static: the W8A8 product for callers that are not allowed to allocate.
//
// Some hosts of this library run inside a memory budget that is fixed before inference starts: a
// serving process that hands each model a pre-sized arena, or a real-time loop where a cudaMalloc
// (which may synchronise the whole device and can fail late) is forbidden once the loop is running.
// pg_matmul_quantized keeps its intermediates -- the quantised activations [M,K] i8 and their
// per-row scales [M] f32 -- in context scratch memory that grows on demand with cudaMalloc.  This
// variant keeps them in a fixed array that is part of the library image instead, so the call
// itself never allocates, frees or resizes anything.
//
// The array lives in every GPU's memory from the moment the library is loaded on it until the
// process exits (PG_STATIC_SCRATCH_BYTES, about 257 KiB per GPU).  All calls on a GPU share it, and
// it keeps whatever the previous call left: nothing in this path needs zeroed memory, every byte
// that is read has been written by the same call.  Two calls that can overlap on the GPU (different
// streams, or different contexts on one GPU) race on it; callers must order them.
#include <mutex>

#include "pg_internal.cuh"

namespace {

constexpr size_t STATIC_Q_BYTES = 256 * 1024;      // quantised activations: M*K <= 262144
constexpr size_t STATIC_S_BYTES = 1024;            // row scales: M <= 256
constexpr size_t PG_STATIC_SCRATCH_BYTES = STATIC_Q_BYTES + STATIC_S_BYTES;

// In host code this name is only a handle for the symbol, not an address the GPU can use: the
// device address is looked up once per device with cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_static_scratch[PG_STATIC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
std::mutex g_setup_mutex;
void *g_scratch_addr[MAX_DEVICES] = {};

// Device address of the array on `device`; resolves it on the first call for that device.
int32_t static_scratch(int device, void **out)
{
    PG_REQUIRE(device >= 0 && device < MAX_DEVICES, "device index %d is outside 0..%d", device, MAX_DEVICES - 1);
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_addr[device]) {
        int prev = -1;
        PG_CUDA(cudaGetDevice(&prev));
        if (prev != device) PG_CUDA(cudaSetDevice(device));
        void *p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (prev != device) cudaSetDevice(prev);
        if (e != cudaSuccess || !p) PG_FAIL(PG_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed on device %d: %s", device, cudaGetErrorString(e));
        g_scratch_addr[device] = p;
    }
    *out = g_scratch_addr[device];
    return PG_OK;
}

}  // namespace

extern "C" PG_API int64_t pg_static_scratch_bytes(void) { return (int64_t)PG_STATIC_SCRATCH_BYTES; }

extern "C" PG_API int32_t pg_matmul_quantized_static(pg_ctx *ctx, const float *d_x, int64_t m, int64_t k, const pg_qtensor *w,
                                                     float *d_y)
{
    PG_REQUIRE(ctx != nullptr, "null context");
    PG_REQUIRE(w != nullptr, "matmul_quantized: weights not on GPU");
    PG_REQUIRE(m >= 0 && k >= 0, "matmul_quantized: negative shape");
    PG_REQUIRE(w->rows == k, "matmul_quantized: w.rows (%lld) != k (%lld)", (long long)w->rows, (long long)k);
    if (m == 0 || w->cols == 0) return PG_OK;
    PG_REQUIRE(d_y && (k == 0 || d_x), "matmul_quantized: null pointer");
    if ((size_t)m * (size_t)k > STATIC_Q_BYTES || (size_t)m * sizeof(float) > STATIC_S_BYTES)
        PG_FAIL(PG_ERR_UNSUPPORTED,
                "pg_matmul_quantized_static: M*K = %lld exceeds the built-in scratch (M*K <= %zu, M <= %zu); "
                "use pg_matmul_quantized, which allocates",
                (long long)(m * k), STATIC_Q_BYTES, STATIC_S_BYTES / sizeof(float));
    void *base = nullptr;
    const int32_t rc = static_scratch(ctx->device, &base);
    if (rc != PG_OK) return rc;
    int8_t *a_i8 = reinterpret_cast<int8_t *>(base);
    float *a_scales = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(base) + STATIC_Q_BYTES);
    const int32_t rq = pg_quantize_activations(ctx, d_x, m, k, a_i8, a_scales);
    if (rq != PG_OK) return rq;
    ctx->no_growth = true;          // the split-K form of the tensor-core kernel would reserve a workspace
    const int32_t rg = pg_gemm_i8(ctx, a_i8, a_scales, m, k, w, d_y, nullptr, PG_ALGO_AUTO);
    ctx->no_growth = false;
    return rg;
}
