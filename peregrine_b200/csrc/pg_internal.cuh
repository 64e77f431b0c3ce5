// Internal declarations shared by the translation units of libperegrine_b200.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <atomic>

#include "peregrine_b200.h"

// ---------------------------------------------------------------- errors ----
void pg_set_error(const char *fmt, ...);
extern std::atomic<uint64_t> g_pg_launches;

#define PG_FAIL(code, ...)          \
    do {                            \
        pg_set_error(__VA_ARGS__);  \
        return (code);              \
    } while (0)

#define PG_REQUIRE(cond, ...)                          \
    do {                                               \
        if (!(cond)) PG_FAIL(PG_ERR_INVALID, __VA_ARGS__); \
    } while (0)

#define PG_CUDA(expr)                                                                         \
    do {                                                                                      \
        cudaError_t _e = (expr);                                                              \
        if (_e != cudaSuccess) {                                                              \
            pg_set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
            return _e == cudaErrorMemoryAllocation ? PG_ERR_NOMEM : PG_ERR_CUDA;              \
        }                                                                                     \
    } while (0)

// Call after every kernel launch: counts it and turns a launch error into a status.
#define PG_LAUNCHED()                       \
    do {                                    \
        g_pg_launches.fetch_add(1);         \
        PG_CUDA(cudaGetLastError());        \
    } while (0)

// ------------------------------------------------- loads across kernels ----
// The kernels of this library are launched with programmatic stream serialisation and signal
// griddepcontrol.launch_dependents first thing, so a kernel is usually resident while its
// predecessor still runs (and while older kernels' lines sit in that SM's L1).  Data that a
// preceding kernel of the stream produced is therefore read, after griddepcontrol.wait, with
// loads that go to L2: never through the non-coherent path (ld.global.nc / __ldg, which the
// compiler also chooses by itself for `const __restrict__` pointers) and never from L1.
#ifdef __CUDACC__
template <typename T>
__device__ __forceinline__ T pg_ld_fresh(const T *p)
{
    return __ldcg(p);
}
#endif

#ifdef __CUDACC__
// ---- a row spread over the CTAs of a thread-block cluster ----------------------------------------
// With a handful of sequences per step a kernel of one CTA per row leaves most SMs idle and is bound
// by the latency of one CTA walking its row.  The row kernels below therefore cut a row into `cs`
// column segments (cs = cluster size, 1..8), one CTA each, and exchange their partial sums / maxima
// through distributed shared memory: every CTA stores its value into slot [rank] of every peer, one
// cluster barrier, every CTA reduces the cs slots itself.
__device__ __forceinline__ uint32_t cl_rank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cl_size()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cl_sync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void cl_store_f32(float *local_slot, uint32_t cta, float v)
{
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local_slot)), "r"(cta));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}
__device__ __forceinline__ void cl_store_s32(int *local_slot, uint32_t cta, int v)
{
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local_slot)), "r"(cta));
    asm volatile("st.shared::cluster.s32 [%0], %1;" ::"r"(remote), "r"(v) : "memory");
}
// v: this CTA's value (the same in every thread).  slots: 8 floats of shared memory not used by another exchange in flight.
template <bool MAX>
__device__ __forceinline__ float cl_allreduce(float v, float *slots, uint32_t cs, uint32_t rank)
{
    if (cs == 1) return v;
    if (threadIdx.x < cs) cl_store_f32(slots + rank, threadIdx.x, v);
    cl_sync();
    float r = slots[0];
    for (uint32_t i = 1; i < cs; i++) r = MAX ? fmaxf(r, slots[i]) : r + slots[i];
    return r;
}
#endif

// --------------------------------------------------------------- objects ----
struct pg_ctx {
    int device = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    // scratch for intermediates (quantised activations, split-K partial sums); grows on demand
    void *scratch = nullptr;
    size_t scratch_bytes = 0;
    // device copies of host arguments for the *_host entry points; separate from `scratch`, which
    // kernels launched inside those calls may resize or overwrite
    void *staging = nullptr;
    size_t staging_bytes = 0;
    // zero-initialised workspace of the split-K paths (int32 partial sums + arrival counters); every
    // kernel that uses it leaves it zeroed again
    void *splitk = nullptr;
    size_t splitk_bytes = 0;
    int32_t *d_status = nullptr;  // device status word for bounded waits
    void *h_pinned = nullptr;     // pinned staging for *_host calls
    size_t h_pinned_bytes = 0;
    bool capturing = false;       // between pg_graph_begin and pg_graph_end
};

struct pg_graph {
    cudaGraphExec_t exec = nullptr;
};

struct pg_qtensor {
    const int8_t *d_data_i8 = nullptr;    // [K,N] (optional)
    const int8_t *d_data_i8_t = nullptr;  // [N,K]
    const float *d_scales = nullptr;      // [N]
    int64_t rows = 0;                     // K
    int64_t cols = 0;                     // N held on this GPU
    bool owned = false;
    void *block = nullptr;                // where the three arrays are parts of one allocation: that allocation
    // TMA descriptor of data_i8_t for the tcgen05 path, built on first use (128 B, opaque)
    alignas(64) unsigned char tmap_b[128];
    int tmap_b_box_rows = 0;
};

struct pg_gguf_weight {
    int32_t type = 0;
    int64_t n = 0, k = 0;       // rows held on this GPU, columns
    // Repacked at upload: quants and scales in separate, 16-byte aligned planes.
    //   Q8_0: qs [N][K] i8                         d [N][K/32] f16
    //   Q4_0: qs [N][K/2] u8 (block-local order)   d [N][K/32] f16
    //   Q4_1: as Q4_0                              d, m [N][K/32] f16
    uint8_t *d_qs = nullptr;
    uint16_t *d_d = nullptr;
    uint16_t *d_m = nullptr;
    int interleaved = 0;        // quants stored in the tensor-core kernel's chunk order (see repack_kernel)
};

int32_t pg_scratch_reserve(pg_ctx *ctx, size_t bytes);
int32_t pg_pinned_reserve(pg_ctx *ctx, size_t bytes);
int32_t pg_staging_reserve(pg_ctx *ctx, size_t bytes);
int32_t pg_splitk_reserve(pg_ctx *ctx, size_t bytes);

// ------------------------------------------------------- kernel launchers ----
// pg_quantize.cu
int32_t pgk_quantize_activations(pg_ctx *ctx, const float *d_x, int64_t rows, int64_t cols, int8_t *d_q, float *d_scales);
int32_t pgk_quantize_weights(pg_ctx *ctx, const float *d_w, int64_t rows, int64_t cols, int8_t *d_q, int8_t *d_qt, float *d_scales);
int32_t pgk_transpose_i8(pg_ctx *ctx, const int8_t *d_in, int64_t rows, int64_t cols, int8_t *d_out);
// device -> device-visible memory by a kernel, 16-byte words (both pointers 16-byte aligned)
int32_t pgk_copy_words(pg_ctx *ctx, const void *d_src, void *dst, size_t bytes);
// Huffman streams (back to back in host memory) -> int8 symbols back to back on the device
int32_t pgk_huffman_decode(pg_ctx *ctx, const uint8_t *bit_lengths, int64_t num_streams, const uint64_t *stream_symbols,
                           const uint64_t *stream_bytes, const uint8_t *h_data, int8_t *d_out);
int32_t pgk_dequantize(pg_ctx *ctx, const int8_t *d_q, const float *d_scales, int64_t rows, int64_t cols, float *d_out);
int32_t pgk_matmul_f32(pg_ctx *ctx, const float *d_a, const float *d_b, int64_t m, int64_t k, int64_t n, float *d_out);
// pg_gemm_naive.cu
int32_t pgk_gemm_i8_naive(pg_ctx *ctx, const int8_t *d_a, const float *d_as, int64_t m, int64_t k, const int8_t *d_bt,
                          const float *d_ws, int64_t n, float *d_y, int32_t *d_acc);
// pg_gemv_w8a8.cu
bool pgk_gemm_i8_stream_supports(int64_t m, int64_t k, int64_t n);
int32_t pgk_gemm_i8_stream(pg_ctx *ctx, const int8_t *d_a, const float *d_as, int64_t m, int64_t k, const int8_t *d_bt,
                           const float *d_ws, int64_t n, float *d_y, int32_t *d_acc);
// pg_gemv_wstream.cu
bool pgk_gemm_i8_wstream_supports(int64_t m, int64_t k, int64_t n);
int32_t pgk_gemm_i8_wstream(pg_ctx *ctx, const int8_t *d_a, const float *d_as, int64_t m, int64_t k, const int8_t *d_bt,
                            const float *d_ws, int64_t n, float *d_y, int32_t *d_acc);
// pg_llama_attn.cu
int pgk_gqa_stream_splits(const pg_ctx *ctx, int64_t B, int64_t Hkv, int64_t cap);
bool pgk_gqa_stream_supports(int64_t G);
int32_t pgk_gqa_decode_stream(pg_ctx *ctx, const float *d_q, float *d_k, float *d_v, const int32_t *d_pos, const float *d_cos,
                              const float *d_sin, int64_t B, int64_t Hq, int64_t Hkv, int64_t cap, int S, float scale, float *part_o,
                              float *part_ml);
// pg_gemm_tcgen05.cu
bool pgk_gemm_i8_tcgen05_supports(int64_t m, int64_t k, int64_t n);
int32_t pgk_gemm_i8_tcgen05(pg_ctx *ctx, const int8_t *d_a, const float *d_as, int64_t m, int64_t k, pg_qtensor *w,
                            float *d_y, int32_t *d_acc);
// pg_gemm_tcgen05_2cta.cu
int32_t pgk_gemm_i8_tcgen05_2cta(pg_ctx *ctx, const int8_t *d_a, const float *d_as, int64_t m, int64_t k, pg_qtensor *w,
                                 float *d_y, int32_t *d_acc);
// pg_gguf.cu
int32_t pgk_dequant_blocks(pg_ctx *ctx, int32_t type, const uint8_t *d_raw, int64_t num_blocks, float *d_out);
int32_t pgk_f16_to_f32(pg_ctx *ctx, const uint16_t *d_bits, int64_t count, float *d_out);
int32_t pgk_gguf_repack(pg_ctx *ctx, int32_t type, const uint8_t *d_raw, int64_t n, int64_t k, pg_gguf_weight *w);
int32_t pgk_matmul_gguf(pg_ctx *ctx, const float *d_x, int64_t m, const pg_gguf_weight *w, float *d_y);
// pg_gguf_mma.cu
bool pgk_matmul_gguf_mma_supports(const pg_gguf_weight *w, int64_t m);
int32_t pgk_matmul_gguf_mma(pg_ctx *ctx, const float *d_x, int64_t m, const pg_gguf_weight *w, float *d_y);

// ------------------------------------------------------- device helpers ----
// Rust `(v.round().clamp(-127.0, 127.0)) as i8`: roundf is half away from zero; the
// float->int conversion maps NaN to 0 and saturates, so the clamp can be done on the
// integer and NaN never meets a float min/max (which would drop it).
__device__ __forceinline__ int pg_round_clamp_i8(float v)
{
    int i = __float2int_rz(roundf(v));
    return max(-127, min(127, i));
}
