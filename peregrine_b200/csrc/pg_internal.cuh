// Internal declarations shared by the translation units of libperegrine_b200.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <atomic>
#include <vector>

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

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) sticks to a kernel for the life of the process (per device): set it
// once per kernel instantiation and device instead of on every launch.  `mask` is a static of the calling launcher
// (one per instantiation); bit d = done on device d.
template <typename K>
inline cudaError_t pg_max_smem_once(K kern, int bytes, int device, std::atomic<uint64_t> &mask)
{
    const uint64_t bit = 1ull << (device & 63);
    if (mask.load(std::memory_order_acquire) & bit) return cudaSuccess;
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) mask.fetch_or(bit, std::memory_order_release);
    return e;
}

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
    // Bounded waits inside kernels (mbarrier waits, flag waits on other GPUs) give up after this long and record
    // PG_ERR_DEVICE_TIMEOUT in d_status; a kernel argument, so a caller (or a test) can shorten it per context.
    unsigned long long wait_limit_ns = 1000ull * 1000ull * 1000ull;
    // A recorded graph keeps the scratch / staging / split-K addresses it was recorded with.  While graphs of this
    // context are alive, a block that has to grow is not freed but parked here, and freed when the last graph goes
    // (or with the context), so that replaying an older graph never touches freed memory.
    // pg_matmul_quantized_host with page-locked buffers: the launches of a call that comes back with the same buffers,
    // shape and weights are recorded once and replayed as one graph (a third less submission work per blocking call)
    struct HostCall {
        const void *x = nullptr, *y = nullptr, *w = nullptr, *wt = nullptr, *ws = nullptr, *staging = nullptr, *scratch = nullptr, *splitk = nullptr;
        int64_t m = 0, k = 0, n = 0;
        unsigned long long limit = 0;
        int mode = 0;
        cudaGraphExec_t exec = nullptr;   // null: seen once, not yet recorded
        uint64_t stamp = 0, kernels = 0;
    };
    std::vector<HostCall> host_calls;
    uint64_t host_stamp = 0;
    bool no_growth = false;         // set around a call that may not allocate: kernels choose forms that need no new workspace
    int live_graphs = 0;
    std::vector<void *> retired;
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
    // tiled = 1 (Q4_0 / Q8_0 with K % 256 == 0): d_qs holds the streaming kernel's layout instead of the planes above --
    // one contiguous "fill" per (tile of 16 rows, slice of 8 blocks): 16 rows x {128, 256} quant bytes, then 16 rows x
    // eight f16 scales (csrc/pg_gguf.cu: repack_kernel).  Rows past N are zero.
    int tiled = 0;
};

// ---- exchange between the GPUs of a node (csrc/pg_peer.cu) ----------------------------------------------------
// One symmetric block per rank: a plain result buffer, a buffer of flagged cells and control words.
//
// Flagged cells (the form the step kernels use): every f32 of the gathered matrix travels as an 8-byte cell
// {value bits, number of the exchange}, written by the producing kernel's epilogue into EVERY rank's cell buffer with
// one plain 8-byte store per cell (two cells per 16-byte store where aligned).  An 8-byte store arrives whole, so a
// consumer that reads a cell and finds the number it expects has the value: no fence, no separate flag, no counter
// crosses NVLink, and an exchange costs one store latency.  Consumers poll the cells they need (bounded).
// The number of an exchange is kept on the device (PG_CTL_SENT, bumped by the producer's last CTA with a local atomic
// counter), so the kernels replay from a graph; every rank enqueues the same sequence, so a consumer finds its own
// producer's count in PG_CTL_SENT and waits for cells of exactly that number.
//
// Separate flags (pg_exchange_store / pg_exchange_wait, for slices some other kernel produced): plain floats into
// every rank's result buffer, a system-scope fence, then flag[producer] raised on every rank; consumers spin, bounded,
// on the flags of their own block.
constexpr int PG_MAX_PEERS = 8;
enum { PG_CTL_FLAG0 = 0, PG_CTL_SENT = 8, PG_CTL_WAITED = 9, PG_CTL_DONE = 10, PG_CTL_CELL_SENT = 11, PG_CTL_CELL_DONE = 12, PG_CTL_WORDS = 64 };

// what a producing kernel gets (by value, in its arguments)
struct PgPeerOut {
    float *y[PG_MAX_PEERS];          // plain result buffer of each rank (own included)
    uint2 *cells[PG_MAX_PEERS];      // cell buffer of each rank
    uint32_t *ctl[PG_MAX_PEERS];     // control block of each rank
    int32_t world, rank;
    int64_t ld, col0;                // row stride of the result (total columns) and this rank's first column
};
// what a consuming kernel gets: its own cell buffer and control block; cells == nullptr means "nothing to wait for"
struct PgPeerWait {
    const uint2 *cells;
    const uint32_t *ctl;
    int32_t world;
    int32_t *status;
    unsigned long long limit_ns;
};

struct pg_exchange {
    int world = 0, rank = 0;
    float *y_local = nullptr;       // own plain result buffer (start of the symmetric block)
    uint2 *cells_local = nullptr;   // own cell buffer (behind it)
    uint32_t *ctl_local = nullptr;  // own control block (behind that)
    void *base_local = nullptr;
    size_t bytes = 0, y_bytes = 0;
    void *peer_base[PG_MAX_PEERS] = {};
    float *y[PG_MAX_PEERS] = {};
    uint2 *cells[PG_MAX_PEERS] = {};
    uint32_t *ctl[PG_MAX_PEERS] = {};
    bool connected = false;
};
PgPeerOut pg_peer_out(const pg_exchange *ex, int64_t ld, int64_t col0);
PgPeerWait pg_peer_wait_of(const pg_ctx *ctx, const pg_exchange *ex);

#ifdef __CUDACC__
__device__ __forceinline__ unsigned long long pg_globaltimer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---- flagged cells: producer side ----
// number of the exchange this kernel produces (read once per thread that stores, after griddepcontrol.wait)
__device__ __forceinline__ uint32_t pg_cell_seq(const PgPeerOut &o) { return __ldcg(o.ctl[o.rank] + PG_CTL_CELL_SENT) + 1; }
// one value to column `col` (local numbering) of row `m` of every rank
__device__ __forceinline__ void pg_cell_store(const PgPeerOut &o, uint32_t seq, int64_t m, int64_t col, float v)
{
    const int64_t at = m * o.ld + o.col0 + col;
    for (int p = 0; p < o.world; p++)
        asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(o.cells[p] + at), "r"(__float_as_uint(v)), "r"(seq) : "memory");
}
// two adjacent columns in one 16-byte store (each half carries its own number); the cell index must be even
__device__ __forceinline__ void pg_cell_store2(const PgPeerOut &o, uint32_t seq, int64_t m, int64_t col, float v0, float v1)
{
    const int64_t at = m * o.ld + o.col0 + col;
    for (int p = 0; p < o.world; p++)
        asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %2};" ::"l"(o.cells[p] + at), "r"(__float_as_uint(v0)), "r"(seq),
                     "r"(__float_as_uint(v1))
                     : "memory");
}
// Called once by every thread of EVERY CTA of the producing grid after its last cell store: the last CTA to be counted
// (a local counter, nothing crosses NVLink) records the number for this rank's consumers.
__device__ __forceinline__ void pg_cell_finish(const PgPeerOut &o, uint32_t seq, int tid)
{
    __syncthreads();
    if (tid == 0) {
        uint32_t *ctl = o.ctl[o.rank];
        const unsigned ctas = gridDim.x * gridDim.y * gridDim.z;
        __threadfence();
        if (atomicAdd(&ctl[PG_CTL_CELL_DONE], 1u) == ctas - 1) {
            ctl[PG_CTL_CELL_DONE] = 0;
            __stcg(ctl + PG_CTL_CELL_SENT, seq);
        }
    }
}

// ---- flagged cells: consumer side ----
// the number this rank's consumers wait for: its own producer's last exchange (the producer ran earlier in the stream)
// (limit_ns == 0 is the solo diagnostic of pg_peer.cu: every cell counts as delivered)
__device__ __forceinline__ uint32_t pg_cell_want(const PgPeerWait &w) { return w.limit_ns ? __ldcg(w.ctl + PG_CTL_CELL_SENT) : 0x80000000u; }
__device__ __forceinline__ bool pg_cell_fresh(uint32_t got, uint32_t want) { return want == 0x80000000u || (int32_t)(got - want) >= 0; }
// gives up after limit_ns: PG_ERR_DEVICE_TIMEOUT goes to the status word and the caller carries on with what it has
__device__ __forceinline__ bool pg_cell_expired(unsigned long long &t0, uint32_t it, const PgPeerWait &w)
{
    if ((it & 63) != 63) return false;
    const unsigned long long now = pg_globaltimer_ns();
    if (t0 == 0) {
        t0 = now;
        return false;
    }
    if (now - t0 <= w.limit_ns) return false;
    atomicExch(w.status, (int32_t)PG_ERR_DEVICE_TIMEOUT);
    return true;
}
// Four consecutive values starting at cell `at` (a multiple of 2: 16-byte aligned), in two steps so that a thread can
// have the loads of several groups in flight before it looks at any of them (a loop that polls one group to the end
// before it asks for the next one pays a full memory latency per group):
//   pg_cell_issue4   the two 16-byte loads, no dependence on their results
//   pg_cell_settle4  checks the numbers and polls again (bounded) only while a cell is still the previous exchange's
__device__ __forceinline__ void pg_cell_issue4(const PgPeerWait &w, int64_t at, uint4 &a, uint4 &b)
{
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(w.cells + at) : "memory");
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(w.cells + at + 2) : "memory");
}
__device__ __forceinline__ float4 pg_cell_settle4(const PgPeerWait &w, uint32_t want, int64_t at, uint4 a, uint4 b)
{
    unsigned long long t0 = 0;
    for (uint32_t it = 0;; ++it) {
        if (pg_cell_fresh(a.y, want) && pg_cell_fresh(a.w, want) && pg_cell_fresh(b.y, want) && pg_cell_fresh(b.w, want)) break;
        if (pg_cell_expired(t0, it, w)) break;
        pg_cell_issue4(w, at, a, b);
    }
    return make_float4(__uint_as_float(a.x), __uint_as_float(a.z), __uint_as_float(b.x), __uint_as_float(b.z));
}
__device__ __forceinline__ float4 pg_cell_load4(const PgPeerWait &w, uint32_t want, int64_t at)
{
    uint4 a, b;
    pg_cell_issue4(w, at, a, b);
    return pg_cell_settle4(w, want, at, a, b);
}
__device__ __forceinline__ float pg_cell_load(const PgPeerWait &w, uint32_t want, int64_t at)
{
    unsigned long long t0 = 0;
    uint2 a;
    for (uint32_t it = 0;; ++it) {
        asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(a.x), "=r"(a.y) : "l"(w.cells + at) : "memory");
        if (pg_cell_fresh(a.y, want)) break;
        if (pg_cell_expired(t0, it, w)) break;
    }
    return __uint_as_float(a.x);
}

// ---- separate flags ----
// Producer side, called once by every thread of EVERY CTA of the grid after its last plain store into the peers'
// buffers.  The CTA barrier orders the CTA's stores before thread 0's system-scope fence (fences are cumulative); the
// last CTA to be counted numbers the exchange and raises this rank's flag on every rank.
__device__ __forceinline__ void pg_peer_publish(const PgPeerOut &o, int tid)
{
    __syncthreads();
    if (tid == 0) {
        __threadfence_system();
        uint32_t *ctl = o.ctl[o.rank];
        const unsigned ctas = gridDim.x * gridDim.y * gridDim.z;
        if (atomicAdd(&ctl[PG_CTL_DONE], 1u) == ctas - 1) {
            ctl[PG_CTL_DONE] = 0;
            const uint32_t seq = __ldcg(ctl + PG_CTL_SENT) + 1;
            __stcg(ctl + PG_CTL_SENT, seq);
            __threadfence_system();
            for (int p = 0; p < o.world; p++)
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(o.ctl[p] + PG_CTL_FLAG0 + o.rank), "r"(seq) : "memory");
        }
    }
}
// one value to column `col` (local numbering) of row `m` of every rank's plain buffer
__device__ __forceinline__ void pg_peer_store(const PgPeerOut &o, int64_t m, int64_t col, float v)
{
    const int64_t at = m * o.ld + o.col0 + col;
    for (int p = 0; p < o.world; p++) o.y[p][at] = v;
}
__device__ __forceinline__ void pg_peer_store4(const PgPeerOut &o, int64_t m, int64_t col, float4 v)   // 16-byte aligned
{
    const int64_t at = m * o.ld + o.col0 + col;
    for (int p = 0; p < o.world; p++) *reinterpret_cast<float4 *>(o.y[p] + at) = v;
}
#endif

int32_t pg_scratch_reserve(pg_ctx *ctx, size_t bytes);
int32_t pg_pinned_reserve(pg_ctx *ctx, size_t bytes);
int32_t pg_staging_reserve(pg_ctx *ctx, size_t bytes);
int32_t pg_splitk_reserve(pg_ctx *ctx, size_t bytes);

// Makes the context's device current for the duration of an entry point and restores the caller's afterwards.
struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev)
    {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != dev) ok = (cudaSetDevice(dev) == cudaSuccess);
    }
    ~DeviceGuard()
    {
        int cur = -1;
        if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
    }
};

#define PG_ENTER(ctx)                                                   \
    PG_REQUIRE((ctx) != nullptr, "null context");                       \
    DeviceGuard _guard((ctx)->device);                                  \
    if (!_guard.ok) PG_FAIL(PG_ERR_CUDA, "cudaSetDevice(%d) failed", (ctx)->device)

// ------------------------------------------------------- kernel launchers ----
// pg_quantize.cu
int32_t pgk_quantize_activations(pg_ctx *ctx, const float *d_x, int64_t rows, int64_t cols, int8_t *d_q, float *d_scales);
int32_t pgk_quantize_activations_wait(pg_ctx *ctx, const float *d_x, int64_t rows, int64_t cols, int8_t *d_q, float *d_scales,
                                      const PgPeerWait *wait);
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
// the same product with its outputs stored into every rank's exchange buffer and the exchange published by the kernel
int32_t pgk_gemm_i8_wstream_peer(pg_ctx *ctx, const int8_t *d_a, const float *d_as, int64_t m, int64_t k, const int8_t *d_bt,
                                 const float *d_ws, int64_t n, const PgPeerOut &out);
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
// pg_gguf_stream.cu
bool pgk_matmul_gguf_stream_supports(const pg_gguf_weight *w, int64_t m);
int32_t pgk_matmul_gguf_stream(pg_ctx *ctx, const float *d_x, int64_t m, const pg_gguf_weight *w, float *d_y);
// bytes of d_qs for `rows` rows of `k` columns, and whether the tiled layout applies
size_t pgk_gguf_qs_bytes(int32_t type, int64_t rows, int64_t k, int *tiled);

// ------------------------------------------------------- device helpers ----
// Rust `(v.round().clamp(-127.0, 127.0)) as i8`: roundf is half away from zero; the
// float->int conversion maps NaN to 0 and saturates, so the clamp can be done on the
// integer and NaN never meets a float min/max (which would drop it).
__device__ __forceinline__ int pg_round_clamp_i8(float v)
{
    int i = __float2int_rz(roundf(v));
    return max(-127, min(127, i));
}
