// All-gather of output slices by direct stores into peer GPUs' memory over NVLink.
//
// Column-sharded linears end with one exchange: every rank holds Y[:, n0:n1] and every rank needs
// all of Y.  (API precedent in the reference: Communicator::allgather, src/comm/communicator.rs:162-191,
// a CPU shared-memory ring.)  At decode sizes the slices are 16 KB - 1 MB, where a library collective
// costs mostly launch latency and cannot be recorded into this library's step graph.  Here each rank
// instead writes its slice straight into every rank's [M, N] result buffer (plain st.global to
// peer pointers obtained through CUDA IPC), then raises one flag per destination; consumers wait on
// their local flags.  No multimem, no TMA, no library kernel touches peer memory.
//
// Protocol, per exchange object (one per linear), all words in the symmetric block of each rank:
//   flag[src]   written remotely by rank `src`: the number of the last exchange it has delivered
//   sent        local count of exchanges this rank has produced (bumped by the producer kernel)
//   waited      local count of exchanges this rank has consumed (bumped by the wait kernel)
//   done        CTA counter of the producer kernel
// Counting on the device (not in kernel arguments) keeps the kernels replayable from a graph.
// The consumer's wait is bounded (about a second): on expiry it records PG_ERR_DEVICE_TIMEOUT in the
// context's status word and returns, so a missing peer never hangs a GPU.
#include <string.h>

#include <new>

#include "pg_internal.cuh"

namespace {

constexpr int PG_MAX_PEERS = 8;
constexpr unsigned long long PEER_WAIT_LIMIT_NS = 1000ull * 1000ull * 1000ull;

struct PeerDst {
    float *y[PG_MAX_PEERS];          // [M, n_total] result buffer of each rank (own included)
    uint32_t *ctl[PG_MAX_PEERS];     // control block of each rank: flag[8], sent, waited, done
};

__device__ __forceinline__ unsigned long long globaltimer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// grid-stride copy of the local slice [M, n_local] into column range [col0, col0 + n_local) of every
// rank's [M, n_total]; the last CTA to finish publishes the exchange number to every rank.
__global__ void __launch_bounds__(256) peer_allgather_store_kernel(const float *__restrict__ slice, int M, int64_t n_local,
                                                                   int64_t n_total, int64_t col0, PeerDst dst, int world, int rank)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int64_t total = (int64_t)M * n_local;
    const bool vec = ((n_local | n_total | col0) & 3) == 0;
    if (vec) {
        const int64_t nv = total >> 2, rowv = n_local >> 2;
        for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < nv; i += (int64_t)gridDim.x * 256) {
            const int64_t m = i / rowv, c = (i - m * rowv) << 2;
            const float4 v = *reinterpret_cast<const float4 *>(slice + m * n_local + c);
            for (int p = 0; p < world; p++) *reinterpret_cast<float4 *>(dst.y[p] + m * n_total + col0 + c) = v;
        }
    } else {
        for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
            const int64_t m = i / n_local, c = i - m * n_local;
            const float v = pg_ld_fresh(slice + i);
            for (int p = 0; p < world; p++) dst.y[p][m * n_total + col0 + c] = v;
        }
    }
    // The CTA barrier orders every thread's peer stores before thread 0's system-scope fence, which
    // (fences are cumulative) makes them visible to the other GPUs before the CTA is counted.
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        uint32_t *ctl = dst.ctl[rank];
        if (atomicAdd(&ctl[PG_MAX_PEERS + 2], 1u) == gridDim.x - 1) {
            ctl[PG_MAX_PEERS + 2] = 0;
            const uint32_t seq = ++ctl[PG_MAX_PEERS + 0];
            __threadfence_system();
            for (int p = 0; p < world; p++) {
                uint32_t *f = dst.ctl[p] + rank;
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(seq) : "memory");
            }
        }
    }
}

// one warp: lane r waits until rank r has delivered this rank's next exchange
__global__ void __launch_bounds__(32) peer_wait_kernel(uint32_t *ctl, int world, int32_t *status)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int lane = threadIdx.x;
    uint32_t want = 0;
    if (lane == 0) want = ++ctl[PG_MAX_PEERS + 1];
    want = __shfl_sync(0xffffffffu, want, 0);
    if (lane < world) {
        const unsigned long long t0 = globaltimer_ns();
        for (uint32_t it = 0;; ++it) {
            uint32_t got;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(got) : "l"(ctl + lane) : "memory");
            if ((int32_t)(got - want) >= 0) break;
            if ((it & 63) == 63 && globaltimer_ns() - t0 > PEER_WAIT_LIMIT_NS) {
                atomicExch(status, (int32_t)PG_ERR_DEVICE_TIMEOUT);
                break;
            }
        }
    }
    __threadfence_system();
}

}  // namespace

struct pg_exchange {
    int world = 0, rank = 0;
    float *y_local = nullptr;       // own [M_max, n_total] buffer (symmetric allocation)
    uint32_t *ctl_local = nullptr;  // own control block (part of the same allocation)
    void *base_local = nullptr;
    size_t bytes = 0, y_bytes = 0;
    void *peer_base[PG_MAX_PEERS] = {};
    PeerDst dst = {};
};

extern "C" {

// Allocates this rank's symmetric block (result buffer of `y_bytes` + control words) and writes its
// 64-byte CUDA IPC handle to `handle_out`.  Every rank then passes all ranks' handles, in rank order,
// to pg_exchange_connect.
PG_API int32_t pg_exchange_create(pg_ctx *ctx, int32_t rank, int32_t world, size_t y_bytes, void *handle_out, pg_exchange **out)
{
    PG_REQUIRE(ctx && out && handle_out, "exchange_create: null argument");
    *out = nullptr;
    PG_REQUIRE(world >= 1 && world <= PG_MAX_PEERS && rank >= 0 && rank < world, "exchange_create: rank %d / world %d (max %d)", rank, world,
               PG_MAX_PEERS);
    int prev = -1;
    cudaGetDevice(&prev);
    if (prev != ctx->device) PG_CUDA(cudaSetDevice(ctx->device));
    pg_exchange *ex = new (std::nothrow) pg_exchange();
    if (!ex) PG_FAIL(PG_ERR_NOMEM, "out of host memory");
    ex->world = world;
    ex->rank = rank;
    ex->y_bytes = (y_bytes + 255) & ~(size_t)255;
    ex->bytes = ex->y_bytes + 256;
    cudaError_t e = cudaMalloc(&ex->base_local, ex->bytes);
    if (e == cudaSuccess) e = cudaMemset(ex->base_local, 0, ex->bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, ex->base_local);
    if (e != cudaSuccess) {
        pg_set_error("exchange_create: %s", cudaGetErrorString(e));
        if (ex->base_local) cudaFree(ex->base_local);
        delete ex;
        return e == cudaErrorMemoryAllocation ? PG_ERR_NOMEM : PG_ERR_CUDA;
    }
    memcpy(handle_out, &h, sizeof(h));
    ex->y_local = reinterpret_cast<float *>(ex->base_local);
    ex->ctl_local = reinterpret_cast<uint32_t *>(reinterpret_cast<char *>(ex->base_local) + ex->y_bytes);
    *out = ex;
    return PG_OK;
}

// handles: world x 64 bytes in rank order (this rank's own entry is ignored).
PG_API int32_t pg_exchange_connect(pg_ctx *ctx, pg_exchange *ex, const void *handles)
{
    PG_REQUIRE(ctx && ex && handles, "exchange_connect: null argument");
    int prev = -1;
    cudaGetDevice(&prev);
    if (prev != ctx->device) PG_CUDA(cudaSetDevice(ctx->device));
    for (int p = 0; p < ex->world; p++) {
        void *base = ex->base_local;
        if (p != ex->rank) {
            cudaIpcMemHandle_t h;
            memcpy(&h, reinterpret_cast<const char *>(handles) + (size_t)p * sizeof(h), sizeof(h));
            PG_CUDA(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
            ex->peer_base[p] = base;
        }
        ex->dst.y[p] = reinterpret_cast<float *>(base);
        ex->dst.ctl[p] = reinterpret_cast<uint32_t *>(reinterpret_cast<char *>(base) + ex->y_bytes);
    }
    return PG_OK;
}

PG_API float *pg_exchange_result(const pg_exchange *ex) { return ex ? ex->y_local : nullptr; }

// Enqueues the store half: copy slice [M, n_local] into columns [col0, col0 + n_local) of every rank's
// result buffer ([M, n_total]) and publish.  Returns without waiting for the other ranks.
PG_API int32_t pg_exchange_store(pg_ctx *ctx, pg_exchange *ex, const float *d_slice, int64_t m, int64_t n_local, int64_t n_total,
                                 int64_t col0)
{
    PG_REQUIRE(ctx && ex, "exchange_store: null argument");
    PG_REQUIRE(m >= 0 && n_local >= 0 && col0 >= 0 && col0 + n_local <= n_total, "exchange_store: bad column range");
    PG_REQUIRE((size_t)m * (size_t)n_total * sizeof(float) <= ex->y_bytes, "exchange_store: result does not fit the exchange buffer");
    PG_REQUIRE(ex->dst.y[ex->world - 1] != nullptr, "exchange_store: pg_exchange_connect has not been called");
    const int64_t total = m * n_local;
    int64_t blocks = (total / 4 + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > 2 * (int64_t)ctx->sm_count) blocks = 2 * (int64_t)ctx->sm_count;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = ctx->stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    PG_CUDA(cudaLaunchKernelEx(&cfg, peer_allgather_store_kernel, d_slice, (int)m, n_local, n_total, col0, ex->dst, ex->world, ex->rank));
    PG_LAUNCHED();
    return PG_OK;
}

// Enqueues the wait half: a bounded wait until every rank has delivered its slice of this rank's next
// exchange on `ex`.  One wait per store, in the same order on every rank.
PG_API int32_t pg_exchange_wait(pg_ctx *ctx, pg_exchange *ex)
{
    PG_REQUIRE(ctx && ex, "exchange_wait: null argument");
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t wc = {};
    wc.gridDim = dim3(1);
    wc.blockDim = dim3(32);
    wc.stream = ctx->stream;
    wc.attrs = attr;
    wc.numAttrs = 1;
    PG_CUDA(cudaLaunchKernelEx(&wc, peer_wait_kernel, ex->ctl_local, ex->world, ctx->d_status));
    PG_LAUNCHED();
    return PG_OK;
}

// store + wait
PG_API int32_t pg_exchange_allgather(pg_ctx *ctx, pg_exchange *ex, const float *d_slice, int64_t m, int64_t n_local, int64_t n_total,
                                     int64_t col0)
{
    const int32_t rc = pg_exchange_store(ctx, ex, d_slice, m, n_local, n_total, col0);
    if (rc != PG_OK) return rc;
    return pg_exchange_wait(ctx, ex);
}

PG_API int32_t pg_exchange_destroy(pg_ctx *ctx, pg_exchange *ex)
{
    if (!ex) return PG_OK;
    PG_REQUIRE(ctx != nullptr, "null context");
    cudaStreamSynchronize(ctx->stream);
    for (int p = 0; p < ex->world; p++)
        if (ex->peer_base[p]) cudaIpcCloseMemHandle(ex->peer_base[p]);
    if (ex->base_local) cudaFree(ex->base_local);
    delete ex;
    return PG_OK;
}

}  // extern "C"
