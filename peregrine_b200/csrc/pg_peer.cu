// All-gather of output slices by direct stores into peer GPUs' memory over NVLink.
//
// Column-sharded linears end with one exchange: every rank holds Y[:, n0:n1] and every rank needs
// all of Y.  (API precedent in the reference: Communicator::allgather, src/comm/communicator.rs:162-191,
// a CPU shared-memory ring.)  At decode sizes the slices are 16 KB - 1 MB, where a library collective
// costs mostly launch latency and cannot be recorded into this library's step graph.  Here each rank
// instead writes its slice straight into every rank's buffer (plain stores to peer pointers obtained
// through CUDA IPC).  No multimem, no TMA, no library kernel touches peer memory; only stores cross NVLink.
//
// Two forms (the protocols are described with the structures in pg_internal.cuh):
//   * flagged cells (pg_gemm_i8_exchange and the *_exchange glue entry points of pg_llama.cu): the producing
//     kernel's own epilogue stores {value, number of the exchange} cells into every rank; the consuming kernel (the
//     next quantiser / RMSNorm of the step, or pg_exchange_gather) polls the cells it reads.  No extra launch, no
//     fence and no flag per exchange: one store latency.  (With a system-scope fence, a flag per rank and an
//     acquire-poll the same exchange took 12-15 us on two B200s, as much as the product it followed.)
//   * separate flags (pg_exchange_store / pg_exchange_wait): a copy kernel and a one-warp wait kernel, for slices
//     that some other kernel produced into plain memory.
//
// An exchange object may be reused once every rank has consumed its previous result: two other exchanges that all
// ranks take part in between two uses are enough (a decode layer has four).  Every wait is bounded
// (pg_ctx_set_wait_limit_ns, a second by default): on expiry the kernel records PG_ERR_DEVICE_TIMEOUT in the
// context's status word and goes on, so a missing peer never hangs a GPU.
#include <string.h>

#include <new>

#include "pg_internal.cuh"

namespace {

// grid-stride copy of the local slice [M, n_local] into column range [col0, col0 + n_local) of every
// rank's [M, ld]; the last CTA to finish publishes the exchange number to every rank.
__global__ void __launch_bounds__(256) peer_allgather_store_kernel(const float *slice, int M, int64_t n_local, const PgPeerOut dst, int vec)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int64_t total = (int64_t)M * n_local;
    // the slice comes from the kernel before this one: read it through L2 (see pg_ld_fresh)
    if (vec) {
        const int64_t nv = total >> 2, rowv = n_local >> 2;
        for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < nv; i += (int64_t)gridDim.x * 256) {
            const int64_t m = i / rowv, c = (i - m * rowv) << 2;
            pg_peer_store4(dst, m, c, pg_ld_fresh(reinterpret_cast<const float4 *>(slice + m * n_local + c)));
        }
    } else {
        for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
            const int64_t m = i / n_local, c = i - m * n_local;
            pg_peer_store(dst, m, c, pg_ld_fresh(slice + i));
        }
    }
    pg_peer_publish(dst, threadIdx.x);
}

// the same copy into every rank's flagged cells (for a slice that an ordinary kernel produced)
__global__ void __launch_bounds__(256) peer_cells_store_kernel(const float *slice, int M, int64_t n_local, const PgPeerOut dst)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t seq = pg_cell_seq(dst);
    const int64_t total = (int64_t)M * n_local;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
        const int64_t m = i / n_local, c = i - m * n_local;
        pg_cell_store(dst, seq, m, c, pg_ld_fresh(slice + i));
    }
    pg_cell_finish(dst, seq, threadIdx.x);
}

// waits (bounded, per cell) for every rank's cells of this rank's last exchange and writes the plain [rows, cols] matrix
__global__ void __launch_bounds__(256) peer_cells_gather_kernel(float *out, int64_t total, const PgPeerWait wt)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t want = pg_cell_want(wt);
    const int64_t nv = total >> 2;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < nv; i += (int64_t)gridDim.x * 256)
        reinterpret_cast<float4 *>(out)[i] = pg_cell_load4(wt, want, i * 4);
    for (int64_t i = (nv << 2) + (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256)
        out[i] = pg_cell_load(wt, want, i);
}

// The same for several exchanges in one launch (results that nothing consumes one by one: the independent products of a
// batch of requests).  The concatenation of the matrices is walked in units of four values; each matrix has a multiple
// of four of them.
constexpr int PG_GATHER_MAX = 16;
struct PgGatherMany {
    PgPeerWait wt[PG_GATHER_MAX];
    float *out[PG_GATHER_MAX];
    int64_t end4[PG_GATHER_MAX];    // running sum of the matrices' sizes, in units of four values
    int count;
};
__global__ void __launch_bounds__(256) peer_cells_gather_many_kernel(const __grid_constant__ PgGatherMany p)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int64_t all = p.end4[p.count - 1];
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < all; i += (int64_t)gridDim.x * 256) {
        int e = 0;
        while (i >= p.end4[e]) e++;
        const int64_t at = (i - (e ? p.end4[e - 1] : 0)) * 4;
        const uint32_t want = pg_cell_want(p.wt[e]);
        *reinterpret_cast<float4 *>(p.out[e] + at) = pg_cell_load4(p.wt[e], want, at);
    }
}

// one warp: lane r waits until rank r has delivered this rank's next exchange
__global__ void __launch_bounds__(32) peer_wait_kernel(uint32_t *ctl, int world, int32_t *status, unsigned long long limit_ns)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int lane = threadIdx.x;
    uint32_t want = 0;
    if (lane == 0) {
        want = __ldcg(ctl + PG_CTL_WAITED) + 1;
        __stcg(ctl + PG_CTL_WAITED, want);
    }
    want = __shfl_sync(0xffffffffu, want, 0);
    if (lane < world) {
        const unsigned long long t0 = pg_globaltimer_ns();
        for (uint32_t it = 0;; ++it) {
            uint32_t got;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(got) : "l"(ctl + PG_CTL_FLAG0 + lane) : "memory");
            if ((int32_t)(got - want) >= 0) break;
            if ((it & 63) == 63 && pg_globaltimer_ns() - t0 > limit_ns) {
                atomicExch(status, (int32_t)PG_ERR_DEVICE_TIMEOUT);
                break;
            }
        }
    }
    __threadfence_system();
}

}  // namespace

// Diagnostic (pg_tune_exchange_solo): a rank of a sharded step run WITHOUT its peers -- producers store into their own
// buffer only, consumers take every cell as delivered.  The results are meaningless; the step's time is what one rank's
// kernels and launches cost at the sharded shapes with nothing crossing NVLink and nobody waited for.
static int g_exchange_solo = 0;
extern "C" PG_API void pg_tune_exchange_solo(int on) { g_exchange_solo = on; }

PgPeerOut pg_peer_out(const pg_exchange *ex, int64_t ld, int64_t col0)
{
    PgPeerOut o = {};
    if (g_exchange_solo) {
        o.y[0] = ex->y_local;
        o.cells[0] = ex->cells_local;
        o.ctl[0] = ex->ctl_local;
        o.world = 1;
        o.rank = 0;
        o.ld = ld;
        o.col0 = col0;
        return o;
    }
    for (int p = 0; p < ex->world; p++) {
        o.y[p] = ex->y[p];
        o.cells[p] = ex->cells[p];
        o.ctl[p] = ex->ctl[p];
    }
    o.world = ex->world;
    o.rank = ex->rank;
    o.ld = ld;
    o.col0 = col0;
    return o;
}

PgPeerWait pg_peer_wait_of(const pg_ctx *ctx, const pg_exchange *ex)
{
    PgPeerWait w = {};
    w.cells = ex ? ex->cells_local : nullptr;
    w.ctl = ex ? ex->ctl_local : nullptr;
    w.world = ex ? ex->world : 0;
    w.status = ctx->d_status;
    w.limit_ns = g_exchange_solo ? 0ull : ctx->wait_limit_ns;   // solo: limit 0 marks "take every cell as delivered"
    return w;
}

extern "C" {

// Allocates this rank's symmetric block (result buffer of `y_bytes` + control words) and writes its
// 64-byte CUDA IPC handle to `handle_out`.  Every rank then passes all ranks' handles, in rank order,
// to pg_exchange_connect.
PG_API int32_t pg_exchange_create(pg_ctx *ctx, int32_t rank, int32_t world, size_t y_bytes, void *handle_out, pg_exchange **out)
{
    PG_ENTER(ctx);
    PG_REQUIRE(out && handle_out, "exchange_create: null argument");
    *out = nullptr;
    PG_REQUIRE(world >= 1 && world <= PG_MAX_PEERS && rank >= 0 && rank < world, "exchange_create: rank %d / world %d (max %d)", rank, world,
               PG_MAX_PEERS);
    pg_exchange *ex = new (std::nothrow) pg_exchange();
    if (!ex) PG_FAIL(PG_ERR_NOMEM, "out of host memory");
    ex->world = world;
    ex->rank = rank;
    ex->y_bytes = (y_bytes + 255) & ~(size_t)255;
    ex->bytes = 3 * ex->y_bytes + PG_CTL_WORDS * sizeof(uint32_t);   // plain floats | cells (8 bytes per float) | control words
    cudaError_t e = cudaMalloc(&ex->base_local, ex->bytes);
    if (e == cudaSuccess) e = cudaMemset(ex->base_local, 0, ex->bytes);
    cudaIpcMemHandle_t h;
    memset(&h, 0, sizeof(h));
    if (e == cudaSuccess && world > 1) e = cudaIpcGetMemHandle(&h, ex->base_local);
    if (e != cudaSuccess) {
        pg_set_error("exchange_create: %s", cudaGetErrorString(e));
        if (ex->base_local) cudaFree(ex->base_local);
        delete ex;
        return e == cudaErrorMemoryAllocation ? PG_ERR_NOMEM : PG_ERR_CUDA;
    }
    memcpy(handle_out, &h, sizeof(h));
    ex->y_local = reinterpret_cast<float *>(ex->base_local);
    ex->cells_local = reinterpret_cast<uint2 *>(reinterpret_cast<char *>(ex->base_local) + ex->y_bytes);
    ex->ctl_local = reinterpret_cast<uint32_t *>(reinterpret_cast<char *>(ex->base_local) + 3 * ex->y_bytes);
    *out = ex;
    return PG_OK;
}

// handles: world x 64 bytes in rank order (this rank's own entry is ignored).
PG_API int32_t pg_exchange_connect(pg_ctx *ctx, pg_exchange *ex, const void *handles)
{
    PG_ENTER(ctx);
    PG_REQUIRE(ex && (handles || ex->world == 1), "exchange_connect: null argument");
    for (int p = 0; p < ex->world; p++) {
        void *base = ex->base_local;
        if (p != ex->rank) {
            cudaIpcMemHandle_t h;
            memcpy(&h, reinterpret_cast<const char *>(handles) + (size_t)p * sizeof(h), sizeof(h));
            PG_CUDA(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
            ex->peer_base[p] = base;
        }
        ex->y[p] = reinterpret_cast<float *>(base);
        ex->cells[p] = reinterpret_cast<uint2 *>(reinterpret_cast<char *>(base) + ex->y_bytes);
        ex->ctl[p] = reinterpret_cast<uint32_t *>(reinterpret_cast<char *>(base) + 3 * ex->y_bytes);
    }
    ex->connected = true;
    return PG_OK;
}

// Ranks inside one process: the peers' blocks are ordinary device pointers of this process.
PG_API int32_t pg_exchange_connect_local(pg_ctx *ctx, pg_exchange *ex, pg_exchange *const *all)
{
    PG_ENTER(ctx);
    PG_REQUIRE(ex && (all || g_exchange_solo), "exchange_connect_local: null argument");
    for (int p = 0; all && p < ex->world; p++) {
        PG_REQUIRE(all[p] && all[p]->world == ex->world && all[p]->rank == p && all[p]->y_bytes == ex->y_bytes,
                   "exchange_connect_local: entry %d is not rank %d of the same exchange", p, p);
        ex->y[p] = all[p]->y_local;
        ex->cells[p] = all[p]->cells_local;
        ex->ctl[p] = all[p]->ctl_local;
    }
    ex->connected = true;
    return PG_OK;
}

PG_API float *pg_exchange_result(const pg_exchange *ex) { return ex ? ex->y_local : nullptr; }

// Enqueues the store half: copy slice [M, n_local] into columns [col0, col0 + n_local) of every rank's
// result buffer ([M, n_total]) and publish.  Returns without waiting for the other ranks.
PG_API int32_t pg_exchange_store(pg_ctx *ctx, pg_exchange *ex, const float *d_slice, int64_t m, int64_t n_local, int64_t n_total,
                                 int64_t col0)
{
    PG_ENTER(ctx);
    PG_REQUIRE(ex != nullptr, "exchange_store: null argument");
    PG_REQUIRE(m >= 0 && n_local >= 0 && col0 >= 0 && col0 + n_local <= n_total, "exchange_store: bad column range");
    PG_REQUIRE((size_t)m * (size_t)n_total * sizeof(float) <= ex->y_bytes, "exchange_store: result does not fit the exchange buffer");
    PG_REQUIRE(ex->connected, "exchange_store: pg_exchange_connect has not been called");
    PG_REQUIRE(m * n_local == 0 || d_slice, "exchange_store: slice is null");
    const int64_t total = m * n_local;
    int64_t blocks = (total / 4 + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > 2 * (int64_t)ctx->sm_count) blocks = 2 * (int64_t)ctx->sm_count;
    // 16-byte accesses only where every row segment starts on a 16-byte boundary on both sides
    const int vec = ((n_local | n_total | col0) & 3) == 0 && ((uintptr_t)d_slice & 15) == 0;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = ctx->stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    PG_CUDA(cudaLaunchKernelEx(&cfg, peer_allgather_store_kernel, d_slice, (int)m, n_local, pg_peer_out(ex, n_total, col0), vec));
    PG_LAUNCHED();
    return PG_OK;
}

// Enqueues the wait half: a bounded wait until every rank has delivered its slice of this rank's next
// exchange on `ex`.  One wait per store, in the same order on every rank.
PG_API int32_t pg_exchange_wait(pg_ctx *ctx, pg_exchange *ex)
{
    PG_ENTER(ctx);
    PG_REQUIRE(ex != nullptr, "exchange_wait: null argument");
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t wc = {};
    wc.gridDim = dim3(1);
    wc.blockDim = dim3(32);
    wc.stream = ctx->stream;
    wc.attrs = attr;
    wc.numAttrs = 1;
    PG_CUDA(cudaLaunchKernelEx(&wc, peer_wait_kernel, ex->ctl_local, ex->world, ctx->d_status, ctx->wait_limit_ns));
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

// The producer of a flagged-cell exchange for a slice that lies in plain device memory (any kernel's output): copies
// d_slice [M, n_local] into columns [col0, col0 + n_local) of every rank's [M, n_total] cells.  One per exchange and
// rank, like pg_gemm_i8_exchange; consumers: pg_exchange_gather and the *_exchange entry points.
PG_API int32_t pg_exchange_store_cells(pg_ctx *ctx, pg_exchange *ex, const float *d_slice, int64_t m, int64_t n_local, int64_t n_total,
                                       int64_t col0)
{
    PG_ENTER(ctx);
    PG_REQUIRE(ex && ex->connected, "exchange_store_cells: null argument or unconnected exchange");
    PG_REQUIRE(m >= 0 && m <= 0x7fffffff && n_local >= 0 && col0 >= 0 && col0 + n_local <= n_total, "exchange_store_cells: bad column range");
    PG_REQUIRE((size_t)m * (size_t)n_total * sizeof(float) <= ex->y_bytes, "exchange_store_cells: result does not fit the exchange buffer");
    PG_REQUIRE(m * n_local == 0 || d_slice, "exchange_store_cells: slice is null");
    int64_t blocks = (m * n_local + 255) / 256;
    blocks = blocks < 1 ? 1 : (blocks > 2 * (int64_t)ctx->sm_count ? 2 * (int64_t)ctx->sm_count : blocks);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = ctx->stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    PG_CUDA(cudaLaunchKernelEx(&cfg, peer_cells_store_kernel, d_slice, (int)m, n_local, pg_peer_out(ex, n_total, col0)));
    PG_LAUNCHED();
    return PG_OK;
}

// One rank's part of a column-sharded integer GEMM with the all-gather inside it: the product of a_i8 [M, K] with
// this rank's columns `w` ([K, n_local]) lands in columns [col0, col0 + n_local) of EVERY rank's [M, n_total] exchange
// buffer and the exchange is published.  At decode sizes (M <= 16, K % 64 == 0) the product kernel's own epilogue does
// the peer stores; other shapes run the ordinary product into `d_slice_tmp` ([M, n_local] floats of the caller's)
// followed by the copy kernel.  Consumers wait with pg_exchange_wait or one of the *_exchange glue entry points.
PG_API int32_t pg_gemm_i8_exchange(pg_ctx *ctx, const int8_t *d_a_i8, const float *d_a_scales, int64_t m, int64_t k, const pg_qtensor *w,
                                   pg_exchange *ex, int64_t n_total, int64_t col0, float *d_slice_tmp)
{
    PG_ENTER(ctx);
    PG_REQUIRE(w && ex, "gemm_i8_exchange: null argument");
    PG_REQUIRE(ex->connected, "gemm_i8_exchange: pg_exchange_connect has not been called");
    PG_REQUIRE(m >= 0 && k >= 0 && w->rows == k, "gemm_i8_exchange: w.rows (%lld) != k (%lld)", (long long)w->rows, (long long)k);
    const int64_t n = w->cols;
    PG_REQUIRE(col0 >= 0 && col0 + n <= n_total, "gemm_i8_exchange: columns [%lld, %lld) outside [0, %lld)", (long long)col0,
               (long long)(col0 + n), (long long)n_total);
    PG_REQUIRE((size_t)m * (size_t)n_total * sizeof(float) <= ex->y_bytes, "gemm_i8_exchange: result does not fit the exchange buffer");
    PG_REQUIRE(m * k == 0 || (d_a_i8 && d_a_scales), "gemm_i8_exchange: activations are null");
    const bool aligned = (((uintptr_t)d_a_i8 | (uintptr_t)w->d_data_i8_t) & 15) == 0;
    if (m > 0 && n > 0 && aligned && pgk_gemm_i8_wstream_supports(m, k, n))
        return pgk_gemm_i8_wstream_peer(ctx, d_a_i8, d_a_scales, m, k, w->d_data_i8_t, w->d_scales, n, pg_peer_out(ex, n_total, col0));
    PG_REQUIRE(m * n == 0 || d_slice_tmp, "gemm_i8_exchange: this shape needs the slice buffer");
    const int32_t rc = pg_gemm_i8(ctx, d_a_i8, d_a_scales, m, k, w, d_slice_tmp, nullptr, PG_ALGO_AUTO);
    if (rc != PG_OK) return rc;
    return pg_exchange_store_cells(ctx, ex, d_slice_tmp, m, n, n_total, col0);
}

// pg_matmul_quantized with the all-gather inside: f32 activations in, this rank's columns of the product into every rank's
// exchange buffer: the activation quantiser into the context's scratch, then pg_gemm_i8_exchange.  (Running the quantiser
// inside the product kernel for up to four rows was measured: 121.7 against 109.5 us per nine-case sweep on 2 GPUs, 86.2
// against 77.1 us on 8: the separate launch hides behind the preceding product, the prologue inside the kernel does not.)
PG_API int32_t pg_matmul_quantized_exchange(pg_ctx *ctx, const float *d_x, int64_t m, int64_t k, const pg_qtensor *w, pg_exchange *ex,
                                            int64_t n_total, int64_t col0, float *d_slice_tmp)
{
    PG_ENTER(ctx);
    PG_REQUIRE(w && ex && ex->connected, "matmul_quantized_exchange: null argument or unconnected exchange");
    PG_REQUIRE(m >= 0 && k >= 0 && w->rows == k, "matmul_quantized_exchange: w.rows (%lld) != k (%lld)", (long long)w->rows, (long long)k);
    const int64_t n = w->cols;
    PG_REQUIRE(n_total >= n && col0 >= 0 && col0 + n <= n_total, "matmul_quantized_exchange: columns outside the result");
    PG_REQUIRE((size_t)m * (size_t)n_total * sizeof(float) <= ex->y_bytes, "matmul_quantized_exchange: result does not fit the exchange buffer");
    PG_REQUIRE(m * k == 0 || d_x, "matmul_quantized_exchange: activations are null");
    if (m == 0 || n == 0) return PG_OK;
    const size_t nq = ((size_t)m * (size_t)k + 16 + 255) & ~(size_t)255;
    const int32_t rs = pg_scratch_reserve(ctx, nq + (size_t)m * sizeof(float) + 256);
    if (rs != PG_OK) return rs;
    int8_t *d_q = reinterpret_cast<int8_t *>(ctx->scratch);
    float *d_s = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(ctx->scratch) + nq);
    const int32_t rq = pgk_quantize_activations(ctx, d_x, m, k, d_q, d_s);
    if (rq != PG_OK) return rq;
    return pg_gemm_i8_exchange(ctx, d_q, d_s, m, k, w, ex, n_total, col0, d_slice_tmp);
}

// Consumer of a flagged-cell exchange for callers that want the gathered matrix as plain floats: waits (bounded, per
// cell) for every rank's part of the exchange this rank produced last on `ex` (enqueue it behind this rank's own
// producer) and writes [rows, cols] f32 to d_out, or to the exchange's own result buffer (pg_exchange_result) when
// d_out is NULL.
PG_API int32_t pg_exchange_gather(pg_ctx *ctx, pg_exchange *ex, int64_t rows, int64_t cols, float *d_out)
{
    PG_ENTER(ctx);
    PG_REQUIRE(ex && ex->connected, "exchange_gather: null argument or unconnected exchange");
    PG_REQUIRE(rows >= 0 && cols >= 0 && (size_t)rows * (size_t)cols * sizeof(float) <= ex->y_bytes, "exchange_gather: result does not fit the exchange buffer");
    float *out = d_out ? d_out : ex->y_local;
    PG_REQUIRE(((uintptr_t)out & 15) == 0, "exchange_gather: the output must be 16-byte aligned");
    const int64_t total = rows * cols;
    if (total == 0) return PG_OK;
    int64_t blocks = (total / 4 + 255) / 256;
    blocks = blocks < 1 ? 1 : (blocks > 2 * (int64_t)ctx->sm_count ? 2 * (int64_t)ctx->sm_count : blocks);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = ctx->stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    PG_CUDA(cudaLaunchKernelEx(&cfg, peer_cells_gather_kernel, out, total, pg_peer_wait_of(ctx, ex)));
    PG_LAUNCHED();
    return PG_OK;
}

// pg_exchange_gather for up to 16 exchanges in one launch: exchange i's [rows[i], cols[i]] matrix goes to d_outs[i] (or, where
// d_outs or d_outs[i] is NULL, to that exchange's own result buffer).  rows[i] * cols[i] must be a multiple of four.
PG_API int32_t pg_exchange_gather_many(pg_ctx *ctx, pg_exchange *const *exs, const int64_t *rows, const int64_t *cols, float *const *d_outs,
                                       int32_t count)
{
    PG_ENTER(ctx);
    PG_REQUIRE(count >= 0 && count <= PG_GATHER_MAX, "exchange_gather_many: between 0 and %d exchanges per call", PG_GATHER_MAX);
    PG_REQUIRE(count == 0 || (exs && rows && cols), "exchange_gather_many: null argument");
    PgGatherMany p = {};
    int64_t sum4 = 0;
    for (int i = 0; i < count; i++) {
        pg_exchange *ex = exs[i];
        PG_REQUIRE(ex && ex->connected, "exchange_gather_many: exchange %d is null or unconnected", i);
        PG_REQUIRE(rows[i] >= 0 && cols[i] >= 0 && (size_t)rows[i] * (size_t)cols[i] * sizeof(float) <= ex->y_bytes,
                   "exchange_gather_many: result %d does not fit its exchange buffer", i);
        const int64_t total = rows[i] * cols[i];
        PG_REQUIRE(total % 4 == 0, "exchange_gather_many: matrix %d has %lld values, not a multiple of four", i, (long long)total);
        float *out = (d_outs && d_outs[i]) ? d_outs[i] : ex->y_local;
        PG_REQUIRE(((uintptr_t)out & 15) == 0, "exchange_gather_many: output %d must be 16-byte aligned", i);
        if (total == 0) continue;
        p.wt[p.count] = pg_peer_wait_of(ctx, ex);
        p.out[p.count] = out;
        sum4 += total / 4;
        p.end4[p.count] = sum4;
        p.count++;
    }
    if (p.count == 0) return PG_OK;
    int64_t blocks = (sum4 + 255) / 256;
    blocks = blocks > 4 * (int64_t)ctx->sm_count ? 4 * (int64_t)ctx->sm_count : blocks;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = ctx->stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    PG_CUDA(cudaLaunchKernelEx(&cfg, peer_cells_gather_many_kernel, p));
    PG_LAUNCHED();
    return PG_OK;
}

PG_API int32_t pg_exchange_destroy(pg_ctx *ctx, pg_exchange *ex)
{
    if (!ex) return PG_OK;
    PG_ENTER(ctx);
    cudaStreamSynchronize(ctx->stream);
    for (int p = 0; p < ex->world; p++)
        if (ex->peer_base[p]) cudaIpcCloseMemHandle(ex->peer_base[p]);
    if (ex->base_local) cudaFree(ex->base_local);
    delete ex;
    return PG_OK;
}

}  // extern "C"
