/*
 * peregrine_b200 -- C ABI of the B200 (sm_100a) quantized-inference path.
 *
 * This is the boundary a host-language binding (Rust `extern "C"`, ctypes, cgo)
 * links against.  Each entry point names the function of the reference
 * (etam103/peregrine, paths relative to that project) whose work it takes
 * over.  The reference's seam for a GPU backend is its `metal` cargo feature:
 * device buffers cached inside `QuantizedTensor` (src/quant.rs:19-22,172-191),
 * per-call upload of the activations and an unsynchronised device result
 * (src/quant.rs:195-218), dispatch in `Tensor::matmul_quantized`
 * (src/tensor.rs:1382-1408).  The same shape is kept here.
 *
 * Conventions
 *   - Every function returns 0 (PG_OK) or a negative pg_status.  Nothing
 *     aborts, traps or throws across the boundary; `pg_last_error()` returns a
 *     thread-local message for the last failure on the calling thread.  The
 *     reference panics (assert!/expect) where these return PG_ERR_INVALID.
 *   - Pointers named d_* are device pointers on the context's GPU; all others
 *     are host pointers.  Plain pointers and sizes only.
 *   - Work is enqueued on the context's stream and is NOT synchronised unless
 *     the name ends in `_host` (those copy results back and block), matching
 *     the reference's "caller syncs" rule (tests/quant_parity.rs:102-107).
 *   - A context belongs to one thread at a time (the reference's GPU context is
 *     a thread-local singleton, src/metal/context.rs:2472-2510).
 *   - There is no CPU fallback: without a usable sm_100 device pg_ctx_create fails.
 *
 * Matrix layouts are the reference's: activations [M,K] row-major f32;
 * QuantizedTensor data_i8 [K,N] row-major, data_i8_t [N,K] row-major,
 * scales [N]; outputs [M,N] row-major f32.
 */
#ifndef PEREGRINE_B200_H
#define PEREGRINE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define PG_API
#else
#define PG_API __attribute__((visibility("default")))
#endif

typedef struct pg_ctx pg_ctx;
typedef struct pg_qtensor pg_qtensor;
typedef struct pg_gguf_weight pg_gguf_weight;
typedef struct pg_graph pg_graph;
typedef struct pg_exchange pg_exchange;

typedef enum pg_status {
    PG_OK = 0,
    PG_ERR_INVALID = -1,        /* shape/argument check failed (reference: assert!/panic) */
    PG_ERR_CUDA = -2,           /* a CUDA runtime/driver call failed */
    PG_ERR_NOMEM = -3,          /* device or host allocation failed */
    PG_ERR_UNSUPPORTED = -4,    /* no sm_100 device, or a shape the requested kernel cannot take */
    PG_ERR_DEVICE_TIMEOUT = -5  /* a bounded wait inside a kernel ran out; the context stays usable */
} pg_status;

/* GGUF block formats (reference: GgmlType, src/gguf.rs:15-21, same numbering) */
typedef enum pg_gguf_type { PG_GGUF_Q4_0 = 2, PG_GGUF_Q4_1 = 3, PG_GGUF_Q8_0 = 8 } pg_gguf_type;

/* Kernel selection for pg_gemm_i8 / pg_matmul_quantized_algo. */
typedef enum pg_gemm_algo {
    PG_ALGO_AUTO = 0,      /* M <= 16 and K % 64 == 0: warp-stream kernel; 17 <= M <= 32 on narrow layers with K < 8192
                              (and M <= 64 where K % 64 != 0): per-lane streaming kernel; otherwise tcgen05 (with K
                              divided over CTAs where one row of tiles leaves SMs idle and K is long); shapes none of
                              them takes (K % 16 != 0, unaligned operands): the naive kernel */
    PG_ALGO_NAIVE = 1,     /* one thread per output, dp4a; the on-device checker */
    PG_ALGO_STREAM = 2,    /* bandwidth-bound decode kernel (per-lane cp.async FIFO + int8 mma.sync), M <= 64 */
    PG_ALGO_TCGEN05 = 3,   /* tcgen05.mma kind::i8, TMEM accumulators, TMA-fed; at M <= 128 it may reserve a workspace for
                              partial sums (context memory, grown outside graph recording like the scratch) */
    PG_ALGO_WSTREAM = 4    /* persistent decode kernel, M <= 16, K % 64 == 0: bulk copies into per-warp rings, activations
                              resident in shared memory, K split inside the CTA (and over a cluster when the
                              activations do not fit beside the rings), sums added in shared memory */
} pg_gemm_algo;

PG_API const char *pg_last_error(void);
PG_API int32_t pg_version(void);
/* Number of kernels this library has launched in the calling process (for benchmarks). */
PG_API uint64_t pg_launch_count(void);

/* ---- context, replaces metal::init_gpu / GpuContext (src/metal/context.rs:45,2472-2510) ----
 * `stream` is a cudaStream_t to enqueue on (not owned), or NULL to create one. */
PG_API int32_t pg_ctx_create(int32_t device, void *stream, pg_ctx **out);
PG_API int32_t pg_ctx_destroy(pg_ctx *ctx);
/* GpuContext::sync (src/metal/context.rs:188-204) */
PG_API int32_t pg_ctx_sync(pg_ctx *ctx);
PG_API void *pg_ctx_stream(pg_ctx *ctx);
/* Status word written by kernels whose waits are bounded; 0 if none gave up. Clears it. */
PG_API int32_t pg_ctx_device_status(pg_ctx *ctx, int32_t *status_out);
/* How long a bounded wait inside a kernel (an mbarrier of a copy ring, another GPU's flag) may last before the kernel
 * gives up with PG_ERR_DEVICE_TIMEOUT in the status word.  Default one second; at least a microsecond.  Applies to
 * launches made after the call (recorded graphs keep the value they were recorded with).  The reference has no
 * counterpart: its ring collectives spin without a limit (src/comm/signal.rs:61-63, 84-86). */
PG_API int32_t pg_ctx_set_wait_limit_ns(pg_ctx *ctx, uint64_t ns);
/* Device memory the context has allocated so far for its own intermediates (scratch, staging of *_host calls,
 * split-K workspace): grows on demand, never shrinks before pg_ctx_destroy.  0 for a context that has only served
 * calls which bring their own buffers (pg_gemm_i8, pg_matmul_quantized_ex with both buffers, pg_matmul_quantized_static). */
PG_API uint64_t pg_ctx_scratch_bytes(const pg_ctx *ctx);

/* ---- batched submission, replaces the pending command buffer of GpuContext
 *      (src/metal/context.rs:188-204: commands accumulate and are submitted together) ----
 * Everything enqueued on the context between begin and end is recorded into a CUDA graph
 * instead of running; pg_graph_launch then submits the whole batch with one call.  Run the same
 * calls once before recording: a call that has to grow the context's scratch memory cannot
 * be recorded.  *_host calls (they block) cannot be recorded.  A graph keeps the scratch addresses it was
 * recorded with: when a later, larger call makes the context's scratch grow while graphs are alive, the old
 * block stays allocated until the context's last graph is freed, so older graphs stay valid to launch. */
PG_API int32_t pg_graph_begin(pg_ctx *ctx);
PG_API int32_t pg_graph_end(pg_ctx *ctx, pg_graph **out);
PG_API int32_t pg_graph_launch(pg_ctx *ctx, pg_graph *graph);
PG_API int32_t pg_graph_free(pg_ctx *ctx, pg_graph *graph);

/* ---- device memory, replaces GpuContext::alloc/upload and GpuBuffer::read
 *      (src/metal/context.rs; used at src/quant.rs:176-187,207-210) ---- */
PG_API int32_t pg_mem_alloc(pg_ctx *ctx, size_t bytes, void **d_out);
PG_API int32_t pg_mem_free(pg_ctx *ctx, void *d_ptr);
PG_API int32_t pg_mem_upload(pg_ctx *ctx, void *d_dst, const void *src, size_t bytes);   /* async */
PG_API int32_t pg_mem_download(pg_ctx *ctx, void *dst, const void *d_src, size_t bytes); /* blocks */

/* ---- quant::quantize_activations (src/quant.rs:79-112, scalar branch :97-109) ----
 * x [M,K] f32 -> q [M,K] i8, scales [M] f32.  Bit-exact with the scalar branch. */
PG_API int32_t pg_quantize_activations(pg_ctx *ctx, const float *d_x, int64_t rows, int64_t cols,
                                       int8_t *d_q, float *d_scales);
PG_API int32_t pg_quantize_activations_host(pg_ctx *ctx, const float *x, int64_t rows, int64_t cols,
                                            int8_t *q, float *scales);

/* ---- quant::quantize_weights (src/quant.rs:27-75) ----
 * w [K,N] f32 -> data_i8 [K,N], data_i8_t [N,K] (either may be NULL), scales [N]. */
PG_API int32_t pg_quantize_weights(pg_ctx *ctx, const float *d_w, int64_t rows, int64_t cols,
                                   int8_t *d_data_i8, int8_t *d_data_i8_t, float *d_scales);
PG_API int32_t pg_quantize_weights_host(pg_ctx *ctx, const float *w, int64_t rows, int64_t cols,
                                        int8_t *data_i8, int8_t *data_i8_t, float *scales);

/* ---- quant::dequantize (src/quant.rs:115-123) ---- */
PG_API int32_t pg_dequantize(pg_ctx *ctx, const int8_t *d_data_i8, const float *d_scales,
                             int64_t rows, int64_t cols, float *d_out);

/* ---- QuantizedTensor::to_gpu / from_gpu (src/quant.rs:172-191) ----
 * Uploads host data_i8_t [N,K] (required), data_i8 [K,N] (optional, may be NULL) and
 * scales [N].  Columns [col_begin, col_end) only are kept on this GPU (pass 0, cols for
 * the whole tensor): the column shard of one rank. */
PG_API int32_t pg_qtensor_upload(pg_ctx *ctx, const int8_t *data_i8, const int8_t *data_i8_t,
                                 const float *scales, int64_t rows, int64_t cols,
                                 int64_t col_begin, int64_t col_end, pg_qtensor **out);
/* Wraps device arrays the caller already holds (not owned, not copied). d_data_i8 may be NULL. */
PG_API int32_t pg_qtensor_wrap(pg_ctx *ctx, const int8_t *d_data_i8, const int8_t *d_data_i8_t,
                               const float *d_scales, int64_t rows, int64_t cols, pg_qtensor **out);
/* Quantises f32 weights [K,N] already on the device and keeps the result on the device. */
PG_API int32_t pg_qtensor_from_f32(pg_ctx *ctx, const float *d_w, int64_t rows, int64_t cols,
                                   int32_t keep_data_i8, pg_qtensor **out);
PG_API int32_t pg_qtensor_download(pg_ctx *ctx, const pg_qtensor *t, int8_t *data_i8, int8_t *data_i8_t,
                                   float *scales);
PG_API int32_t pg_qtensor_free(pg_ctx *ctx, pg_qtensor *t);
PG_API int64_t pg_qtensor_rows(const pg_qtensor *t);
PG_API int64_t pg_qtensor_cols(const pg_qtensor *t);
PG_API const int8_t *pg_qtensor_data_i8_t(const pg_qtensor *t);
PG_API const float *pg_qtensor_scales(const pg_qtensor *t);

/* ---- quant::matmul_quantized (src/quant.rs:129-169), Tensor::matmul_quantized
 *      (src/tensor.rs:1382-1408), quant::matmul_quantized_gpu (src/quant.rs:195-218) ----
 * y[M,N] = ((i32 sum_k q(x)[m,k] * w_t[n,k]) as f32 * a_scale[m]) * w_scale[n].
 * d_acc (nullable) receives the i32 sums [M,N]; d_a_i8 / d_a_scales (nullable) receive the
 * quantised activations.  Without them the context's own scratch holds the intermediates. */
PG_API int32_t pg_matmul_quantized(pg_ctx *ctx, const float *d_x, int64_t m, int64_t k,
                                   const pg_qtensor *w, float *d_y);
PG_API int32_t pg_matmul_quantized_ex(pg_ctx *ctx, const float *d_x, int64_t m, int64_t k,
                                      const pg_qtensor *w, float *d_y, int32_t *d_acc,
                                      int8_t *d_a_i8, float *d_a_scales, int32_t algo);
/* Host slices in, host result out: the exact shape of quant::matmul_quantized. Blocks.
 * Any host memory is accepted.  With page-locked, 16-byte aligned buffers of up to 1 MiB the kernels reach x and y
 * themselves (no copy engine), and a call that comes back with the same buffers, shape and weights is recorded the
 * second time it is seen and replayed as one graph of its launches from then on; the same bits on every route. */
PG_API int32_t pg_matmul_quantized_host(pg_ctx *ctx, const float *x, int64_t m, int64_t k,
                                        const pg_qtensor *w, float *y);

/* ---- quant::matmul_quantized_gpu (src/quant.rs:195-218) as the reference's GPU kernels compute it: matmul_dequant_i8 /
 *      matmul_dequant_simd_i8 (src/metal/shaders.rs:2329-2465, selector src/metal/context.rs:2226-2306) ----
 * y[M,N] = sum_k x[m,k] * (float(w_i8[k,n]) * w_scale[n]), f32 throughout: the activations are NOT quantised ("W8A32"),
 * unlike the CPU path above.  sequential != 0: one thread per output, ascending k with separately rounded multiply and
 * add (the order of the 16 x 16 kernel's loops; bit-exact against the CPU restatement); 0: the bandwidth-bound form
 * (one pass over data_i8_t per eight rows, f32 sums in another order).  Enqueued, not synchronised, like the Metal
 * dispatch (tests/quant_parity.rs:102-107). */
PG_API int32_t pg_matmul_dequant_w8a32(pg_ctx *ctx, const float *d_x, int64_t m, int64_t k, const pg_qtensor *w, float *d_y,
                                       int32_t sequential);

/* ---- the same product for callers that must not allocate (no counterpart in the reference) ----
 * For hosts that run inside a memory budget fixed before inference starts (a pre-sized arena per
 * model, a real-time loop in which cudaMalloc is forbidden): identical to pg_matmul_quantized, but
 * the quantised activations and their row scales live in an array built into the library image
 * (pg_static_scratch_bytes() bytes on every GPU that loads the library, held until the process
 * exits) instead of context scratch that grows with cudaMalloc.  The call allocates, frees and
 * resizes nothing.  Limit: M*K <= 262144 and M <= 256; larger shapes return PG_ERR_UNSUPPORTED.
 * The first call on each GPU looks up the array's device address: make that call before any
 * stream capture begins.  All calls on a GPU share the array (it keeps the previous call's bytes;
 * nothing here needs it zeroed), so calls that can overlap on the GPU race and must be ordered by
 * the caller. */
PG_API int32_t pg_matmul_quantized_static(pg_ctx *ctx, const float *d_x, int64_t m, int64_t k,
                                          const pg_qtensor *w, float *d_y);
PG_API int64_t pg_static_scratch_bytes(void);

/* ---- the integer GEMM alone: simd_kernels::gemm_i8_sdot (src/simd_kernels.rs:1087-1214),
 *      scalar form src/quant.rs:154-166 ---- */
PG_API int32_t pg_gemm_i8(pg_ctx *ctx, const int8_t *d_a_i8, const float *d_a_scales, int64_t m, int64_t k,
                          const pg_qtensor *w, float *d_y, int32_t *d_acc, int32_t algo);

/* ---- gguf::dequant_q8_0 / dequant_q4_0 / dequant_q4_1 / f16_to_f32
 *      (src/gguf.rs:286-302, 307-326, 331-351, 354-382) ----
 * raw block stream -> f32.  num_elements % 32 != 0 or a short buffer is PG_ERR_INVALID. */
PG_API int32_t pg_dequant_blocks(pg_ctx *ctx, int32_t type, const uint8_t *d_raw, size_t raw_len,
                                 int64_t num_elements, float *d_out);
PG_API int32_t pg_dequant_blocks_host(pg_ctx *ctx, int32_t type, const uint8_t *raw, size_t raw_len,
                                      int64_t num_elements, float *out);
PG_API int32_t pg_f16_to_f32(pg_ctx *ctx, const uint16_t *d_bits, int64_t count, float *d_out);

/* ---- the Llama linear on a GGUF weight: GgufFile::load_tensor_f32 (src/gguf.rs:485-517) +
 *      load_transposed_weight (src/models/llama/model.rs:243-257) + Tensor::matmul
 *      (src/tensor.rs:1342-1354), done without materialising the f32 weight ----
 * raw: [N rows][K/32 blocks] in GGUF [out,in] order; rows [row_begin,row_end) are kept
 * (0, n for all).  y[M,N] = x[M,K] . dequant(W)[N,K]^T in f32. */
PG_API int32_t pg_gguf_upload(pg_ctx *ctx, int32_t type, const uint8_t *raw, size_t raw_len,
                              int64_t n, int64_t k, int64_t row_begin, int64_t row_end,
                              pg_gguf_weight **out);
PG_API int32_t pg_gguf_free(pg_ctx *ctx, pg_gguf_weight *w);
PG_API int64_t pg_gguf_rows(const pg_gguf_weight *w);
PG_API int64_t pg_gguf_cols(const pg_gguf_weight *w);
PG_API int32_t pg_matmul_gguf(pg_ctx *ctx, const float *d_x, int64_t m, const pg_gguf_weight *w, float *d_y);
PG_API int32_t pg_matmul_gguf_host(pg_ctx *ctx, const float *x, int64_t m, const pg_gguf_weight *w, float *y);
/* gguf::load_tensor_q8_as_quantized (src/gguf.rs:386-401): Q8_0 blocks [rows,cols] ->
 * dequantise -> quantize_weights(rows, cols), all on the device. */
PG_API int32_t pg_qtensor_from_q8_0(pg_ctx *ctx, const uint8_t *raw, size_t raw_len, int64_t rows, int64_t cols,
                                    pg_qtensor **out);
/* serial::read_quantized_tensor (src/serial.rs:161-222) keeps data_i8 [rows, cols] and scales [cols] in the file and
   rebuilds data_i8_t on load: here the transposition runs on the device.  Host arrays in, resident tensor out. */
PG_API int32_t pg_qtensor_from_i8(pg_ctx *ctx, const int8_t *data_i8, const float *scales, int64_t rows, int64_t cols,
                                  pg_qtensor **out);

/* Huffman-coded int8 weights (src/huffman.rs).  One canonical code (256 bit lengths, the code book of
 * HuffmanTable::to_bytes / from_bytes, src/huffman.rs:287-307) shared by `num_streams` bitstreams that lie back to
 * back in `streams` (the layout of serial::write_huffman_tensor, src/serial.rs:320-365); stream s holds
 * stream_symbols[s] code words in stream_bytes[s] bytes.
 *   pg_huffman_decode_host   HuffmanTable::decode (src/huffman.rs:254-284) over every stream: host in, host out
 *                            (sum of stream_symbols bytes), the decode itself on the device.
 *   pg_qtensor_from_huffman  HuffmanTensor::decode_to_quantized + to_gpu (src/huffman.rs:374-437): the compressed
 *                            bytes are uploaded, decoded and transposed on the device; the tensor comes back resident,
 *                            ready for pg_matmul_quantized (what matmul_huffman does, src/huffman.rs:465-476).
 * The symbols must add up to rows * cols (the reference asserts it), else PG_ERR_INVALID. */
PG_API int32_t pg_huffman_decode_host(pg_ctx *ctx, const uint8_t *bit_lengths, int64_t num_streams, const uint64_t *stream_symbols,
                                      const uint64_t *stream_bytes, const uint8_t *streams, int8_t *out);
PG_API int32_t pg_qtensor_from_huffman(pg_ctx *ctx, const uint8_t *bit_lengths, int64_t num_streams, const uint64_t *stream_symbols,
                                       const uint64_t *stream_bytes, const uint8_t *streams, const float *scales, int64_t rows,
                                       int64_t cols, pg_qtensor **out);

/* ---- all-gather of output slices between the GPUs of one node; API precedent:
 *      Communicator::allgather (src/comm/communicator.rs:162-191, a CPU shared-memory ring) ----
 * One process per GPU.  Every rank creates an exchange (a result buffer of y_bytes plus control words,
 * shareable through CUDA IPC), the ranks swap the 64-byte handles by any means (the tests use
 * torch.distributed), and connect.  pg_exchange_allgather then stores this rank's slice
 * [M, n_local] into columns [col0, col0+n_local) of EVERY rank's [M, n_total] buffer with plain
 * stores over NVLink and waits, bounded (about a second; PG_ERR_DEVICE_TIMEOUT in the status word on
 * expiry), until all ranks have delivered theirs; pg_exchange_result is then the full matrix.  The
 * kernels count exchanges on the device, so the call can be recorded with pg_graph_begin/end.  An
 * exchange may be reused only after every rank has consumed its previous result (use one per
 * linear of a layer, or alternate two). */
PG_API int32_t pg_exchange_create(pg_ctx *ctx, int32_t rank, int32_t world, size_t y_bytes, void *handle_out,
                                  pg_exchange **out);
PG_API int32_t pg_exchange_connect(pg_ctx *ctx, pg_exchange *ex, const void *handles);
PG_API float *pg_exchange_result(const pg_exchange *ex);
PG_API int32_t pg_exchange_allgather(pg_ctx *ctx, pg_exchange *ex, const float *d_slice, int64_t m, int64_t n_local,
                                     int64_t n_total, int64_t col0);
/* The two halves of pg_exchange_allgather, for callers that have independent work to enqueue between
 * handing over their slice and needing everybody's: one wait per store, same order on every rank. */
PG_API int32_t pg_exchange_store(pg_ctx *ctx, pg_exchange *ex, const float *d_slice, int64_t m, int64_t n_local,
                                 int64_t n_total, int64_t col0);
PG_API int32_t pg_exchange_wait(pg_ctx *ctx, pg_exchange *ex);
PG_API int32_t pg_exchange_destroy(pg_ctx *ctx, pg_exchange *ex);
/* Ranks that live in ONE process (several contexts of one process, one per GPU, or a test that plays all ranks on one
 * GPU): `all` holds the `world` exchange objects in rank order; no IPC handle is opened. */
PG_API int32_t pg_exchange_connect_local(pg_ctx *ctx, pg_exchange *ex, pg_exchange *const *all);
/* The column-sharded integer GEMM with its all-gather inside: this rank's columns `w` ([K, n_local]) of the product
 * land in columns [col0, col0 + n_local) of EVERY rank's [M, n_total] exchange buffer, stored by the product kernel's
 * own epilogue (M <= 16, K % 64 == 0; plain stores over NVLink, all loads local).  Other shapes run pg_gemm_i8 into
 * d_slice_tmp ([M, n_local] floats, may be NULL for decode shapes) followed by a copy kernel.  Integer sums and the
 * per-column epilogue make the gathered matrix bit-identical to the unsharded product.  The exchange buffer holds
 * y_bytes / 4 values (pg_exchange_create). */
PG_API int32_t pg_gemm_i8_exchange(pg_ctx *ctx, const int8_t *d_a_i8, const float *d_a_scales, int64_t m, int64_t k,
                                   const pg_qtensor *w, pg_exchange *ex, int64_t n_total, int64_t col0, float *d_slice_tmp);
/* pg_matmul_quantized (f32 activations in) with the all-gather inside: quant::matmul_quantized (src/quant.rs:129-169) for a
 * weight sharded by output column: the activation quantiser (into the context's scratch), then pg_gemm_i8_exchange; the
 * gathered matrix is bit-identical to the unsharded call. */
PG_API int32_t pg_matmul_quantized_exchange(pg_ctx *ctx, const float *d_x, int64_t m, int64_t k, const pg_qtensor *w, pg_exchange *ex,
                                            int64_t n_total, int64_t col0, float *d_slice_tmp);
/* The slices travel as flagged cells (8 bytes per value: the value and the number of the exchange), which lets a
 * consumer poll the very cells it reads: no fence, no flag, no launch per exchange.  Consumers (enqueue them behind this
 * rank's own producer on the same exchange; their waits are bounded): pg_exchange_gather, which writes the gathered
 * [rows, cols] matrix as plain floats to d_out (NULL: to pg_exchange_result); the quantiser of src/quant.rs:97-109 over
 * the gathered matrix; pg_add_rmsnorm_quantize with the gathered matrix as the residual delta. */
PG_API int32_t pg_exchange_gather(pg_ctx *ctx, pg_exchange *ex, int64_t rows, int64_t cols, float *d_out);
/* the same for up to 16 exchanges in one launch (independent products whose results nothing consumes one by one);
 * rows[i] * cols[i] must be a multiple of four; d_outs or d_outs[i] NULL: that exchange's own result buffer */
PG_API int32_t pg_exchange_gather_many(pg_ctx *ctx, pg_exchange *const *exs, const int64_t *rows, const int64_t *cols,
                                       float *const *d_outs, int32_t count);
/* the producer of such an exchange for a slice that lies in plain device memory (any kernel's output) */
PG_API int32_t pg_exchange_store_cells(pg_ctx *ctx, pg_exchange *ex, const float *d_slice, int64_t m, int64_t n_local,
                                       int64_t n_total, int64_t col0);
PG_API int32_t pg_quantize_activations_exchange(pg_ctx *ctx, pg_exchange *ex, int64_t rows, int64_t cols, int8_t *d_q,
                                                float *d_scales);
PG_API int32_t pg_add_rmsnorm_quantize_exchange(pg_ctx *ctx, float *d_x, pg_exchange *ex_delta, const float *d_w, int64_t rows,
                                                int64_t dim, float eps, int8_t *d_q, float *d_scales, float *d_normed);

/* ---- the glue of one Llama decode step between the quantised linears (what the reference runs on the
 *      host in f32: src/models/llama/decoder.rs:69-155, src/models/llama/attention.rs:73-195,
 *      src/models/llama/model.rs:223-237).  Rows are independent sequences; the position is read from
 *      device memory so that a step can be recorded once and replayed. ----
 * residual add + RMSNorm (src/nn.rs:577-652) + per-row int8 quantiser (src/quant.rs:97-109), fused */
PG_API int32_t pg_add_rmsnorm_quantize(pg_ctx *ctx, float *d_x, const float *d_delta, const float *d_w, int64_t rows,
                                       int64_t dim, float eps, int8_t *d_q, float *d_scales, float *d_normed);
/* silu(gate) * up (src/models/llama/decoder.rs:143-150) on the fused [gate | up] output + quantiser */
PG_API int32_t pg_swiglu_quantize(pg_ctx *ctx, const float *d_gate_up, int64_t rows, int64_t F, int8_t *d_q,
                                  float *d_scales, float *d_act);
/* RoPE (src/nn.rs:1322-1338) on q and k, append of k and v to the f32 KV cache (src/attention.rs:65-83) */
PG_API int32_t pg_rope_kv_append(pg_ctx *ctx, const float *d_qkv, const int32_t *d_pos, const float *d_cos,
                                 const float *d_sin, int64_t B, int64_t Hq, int64_t Hkv, int64_t hd, int64_t cap,
                                 float *d_q_rot, float *d_kcache, float *d_vcache);
/* GQA attention of one new token per sequence (src/attention.rs:141-265), head_dim 128 */
/* slices of the context per (sequence, KV head); the work buffer of pg_gqa_attention_decode holds B * Hq * S * 130 floats */
PG_API int32_t pg_gqa_decode_splits(pg_ctx *ctx, int64_t B, int64_t Hq, int64_t Hkv, int64_t cap);
PG_API int32_t pg_gqa_attention_decode(pg_ctx *ctx, const float *d_q_rot, const float *d_kcache, const float *d_vcache,
                                       const int32_t *d_pos, int64_t B, int64_t Hq, int64_t Hkv, int64_t hd, int64_t cap,
                                       float *d_work, float *d_out /* [B, Hq*hd] f32, nullable when the int8 form is taken */,
                                       int8_t *d_out_i8 /* nullable: the same rows through the activation quantiser */,
                                       float *d_out_scales /* [B], with d_out_i8 */);
/* pg_rope_kv_append + pg_gqa_attention_decode in one launch (4 or 8 query heads per KV head): d_qkv is the raw
   [B, (Hq + 2 Hkv) * hd] output of the fused Q|K|V projection; the newest token's rotated key and its value are written
   at position *d_pos of the caches */
PG_API int32_t pg_gqa_attention_decode_fused(pg_ctx *ctx, const float *d_qkv, const int32_t *d_pos, const float *d_cos,
                                             const float *d_sin, float *d_kcache, float *d_vcache, int64_t B, int64_t Hq,
                                             int64_t Hkv, int64_t hd, int64_t cap, float *d_work, float *d_out,
                                             int8_t *d_out_i8, float *d_out_scales);
/* embedding gather (src/nn.rs:217-227); greedy argmax, first maximum (examples/llama/main.rs:15-26).  *d_pos is
   advanced by one but never beyond pos_limit (pass the KV capacity; 0 = no limit).  The kernels that read *d_pos
   (pg_rope_kv_append, the attention entry points) touch neither the caches nor the rotation tables when it lies outside
   [0, cap): they record PG_ERR_INVALID in the context's status word (pg_ctx_device_status) instead. */
PG_API int32_t pg_embedding(pg_ctx *ctx, const float *d_table, const int32_t *d_tokens, int64_t B, int64_t dim,
                            float *d_out);
PG_API int32_t pg_argmax_advance(pg_ctx *ctx, const float *d_logits, int64_t B, int64_t V, int32_t *d_tokens,
                                 int32_t *d_pos, int64_t pos_limit);
/* ---- the same step with every linear sharded by output column over the ranks of a node (one process per GPU):
 *      whole KV heads with their query heads per rank (fuse_qkv's column order, src/models/llama/attention.rs:51-71,
 *      regrouped per rank), the same channel range of gate and up per rank (src/models/llama/decoder.rs:49-67), the
 *      vocabulary by column range.  Four exchanges per layer (attention rows, O, SwiGLU rows, down), each stored by the
 *      kernel that produces the slice and awaited by the kernel that consumes the rows. ----
 * attention on this rank's heads (see pg_gqa_attention_decode_fused); merged f32 rows -> columns [col0, col0 + Hq*hd)
 * of every rank's [B, n_total] buffer.  splits: context slices per (sequence, KV head); the unsharded shape's
 * pg_gqa_decode_splits value reproduces the single-GPU sums bit for bit, 0 = this rank's own choice. */
PG_API int32_t pg_gqa_attention_decode_fused_exchange(pg_ctx *ctx, const float *d_qkv, const int32_t *d_pos, const float *d_cos,
                                                      const float *d_sin, float *d_kcache, float *d_vcache, int64_t B,
                                                      int64_t Hq, int64_t Hkv, int64_t hd, int64_t cap, float *d_work,
                                                      int32_t splits, pg_exchange *ex, int64_t n_total, int64_t col0);
/* silu(gate) * up on this rank's [rows, 2 F_local] = [gate columns | up columns]; f32 rows -> columns
 * [col0, col0 + F_local) of every rank's [rows, F_total] buffer */
PG_API int32_t pg_swiglu_exchange(pg_ctx *ctx, const float *d_gate_up_local, int64_t rows, int64_t F_local, pg_exchange *ex,
                                  int64_t F_total, int64_t col0);
/* greedy choice over a vocabulary sharded by column: this rank's (maximum, index) pair per sequence goes to every
 * rank (exchange buffer of B * world * 8 bytes); pg_pick_embed waits, takes the first maximum, advances *d_pos and
 * gathers the chosen tokens' embedding rows (d_table nullable) */
PG_API int32_t pg_argmax_exchange(pg_ctx *ctx, const float *d_logits_local, int64_t B, int64_t V_local, int64_t v0,
                                  pg_exchange *ex);
PG_API int32_t pg_pick_embed(pg_ctx *ctx, pg_exchange *ex, int64_t B, int32_t *d_tokens, int32_t *d_pos, int64_t pos_limit,
                             const float *d_table, int64_t dim, float *d_out);

/* ---- Tensor::matmul, naive branch (src/tensor.rs:1342-1354): [M,K] x [K,N] f32,
 *      ascending-p accumulation with separately rounded multiply and add ---- */
PG_API int32_t pg_matmul_f32(pg_ctx *ctx, const float *d_a, const float *d_b, int64_t m, int64_t k, int64_t n,
                             float *d_out);

#ifdef __cplusplus
}
#endif
#endif /* PEREGRINE_B200_H */
