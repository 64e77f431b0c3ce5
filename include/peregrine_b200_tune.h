/*
 * peregrine_b200 -- tuning and diagnostic knobs of the library (NOT part of the path's API).
 *
 * These switches force a kernel variant or a blocking factor that the library otherwise chooses by itself.  They
 * exist so that tests can drive every variant through the same entry points and so that a profiling run can
 * compare variants; a host binding does not need them.
 *
 * Thread safety: every knob is one plain process-wide variable, read without synchronisation by the launch
 * functions of EVERY context.  Set a knob only while no other thread is inside the library, and put it back to its
 * default (0, or negative where stated) afterwards.  Results never depend on a knob -- every variant is bit-exact
 * against the same oracle -- only speed and the choice of kernel do.
 */
#ifndef PEREGRINE_B200_TUNE_H
#define PEREGRINE_B200_TUNE_H

#include "peregrine_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* per-lane streaming product (PG_ALGO_STREAM): column groups per CTA, FIFO depth, shared-memory carve-out in
 * percent (-1 = the driver's choice), K split over a cluster; 0 = the library's choice */
PG_API void pg_tune_stream_ng(int ng);
PG_API void pg_tune_stream_depth(int depth);
PG_API void pg_tune_stream_carveout(int pct);
PG_API void pg_tune_stream_split(int split);
/* warp-stream decode product (PG_ALGO_WSTREAM): warps that share a tile's K range (1, 2, 4, 8, 16) and the cluster
 * size over which K is split (1, 2, 4); 0 = the library's choice */
PG_API void pg_tune_wstream_kw(int kw);
PG_API void pg_tune_wstream_cluster(int cs);
/* tcgen05 product: tile width in columns (32, 64, 128, 256; 0 = choice); CTA pairs: 0 = choice, 1 = never, 2 = always */
PG_API void pg_tune_tcgen05_bn(int bn);
PG_API void pg_tune_tcgen05_pair(int mode);
/* tcgen05 kernel at M <= 128: parts of K per tile; 0 heuristic, 1 never split, 2 / 4 / 8 that many */
PG_API void pg_tune_tcgen05_split(int mode);
/* GGUF weights uploaded while this is 1 keep the plain block planes and take the CUDA-core product kernel (otherwise
 * Q4_0 / Q8_0 weights with K % 256 == 0 are laid out for, and served by, the streaming tensor-core kernel) */
PG_API void pg_tune_gguf_simple(int on);
/* pg_matmul_quantized_host with page-locked buffers: up to how many bytes the quantiser reads x itself / the product
 * writes y itself / a copy kernel pushes y (0 = path off, negative = default) */
PG_API void pg_tune_host_direct(int x_bytes, int y_bytes);
PG_API void pg_tune_host_push(int y_bytes);
/* pg_matmul_quantized_host: replay a repeated call (same page-locked buffers, shape, weights) from a graph of its own
 * launches; 1 (default) / 0 */
PG_API void pg_tune_host_graph(int on);
/* diagnostic: one rank of a sharded step without its peers (stores stay local, no cell is waited for; results are
 * meaningless, the time is one rank's kernels and launches alone) */
PG_API void pg_tune_exchange_solo(int on);
/* diagnostic: sweeps over the subsequence starts that the last Huffman decode of this process took */
PG_API int pg_huffman_last_sweeps(void);

#ifdef __cplusplus
}
#endif
#endif /* PEREGRINE_B200_TUNE_H */
