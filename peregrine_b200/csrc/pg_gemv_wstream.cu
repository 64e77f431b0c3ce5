// Decode-size W8A8 product for M <= 16: the integer GEMM of src/quant.rs:154-166 /
// simd_kernels::gemm_i8_sdot (src/simd_kernels.rs:1087-1214), built so that the only traffic that
// matters is one pass over data_i8_t [N,K].
//
//   * One persistent CTA of 16 warps per SM.  The quantised activations [M,K] are copied into
//     shared memory ONCE per CTA, so they cost #SMs x M x K bytes of L2 reads per call instead of
//     one copy per 16 output columns.
//   * An output tile is 8 columns (8 rows of data_i8_t).  `kw` warps (1, 2, 4, 8 or 16) share a
//     tile, each taking one contiguous part of K; kw > 1 is chosen when N alone gives fewer tiles
//     than the GPU has warps, so that a small matrix is requested from HBM in one go.
//   * A warp streams its 8 row segments through a private two-slot ring in shared memory with
//     bulk asynchronous copies (cp.async.bulk, one row segment per lane 0..7, completion on an
//     mbarrier).  There is no block-wide barrier after start-up; the tile's sums live in the
//     warp's MMA accumulators.  With kw > 1 the partial sums meet in shared memory (integer adds:
//     exact in any order) behind a named barrier of just those kw warps, in the padding of the
//     ring rows, double-buffered by tile parity.
//   * The dot products run on the warp-level int8 MMA m16n8k32 with the same K permutation as the
//     other streaming kernel: a lane's 16 contiguous K bytes of a weight row and of an activation
//     row feed two MMAs directly.
//   * Rows of both shared-memory tiles are padded so that the stride is 64 mod 128 bytes: the
//     128-bit fragment loads are then free of bank conflicts.
//
// Weights never depend on the preceding kernel, so the first ring slots are requested before
// griddepcontrol.wait.  Every mbarrier wait is bounded (about a second): on expiry the kernel
// records PG_ERR_DEVICE_TIMEOUT in the context's status word, stops computing and leaves through
// the remaining named barriers.
#include <algorithm>

#include "pg_internal.cuh"

namespace {

constexpr int WS_WARPS = 16;
constexpr int WS_THREADS = WS_WARPS * 32;
constexpr int WS_SLOTS = 2;
constexpr int WS_SMEM_MAX = 227 * 1024;

// SEG: bytes of one weight row per ring slot.  512 keeps 128 KB in flight per SM; 256 leaves room
// for activations of up to 146 KB.
template <int SEG>
struct WsCfg {
    static constexpr int SEG_STRIDE = SEG + 64;               // 64 mod 128
    static constexpr int SLOT_BYTES = 8 * SEG_STRIDE;
    static constexpr int RING_BYTES = WS_WARPS * WS_SLOTS * SLOT_BYTES;
    static constexpr int BAR_BYTES = (WS_WARPS * WS_SLOTS + 1) * 8 + 8;
    static constexpr int A_MAX = (WS_SMEM_MAX - RING_BYTES - BAR_BYTES) & ~127;
};

__device__ __forceinline__ unsigned long long ws_globaltimer()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void ws_mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void ws_mbar_expect(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool ws_mbar_try(uint32_t bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}
__device__ __forceinline__ bool ws_mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int32_t *status,
                                             unsigned long long limit_ns)
{
    unsigned long long t0 = 0;
    for (uint32_t it = 1;; ++it) {
        if (ws_mbar_try(bar, parity)) return true;
        if ((it & 0xff) == 0) {
            if (*abort_flag) return false;
            const unsigned long long now = ws_globaltimer();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > limit_ns) {
                *abort_flag = 1;
                atomicExch(status, (int32_t)PG_ERR_DEVICE_TIMEOUT);
                return false;
            }
        }
    }
}
__device__ __forceinline__ void ws_bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ uint4 ws_lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void ws_mma(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t ws_mapa(uint32_t local_addr, uint32_t cta)
{
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(cta));
    return remote;
}

// HI: activation rows 8..15 exist (M > 8).
// CL: the activations do not fit beside the rings of one CTA.  The kernel then runs as clusters of cs = 2 or 4 CTAs
// that work on the SAME tiles: CTA c of a cluster holds columns [c * KH, (c + 1) * KH) of the activations and streams
// that part of K of every tile.  Per round of tiles the other CTAs add their sums into cells in the first CTA's shared
// memory (red.shared::cluster, 512 bytes per tile, two sets used by round parity), one cluster barrier, and the first
// CTA finishes the tiles and clears the cells it read.
// Warp w: tile slot w / kw, K part w % kw (KW bytes each) of the CTA's K range.
// CTA b (unit u = b / cs; U = number of clusters or CTAs): tiles  u + U * (slot + (16 / kw) * j).
// Shared memory: activations (a_bytes, row stride a_stride) | rings | mbarriers | CL: exchange cells [2][16 / kw][512 B].
// PEER: the kernel is one rank's part of a column-sharded product.  Its outputs go straight into every rank's [M, ld]
// buffer of flagged cells (pg_internal.cuh: 8 bytes per value, the value with the number of the exchange, plain stores
// to peer pointers over NVLink, columns col0 + n): no separate all-gather launch, no fence, and the consumers need no
// flag beyond the cells themselves.  Only stores cross NVLink; every load, bulk copies included, reads this GPU's own
// memory.
template <bool HI, int SEG, bool CL, bool PEER>
__global__ void __launch_bounds__(WS_THREADS, 1)
    gemv_wstream_kernel(const int8_t *__restrict__ a, const float *__restrict__ a_scales, int M, int K, const int8_t *__restrict__ bt,
                        const float *__restrict__ w_scales, int64_t N, float *__restrict__ y, int32_t *__restrict__ acc_out, int kw,
                        int KW, int a_stride, int a_bytes, int KH, int32_t *status, unsigned long long limit_ns, const PgPeerOut po)
{
    using C = WsCfg<SEG>;
    extern __shared__ __align__(128) unsigned char smem[];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = lane >> 2, t = lane & 3;
    const uint32_t a_base = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t ring0 = a_base + (uint32_t)a_bytes;
    const uint32_t fifo = ring0 + (uint32_t)warp * (WS_SLOTS * C::SLOT_BYTES);
    const uint32_t bars = ring0 + C::RING_BYTES;
    const uint32_t my_bar = bars + (uint32_t)warp * (WS_SLOTS * 8);
    const uint32_t a_bar = bars + WS_WARPS * WS_SLOTS * 8;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + a_bytes + C::RING_BYTES + (WS_WARPS * WS_SLOTS + 1) * 8);

    if (threadIdx.x == 0) {
        for (int i = 0; i < WS_WARPS * WS_SLOTS + 1; i++) ws_mbar_init(bars + 8 * i, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    uint32_t my_rank = 0, cs = 1;
    if (CL) {
        asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(my_rank));
        asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(cs));
    }
    const int ka0 = CL ? (int)my_rank * KH : 0;             // the K range of this CTA: [ka0, ka0 + kalen)
    const int kalen = CL ? max(0, min(KH, K - ka0)) : K;
    const int groups = WS_WARPS / kw, slot_idx = warp / kw, kpart = warp - slot_idx * kw;
    const int k0 = ka0 + kpart * KW;
    const int klen = max(0, min(KW, ka0 + kalen - k0));     // > 0 without CL; a part of the last, shorter range may be empty
    const int nsub = (klen + SEG - 1) / SEG;
    const int64_t tiles = (N + 7) >> 3;
    const int64_t unit = blockIdx.x / cs, units = gridDim.x / cs;
    const int64_t first = unit + units * slot_idx, tstep = units * groups;
    const int my_tiles = first < tiles ? (int)((tiles - first + tstep - 1) / tstep) : 0;
    const int rounds = unit < tiles ? (int)((tiles - unit + tstep - 1) / tstep) : 0;   // of the CTA: those of its slot 0
    const int total = my_tiles * nsub;                      // ring fills of this warp
    const uint32_t xcell = bars + C::BAR_BYTES;             // CL: [2][groups][512 B], used in the first CTA of the cluster

    // ring fill q: tile j = q / nsub, K segment sc = q % nsub
    auto issue = [&](int q) {
        const int j = q / nsub, sc = q - j * nsub;
        const uint32_t bytes = (uint32_t)min(SEG, klen - sc * SEG);
        const uint32_t bar = my_bar + (uint32_t)(q % WS_SLOTS) * 8;
        if (lane == 0) ws_mbar_expect(bar, 8 * bytes);
        __syncwarp();
        if (lane < 8) {
            int64_t n = (first + (int64_t)j * tstep) * 8 + lane;
            if (n >= N) n = N - 1;                          // rows past the edge repeat the last one; their sums are dropped
            ws_bulk_load(fifo + (uint32_t)(q % WS_SLOTS) * C::SLOT_BYTES + (uint32_t)lane * C::SEG_STRIDE,
                         bt + n * (int64_t)K + k0 + sc * SEG, bytes, bar);
        }
    };
#pragma unroll
    for (int q = 0; q < WS_SLOTS; q++)
        if (q < total) issue(q);

    // the activations come from the preceding kernel
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x == 0) ws_mbar_expect(a_bar, (uint32_t)M * (uint32_t)kalen);
    __syncthreads();
    if ((int)threadIdx.x < M)
        ws_bulk_load(a_base + threadIdx.x * (uint32_t)a_stride, a + (int64_t)threadIdx.x * K + ka0, (uint32_t)kalen, a_bar);
    bool ok = ws_mbar_wait(a_bar, 0, abort_flag, status, limit_ns);   // also keeps the shared memory alive until the copy has landed
    if (CL) {
        // the cells start from zero, and nobody adds into them before that
        if (my_rank == 0)
            for (int i = threadIdx.x; i < 2 * groups * 128; i += WS_THREADS) asm volatile("st.shared.u32 [%0], %1;" ::"r"(xcell + i * 4), "r"(0) : "memory");
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    }

    // rows past M read row 0 (their sums are dropped): nothing outside the loaded region is touched
    const uint32_t a_lo = a_base + (uint32_t)(r < M ? r : 0) * a_stride + (k0 - ka0) + t * 16;
    const uint32_t a_hi = a_base + (uint32_t)(r + 8 < M ? r + 8 : 0) * a_stride + (k0 - ka0) + t * 16;
    const uint32_t w_off = (uint32_t)r * C::SEG_STRIDE + t * 16;
    const uint32_t pad_off = (uint32_t)r * C::SEG_STRIDE + SEG + t * 16;   // this lane's 16 bytes of row padding
    // scales of the two activation rows this lane's accumulators belong to (written by the preceding kernel: one L2
    // load each, here, instead of one per output)
    const float as_lo = (r < M) ? pg_ld_fresh(a_scales + r) : 0.0f;
    const float as_hi = (HI && r + 8 < M) ? pg_ld_fresh(a_scales + r + 8) : 0.0f;
    const uint32_t peer_seq = PEER ? pg_cell_seq(po) : 0u;   // after griddepcontrol.wait
    int acc[4] = {0, 0, 0, 0};
    int q = 0;
    // Rounds of the CTA: in round j a warp streams its part of its j-th tile, if it has one.  Warps without a tile in
    // the last round still meet the others at the cluster's barrier.
    for (int j = 0; j < (CL ? rounds : my_tiles); j++) {
        if (j < my_tiles) {
            for (int sc = 0; sc < nsub; sc++, q++) {
                const uint32_t slot = fifo + (uint32_t)(q % WS_SLOTS) * C::SLOT_BYTES;
                ok = ok && ws_mbar_wait(my_bar + (uint32_t)(q % WS_SLOTS) * 8, (uint32_t)(q / WS_SLOTS) & 1u, abort_flag, status, limit_ns);
                if (ok) {
                    const int steps = min(SEG, klen - sc * SEG) >> 6;
                    const uint32_t ak = (uint32_t)sc * SEG;
#pragma unroll
                    for (int s = 0; s < SEG / 64; s++) {
                        if (s < steps) {
                            const uint4 w = ws_lds128(slot + w_off + s * 64);
                            const uint4 xl = ws_lds128(a_lo + ak + s * 64);
                            uint4 xh = make_uint4(0u, 0u, 0u, 0u);
                            if (HI) xh = ws_lds128(a_hi + ak + s * 64);
                            ws_mma(acc, xl.x, xh.x, xl.y, xh.y, w.x, w.y);
                            ws_mma(acc, xl.z, xh.z, xl.w, xh.w, w.z, w.w);
                        }
                    }
                    __syncwarp();                           // every lane has read the slot
                    if (q + WS_SLOTS < total) issue(q + WS_SLOTS);
                }
            }
            // tile finished for this warp's part of K: the kw warps of the slot add up in the first one
            if (kw > 1) {
                const uint32_t buf = (uint32_t)(j & 1) * C::SLOT_BYTES + pad_off;
                if (kpart != 0)
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(fifo + buf), "r"(acc[0]), "r"(acc[1]), "r"(acc[2]), "r"(acc[3])
                                 : "memory");
                asm volatile("bar.sync %0, %1;" ::"r"(1 + slot_idx), "r"(kw * 32) : "memory");
                if (kpart == 0) {
                    for (int p = 1; p < kw; p++) {
                        const uint4 v = ws_lds128(fifo + (uint32_t)p * (WS_SLOTS * C::SLOT_BYTES) + buf);
                        acc[0] += (int)v.x;
                        acc[1] += (int)v.y;
                        acc[2] += (int)v.z;
                        acc[3] += (int)v.w;
                    }
                }
            }
        }
        if (CL) {
            // the other CTAs' sums of this round are added into the first CTA's cells
            const uint32_t cell = xcell + ((uint32_t)(j & 1) * groups + slot_idx) * 512 + lane * 16;
            if (my_rank != 0 && kpart == 0 && j < my_tiles) {
                const uint32_t remote = ws_mapa(cell, 0);
#pragma unroll
                for (int c = 0; c < 4; c++) asm volatile("red.shared::cluster.add.s32 [%0], %1;" ::"r"(remote + 4 * c), "r"(acc[c]) : "memory");
            }
            asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
            if (my_rank == 0 && kpart == 0 && j < my_tiles) {
                const uint4 v = ws_lds128(cell);
                acc[0] += (int)v.x;
                acc[1] += (int)v.y;
                acc[2] += (int)v.z;
                acc[3] += (int)v.w;
                // this set is added into again two rounds on, behind the next round's barrier
                asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(cell), "r"(0) : "memory");
            }
        }
        if (j < my_tiles && kpart == 0 && ok && (!CL || my_rank == 0)) {
            // C fragment: acc[0], acc[1] -> (row r, cols 2t, 2t+1); acc[2], acc[3] -> row r + 8
            const int64_t n = (first + (int64_t)j * tstep) * 8 + 2 * t;
#pragma unroll
            for (int h = 0; h < (HI ? 2 : 1); h++) {
                const int m = r + 8 * h;
                if (m < M) {
                    if (PEER) {
                        // two adjacent columns per lane: one 16-byte store of two cells per rank where the pair exists and is aligned
                        const float as = h ? as_hi : as_lo;
                        const float v0 = (n < N) ? __fmul_rn(__fmul_rn(__int2float_rn(acc[2 * h]), as), __ldg(w_scales + n)) : 0.0f;
                        const float v1 = (n + 1 < N) ? __fmul_rn(__fmul_rn(__int2float_rn(acc[2 * h + 1]), as), __ldg(w_scales + n + 1)) : 0.0f;
                        if (n + 1 < N && ((po.ld | po.col0) & 1) == 0) {
                            pg_cell_store2(po, peer_seq, m, n, v0, v1);
                        } else {
                            if (n < N) pg_cell_store(po, peer_seq, m, n, v0);
                            if (n + 1 < N) pg_cell_store(po, peer_seq, m, n + 1, v1);
                        }
                    } else {
#pragma unroll
                        for (int c = 0; c < 2; c++) {
                            if (n + c < N) {
                                const int32_t sum = acc[2 * h + c];
                                if (acc_out) acc_out[(int64_t)m * N + n + c] = sum;
                                if (y) y[(int64_t)m * N + n + c] = __fmul_rn(__fmul_rn(__int2float_rn(sum), h ? as_hi : as_lo), __ldg(w_scales + n + c));
                            }
                        }
                    }
                }
            }
        }
        acc[0] = acc[1] = acc[2] = acc[3] = 0;
    }
    if (PEER) pg_cell_finish(po, peer_seq, threadIdx.x);
}

int g_force_kw = 0;    // tuning override, 0 = heuristic
int g_force_cs = 0;    // 0 = heuristic, else the cluster size (1, 2, 4) over which K is split

template <bool HI, int SEG, bool CL, bool PEER>
int32_t ws_launch(pg_ctx *ctx, const int8_t *d_a, const float *d_as, int M, int K, const int8_t *d_bt, const float *d_ws, int64_t n,
                  float *d_y, int32_t *d_acc, int kw, int KW, int a_stride, int a_bytes, int KH, int grid, int cs, const PgPeerOut &po)
{
    using C = WsCfg<SEG>;
    auto kern = gemv_wstream_kernel<HI, SEG, CL, PEER>;
    const int smem = a_bytes + C::RING_BYTES + C::BAR_BYTES + (CL ? 2 * (WS_WARPS / kw) * 512 : 0);
    static std::atomic<uint64_t> smem_set{0};
    PG_CUDA(pg_max_smem_once(kern, WS_SMEM_MAX, ctx->device, smem_set));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(WS_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = (unsigned)cs;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = CL ? 2 : 1;
    PG_CUDA(cudaLaunchKernelEx(&cfg, kern, d_a, d_as, M, K, d_bt, d_ws, n, d_y, d_acc, kw, KW, a_stride, a_bytes, KH, ctx->d_status,
                               ctx->wait_limit_ns, po));
    PG_LAUNCHED();
    return PG_OK;
}

inline int ws_a_stride(int64_t k) { return (int)(((k + 127) & ~(int64_t)127) + 64); }
// K range of one CTA of a cluster of cs, a whole number of 512-byte ring segments
inline int64_t ws_range(int64_t k, int cs) { return (((k + cs - 1) / cs) + 511) & ~(int64_t)511; }

}  // namespace

extern "C" PG_API void pg_tune_wstream_kw(int kw) { g_force_kw = kw; }
extern "C" PG_API void pg_tune_wstream_cluster(int cs) { g_force_cs = cs; }

constexpr int WS_CELL_BYTES = 2 * WS_WARPS * 512;   // most the exchange cells of a cluster can take

// smallest cluster (1, 2, 4) whose per-CTA share of the activations fits beside a ring of SEG-byte segments; 0 = none
template <int SEG>
int ws_cluster_for(int64_t m, int64_t k)
{
    if (m * ws_a_stride(k) <= WsCfg<SEG>::A_MAX) return 1;
    for (int cs = 2; cs <= 4; cs *= 2)
        if ((cs - 1) * ws_range(k, cs) < k && m * ws_a_stride(ws_range(k, cs)) <= WsCfg<SEG>::A_MAX - WS_CELL_BYTES) return cs;
    return 0;
}

bool pgk_gemm_i8_wstream_supports(int64_t m, int64_t k, int64_t n)
{
    if (!(m >= 1 && m <= 16 && n >= 1 && k >= 64 && (k % 64 == 0) && k <= (1 << 20))) return false;
    return ws_cluster_for<512>(m, k) != 0 || ws_cluster_for<256>(m, k) != 0;
}

static int32_t ws_dispatch(pg_ctx *ctx, const int8_t *d_a, const float *d_as, int64_t m, int64_t k, const int8_t *d_bt,
                           const float *d_ws, int64_t n, float *d_y, int32_t *d_acc, const PgPeerOut *peer)
{
    if (!pgk_gemm_i8_wstream_supports(m, k, n) || ((uintptr_t)d_a & 15) || ((uintptr_t)d_bt & 15))
        PG_FAIL(PG_ERR_UNSUPPORTED,
                "gemm_i8 warp-stream kernel needs 1<=M<=16, K%%64==0, M*K within shared memory and 16-byte aligned operands (M=%lld K=%lld)",
                (long long)m, (long long)k);
    const int M = (int)m, K = (int)k;
    const bool hi = M > 8;
    const int sms = ctx->sm_count;
    const int64_t tiles = (n + 7) / 8;
    // K is split over a cluster when that is what it takes to keep the deep ring (512-byte segments) beside the activations
    int cs = ws_cluster_for<512>(m, k);
    if (cs == 0) cs = ws_cluster_for<256>(m, k);
    if (g_force_cs) cs = g_force_cs;
    PG_REQUIRE(cs == 1 || cs == 2 || cs == 4, "gemm_i8 warp-stream: cluster size must be 1, 2 or 4");
    const int KH = cs > 1 ? (int)ws_range(K, cs) : K;       // K range of one CTA
    PG_REQUIRE(cs == 1 || (int64_t)(cs - 1) * KH < K, "gemm_i8 warp-stream: K too short for a cluster of %d", cs);
    const int64_t units = sms / cs;                         // CTAs or clusters that take tiles
    // more warps per tile while every (tile, K part) still finds a warp of its own: the whole matrix is then requested at once
    int kw = 1;
    while (kw < WS_WARPS && KH / (kw * 2) >= 512 && tiles * (kw * 2) <= units * WS_WARPS) kw *= 2;
    auto part_bytes = [&](int parts) { return (((KH + parts - 1) / parts) + 63) & ~63; };
    while (kw > 1 && (int64_t)(kw - 1) * part_bytes(kw) >= KH) kw /= 2;   // rounding to k-steps must leave no part of a full range empty
    if (g_force_kw) kw = g_force_kw;
    PG_REQUIRE(kw == 1 || kw == 2 || kw == 4 || kw == 8 || kw == 16, "gemm_i8 warp-stream: kw must be a power of two <= 16");
    const int KW = part_bytes(kw);
    PG_REQUIRE((int64_t)(kw - 1) * KW < KH, "gemm_i8 warp-stream: K too short for %d parts", kw);
    const int groups = WS_WARPS / kw;
    // CTAs with every warp busy, the rest of the SMs idle: spreading 1792 tiles as 12 or 13 per CTA over all 148 SMs instead of 16 over
    // 112 was measured slower (127.5 against 113.9 us for the nine-case decode sweep)
    const int grid = (int)std::min<int64_t>(units, (tiles + groups - 1) / groups) * cs;
    const int a_stride = ws_a_stride(KH);
    const int a_bytes = (M * a_stride + 127) & ~127;
    const int cells = cs > 1 ? 2 * groups * 512 : 0;
    const bool big_ring = a_bytes + cells <= WsCfg<512>::A_MAX;
    PG_REQUIRE(a_bytes + cells <= WsCfg<256>::A_MAX, "gemm_i8 warp-stream: activations do not fit in shared memory");
    static const PgPeerOut no_peer = {};
#define PG_WS_CASE(HI, SEG, CL)                                                                                                      \
    return peer ? ws_launch<HI, SEG, CL, true>(ctx, d_a, d_as, M, K, d_bt, d_ws, n, d_y, d_acc, kw, KW, a_stride, a_bytes, KH, grid, \
                                               cs, *peer)                                                                            \
                : ws_launch<HI, SEG, CL, false>(ctx, d_a, d_as, M, K, d_bt, d_ws, n, d_y, d_acc, kw, KW, a_stride, a_bytes, KH,      \
                                                grid, cs, no_peer)
    if (cs > 1) {
        if (hi) {
            if (big_ring) PG_WS_CASE(true, 512, true);
            PG_WS_CASE(true, 256, true);
        }
        if (big_ring) PG_WS_CASE(false, 512, true);
        PG_WS_CASE(false, 256, true);
    }
    if (hi) {
        if (big_ring) PG_WS_CASE(true, 512, false);
        PG_WS_CASE(true, 256, false);
    }
    if (big_ring) PG_WS_CASE(false, 512, false);
    PG_WS_CASE(false, 256, false);
#undef PG_WS_CASE
}

int32_t pgk_gemm_i8_wstream(pg_ctx *ctx, const int8_t *d_a, const float *d_as, int64_t m, int64_t k, const int8_t *d_bt,
                            const float *d_ws, int64_t n, float *d_y, int32_t *d_acc)
{
    return ws_dispatch(ctx, d_a, d_as, m, k, d_bt, d_ws, n, d_y, d_acc, nullptr);
}

int32_t pgk_gemm_i8_wstream_peer(pg_ctx *ctx, const int8_t *d_a, const float *d_as, int64_t m, int64_t k, const int8_t *d_bt,
                                 const float *d_ws, int64_t n, const PgPeerOut &out)
{
    return ws_dispatch(ctx, d_a, d_as, m, k, d_bt, d_ws, n, nullptr, nullptr, &out);
}
