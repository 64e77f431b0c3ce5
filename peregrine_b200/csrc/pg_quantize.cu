// Quantisers of the int8 path.
//
//   quantize_rows_kernel     quant::quantize_activations, scalar branch (src/quant.rs:97-109)
//   col_absmax_kernel +
//   quantize_cols_kernel     quant::quantize_weights (src/quant.rs:27-75)
//   dequantize_kernel        quant::dequantize (src/quant.rs:115-123)
//   matmul_f32_kernel        Tensor::matmul naive branch (src/tensor.rs:1342-1354)
//
// All float steps use the explicitly rounded intrinsics (__fdiv_rn, __fmul_rn, __fadd_rn)
// so that no FMA contraction or approximate division can change a bit; denormals are kept
// (the library is built without -use_fast_math / -ftz).
#include "pg_internal.cuh"

namespace {

constexpr int QR_THREADS = 256;

__device__ __forceinline__ float block_max(float v, float *smem)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float r = (lane < (blockDim.x >> 5)) ? smem[lane] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r = fmaxf(r, __shfl_xor_sync(0xffffffffu, r, o));
    return r;  // every thread holds the block maximum
}

// A cluster of cs CTAs (1..8) per row, each with cols / cs columns: with a handful of rows one CTA per
// row would leave the GPU idle and be bound by one CTA's walk along its row.  The segment is read
// once with 128-bit loads and kept in registers (up to VPT float4 per thread); the absmax is a
// warp-shuffle + shared-memory reduction, then an exchange through distributed shared memory (max is
// order-independent, fmaxf drops NaN like f32::max); the i8 results leave as packed 32-bit stores.
// Columns of a segment past THREADS*VPT*4 are re-read in the second pass.
template <int VPT>
__global__ void __launch_bounds__(QR_THREADS) quantize_rows_kernel(const float *__restrict__ x, int64_t cols,
                                                                    int8_t *__restrict__ q, float *__restrict__ scales,
                                                                    const PgPeerWait wt)
{
    __shared__ float red[32];
    __shared__ float xm[8];
    // x comes from the preceding kernel; once this grid runs, the one after it may start its own
    // independent prologue (the product kernel prefetches weights)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t cs = cl_size(), rank = cl_rank();
    const int64_t row = blockIdx.x / cs;
    const int64_t nvec = (cols >> 2) / cs;        // float4 per segment (the host picks cs so that this is exact)
    const float4 *xr = reinterpret_cast<const float4 *>(x + row * cols) + rank * nvec;
    // wt.cells != nullptr: the rows are an exchange's flagged cells that all GPUs fill; a load returns once the cells
    // carry the number of the exchange this rank's own producer counted last (bounded wait)
    const bool cells = wt.cells != nullptr;
    const uint32_t want = cells ? pg_cell_want(wt) : 0u;
    const int64_t cell0 = row * cols + (int64_t)rank * nvec * 4;
    auto load = [&](int64_t c) -> float4 { return cells ? pg_cell_load4(wt, want, cell0 + c * 4) : pg_ld_fresh(xr + c); };
    float4 v[VPT];
    float amax = 0.0f;
    if (cells) {
        // up to four groups of cells per thread are requested before the first one is looked at
        constexpr int BATCH = VPT < 4 ? VPT : 4;
#pragma unroll
        for (int i0 = 0; i0 < VPT; i0 += BATCH) {
            uint4 ca[BATCH], cb[BATCH];
#pragma unroll
            for (int j = 0; j < BATCH; j++) {
                const int64_t c = (int64_t)(i0 + j) * QR_THREADS + threadIdx.x;
                if (c < nvec) pg_cell_issue4(wt, cell0 + c * 4, ca[j], cb[j]);
            }
#pragma unroll
            for (int j = 0; j < BATCH; j++) {
                const int64_t c = (int64_t)(i0 + j) * QR_THREADS + threadIdx.x;
                v[i0 + j] = (c < nvec) ? pg_cell_settle4(wt, want, cell0 + c * 4, ca[j], cb[j]) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < VPT; i++) {
            const int64_t c = (int64_t)i * QR_THREADS + threadIdx.x;
            v[i] = (c < nvec) ? pg_ld_fresh(xr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
#pragma unroll
    for (int i = 0; i < VPT; i++)
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[i].x), fabsf(v[i].y)), fmaxf(fabsf(v[i].z), fabsf(v[i].w))));
    for (int64_t c = (int64_t)VPT * QR_THREADS + threadIdx.x; c < nvec; c += QR_THREADS) {
        const float4 t = load(c);
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(t.x), fabsf(t.y)), fmaxf(fabsf(t.z), fabsf(t.w))));
    }
    amax = cl_allreduce<true>(block_max(amax, red), xm, cs, rank);
    const float scale = (amax == 0.0f) ? 1.0f : __fdiv_rn(amax, 127.0f);
    const float inv = __fdiv_rn(1.0f, scale);
    if (threadIdx.x == 0 && rank == 0) scales[row] = scale;
    uint32_t *qr = reinterpret_cast<uint32_t *>(q + row * cols) + rank * nvec;
    auto pack = [&](const float4 &t) -> uint32_t {
        const int a = pg_round_clamp_i8(__fmul_rn(t.x, inv));
        const int b = pg_round_clamp_i8(__fmul_rn(t.y, inv));
        const int c = pg_round_clamp_i8(__fmul_rn(t.z, inv));
        const int d = pg_round_clamp_i8(__fmul_rn(t.w, inv));
        return (uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8) | ((uint32_t)(c & 0xff) << 16) | ((uint32_t)(d & 0xff) << 24);
    };
#pragma unroll
    for (int i = 0; i < VPT; i++) {
        const int64_t c = (int64_t)i * QR_THREADS + threadIdx.x;
        if (c < nvec) qr[c] = pack(v[i]);
    }
    for (int64_t c = (int64_t)VPT * QR_THREADS + threadIdx.x; c < nvec; c += QR_THREADS) qr[c] = pack(load(c));
}

// Any cols / any alignment: scalar loads, two passes.
__global__ void __launch_bounds__(QR_THREADS) quantize_rows_scalar_kernel(const float *__restrict__ x, int64_t cols,
                                                                           int8_t *__restrict__ q, float *__restrict__ scales)
{
    __shared__ float red[32];
    const int64_t row = blockIdx.x;
    const float *xr = x + row * cols;
    float amax = 0.0f;
    for (int64_t c = threadIdx.x; c < cols; c += QR_THREADS) amax = fmaxf(amax, fabsf(xr[c]));
    amax = block_max(amax, red);
    const float scale = (amax == 0.0f) ? 1.0f : __fdiv_rn(amax, 127.0f);
    const float inv = __fdiv_rn(1.0f, scale);
    if (threadIdx.x == 0) scales[row] = scale;
    for (int64_t c = threadIdx.x; c < cols; c += QR_THREADS) q[row * cols + c] = (int8_t)pg_round_clamp_i8(__fmul_rn(xr[c], inv));
}

// ---- weights: per-column absmax over [K,N] ---------------------------------
// Thread = one column (a warp reads 128 contiguous bytes of a row); grid.y splits the rows.
// Partial maxima meet in an integer atomicMax on the bit pattern, which orders non-negative
// floats correctly.  `v > m` is false for NaN, so NaN never becomes a maximum (quant.rs:35).
constexpr int CA_THREADS = 256;
constexpr int CA_ROWS = 128;
__global__ void __launch_bounds__(CA_THREADS) col_absmax_kernel(const float *__restrict__ w, int64_t rows, int64_t cols,
                                                                 int *__restrict__ amax_bits)
{
    const int64_t n = (int64_t)blockIdx.x * CA_THREADS + threadIdx.x;
    if (n >= cols) return;
    const int64_t r0 = (int64_t)blockIdx.y * CA_ROWS;
    const int64_t r1 = min(rows, r0 + CA_ROWS);
    float m = 0.0f;
    for (int64_t r = r0; r < r1; r++) {
        const float v = fabsf(__ldg(w + r * cols + n));
        if (v > m) m = v;
    }
    atomicMax(amax_bits + n, __float_as_int(m));
}

// ---- weights: quantise a 32x32 tile and write both layouts coalesced --------
__global__ void __launch_bounds__(256) quantize_cols_kernel(const float *__restrict__ w, int64_t rows, int64_t cols,
                                                             const int *__restrict__ amax_bits, int8_t *__restrict__ q,
                                                             int8_t *__restrict__ qt, float *__restrict__ scales)
{
    __shared__ int8_t tile[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    const int64_t n = (int64_t)blockIdx.x * 32 + tx;
    const int64_t k0 = (int64_t)blockIdx.y * 32;
    float scale = 1.0f;
    if (n < cols) {
        const float amax = __int_as_float(amax_bits[n]);
        scale = (amax == 0.0f) ? 1.0f : __fdiv_rn(amax, 127.0f);
        if (blockIdx.y == 0 && ty == 0) scales[n] = scale;
    }
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int kk = ty + j * 8;
        const int64_t k = k0 + kk;
        int8_t v = 0;
        if (n < cols && k < rows) {
            v = (int8_t)pg_round_clamp_i8(__fdiv_rn(__ldg(w + k * cols + n), scale));
            if (q) q[k * cols + n] = v;
        }
        tile[kk][tx] = v;
    }
    __syncthreads();
    if (qt) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int nn = ty + j * 8;
            const int64_t no = (int64_t)blockIdx.x * 32 + nn;
            const int64_t k = k0 + tx;
            if (no < cols && k < rows) qt[no * rows + k] = tile[tx][nn];
        }
    }
}

__global__ void __launch_bounds__(256) dequantize_kernel(const int8_t *__restrict__ q, const float *__restrict__ scales,
                                                          int64_t total, int64_t cols, float *__restrict__ out)
{
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i < total) out[i] = __fmul_rn((float)q[i], __ldg(scales + (i % cols)));
}

// One thread per output; the sum runs in ascending p with the multiply and the add rounded
// separately, so the result is bit-identical to the reference's naive loop.
__global__ void __launch_bounds__(256) matmul_f32_kernel(const float *__restrict__ a, const float *__restrict__ b, int64_t m,
                                                          int64_t k, int64_t n, float *__restrict__ out)
{
    const int64_t j = (int64_t)blockIdx.x * 256 + threadIdx.x;
    const int64_t i = blockIdx.y;
    if (j >= n || i >= m) return;
    float sum = 0.0f;
    for (int64_t p = 0; p < k; p++) sum = __fadd_rn(sum, __fmul_rn(__ldg(a + i * k + p), __ldg(b + p * n + j)));
    out[i * n + j] = sum;
}

}  // namespace

int32_t pgk_quantize_activations(pg_ctx *ctx, const float *d_x, int64_t rows, int64_t cols, int8_t *d_q, float *d_scales)
{
    return pgk_quantize_activations_wait(ctx, d_x, rows, cols, d_q, d_scales, nullptr);
}

// wait != nullptr: d_x is this rank's exchange buffer; the kernel first waits (bounded) for every rank's flags
int32_t pgk_quantize_activations_wait(pg_ctx *ctx, const float *d_x, int64_t rows, int64_t cols, int8_t *d_q, float *d_scales,
                                      const PgPeerWait *wait)
{
    if (rows == 0) return PG_OK;
    PG_REQUIRE(rows <= 0x7fffffff, "quantize_activations: rows=%lld exceeds the grid limit", (long long)rows);
    const bool vec = (cols % 4 == 0) && (((uintptr_t)d_x & 15) == 0) && (((uintptr_t)d_q & 3) == 0);
    PG_REQUIRE(!wait || (vec && cols > 0), "quantize_activations: rows taken from an exchange need cols %% 4 == 0 and aligned buffers");
    PgPeerWait wt = {};
    if (wait) wt = *wait;
    if (cols == 0) {
        // scale of an empty row is 1.0 (amax == 0)
        quantize_rows_scalar_kernel<<<(unsigned)rows, QR_THREADS, 0, ctx->stream>>>(d_x, 0, d_q, d_scales);
    } else if (!vec) {
        quantize_rows_scalar_kernel<<<(unsigned)rows, QR_THREADS, 0, ctx->stream>>>(d_x, cols, d_q, d_scales);
    } else {
        // CTAs per row: one, unless the row is long enough (8192 columns per CTA) for the exchange between the CTAs
        // of a cluster to cost less than one CTA's walk along the row (measured: at 4096 and 14336 columns one CTA wins)
        int cs = 8;
        const int64_t nvec = cols / 4;
        // (rows read from an exchange's cells are polled, which costs a memory latency per group of cells and thread:
        // there a row is spread as widely as the cluster allows)
        const int64_t min_seg = wait ? 256 : 2048;
        while (cs > 1 && (rows * cs > 2 * (int64_t)ctx->sm_count || nvec % cs != 0 || nvec / cs < min_seg)) cs >>= 1;
        PG_REQUIRE(rows * cs <= 0x7fffffff, "quantize_activations: rows=%lld exceeds the grid limit", (long long)rows);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(rows * cs));
        cfg.blockDim = dim3(QR_THREADS);
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = (unsigned)cs;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = cs > 1 ? 2 : 1;
        const int64_t seg = cols / cs;
        if (seg <= 4 * QR_THREADS)
            PG_CUDA(cudaLaunchKernelEx(&cfg, quantize_rows_kernel<1>, d_x, cols, d_q, d_scales, wt));
        else if (seg <= 4 * QR_THREADS * 4)
            PG_CUDA(cudaLaunchKernelEx(&cfg, quantize_rows_kernel<4>, d_x, cols, d_q, d_scales, wt));
        else
            PG_CUDA(cudaLaunchKernelEx(&cfg, quantize_rows_kernel<16>, d_x, cols, d_q, d_scales, wt));
    }
    PG_LAUNCHED();
    return PG_OK;
}

int32_t pgk_quantize_weights(pg_ctx *ctx, const float *d_w, int64_t rows, int64_t cols, int8_t *d_q, int8_t *d_qt,
                             float *d_scales)
{
    if (cols == 0) return PG_OK;
    const int32_t rc = pg_scratch_reserve(ctx, (size_t)cols * sizeof(int));
    if (rc != PG_OK) return rc;
    int *amax = reinterpret_cast<int *>(ctx->scratch);
    PG_CUDA(cudaMemsetAsync(amax, 0, (size_t)cols * sizeof(int), ctx->stream));
    if (rows > 0) {
        dim3 g1((unsigned)((cols + CA_THREADS - 1) / CA_THREADS), (unsigned)((rows + CA_ROWS - 1) / CA_ROWS));
        PG_REQUIRE(g1.y <= 65535, "quantize_weights: rows=%lld too large", (long long)rows);
        col_absmax_kernel<<<g1, CA_THREADS, 0, ctx->stream>>>(d_w, rows, cols, amax);
        PG_LAUNCHED();
    }
    dim3 g2((unsigned)((cols + 31) / 32), (unsigned)((rows + 31) / 32 > 0 ? (rows + 31) / 32 : 1));
    PG_REQUIRE(g2.y <= 65535, "quantize_weights: rows=%lld too large", (long long)rows);
    quantize_cols_kernel<<<g2, 256, 0, ctx->stream>>>(d_w, rows, cols, amax, d_q, d_qt, d_scales);
    PG_LAUNCHED();
    return PG_OK;
}

// [rows, cols] i8 -> [cols, rows] i8 through a 64 x 64 tile in shared memory (one byte of padding per row keeps the
// column reads off a single bank): what read_quantized_tensor does on the host to rebuild data_i8_t (src/serial.rs:203-208).
__global__ void __launch_bounds__(256) transpose_i8_kernel(const int8_t *__restrict__ in, int64_t rows, int64_t cols, int8_t *__restrict__ out)
{
    __shared__ int8_t tile[64][65];
    const int64_t r0 = (int64_t)blockIdx.y * 64, c0 = (int64_t)blockIdx.x * 64;
    for (int i = threadIdx.x; i < 64 * 64; i += 256) {
        const int r = i >> 6, c = i & 63;
        if (r0 + r < rows && c0 + c < cols) tile[r][c] = in[(r0 + r) * cols + c0 + c];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 64 * 64; i += 256) {
        const int c = i >> 6, r = i & 63;
        if (r0 + r < rows && c0 + c < cols) out[(c0 + c) * rows + r0 + r] = tile[r][c];
    }
}

// The same for shapes and pointers that allow 32-bit accesses: a 128 x 128 tile, rows read and written as whole
// 128-byte lines.  The tile's row stride of 129 bytes puts the four bytes a thread gathers for one output word, and
// the words of the 32 lanes, in different banks.
__global__ void __launch_bounds__(256) transpose_i8_words_kernel(const int8_t *__restrict__ in, int64_t rows, int64_t cols, int8_t *__restrict__ out)
{
    __shared__ uint8_t tile[128 * 129];
    const int64_t r0 = (int64_t)blockIdx.y * 128, c0 = (int64_t)blockIdx.x * 128;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t v[16];
#pragma unroll
    for (int i = 0; i < 16; i++) {
        const int r = warp * 16 + i;
        v[i] = (r0 + r < rows && c0 + 4 * lane < cols) ? __ldg((const uint32_t *)(in + (r0 + r) * cols + c0) + lane) : 0u;
    }
#pragma unroll
    for (int i = 0; i < 16; i++) {
        uint8_t *t = tile + (warp * 16 + i) * 129 + 4 * lane;
        t[0] = (uint8_t)v[i];
        t[1] = (uint8_t)(v[i] >> 8);
        t[2] = (uint8_t)(v[i] >> 16);
        t[3] = (uint8_t)(v[i] >> 24);
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 16; i++) {
        const int c = warp * 16 + i;
        if (c0 + c >= cols || r0 + 4 * lane >= rows) continue;
        const uint8_t *t = tile + (4 * lane) * 129 + c;
        const uint32_t w = (uint32_t)t[0] | ((uint32_t)t[129] << 8) | ((uint32_t)t[258] << 16) | ((uint32_t)t[387] << 24);
        *((uint32_t *)(out + (c0 + c) * rows + r0) + lane) = w;
    }
}

int32_t pgk_transpose_i8(pg_ctx *ctx, const int8_t *d_in, int64_t rows, int64_t cols, int8_t *d_out)
{
    if (rows == 0 || cols == 0) return PG_OK;
    if (rows % 4 == 0 && cols % 4 == 0 && (((uintptr_t)d_in | (uintptr_t)d_out) & 3) == 0 && (rows + 127) / 128 <= 65535) {
        const dim3 grid((unsigned)((cols + 127) / 128), (unsigned)((rows + 127) / 128));
        transpose_i8_words_kernel<<<grid, 256, 0, ctx->stream>>>(d_in, rows, cols, d_out);
        PG_LAUNCHED();
        return PG_OK;
    }
    const dim3 grid((unsigned)((cols + 63) / 64), (unsigned)((rows + 63) / 64));
    PG_REQUIRE(grid.y <= 65535, "transpose_i8: rows=%lld too large", (long long)rows);
    transpose_i8_kernel<<<grid, 256, 0, ctx->stream>>>(d_in, rows, cols, d_out);
    PG_LAUNCHED();
    return PG_OK;
}

int32_t pgk_dequantize(pg_ctx *ctx, const int8_t *d_q, const float *d_scales, int64_t rows, int64_t cols, float *d_out)
{
    const int64_t total = rows * cols;
    if (total == 0) return PG_OK;
    dequantize_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>(d_q, d_scales, total, cols, d_out);
    PG_LAUNCHED();
    return PG_OK;
}

int32_t pgk_matmul_f32(pg_ctx *ctx, const float *d_a, const float *d_b, int64_t m, int64_t k, int64_t n, float *d_out)
{
    if (m == 0 || n == 0) return PG_OK;
    PG_REQUIRE(m <= 65535, "matmul_f32: m=%lld exceeds the grid limit of this checker kernel", (long long)m);
    dim3 g((unsigned)((n + 255) / 256), (unsigned)m);
    matmul_f32_kernel<<<g, 256, 0, ctx->stream>>>(d_a, d_b, m, k, n, d_out);
    PG_LAUNCHED();
    return PG_OK;
}

// A plain copy of 16-byte words by the SMs (both pointers 16-byte aligned).  Used to push a small result into
// page-locked host memory: a kernel behind the product in the stream starts sooner than a copy engine does.
__global__ void __launch_bounds__(256) copy_words_kernel(const uint4 *__restrict__ src, uint4 *__restrict__ dst, size_t words, size_t tail_from,
                                                         size_t bytes)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < words; i += stride) {
        const uint4 v = pg_ld_fresh(src + i);
        dst[i] = v;
    }
    if (blockIdx.x == 0 && threadIdx.x < bytes - tail_from)
        ((unsigned char *)dst)[tail_from + threadIdx.x] = pg_ld_fresh((const unsigned char *)src + tail_from + threadIdx.x);
}

int32_t pgk_copy_words(pg_ctx *ctx, const void *d_src, void *dst, size_t bytes)
{
    if (bytes == 0) return PG_OK;
    const size_t words = bytes / 16;
    const unsigned blocks = (unsigned)std::min<size_t>((words + 255) / 256 ? (words + 255) / 256 : 1, 2 * 148);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    PG_CUDA(cudaLaunchKernelEx(&cfg, copy_words_kernel, (const uint4 *)d_src, (uint4 *)dst, words, words * 16, bytes));
    PG_LAUNCHED();
    return PG_OK;
}

