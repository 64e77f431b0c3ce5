// GGUF block formats: decoders and the dequantising product used by the Llama linears.
//
//   dequant_blocks_kernel   gguf::dequant_q8_0 / dequant_q4_0 / dequant_q4_1
//                           (src/gguf.rs:286-302, 307-326, 331-351): raw block stream -> f32
//   f16_to_f32_kernel       gguf::f16_to_f32 (src/gguf.rs:354-382)
//   repack_kernel           upload-time split of the raw stream into 16-byte aligned planes
//                           (the reference also re-lays weights out once at load:
//                           src/quant.rs:56-62, src/models/llama/model.rs:243-257)
//   matmul_gguf_kernel      y = x . dequant(W)^T in f32: what load_tensor_f32 (src/gguf.rs:485-517)
//                           followed by Tensor::matmul (src/tensor.rs:1342-1354) computes, without
//                           ever writing the f32 weight to memory.
//
// Block layouts (little endian): Q8_0 = f16 d, 32 x i8.  Q4_0 = f16 d, 16 bytes; byte i holds
// element 2i in its low nibble and 2i+1 in its high nibble, value = nibble - 8.
// Q4_1 = f16 d, f16 m, 16 bytes; value = nibble * d + m.
#include <cuda_fp16.h>

#include "pg_internal.cuh"

namespace {

// Integer restatement of src/gguf.rs:354-382 (keeps NaN payloads exactly as the reference does).
__device__ __forceinline__ float f16_bits_to_f32(uint32_t bits)
{
    const uint32_t sign = (bits >> 15) & 1u, exp = (bits >> 10) & 0x1Fu, mant = bits & 0x3FFu;
    uint32_t out;
    if (exp == 0) {
        if (mant == 0) {
            out = sign << 31;
        } else {
            const int shift = __clz(mant) - 21;  // moves the leading one to bit 10
            const uint32_t m = (mant << shift) & 0x3FFu;
            out = (sign << 31) | ((uint32_t)(127 - 15 + 1 - shift) << 23) | (m << 13);
        }
    } else if (exp == 31) {
        out = (sign << 31) | (0xFFu << 23) | (mant << 13);
    } else {
        out = (sign << 31) | ((exp + 127 - 15) << 23) | (mant << 13);
    }
    return __uint_as_float(out);
}

__device__ __forceinline__ int block_bytes(int type) { return type == PG_GGUF_Q8_0 ? 34 : (type == PG_GGUF_Q4_0 ? 18 : 20); }

// One warp per block, lane = element: byte loads and f32 stores are both coalesced.
__global__ void __launch_bounds__(256) dequant_blocks_kernel(int type, const uint8_t *__restrict__ raw, int64_t num_blocks,
                                                              float *__restrict__ out)
{
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = ((int64_t)blockIdx.x * 256 + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * 256) >> 5;
    const int bs = block_bytes(type);
    for (int64_t b = warp0; b < num_blocks; b += nwarps) {
        const uint8_t *p = raw + b * bs;
        const float d = f16_bits_to_f32((uint32_t)p[0] | ((uint32_t)p[1] << 8));
        float v;
        if (type == PG_GGUF_Q8_0) {
            v = __fmul_rn((float)(int8_t)p[2 + lane], d);
        } else if (type == PG_GGUF_Q4_0) {
            const uint32_t byte = p[2 + (lane >> 1)];
            const int q = (int)((lane & 1) ? (byte >> 4) : (byte & 0xF)) - 8;
            v = __fmul_rn((float)q, d);
        } else {
            const float mn = f16_bits_to_f32((uint32_t)p[2] | ((uint32_t)p[3] << 8));
            const uint32_t byte = p[4 + (lane >> 1)];
            const float q = (float)((lane & 1) ? (byte >> 4) : (byte & 0xF));
            v = __fadd_rn(__fmul_rn(q, d), mn);
        }
        out[b * 32 + lane] = v;
    }
}

__global__ void __launch_bounds__(256) f16_to_f32_kernel(const uint16_t *__restrict__ bits, int64_t count, float *__restrict__ out)
{
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i < count) out[i] = f16_bits_to_f32(bits[i]);
}

// raw [N][K/32][block] -> qs plane + scale planes.
// Plain planes: qs [N][K/32][16 or 32 quant bytes], d [N][K/32] f16 (Q4_1: also m).
// Tiled layout of the streaming tensor-core kernel (Q4_0 / Q8_0, K % 256 == 0): one contiguous "fill" per (tile of 16 rows,
// slice of 8 blocks), FILL = 16 * SEG + 256 bytes with SEG = 8 * {16, 32} quant bytes per row:
//   row r of the tile at r * SEG, as 16-byte pieces; piece p of a row holds what lane t = p % 4 of a tensor-core fragment
//   needs of block group p / 4 -- Q4_0: word t (elements 8t..8t+7) of the group's four blocks; Q8_0: bytes 8t..8t+7 of
//   the group's two blocks -- and is stored at position p ^ ((r & 1) << 2), so that the eight lanes of a quarter warp
//   (two rows, four pieces each) hit all 32 banks when the fill lies in shared memory as it lies in global memory;
//   then the scales: row r's eight f16 at 16 * SEG + r * 16.
__device__ __forceinline__ int64_t tiled_index(int type, int64_t row, int64_t nslices, int blk_in_row, int byte, bool scale)
{
    const int seg = (type == PG_GGUF_Q8_0) ? 256 : 128;
    const int64_t fill = 16 * seg + 256;
    const int64_t base = ((row >> 4) * nslices + (blk_in_row >> 3)) * fill;
    const int r = (int)(row & 15), bl = blk_in_row & 7;
    if (scale) return base + 16 * seg + r * 16 + bl * 2;
    int piece, within;
    if (type == PG_GGUF_Q8_0) {
        piece = (bl >> 1) * 4 + (byte >> 3);
        within = (bl & 1) * 8 + (byte & 7);
    } else {
        piece = (bl >> 2) * 4 + (byte >> 2);
        within = (bl & 3) * 4 + (byte & 3);
    }
    return base + (int64_t)r * seg + ((piece ^ ((r & 1) << 2)) * 16) + within;
}

__global__ void __launch_bounds__(256) repack_kernel(int type, int tiled, const uint8_t *__restrict__ raw, int64_t num_blocks, int nblk_row,
                                                      uint8_t *__restrict__ qs, uint16_t *__restrict__ dd, uint16_t *__restrict__ mm)
{
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = ((int64_t)blockIdx.x * 256 + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * 256) >> 5;
    const int bs = block_bytes(type);
    for (int64_t b = warp0; b < num_blocks; b += nwarps) {
        const uint8_t *p = raw + b * bs;
        if (tiled) {
            const int64_t row = b / nblk_row;
            const int bir = (int)(b - row * nblk_row);
            const int64_t nslices = nblk_row >> 3;
            if (lane < 2) qs[tiled_index(type, row, nslices, bir, 0, true) + lane] = p[lane];
            if (type == PG_GGUF_Q8_0 || lane < 16) qs[tiled_index(type, row, nslices, bir, lane, false)] = p[2 + lane];
            continue;
        }
        if (lane == 0) dd[b] = (uint16_t)(p[0] | (p[1] << 8));
        if (type == PG_GGUF_Q8_0) {
            qs[b * 32 + lane] = p[2 + lane];
        } else if (type == PG_GGUF_Q4_0) {
            if (lane < 16) qs[b * 16 + lane] = p[2 + lane];
        } else {
            if (lane == 1) mm[b] = (uint16_t)(p[2] | (p[3] << 8));
            if (lane < 16) qs[b * 16 + lane] = p[4 + lane];
        }
    }
}

// ---- dequantising product, CUDA-core form --------------------------------------------
// A warp owns R weight rows; its lanes take interleaved 32-element blocks of K.  Per block a
// lane reads the quants of its R rows with 128-bit loads, unpacks them in registers, and for
// each activation row forms the block's partial sum in f32 before applying the block scale:
// y += d * sum_i x_i q_i  (+ m * sum_i x_i for Q4_1).  Lanes are then summed by shuffles.
template <int TYPE, int R, int MC>
__global__ void __launch_bounds__(256) matmul_gguf_kernel(const float *__restrict__ x, int m0, int M, int K,
                                                           const uint8_t *__restrict__ qs, const uint16_t *__restrict__ dd,
                                                           const uint16_t *__restrict__ mm, int64_t N, float *__restrict__ y)
{
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * 256 + threadIdx.x) >> 5;
    const int64_t nrow0 = warp * R;
    if (nrow0 >= N) return;
    const int nblk = K >> 5;
    float acc[MC][R];
#pragma unroll
    for (int i = 0; i < MC; i++)
#pragma unroll
        for (int j = 0; j < R; j++) acc[i][j] = 0.0f;

    for (int b = lane; b < nblk; b += 32) {
        float q[R][32];
        float d[R], mn[R];
#pragma unroll
        for (int j = 0; j < R; j++) {
            const int64_t row = (nrow0 + j < N) ? nrow0 + j : N - 1;
            const int64_t blk = row * nblk + b;
            d[j] = __half2float(__ushort_as_half(dd[blk]));
            mn[j] = 0.0f;
            if (TYPE == PG_GGUF_Q8_0) {
                uint32_t wds[8];
                const uint4 *p = reinterpret_cast<const uint4 *>(qs + blk * 32);
                const uint4 v0 = __ldg(p), v1 = __ldg(p + 1);
                wds[0] = v0.x; wds[1] = v0.y; wds[2] = v0.z; wds[3] = v0.w;
                wds[4] = v1.x; wds[5] = v1.y; wds[6] = v1.z; wds[7] = v1.w;
#pragma unroll
                for (int wd = 0; wd < 8; wd++)
#pragma unroll
                    for (int e = 0; e < 4; e++) q[j][wd * 4 + e] = (float)(int8_t)((wds[wd] >> (8 * e)) & 0xff);
            } else {
                uint32_t wds[4];
                const uint4 v = __ldg(reinterpret_cast<const uint4 *>(qs + blk * 16));
                wds[0] = v.x; wds[1] = v.y; wds[2] = v.z; wds[3] = v.w;
#pragma unroll
                for (int wd = 0; wd < 4; wd++)
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const uint32_t byte = (wds[wd] >> (8 * e)) & 0xff;
                        const int off = (TYPE == PG_GGUF_Q4_0) ? 8 : 0;
                        q[j][(wd * 4 + e) * 2] = (float)((int)(byte & 0xF) - off);
                        q[j][(wd * 4 + e) * 2 + 1] = (float)((int)(byte >> 4) - off);
                    }
                if (TYPE == PG_GGUF_Q4_1) mn[j] = __half2float(__ushort_as_half(mm[blk]));
            }
        }
#pragma unroll
        for (int i = 0; i < MC; i++) {
            if (m0 + i >= M) break;
            const float4 *xp = reinterpret_cast<const float4 *>(x + (int64_t)(m0 + i) * K + b * 32);
            float ps[R];
#pragma unroll
            for (int j = 0; j < R; j++) ps[j] = 0.0f;
            float xs = 0.0f;
#pragma unroll
            for (int v = 0; v < 8; v++) {
                const float4 xv = __ldg(xp + v);
#pragma unroll
                for (int j = 0; j < R; j++) {
                    ps[j] = fmaf(xv.x, q[j][v * 4 + 0], ps[j]);
                    ps[j] = fmaf(xv.y, q[j][v * 4 + 1], ps[j]);
                    ps[j] = fmaf(xv.z, q[j][v * 4 + 2], ps[j]);
                    ps[j] = fmaf(xv.w, q[j][v * 4 + 3], ps[j]);
                }
                if (TYPE == PG_GGUF_Q4_1) xs += (xv.x + xv.y) + (xv.z + xv.w);
            }
#pragma unroll
            for (int j = 0; j < R; j++) {
                acc[i][j] = fmaf(d[j], ps[j], acc[i][j]);
                if (TYPE == PG_GGUF_Q4_1) acc[i][j] = fmaf(mn[j], xs, acc[i][j]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < MC; i++) {
#pragma unroll
        for (int j = 0; j < R; j++) {
            float v = acc[i][j];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && m0 + i < M && nrow0 + j < N) y[(int64_t)(m0 + i) * N + nrow0 + j] = v;
        }
    }
}

template <int TYPE>
int32_t launch_matmul(pg_ctx *ctx, const float *d_x, int64_t m, const pg_gguf_weight *w, float *d_y)
{
    constexpr int R = 2, MC = 4;
    const int64_t warps = (w->n + R - 1) / R;
    const int64_t blocks = (warps + 7) / 8;
    for (int64_t m0 = 0; m0 < m; m0 += MC) {
        matmul_gguf_kernel<TYPE, R, MC><<<(unsigned)blocks, 256, 0, ctx->stream>>>(d_x, (int)m0, (int)m, (int)w->k, w->d_qs, w->d_d,
                                                                                  w->d_m, w->n, d_y);
        PG_LAUNCHED();
    }
    return PG_OK;
}

}  // namespace

int32_t pgk_dequant_blocks(pg_ctx *ctx, int32_t type, const uint8_t *d_raw, int64_t num_blocks, float *d_out)
{
    if (num_blocks == 0) return PG_OK;
    int64_t blocks = (num_blocks + 7) / 8;
    if (blocks > (int64_t)ctx->sm_count * 64) blocks = (int64_t)ctx->sm_count * 64;
    dequant_blocks_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(type, d_raw, num_blocks, d_out);
    PG_LAUNCHED();
    return PG_OK;
}

int32_t pgk_f16_to_f32(pg_ctx *ctx, const uint16_t *d_bits, int64_t count, float *d_out)
{
    if (count == 0) return PG_OK;
    f16_to_f32_kernel<<<(unsigned)((count + 255) / 256), 256, 0, ctx->stream>>>(d_bits, count, d_out);
    PG_LAUNCHED();
    return PG_OK;
}

static int g_gguf_force_simple = 0;
extern "C" PG_API void pg_tune_gguf_simple(int on) { g_gguf_force_simple = on; }

size_t pgk_gguf_qs_bytes(int32_t type, int64_t rows, int64_t k, int *tiled)
{
    const int64_t nblk = k / 32;
    // the streaming tensor-core kernel's layout whenever that kernel can take the weight
    const bool t = (type == PG_GGUF_Q4_0 || type == PG_GGUF_Q8_0) && k >= 256 && (k % 256 == 0) && !g_gguf_force_simple;
    if (tiled) *tiled = t ? 1 : 0;
    if (t) return (size_t)((rows + 15) / 16) * (size_t)(nblk / 8) * (size_t)(16 * (type == PG_GGUF_Q8_0 ? 256 : 128) + 256);
    return (size_t)rows * nblk * (type == PG_GGUF_Q8_0 ? 32 : 16);
}

// w->d_qs must hold pgk_gguf_qs_bytes(...) bytes
int32_t pgk_gguf_repack(pg_ctx *ctx, int32_t type, const uint8_t *d_raw, int64_t n, int64_t k, pg_gguf_weight *w)
{
    const int64_t num_blocks = n * (k / 32);
    if (num_blocks == 0) return PG_OK;
    int64_t blocks = (num_blocks + 7) / 8;
    if (blocks > (int64_t)ctx->sm_count * 64) blocks = (int64_t)ctx->sm_count * 64;
    int tiled = 0;
    const size_t qbytes = pgk_gguf_qs_bytes(type, n, k, &tiled);
    w->tiled = tiled;
    if (tiled && (n & 15)) PG_CUDA(cudaMemsetAsync(w->d_qs, 0, qbytes, ctx->stream));   // rows past N of the last tile
    repack_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(type, tiled, d_raw, num_blocks, (int)(k / 32), w->d_qs, w->d_d, w->d_m);
    PG_LAUNCHED();
    return PG_OK;
}

int32_t pgk_matmul_gguf(pg_ctx *ctx, const float *d_x, int64_t m, const pg_gguf_weight *w, float *d_y)
{
    if (m == 0 || w->n == 0) return PG_OK;
    PG_REQUIRE(((uintptr_t)d_x & 15) == 0, "matmul_gguf: x must be 16-byte aligned");
    if (w->tiled) return pgk_matmul_gguf_stream(ctx, d_x, m, w, d_y);
    switch (w->type) {
        case PG_GGUF_Q8_0: return launch_matmul<PG_GGUF_Q8_0>(ctx, d_x, m, w, d_y);
        case PG_GGUF_Q4_0: return launch_matmul<PG_GGUF_Q4_0>(ctx, d_x, m, w, d_y);
        case PG_GGUF_Q4_1: return launch_matmul<PG_GGUF_Q4_1>(ctx, d_x, m, w, d_y);
    }
    PG_FAIL(PG_ERR_INVALID, "matmul_gguf: unknown block type %d", w->type);
}
