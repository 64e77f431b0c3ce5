// The glue of one Llama decode step between the quantised linears: what the reference runs on the
// host in f32 around its five matmuls (src/models/llama/decoder.rs:69-155,
// src/models/llama/attention.rs:73-195, src/models/llama/model.rs:223-237).
//
//   add_rmsnorm_quant_kernel   residual add + RMSNorm (src/nn.rs:577-652: x * inv_rms * w with
//                              inv_rms = 1/sqrt(mean(x^2) + eps)) + the per-row int8 quantiser of
//                              src/quant.rs:97-109, fused: the normalised row only ever exists in registers
//   swiglu_quant_kernel        silu(g) * u (src/models/llama/decoder.rs:143-150, g / (1 + exp(-g)))
//                              on the fused [gate | up] output + the same quantiser
//   rope_kv_append_kernel      RoPE on q and k (src/nn.rs:1322-1338: halves rotated with a cos/sin table)
//                              and append of k, v to the f32 KV cache (src/attention.rs:65-83)
//   gqa_decode_*_kernel        GQA attention of one new token against the cache
//                              (src/attention.rs:141-265: dot * 1/sqrt(hd), softmax, weighted sum of V),
//                              split over the context so that all SMs stream the cache, then combined
//   embedding / argmax         src/nn.rs:217-227, examples/llama/main.rs:15-26 (first maximum wins)
//
// Everything is batched over independent sequences (one row per sequence); the position lives in
// device memory so that a whole step can be recorded once and replayed.  f32 sums here run in a
// different order from the reference's sequential loops, so this layer is checked to a tolerance, not
// bit for bit (the linears inside it stay bit-exact for the activations they are given).
#include "pg_internal.cuh"

namespace {

constexpr int LT = 256;  // threads per CTA of the row kernels

__device__ __forceinline__ float block_sum(float v, float *smem)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float r = 0.0f;
#pragma unroll
    for (int i = 0; i < LT / 32; i++) r += smem[i];
    return r;
}
__device__ __forceinline__ float block_max(float v, float *smem)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float r = 0.0f;
#pragma unroll
    for (int i = 0; i < LT / 32; i++) r = fmaxf(r, smem[i]);
    return r;
}
__device__ __forceinline__ uint32_t pack_i8x4(float a, float b, float c, float d, float inv)
{
    const int qa = pg_round_clamp_i8(__fmul_rn(a, inv)), qb = pg_round_clamp_i8(__fmul_rn(b, inv));
    const int qc = pg_round_clamp_i8(__fmul_rn(c, inv)), qd = pg_round_clamp_i8(__fmul_rn(d, inv));
    return (uint32_t)(qa & 0xff) | ((uint32_t)(qb & 0xff) << 8) | ((uint32_t)(qc & 0xff) << 16) | ((uint32_t)(qd & 0xff) << 24);
}

// a cluster of cs CTAs per row, each with dim / cs columns; VPT float4 per thread (dim / cs <= LT * 4 * VPT)
template <int VPT>
__global__ void __launch_bounds__(LT) add_rmsnorm_quant_kernel(float *__restrict__ x, const float *__restrict__ delta,
                                                                const float *__restrict__ w, int dim, float eps,
                                                                int8_t *__restrict__ q, float *__restrict__ scales,
                                                                float *__restrict__ normed)
{
    __shared__ float red[32];
    __shared__ float xs[8], xm[8];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t cs = cl_size(), rank = cl_rank();
    const int64_t row = blockIdx.x / cs;
    const int nseg = (dim >> 2) / (int)cs;       // float4 per segment
    const int c0 = (int)rank * nseg;
    float4 *xr = reinterpret_cast<float4 *>(x + row * dim);
    float4 v[VPT];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; i++) {
        const int c = i * LT + threadIdx.x;
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < nseg) {
            v[i] = pg_ld_fresh(xr + c0 + c);
            if (delta) {
                const float4 d = pg_ld_fresh(reinterpret_cast<const float4 *>(delta + row * dim) + c0 + c);
                v[i].x += d.x; v[i].y += d.y; v[i].z += d.z; v[i].w += d.w;
                xr[c0 + c] = v[i];
            }
            ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
        }
    }
    ss = cl_allreduce<false>(block_sum(ss, red), xs, cs, rank);
    const float inv_rms = __fdiv_rn(1.0f, sqrtf(__fmul_rn(ss, __fdiv_rn(1.0f, (float)dim)) + eps));
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; i++) {
        const int c = i * LT + threadIdx.x;
        if (c < nseg) {
            const float4 ww = __ldg(reinterpret_cast<const float4 *>(w) + c0 + c);
            v[i].x = __fmul_rn(__fmul_rn(v[i].x, inv_rms), ww.x);
            v[i].y = __fmul_rn(__fmul_rn(v[i].y, inv_rms), ww.y);
            v[i].z = __fmul_rn(__fmul_rn(v[i].z, inv_rms), ww.z);
            v[i].w = __fmul_rn(__fmul_rn(v[i].w, inv_rms), ww.w);
            if (normed) reinterpret_cast<float4 *>(normed + row * dim)[c0 + c] = v[i];
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[i].x), fabsf(v[i].y)), fmaxf(fabsf(v[i].z), fabsf(v[i].w))));
        }
    }
    amax = cl_allreduce<true>(block_max(amax, red), xm, cs, rank);
    const float scale = (amax == 0.0f) ? 1.0f : __fdiv_rn(amax, 127.0f);
    const float inv = __fdiv_rn(1.0f, scale);
    if (threadIdx.x == 0 && rank == 0) scales[row] = scale;
    uint32_t *qr = reinterpret_cast<uint32_t *>(q + row * dim);
#pragma unroll
    for (int i = 0; i < VPT; i++) {
        const int c = i * LT + threadIdx.x;
        if (c < nseg) qr[c0 + c] = pack_i8x4(v[i].x, v[i].y, v[i].z, v[i].w, inv);
    }
}

// gate_up [rows, 2F]: gate = [:, :F], up = [:, F:]; a cluster of cs CTAs per row, each with F / cs columns
template <int VPT>
__global__ void __launch_bounds__(LT) swiglu_quant_kernel(const float *__restrict__ gu, int F, int8_t *__restrict__ q,
                                                           float *__restrict__ scales, float *__restrict__ act_out)
{
    __shared__ float red[32];
    __shared__ float xm[8];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t cs = cl_size(), rank = cl_rank();
    const int64_t row = blockIdx.x / cs;
    const int nseg = (F >> 2) / (int)cs;
    const int c0 = (int)rank * nseg;
    const float4 *g4 = reinterpret_cast<const float4 *>(gu + row * 2 * F) + c0;
    const float4 *u4 = reinterpret_cast<const float4 *>(gu + row * 2 * F + F) + c0;
    float4 v[VPT];
    float amax = 0.0f;
    auto silu_mul = [](float g, float u) { return __fmul_rn(__fdiv_rn(g, 1.0f + expf(-g)), u); };
#pragma unroll
    for (int i = 0; i < VPT; i++) {
        const int c = i * LT + threadIdx.x;
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < nseg) {
            const float4 g = pg_ld_fresh(g4 + c), u = pg_ld_fresh(u4 + c);
            v[i] = make_float4(silu_mul(g.x, u.x), silu_mul(g.y, u.y), silu_mul(g.z, u.z), silu_mul(g.w, u.w));
            if (act_out) reinterpret_cast<float4 *>(act_out + row * F)[c0 + c] = v[i];
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[i].x), fabsf(v[i].y)), fmaxf(fabsf(v[i].z), fabsf(v[i].w))));
        }
    }
    amax = cl_allreduce<true>(block_max(amax, red), xm, cs, rank);
    const float scale = (amax == 0.0f) ? 1.0f : __fdiv_rn(amax, 127.0f);
    const float inv = __fdiv_rn(1.0f, scale);
    if (threadIdx.x == 0 && rank == 0) scales[row] = scale;
    uint32_t *qr = reinterpret_cast<uint32_t *>(q + row * F) + c0;
#pragma unroll
    for (int i = 0; i < VPT; i++) {
        const int c = i * LT + threadIdx.x;
        if (c < nseg) qr[c] = pack_i8x4(v[i].x, v[i].y, v[i].z, v[i].w, inv);
    }
}

// grid (Hq + 2*Hkv, B), hd/2 threads.  qkv row = [Q heads | K heads | V heads].
__global__ void rope_kv_append_kernel(const float *__restrict__ qkv, const int *__restrict__ pos_ptr, const float *__restrict__ cos_t,
                                      const float *__restrict__ sin_t, int Hq, int Hkv, int hd, int cap,
                                      float *__restrict__ q_rot, float *__restrict__ kc, float *__restrict__ vc)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int head = blockIdx.x, b = blockIdx.y, i = threadIdx.x, half = hd >> 1;
    const int pos = pg_ld_fresh(pos_ptr);
    const float *src = qkv + ((int64_t)b * (Hq + 2 * Hkv) + head) * hd;
    if (head < Hq + Hkv) {
        const float x0 = pg_ld_fresh(src + i), x1 = pg_ld_fresh(src + half + i);
        const float c = cos_t[(int64_t)pos * half + i], s = sin_t[(int64_t)pos * half + i];
        const float r0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
        const float r1 = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
        float *dst = (head < Hq) ? q_rot + ((int64_t)b * Hq + head) * hd
                                 : kc + (((int64_t)b * Hkv + (head - Hq)) * cap + pos) * hd;
        dst[i] = r0;
        dst[half + i] = r1;
    } else {
        float *dst = vc + (((int64_t)b * Hkv + (head - Hq - Hkv)) * cap + pos) * hd;
        dst[i] = pg_ld_fresh(src + i);
        dst[half + i] = pg_ld_fresh(src + half + i);
    }
}

// ---- attention of one new token per sequence against the cache, head_dim 128 -----------------
// grid (S, Hkv, B): one CTA handles `chunk` cached positions of one KV head for the G query heads that
// share it.  Warp per position, lane = four head-dim elements; scores go to shared memory, then a
// softmax over the chunk, then the weighted sum of V.  Writes unnormalised partial outputs with their
// running maximum and sum; gqa_decode_combine_kernel merges the S partials.
template <int G>
__global__ void __launch_bounds__(256) gqa_decode_partial_kernel(const float *__restrict__ q, const float *__restrict__ kc,
                                                                  const float *__restrict__ vc, const int *__restrict__ pos_ptr, int Hq,
                                                                  int Hkv, int cap, int chunk, float scale, float *__restrict__ part_o,
                                                                  float *__restrict__ part_ml)
{
    constexpr int HD = 128;
    extern __shared__ float sm[];  // sc[chunk][G], then red[8][G][HD]
    float *sc = sm;
    float *red = sm + (((size_t)chunk * G + 3) & ~(size_t)3);   // written as float4: starts on a 16-byte boundary
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int split = blockIdx.x, S = gridDim.x, kvh = blockIdx.y, b = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int len = pg_ld_fresh(pos_ptr) + 1;
    const int t0 = split * chunk, t1 = min(len, t0 + chunk);
    const int n = t1 - t0;
    float *po = part_o + (((int64_t)b * Hq + kvh * G) * S + split) * HD;   // + h * S * HD
    float *pml = part_ml + (((int64_t)b * Hq + kvh * G) * S + split) * 2;  // + h * S * 2
    if (n <= 0) {
        if (threadIdx.x < G) {
            pml[(int64_t)threadIdx.x * S * 2] = -INFINITY;
            pml[(int64_t)threadIdx.x * S * 2 + 1] = 0.0f;
        }
        return;
    }
    const float4 *kbase = reinterpret_cast<const float4 *>(kc + (((int64_t)b * Hkv + kvh) * cap + t0) * HD);
    const float4 *vbase = reinterpret_cast<const float4 *>(vc + (((int64_t)b * Hkv + kvh) * cap + t0) * HD);
    float4 qv[G];
#pragma unroll
    for (int h = 0; h < G; h++) qv[h] = pg_ld_fresh(reinterpret_cast<const float4 *>(q + ((int64_t)b * Hq + kvh * G + h) * HD) + lane);

    // scores
    for (int i0 = warp; i0 < n; i0 += 8 * 4) {
        float4 kv[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int i = i0 + u * 8;
            kv[u] = (i < n) ? pg_ld_fresh(kbase + (int64_t)i * (HD / 4) + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int i = i0 + u * 8;
            float d[G];
#pragma unroll
            for (int h = 0; h < G; h++) d[h] = qv[h].x * kv[u].x + qv[h].y * kv[u].y + qv[h].z * kv[u].z + qv[h].w * kv[u].w;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int h = 0; h < G; h++) d[h] += __shfl_xor_sync(0xffffffffu, d[h], o);
            if (lane == 0 && i < n)
#pragma unroll
                for (int h = 0; h < G; h++) sc[i * G + h] = d[h] * scale;
        }
    }
    __syncthreads();
    // softmax statistics of the chunk: warp h handles head h
    if (warp < G) {
        float m = -INFINITY;
        for (int i = lane; i < n; i += 32) m = fmaxf(m, sc[i * G + warp]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        float l = 0.0f;
        for (int i = lane; i < n; i += 32) {
            const float p = expf(sc[i * G + warp] - m);
            sc[i * G + warp] = p;
            l += p;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
        if (lane == 0) {
            pml[(int64_t)warp * S * 2] = m;
            pml[(int64_t)warp * S * 2 + 1] = l;
        }
    }
    __syncthreads();
    // weighted sum of V
    float4 acc[G];
#pragma unroll
    for (int h = 0; h < G; h++) acc[h] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int i0 = warp; i0 < n; i0 += 8 * 4) {
        float4 vv[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int i = i0 + u * 8;
            vv[u] = (i < n) ? pg_ld_fresh(vbase + (int64_t)i * (HD / 4) + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int i = i0 + u * 8;
            if (i < n) {
#pragma unroll
                for (int h = 0; h < G; h++) {
                    const float p = sc[i * G + h];
                    acc[h].x = fmaf(p, vv[u].x, acc[h].x);
                    acc[h].y = fmaf(p, vv[u].y, acc[h].y);
                    acc[h].z = fmaf(p, vv[u].z, acc[h].z);
                    acc[h].w = fmaf(p, vv[u].w, acc[h].w);
                }
            }
        }
    }
#pragma unroll
    for (int h = 0; h < G; h++) reinterpret_cast<float4 *>(red + ((size_t)warp * G + h) * HD)[lane] = acc[h];
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * HD; idx += 256) {
        const int h = idx / HD, d = idx - h * HD;
        float s = 0.0f;
#pragma unroll
        for (int wv = 0; wv < 8; wv++) s += red[((size_t)wv * G + h) * HD + d];
        po[(int64_t)h * S * HD + d] = s;
    }
}

// grid (Hq, B), 128 threads: out[b, qh*128 + d]
__global__ void __launch_bounds__(128) gqa_decode_combine_kernel(const float *__restrict__ part_o, const float *__restrict__ part_ml, int Hq,
                                                                  int S, float *__restrict__ out)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int qh = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
    const float *ml = part_ml + ((int64_t)b * Hq + qh) * S * 2;
    const float *po = part_o + ((int64_t)b * Hq + qh) * S * 128;
    float m = -INFINITY;
    for (int s = 0; s < S; s++) m = fmaxf(m, pg_ld_fresh(ml + 2 * s));
    float denom = 0.0f, acc = 0.0f;
    for (int s = 0; s < S; s++) {
        const float l = pg_ld_fresh(ml + 2 * s + 1);
        if (l > 0.0f) {
            const float e = expf(pg_ld_fresh(ml + 2 * s) - m);
            denom = fmaf(e, l, denom);
            acc = fmaf(e, pg_ld_fresh(po + (int64_t)s * 128 + d), acc);
        }
    }
    out[((int64_t)b * Hq + qh) * 128 + d] = (denom > 0.0f) ? __fdiv_rn(acc, denom) : 0.0f;
}

__global__ void embedding_kernel(const float *__restrict__ table, const int *__restrict__ tokens, int dim, float *__restrict__ out)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int b = blockIdx.x;
    const float4 *src = reinterpret_cast<const float4 *>(table + (int64_t)pg_ld_fresh(tokens + b) * dim);
    float4 *dst = reinterpret_cast<float4 *>(out + (int64_t)b * dim);
    for (int i = threadIdx.x; i < (dim >> 2); i += blockDim.x) dst[i] = __ldg(src + i);
}

// a cluster of cs CTAs per row, each scanning V / cs logits; the first maximum wins (examples/llama/main.rs:15-26).
// The first CTA of row 0 also advances the position.
__global__ void __launch_bounds__(1024) argmax_kernel(const float *__restrict__ logits, int V, int *__restrict__ tokens, int *pos_ptr)
{
    __shared__ float bv[32];
    __shared__ int bi[32];
    __shared__ float xv[8];
    __shared__ int xi[8];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t cs = cl_size(), rank = cl_rank();
    const int b = blockIdx.x / cs;
    const float *row = logits + (int64_t)b * V;
    const int seg = (V + (int)cs - 1) / (int)cs;
    const int i0 = (int)rank * seg, i1 = min(V, i0 + seg);
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
        const float v = pg_ld_fresh(row + i);
        if (v > best || (v == best && i < idx)) {
            best = v;
            idx = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) {
            best = ov;
            idx = oi;
        }
    }
    if ((threadIdx.x & 31) == 0) {
        bv[threadIdx.x >> 5] = best;
        bi[threadIdx.x >> 5] = idx;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); w++)
            if (bv[w] > best || (bv[w] == best && bi[w] < idx)) {
                best = bv[w];
                idx = bi[w];
            }
        if (cs > 1) {
            cl_store_f32(xv + rank, 0, best);     // everything meets in the first CTA of the cluster
            cl_store_s32(xi + rank, 0, idx);
        }
    }
    if (cs > 1) cl_sync();
    if (threadIdx.x == 0 && rank == 0) {
        for (uint32_t c = 1; c < cs; c++)
            if (xv[c] > best || (xv[c] == best && xi[c] < idx)) {
                best = xv[c];
                idx = xi[c];
            }
        tokens[b] = (idx == 0x7fffffff) ? 0 : idx;   // all-NaN row: the reference keeps index 0
        if (b == 0 && pos_ptr) *pos_ptr = pg_ld_fresh(pos_ptr) + 1;
    }
}

// Merge of the S partial attention outputs of every (sequence, query head), optionally followed by the per-row int8
// quantiser of src/quant.rs:97-109 over the whole row [Hq * 128] (what the output projection takes).
// A cluster of cs CTAs per sequence, each with Hq / cs heads: blockDim = (128, Hq / cs).
__global__ void __launch_bounds__(1024) gqa_combine_quant_kernel(const float *__restrict__ part_o, const float *__restrict__ part_ml, int Hq,
                                                                  int S, float *__restrict__ out, int8_t *__restrict__ q8,
                                                                  float *__restrict__ q8_scales)
{
    constexpr int MAXS = 64;                      // slices per (sequence, KV head) never exceed this (checked on the host)
    __shared__ float red[32];
    __shared__ float xm[8];
    __shared__ float wgt[8][MAXS];                // per head of this CTA: exp(m_s - m), 0 for an empty slice
    __shared__ float den[8];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t cs = cl_size(), rank = cl_rank();
    const int b = blockIdx.x / cs, d = threadIdx.x, qh = (int)rank * blockDim.y + threadIdx.y;
    const float *ml = part_ml + ((int64_t)b * Hq + qh) * S * 2;
    const float *po = part_o + ((int64_t)b * Hq + qh) * S * 128;
    // the first warp of every head turns the S (max, sum) pairs into weights, so that the loads of the partial outputs
    // below do not hang off a chain of exponentials
    if (d < 32) {
        // S <= 64: a lane holds at most two (max, sum) pairs, loaded once
        const float2 p0 = (d < S) ? pg_ld_fresh(reinterpret_cast<const float2 *>(ml) + d) : make_float2(-INFINITY, 0.0f);
        const float2 p1 = (d + 32 < S) ? pg_ld_fresh(reinterpret_cast<const float2 *>(ml) + d + 32) : make_float2(-INFINITY, 0.0f);
        float m = fmaxf(p0.x, p1.x);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
        const float e0 = (p0.y > 0.0f) ? expf(p0.x - m) : 0.0f, e1 = (p1.y > 0.0f) ? expf(p1.x - m) : 0.0f;
        if (d < S) wgt[threadIdx.y][d] = e0;
        if (d + 32 < S) wgt[threadIdx.y][d + 32] = e1;
        float dn = fmaf(e0, p0.y, e1 * p1.y);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) dn += __shfl_xor_sync(0xffffffffu, dn, off);
        if (d == 0) den[threadIdx.y] = dn;
    }
    __syncthreads();
    const float denom = den[threadIdx.y];
    float acc = 0.0f;
#pragma unroll 4
    for (int s = 0; s < S; s++) {
        const float e = wgt[threadIdx.y][s];
        if (e != 0.0f) acc = fmaf(e, pg_ld_fresh(po + (int64_t)s * 128 + d), acc);
    }
    const float o = (denom > 0.0f) ? __fdiv_rn(acc, denom) : 0.0f;
    const int64_t at = ((int64_t)b * Hq + qh) * 128 + d;
    if (out) out[at] = o;
    if (!q8) return;                              // uniform over the cluster: nobody waits at the barrier below
    float amax = fabsf(o);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    const int tid = threadIdx.y * 128 + threadIdx.x, nwarps = (blockDim.x * blockDim.y) >> 5;
    if ((tid & 31) == 0) red[tid >> 5] = amax;
    __syncthreads();
    amax = red[0];
    for (int i = 1; i < nwarps; i++) amax = fmaxf(amax, red[i]);
    if (cs > 1) {
        if (tid < (int)cs) cl_store_f32(xm + rank, tid, amax);
        cl_sync();
        amax = xm[0];
        for (uint32_t i = 1; i < cs; i++) amax = fmaxf(amax, xm[i]);
    }
    const float scale = (amax == 0.0f) ? 1.0f : __fdiv_rn(amax, 127.0f);
    const float inv = __fdiv_rn(1.0f, scale);
    if (tid == 0 && rank == 0) q8_scales[b] = scale;
    q8[at] = (int8_t)pg_round_clamp_i8(__fmul_rn(o, inv));
}

template <typename K, typename... Args>
int32_t launch_pdl_cluster(pg_ctx *ctx, K kern, dim3 grid, dim3 block, size_t smem, int cs, Args... args)
{
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = (unsigned)cs;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cfg.attrs = attr;
    cfg.numAttrs = cs > 1 ? 2 : 1;
    PG_CUDA(cudaLaunchKernelEx(&cfg, kern, args...));
    PG_LAUNCHED();
    return PG_OK;
}

// CTAs per row for the row kernels: as many (up to 8) as keep the grid within about two CTAs per SM, divide the row's
// `units` evenly and leave each CTA at least `min_units`.
int row_cluster(const pg_ctx *ctx, int64_t rows, int64_t units, int64_t min_units)
{
    int cs = 8;
    while (cs > 1 && (rows * cs > 2 * (int64_t)ctx->sm_count || units % cs != 0 || units / cs < min_units)) cs >>= 1;
    return cs;
}

template <typename K, typename... Args>
int32_t launch_pdl(pg_ctx *ctx, K kern, dim3 grid, dim3 block, size_t smem, Args... args)
{
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    PG_CUDA(cudaLaunchKernelEx(&cfg, kern, args...));
    PG_LAUNCHED();
    return PG_OK;
}

}  // namespace

extern "C" {

// x [rows, dim] (updated in place to x + delta when delta != NULL) -> q [rows, dim] i8 + scales [rows] of
// RMSNorm(x) * w; `normed` (nullable) receives the f32 normalised rows.
PG_API int32_t pg_add_rmsnorm_quantize(pg_ctx *ctx, float *d_x, const float *d_delta, const float *d_w, int64_t rows, int64_t dim,
                                       float eps, int8_t *d_q, float *d_scales, float *d_normed)
{
    PG_REQUIRE(ctx && d_x && d_w && d_q && d_scales, "add_rmsnorm_quantize: null pointer");
    PG_REQUIRE(rows >= 0 && dim > 0 && dim % 4 == 0 && dim <= LT * 4 * 16, "add_rmsnorm_quantize: dim must be a multiple of 4, at most %d", LT * 64);
    if (rows == 0) return PG_OK;
    const int cs = row_cluster(ctx, rows, dim / 4, 128);
    const dim3 g((unsigned)(rows * cs)), b(LT);
    if (dim / cs <= LT * 4) return launch_pdl_cluster(ctx, add_rmsnorm_quant_kernel<1>, g, b, 0, cs, d_x, d_delta, d_w, (int)dim, eps, d_q, d_scales, d_normed);
    if (dim / cs <= LT * 16) return launch_pdl_cluster(ctx, add_rmsnorm_quant_kernel<4>, g, b, 0, cs, d_x, d_delta, d_w, (int)dim, eps, d_q, d_scales, d_normed);
    return launch_pdl_cluster(ctx, add_rmsnorm_quant_kernel<16>, g, b, 0, cs, d_x, d_delta, d_w, (int)dim, eps, d_q, d_scales, d_normed);
}

// gate_up [rows, 2F] -> q [rows, F] i8 + scales [rows] of silu(gate) * up; `act` (nullable) receives the f32 rows.
PG_API int32_t pg_swiglu_quantize(pg_ctx *ctx, const float *d_gate_up, int64_t rows, int64_t F, int8_t *d_q, float *d_scales, float *d_act)
{
    PG_REQUIRE(ctx && d_gate_up && d_q && d_scales, "swiglu_quantize: null pointer");
    PG_REQUIRE(rows >= 0 && F > 0 && F % 4 == 0 && F <= LT * 4 * 16, "swiglu_quantize: F must be a multiple of 4, at most %d", LT * 64);
    if (rows == 0) return PG_OK;
    const int cs = row_cluster(ctx, rows, F / 4, 128);
    const dim3 g((unsigned)(rows * cs)), b(LT);
    if (F / cs <= LT * 8) return launch_pdl_cluster(ctx, swiglu_quant_kernel<2>, g, b, 0, cs, d_gate_up, (int)F, d_q, d_scales, d_act);
    if (F / cs <= LT * 16) return launch_pdl_cluster(ctx, swiglu_quant_kernel<4>, g, b, 0, cs, d_gate_up, (int)F, d_q, d_scales, d_act);
    return launch_pdl_cluster(ctx, swiglu_quant_kernel<16>, g, b, 0, cs, d_gate_up, (int)F, d_q, d_scales, d_act);
}

// qkv [B, (Hq + 2 Hkv) * hd] -> q_rot [B, Hq, hd]; k (rotated) and v written at position *d_pos of the caches
// [B, Hkv, cap, hd].  cos/sin tables: [max_pos, hd/2].
PG_API int32_t pg_rope_kv_append(pg_ctx *ctx, const float *d_qkv, const int32_t *d_pos, const float *d_cos, const float *d_sin,
                                 int64_t B, int64_t Hq, int64_t Hkv, int64_t hd, int64_t cap, float *d_q_rot, float *d_kcache,
                                 float *d_vcache)
{
    PG_REQUIRE(ctx && d_qkv && d_pos && d_cos && d_sin && d_q_rot && d_kcache && d_vcache, "rope_kv_append: null pointer");
    PG_REQUIRE(hd % 2 == 0 && hd <= 2048 && B >= 0 && B <= 65535, "rope_kv_append: bad shape");
    if (B == 0) return PG_OK;
    return launch_pdl(ctx, rope_kv_append_kernel, dim3((unsigned)(Hq + 2 * Hkv), (unsigned)B), dim3((unsigned)(hd / 2)), 0, d_qkv, (const int *)d_pos,
                      d_cos, d_sin, (int)Hq, (int)Hkv, (int)hd, (int)cap, d_q_rot, d_kcache, d_vcache);
}

// Attention of one new token per sequence over positions 0..*d_pos (the new one included).
// d_work: B * Hq * S * 130 floats with S = pg_gqa_decode_splits(ctx, B, Hq, Hkv, cap).
PG_API int32_t pg_gqa_decode_splits(pg_ctx *ctx, int64_t B, int64_t Hq, int64_t Hkv, int64_t cap)
{
    if (ctx && Hkv > 0 && Hq % Hkv == 0 && pgk_gqa_stream_supports(Hq / Hkv)) return pgk_gqa_stream_splits(ctx, B, Hkv, cap);
    return cap <= 512 ? 1 : (cap <= 2048 ? 4 : 8);
}

static int32_t attention_decode(pg_ctx *ctx, const float *d_q_rot, float *d_kcache, float *d_vcache, const int32_t *d_pos,
                                const float *d_cos, const float *d_sin, int64_t B, int64_t Hq, int64_t Hkv, int64_t hd, int64_t cap,
                                float *d_work, float *d_out, int8_t *d_out_i8, float *d_out_scales)
{
    PG_REQUIRE(ctx && d_q_rot && d_kcache && d_vcache && d_pos && d_work, "gqa_attention_decode: null pointer");
    PG_REQUIRE(d_out || d_out_i8, "gqa_attention_decode: no output");
    PG_REQUIRE((d_out_i8 == nullptr) == (d_out_scales == nullptr), "gqa_attention_decode: quantised output needs both buffers");
    PG_REQUIRE(hd == 128, "gqa_attention_decode: head_dim %lld is not supported (128 only)", (long long)hd);
    PG_REQUIRE(Hkv > 0 && Hq % Hkv == 0, "gqa_attention_decode: Hkv must divide Hq");
    const int64_t G = Hq / Hkv;
    PG_REQUIRE(G == 1 || G == 2 || G == 4 || G == 8, "gqa_attention_decode: %lld query heads per KV head is not supported (1, 2, 4, 8)", (long long)G);
    if (B == 0) return PG_OK;
    const int S = pg_gqa_decode_splits(ctx, B, Hq, Hkv, cap);
    const float scale = 1.0f / sqrtf((float)hd);
    float *part_o = d_work;
    float *part_ml = d_work + B * Hq * S * 128;
    int32_t rc;
    if (pgk_gqa_stream_supports(G)) {
        rc = pgk_gqa_decode_stream(ctx, d_q_rot, d_kcache, d_vcache, d_pos, d_cos, d_sin, B, Hq, Hkv, cap, S, scale, part_o, part_ml);
    } else {
        PG_REQUIRE(d_cos == nullptr, "gqa_attention_decode_fused: %lld query heads per KV head is not supported (4, 8)", (long long)G);
        const int chunk = (int)((cap + S - 1) / S);
        const size_t smem = ((((size_t)chunk * G + 3) & ~(size_t)3) + 8 * G * 128) * sizeof(float);
        const dim3 grid((unsigned)S, (unsigned)Hkv, (unsigned)B);
#define PG_ATT(GG)                                                                                                              \
    {                                                                                                                           \
        if (smem > 48 * 1024) PG_CUDA(cudaFuncSetAttribute(gqa_decode_partial_kernel<GG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        rc = launch_pdl(ctx, gqa_decode_partial_kernel<GG>, grid, dim3(256), smem, d_q_rot, d_kcache, d_vcache, (const int *)d_pos, (int)Hq, \
                        (int)Hkv, (int)cap, chunk, scale, part_o, part_ml);                                                     \
    }
        if (G == 1) PG_ATT(1) else PG_ATT(2)
#undef PG_ATT
    }
    if (rc) return rc;
    // merge of the partials (+ the quantiser of the output projection's input): a cluster of CTAs per sequence
    int cs = 8;
    while (cs > 1 && (B * cs > 2 * (int64_t)ctx->sm_count || Hq % cs != 0)) cs >>= 1;
    const int64_t hpc = Hq / cs;
    if (hpc <= 8 && S <= 64)
        return launch_pdl_cluster(ctx, gqa_combine_quant_kernel, dim3((unsigned)(B * cs)), dim3(128, (unsigned)hpc), 0, cs, (const float *)part_o,
                                  (const float *)part_ml, (int)Hq, S, d_out, d_out_i8, d_out_scales);
    // many sequences with many heads: merge per head, quantise the rows afterwards
    float *merged = d_out;
    PG_REQUIRE(d_out != nullptr, "gqa_attention_decode: this shape needs the f32 output buffer as well");
    rc = launch_pdl(ctx, gqa_decode_combine_kernel, dim3((unsigned)Hq, (unsigned)B), dim3(128), 0, (const float *)part_o, (const float *)part_ml,
                    (int)Hq, S, merged);
    if (rc || !d_out_i8) return rc;
    return pgk_quantize_activations(ctx, merged, B, Hq * 128, d_out_i8, d_out_scales);
}


PG_API int32_t pg_gqa_attention_decode(pg_ctx *ctx, const float *d_q_rot, const float *d_kcache, const float *d_vcache,
                                       const int32_t *d_pos, int64_t B, int64_t Hq, int64_t Hkv, int64_t hd, int64_t cap, float *d_work,
                                       float *d_out, int8_t *d_out_i8, float *d_out_scales)
{
    // the caches are only read on this path
    return attention_decode(ctx, d_q_rot, const_cast<float *>(d_kcache), const_cast<float *>(d_vcache), d_pos, nullptr, nullptr, B, Hq, Hkv, hd,
                            cap, d_work, d_out, d_out_i8, d_out_scales);
}

// pg_rope_kv_append + pg_gqa_attention_decode in one launch: d_qkv is the raw [B, (Hq + 2 Hkv) * hd] output of the fused
// Q|K|V projection; the newest token's rotated key and its value are written at position *d_pos of the caches.
PG_API int32_t pg_gqa_attention_decode_fused(pg_ctx *ctx, const float *d_qkv, const int32_t *d_pos, const float *d_cos, const float *d_sin,
                                             float *d_kcache, float *d_vcache, int64_t B, int64_t Hq, int64_t Hkv, int64_t hd, int64_t cap,
                                             float *d_work, float *d_out, int8_t *d_out_i8, float *d_out_scales)
{
    PG_REQUIRE(d_cos && d_sin, "gqa_attention_decode_fused: null rotation tables");
    return attention_decode(ctx, d_qkv, d_kcache, d_vcache, d_pos, d_cos, d_sin, B, Hq, Hkv, hd, cap, d_work, d_out, d_out_i8, d_out_scales);
}

PG_API int32_t pg_embedding(pg_ctx *ctx, const float *d_table, const int32_t *d_tokens, int64_t B, int64_t dim, float *d_out)
{
    PG_REQUIRE(ctx && d_table && d_tokens && d_out && dim % 4 == 0, "embedding: bad arguments");
    if (B == 0) return PG_OK;
    return launch_pdl(ctx, embedding_kernel, dim3((unsigned)B), dim3(256), 0, d_table, (const int *)d_tokens, (int)dim, d_out);
}

// tokens[b] = argmax(logits[b, :]) (first maximum); d_pos (nullable) is advanced by one.
PG_API int32_t pg_argmax_advance(pg_ctx *ctx, const float *d_logits, int64_t B, int64_t V, int32_t *d_tokens, int32_t *d_pos)
{
    PG_REQUIRE(ctx && d_logits && d_tokens && V > 0, "argmax: bad arguments");
    if (B == 0) return PG_OK;
    const int cs = row_cluster(ctx, B, V, 4096);
    return launch_pdl_cluster(ctx, argmax_kernel, dim3((unsigned)(B * cs)), dim3(1024), 0, cs, d_logits, (int)V, (int *)d_tokens, (int *)d_pos);
}

}  // extern "C"
