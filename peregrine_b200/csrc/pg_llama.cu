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
                                                                float *__restrict__ normed, const PgPeerWait wt)
{
    __shared__ float red[32];
    __shared__ float xs[8], xm[8];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // wt.cells != nullptr: delta is an exchange's buffer of flagged cells that all GPUs fill (bounded wait per load)
    const bool dcells = wt.cells != nullptr;
    const uint32_t want = dcells ? pg_cell_want(wt) : 0u;
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
            uint4 ca, cb;
            if (dcells) pg_cell_issue4(wt, row * dim + (int64_t)(c0 + c) * 4, ca, cb);
            v[i] = pg_ld_fresh(xr + c0 + c);
            if (delta || dcells) {
                const float4 d = dcells ? pg_cell_settle4(wt, want, row * dim + (int64_t)(c0 + c) * 4, ca, cb)
                                        : pg_ld_fresh(reinterpret_cast<const float4 *>(delta + row * dim) + c0 + c);
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
                                      float *__restrict__ q_rot, float *__restrict__ kc, float *__restrict__ vc, int32_t *status)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int head = blockIdx.x, b = blockIdx.y, i = threadIdx.x, half = hd >> 1;
    const int pos = pg_ld_fresh(pos_ptr);
    if ((unsigned)pos >= (unsigned)cap) {   // the cache and the rotation tables end at cap: record it, touch nothing
        if (i == 0) atomicExch(status, (int32_t)PG_ERR_INVALID);
        return;
    }
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
                                                                  float *__restrict__ part_ml, int32_t *status)
{
    constexpr int HD = 128;
    extern __shared__ float sm[];  // sc[chunk][G], then red[8][G][HD]
    float *sc = sm;
    float *red = sm + (((size_t)chunk * G + 3) & ~(size_t)3);   // written as float4: starts on a 16-byte boundary
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int split = blockIdx.x, S = gridDim.x, kvh = blockIdx.y, b = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int len = pg_ld_fresh(pos_ptr) + 1;
    if ((unsigned)(len - 1) >= (unsigned)cap) {   // position outside the cache: record it, read nothing (empty slices)
        if (threadIdx.x == 0) atomicExch(status, (int32_t)PG_ERR_INVALID);
        len = 0;
    }
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
// PEER (po.world > 0): `logits` holds this rank's V columns of a vocabulary sharded by column; the row's local
// (maximum, index + v0) pair goes to slot [b][rank] of every rank's exchange buffer instead of tokens[b], and
// pick_embed_kernel chooses among the ranks' pairs.
__global__ void __launch_bounds__(1024) argmax_kernel(const float *__restrict__ logits, int V, int *__restrict__ tokens, int *pos_ptr,
                                                       int pos_limit, int v0, const PgPeerOut po)
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
        if (po.world > 0) {
            // an all-NaN (or empty) slice never wins: -inf with the slice's first index
            pg_cell_store2(po, pg_cell_seq(po), b, 0, (idx == 0x7fffffff) ? -INFINITY : best,
                           __int_as_float((idx == 0x7fffffff) ? v0 : idx + v0));
        } else {
            tokens[b] = (idx == 0x7fffffff) ? 0 : idx;   // all-NaN row: the reference keeps index 0
            if (b == 0 && pos_ptr) {
                const int p = pg_ld_fresh(pos_ptr);
                if (pos_limit <= 0 || p < pos_limit) *pos_ptr = p + 1;   // never past the end of the cache
            }
        }
    }
    if (po.world > 0) pg_cell_finish(po, pg_cell_seq(po), threadIdx.x);
}

// One CTA per sequence: waits for every rank's (maximum, index) pair of the sharded vocabulary, takes the first
// maximum in index order (ranks own ascending column ranges, so rank order is index order; strict '>' as in
// examples/llama/main.rs:15-26), stores the token, advances the position (CTA 0) and gathers the token's embedding
// row (src/nn.rs:217-227) for the next step.  pairs: [B][world][2].
__global__ void __launch_bounds__(256) pick_embed_kernel(int world, int *__restrict__ tokens, int *pos_ptr, int pos_limit,
                                                         const float *__restrict__ table, int dim, float *__restrict__ out,
                                                         const PgPeerWait wt)
{
    __shared__ int s_tok;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int b = blockIdx.x;
    if (threadIdx.x < 32) {
        // lane r polls rank r's pair (all pairs in flight at once); lane 0 then walks them in rank order
        const uint32_t want = pg_cell_want(wt);
        const int r = threadIdx.x;
        float v = -INFINITY;
        int i = 0;
        if (r < world) {
            v = pg_cell_load(wt, want, ((int64_t)b * world + r) * 2);
            i = __float_as_int(pg_cell_load(wt, want, ((int64_t)b * world + r) * 2 + 1));
        }
        float best = -INFINITY;
        int idx = 0;
        bool any = false;
        for (int q = 0; q < world; q++) {
            const float vq = __shfl_sync(0xffffffffu, v, q);
            const int iq = __shfl_sync(0xffffffffu, i, q);
            if (vq > best) {
                best = vq;
                idx = iq;
                any = true;
            }
        }
        if (!any) idx = 0;   // every slice all-NaN or -inf: the reference's loop keeps index 0
        if (threadIdx.x == 0) {
            tokens[b] = idx;
            s_tok = idx;
            if (b == 0 && pos_ptr) {
                const int p = pg_ld_fresh(pos_ptr);
                if (pos_limit <= 0 || p < pos_limit) *pos_ptr = p + 1;
            }
        }
    }
    __syncthreads();
    if (table) {
        const float4 *src = reinterpret_cast<const float4 *>(table + (int64_t)s_tok * dim);
        float4 *dst = reinterpret_cast<float4 *>(out + (int64_t)b * dim);
        for (int i = threadIdx.x; i < (dim >> 2); i += blockDim.x) dst[i] = __ldg(src + i);
    }
}

// silu(gate) * up on one rank's columns of a column-sharded [gate | up] product: gu [rows, 2 Fl] holds this rank's Fl
// gate columns followed by its Fl up columns; the f32 results go to columns [col0, col0 + Fl) of every rank's [rows, F]
// exchange buffer (the quantiser of the down projection needs the whole row, so it runs after the exchange).
__global__ void __launch_bounds__(256) swiglu_peer_kernel(const float *__restrict__ gu, int rows, int Fl, const PgPeerOut po)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    auto silu_mul = [](float g, float u) { return __fmul_rn(__fdiv_rn(g, 1.0f + expf(-g)), u); };
    const int nv = Fl >> 2;
    const uint32_t seq = pg_cell_seq(po);
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < (int64_t)rows * nv; i += (int64_t)gridDim.x * 256) {
        const int64_t row = i / nv, c = i - row * nv;
        const float4 g = pg_ld_fresh(reinterpret_cast<const float4 *>(gu + row * 2 * Fl) + c);
        const float4 u = pg_ld_fresh(reinterpret_cast<const float4 *>(gu + row * 2 * Fl + Fl) + c);
        pg_cell_store2(po, seq, row, c * 4, silu_mul(g.x, u.x), silu_mul(g.y, u.y));
        pg_cell_store2(po, seq, row, c * 4 + 2, silu_mul(g.z, u.z), silu_mul(g.w, u.w));
    }
    pg_cell_finish(po, seq, threadIdx.x);
}

// Merge of the S partial attention outputs of every (sequence, query head), optionally followed by the per-row int8
// quantiser of src/quant.rs:97-109 over the whole row [Hq * 128] (what the output projection takes).
// A cluster of cs CTAs per sequence, each with Hq / cs heads: blockDim = (128, Hq / cs).
__global__ void __launch_bounds__(1024) gqa_combine_quant_kernel(const float *__restrict__ part_o, const float *__restrict__ part_ml, int Hq,
                                                                  int S, float *__restrict__ out, int8_t *__restrict__ q8,
                                                                  float *__restrict__ q8_scales, const PgPeerOut peer)
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
    if (S <= 16) {
        // a short chain (13 slices at batch 16, context 2048 on one GPU): measured 3 us per layer faster than the form below
#pragma unroll 4
        for (int s = 0; s < S; s++) {
            const float e = wgt[threadIdx.y][s];
            if (e != 0.0f) acc = fmaf(e, pg_ld_fresh(po + (int64_t)s * 128 + d), acc);
        }
    } else {
        // eight running sums (slice s goes to sum s % 8), added up in a fixed order at the end: eight loads are in flight
        // per thread instead of a chain of S (a rank of a sharded step cuts its few heads into 27 to 34 slices), and the
        // order of the additions depends on S alone, not on how the heads are spread over CTAs or ranks
        float part[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int s0 = 0; s0 < S; s0 += 8) {
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; j++) v[j] = (s0 + j < S && wgt[threadIdx.y][s0 + j] != 0.0f) ? pg_ld_fresh(po + (int64_t)(s0 + j) * 128 + d) : 0.0f;
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (s0 + j < S) part[j] = fmaf(wgt[threadIdx.y][s0 + j], v[j], part[j]);
        }
        acc = ((part[0] + part[1]) + (part[2] + part[3])) + ((part[4] + part[5]) + (part[6] + part[7]));
    }
    const float o = (denom > 0.0f) ? __fdiv_rn(acc, denom) : 0.0f;
    const int64_t at = ((int64_t)b * Hq + qh) * 128 + d;
    if (out) out[at] = o;
    if (peer.world > 0) {
        // column-sharded heads: this rank's Hq heads are columns [col0, col0 + Hq * 128) of every rank's attention row
        const uint32_t seq = pg_cell_seq(peer);
        pg_cell_store(peer, seq, b, (int64_t)qh * 128 + d, o);
        pg_cell_finish(peer, seq, threadIdx.y * 128 + threadIdx.x);
        return;                                   // the quantiser needs the whole row: it runs after the exchange
    }
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

static const PgPeerOut NO_PEER_OUT = {};

// x [rows, dim] (updated in place to x + delta when delta != NULL) -> q [rows, dim] i8 + scales [rows] of
// RMSNorm(x) * w; `normed` (nullable) receives the f32 normalised rows.  wait.ctl != NULL: delta is an exchange buffer.
static int32_t add_rmsnorm_quantize(pg_ctx *ctx, float *d_x, const float *d_delta, const float *d_w, int64_t rows, int64_t dim, float eps,
                                    int8_t *d_q, float *d_scales, float *d_normed, const PgPeerWait &wt)
{
    PG_REQUIRE(ctx && d_x && d_w && d_q && d_scales, "add_rmsnorm_quantize: null pointer");
    PG_REQUIRE(rows >= 0 && dim > 0 && dim % 4 == 0 && dim <= LT * 4 * 16, "add_rmsnorm_quantize: dim must be a multiple of 4, at most %d", LT * 64);
    if (rows == 0) return PG_OK;
    const int cs = row_cluster(ctx, rows, dim / 4, 128);
    const dim3 g((unsigned)(rows * cs)), b(LT);
    if (dim / cs <= LT * 4) return launch_pdl_cluster(ctx, add_rmsnorm_quant_kernel<1>, g, b, 0, cs, d_x, d_delta, d_w, (int)dim, eps, d_q, d_scales, d_normed, wt);
    if (dim / cs <= LT * 16) return launch_pdl_cluster(ctx, add_rmsnorm_quant_kernel<4>, g, b, 0, cs, d_x, d_delta, d_w, (int)dim, eps, d_q, d_scales, d_normed, wt);
    return launch_pdl_cluster(ctx, add_rmsnorm_quant_kernel<16>, g, b, 0, cs, d_x, d_delta, d_w, (int)dim, eps, d_q, d_scales, d_normed, wt);
}

extern "C" {

PG_API int32_t pg_add_rmsnorm_quantize(pg_ctx *ctx, float *d_x, const float *d_delta, const float *d_w, int64_t rows, int64_t dim,
                                       float eps, int8_t *d_q, float *d_scales, float *d_normed)
{
    PG_ENTER(ctx);
    PgPeerWait none = {};
    return add_rmsnorm_quantize(ctx, d_x, d_delta, d_w, rows, dim, eps, d_q, d_scales, d_normed, none);
}

// The same with the residual delta taken from an exchange: the kernel waits (bounded) until every rank has delivered
// its columns of the [rows, dim] result that `ex` gathers, then adds it to x.
PG_API int32_t pg_add_rmsnorm_quantize_exchange(pg_ctx *ctx, float *d_x, pg_exchange *ex_delta, const float *d_w, int64_t rows,
                                                int64_t dim, float eps, int8_t *d_q, float *d_scales, float *d_normed)
{
    PG_ENTER(ctx);
    PG_REQUIRE(ex_delta && ex_delta->connected, "add_rmsnorm_quantize_exchange: the exchange is not connected");
    PG_REQUIRE((size_t)rows * (size_t)dim * sizeof(float) <= ex_delta->y_bytes, "add_rmsnorm_quantize_exchange: rows do not fit the exchange buffer");
    return add_rmsnorm_quantize(ctx, d_x, nullptr, d_w, rows, dim, eps, d_q, d_scales, d_normed, pg_peer_wait_of(ctx, ex_delta));
}

// quant::quantize_activations (src/quant.rs:97-109) on the [rows, cols] matrix an exchange gathers: waits (bounded) for
// every rank's columns first.
PG_API int32_t pg_quantize_activations_exchange(pg_ctx *ctx, pg_exchange *ex, int64_t rows, int64_t cols, int8_t *d_q, float *d_scales)
{
    PG_ENTER(ctx);
    PG_REQUIRE(ex && ex->connected && d_q && d_scales, "quantize_activations_exchange: null argument or unconnected exchange");
    PG_REQUIRE(rows >= 0 && cols > 0 && (size_t)rows * (size_t)cols * sizeof(float) <= ex->y_bytes,
               "quantize_activations_exchange: rows do not fit the exchange buffer");
    const PgPeerWait wt = pg_peer_wait_of(ctx, ex);
    return pgk_quantize_activations_wait(ctx, reinterpret_cast<const float *>(ex->cells_local), rows, cols, d_q, d_scales, &wt);
}

// gate_up [rows, 2F] -> q [rows, F] i8 + scales [rows] of silu(gate) * up; `act` (nullable) receives the f32 rows.
PG_API int32_t pg_swiglu_quantize(pg_ctx *ctx, const float *d_gate_up, int64_t rows, int64_t F, int8_t *d_q, float *d_scales, float *d_act)
{
    PG_ENTER(ctx);
    PG_REQUIRE(d_gate_up && d_q && d_scales, "swiglu_quantize: null pointer");
    PG_REQUIRE(rows >= 0 && F > 0 && F % 4 == 0 && F <= LT * 4 * 16, "swiglu_quantize: F must be a multiple of 4, at most %d", LT * 64);
    if (rows == 0) return PG_OK;
    const int cs = row_cluster(ctx, rows, F / 4, 128);
    const dim3 g((unsigned)(rows * cs)), b(LT);
    if (F / cs <= LT * 8) return launch_pdl_cluster(ctx, swiglu_quant_kernel<2>, g, b, 0, cs, d_gate_up, (int)F, d_q, d_scales, d_act);
    if (F / cs <= LT * 16) return launch_pdl_cluster(ctx, swiglu_quant_kernel<4>, g, b, 0, cs, d_gate_up, (int)F, d_q, d_scales, d_act);
    return launch_pdl_cluster(ctx, swiglu_quant_kernel<16>, g, b, 0, cs, d_gate_up, (int)F, d_q, d_scales, d_act);
}

// One rank's part of silu(gate) * up under column sharding: d_gate_up_local [rows, 2 Fl] = this rank's Fl gate columns,
// then its Fl up columns (the same channel range of both halves).  The f32 results go to columns [col0, col0 + Fl) of
// every rank's [rows, F_total] exchange buffer; pg_quantize_activations_exchange then quantises whole rows.
PG_API int32_t pg_swiglu_exchange(pg_ctx *ctx, const float *d_gate_up_local, int64_t rows, int64_t F_local, pg_exchange *ex,
                                  int64_t F_total, int64_t col0)
{
    PG_ENTER(ctx);
    PG_REQUIRE(d_gate_up_local && ex && ex->connected, "swiglu_exchange: null argument or unconnected exchange");
    PG_REQUIRE(rows >= 0 && rows <= 0x7fffffff && F_local > 0 && F_local % 4 == 0 && F_total % 4 == 0 && col0 % 4 == 0 && col0 >= 0 &&
                   col0 + F_local <= F_total,
               "swiglu_exchange: column ranges must be multiples of 4 inside [0, F_total)");
    PG_REQUIRE((size_t)rows * (size_t)F_total * sizeof(float) <= ex->y_bytes, "swiglu_exchange: rows do not fit the exchange buffer");
    int64_t blocks = (rows * (F_local / 4) + 255) / 256;
    blocks = blocks < 1 ? 1 : (blocks > 2 * (int64_t)ctx->sm_count ? 2 * (int64_t)ctx->sm_count : blocks);
    return launch_pdl(ctx, swiglu_peer_kernel, dim3((unsigned)blocks), dim3(256), 0, d_gate_up_local, (int)rows, (int)F_local,
                      pg_peer_out(ex, F_total, col0));
}

// qkv [B, (Hq + 2 Hkv) * hd] -> q_rot [B, Hq, hd]; k (rotated) and v written at position *d_pos of the caches
// [B, Hkv, cap, hd].  cos/sin tables: [max_pos, hd/2] with max_pos >= cap.  A position outside [0, cap) is not
// written: the kernel records PG_ERR_INVALID in the context's status word instead.
PG_API int32_t pg_rope_kv_append(pg_ctx *ctx, const float *d_qkv, const int32_t *d_pos, const float *d_cos, const float *d_sin,
                                 int64_t B, int64_t Hq, int64_t Hkv, int64_t hd, int64_t cap, float *d_q_rot, float *d_kcache,
                                 float *d_vcache)
{
    PG_ENTER(ctx);
    PG_REQUIRE(d_qkv && d_pos && d_cos && d_sin && d_q_rot && d_kcache && d_vcache, "rope_kv_append: null pointer");
    PG_REQUIRE(hd % 2 == 0 && hd <= 2048 && B >= 0 && B <= 65535 && cap >= 0 && cap <= 0x7fffffff, "rope_kv_append: bad shape");
    if (B == 0) return PG_OK;
    return launch_pdl(ctx, rope_kv_append_kernel, dim3((unsigned)(Hq + 2 * Hkv), (unsigned)B), dim3((unsigned)(hd / 2)), 0, d_qkv, (const int *)d_pos,
                      d_cos, d_sin, (int)Hq, (int)Hkv, (int)hd, (int)cap, d_q_rot, d_kcache, d_vcache, ctx->d_status);
}

// Attention of one new token per sequence over positions 0..*d_pos (the new one included).
// d_work: B * Hq * S * 130 floats with S = pg_gqa_decode_splits(ctx, B, Hq, Hkv, cap).
PG_API int32_t pg_gqa_decode_splits(pg_ctx *ctx, int64_t B, int64_t Hq, int64_t Hkv, int64_t cap)
{
    if (ctx && Hkv > 0 && Hq % Hkv == 0 && pgk_gqa_stream_supports(Hq / Hkv)) return pgk_gqa_stream_splits(ctx, B, Hkv, cap);
    return cap <= 512 ? 1 : (cap <= 2048 ? 4 : 8);
}

// splits: 0 = pg_gqa_decode_splits' choice; peer: where the merged rows go when the heads are sharded over ranks
static int32_t attention_decode(pg_ctx *ctx, const float *d_q_rot, float *d_kcache, float *d_vcache, const int32_t *d_pos,
                                const float *d_cos, const float *d_sin, int64_t B, int64_t Hq, int64_t Hkv, int64_t hd, int64_t cap,
                                float *d_work, float *d_out, int8_t *d_out_i8, float *d_out_scales, int splits, const PgPeerOut *peer)
{
    PG_REQUIRE(ctx && d_q_rot && d_kcache && d_vcache && d_pos && d_work, "gqa_attention_decode: null pointer");
    PG_REQUIRE(d_out || d_out_i8 || peer, "gqa_attention_decode: no output");
    PG_REQUIRE((d_out_i8 == nullptr) == (d_out_scales == nullptr), "gqa_attention_decode: quantised output needs both buffers");
    PG_REQUIRE(hd == 128, "gqa_attention_decode: head_dim %lld is not supported (128 only)", (long long)hd);
    PG_REQUIRE(Hkv > 0 && Hq % Hkv == 0, "gqa_attention_decode: Hkv must divide Hq");
    PG_REQUIRE(cap > 0 && cap <= 0x7fffffff, "gqa_attention_decode: bad capacity");
    const int64_t G = Hq / Hkv;
    PG_REQUIRE(G == 1 || G == 2 || G == 4 || G == 8, "gqa_attention_decode: %lld query heads per KV head is not supported (1, 2, 4, 8)", (long long)G);
    if (B == 0) return PG_OK;
    const int S = splits > 0 ? splits : pg_gqa_decode_splits(ctx, B, Hq, Hkv, cap);
    PG_REQUIRE(S >= 1 && S <= 64, "gqa_attention_decode: %d slices per (sequence, KV head) (1..64)", S);
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
                        (int)Hkv, (int)cap, chunk, scale, part_o, part_ml, ctx->d_status);                                      \
    }
        if (G == 1) PG_ATT(1) else PG_ATT(2)
#undef PG_ATT
    }
    if (rc) return rc;
    // merge of the partials (+ the quantiser of the output projection's input): a cluster of CTAs per sequence
    int cs = 8;
    while (cs > 1 && (B * cs > 2 * (int64_t)ctx->sm_count || Hq % cs != 0)) cs >>= 1;
    while (Hq / cs > 8 && cs < 8 && Hq % (cs * 2) == 0) cs <<= 1;   // at most 8 heads (1024 threads) per CTA
    const int64_t hpc = Hq / cs;
    if (hpc <= 8 && S <= 64)
        return launch_pdl_cluster(ctx, gqa_combine_quant_kernel, dim3((unsigned)(B * cs)), dim3(128, (unsigned)hpc), 0, cs, (const float *)part_o,
                                  (const float *)part_ml, (int)Hq, S, d_out, d_out_i8, d_out_scales, peer ? *peer : NO_PEER_OUT);
    PG_REQUIRE(!peer, "gqa_attention_decode: %lld heads per rank are too many for the sharded form", (long long)Hq);
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
    PG_ENTER(ctx);
    // the caches are only read on this path
    return attention_decode(ctx, d_q_rot, const_cast<float *>(d_kcache), const_cast<float *>(d_vcache), d_pos, nullptr, nullptr, B, Hq, Hkv, hd,
                            cap, d_work, d_out, d_out_i8, d_out_scales, 0, nullptr);
}

// pg_rope_kv_append + pg_gqa_attention_decode in one launch: d_qkv is the raw [B, (Hq + 2 Hkv) * hd] output of the fused
// Q|K|V projection; the newest token's rotated key and its value are written at position *d_pos of the caches.
PG_API int32_t pg_gqa_attention_decode_fused(pg_ctx *ctx, const float *d_qkv, const int32_t *d_pos, const float *d_cos, const float *d_sin,
                                             float *d_kcache, float *d_vcache, int64_t B, int64_t Hq, int64_t Hkv, int64_t hd, int64_t cap,
                                             float *d_work, float *d_out, int8_t *d_out_i8, float *d_out_scales)
{
    PG_ENTER(ctx);
    PG_REQUIRE(d_cos && d_sin, "gqa_attention_decode_fused: null rotation tables");
    return attention_decode(ctx, d_qkv, d_kcache, d_vcache, d_pos, d_cos, d_sin, B, Hq, Hkv, hd, cap, d_work, d_out, d_out_i8, d_out_scales, 0,
                            nullptr);
}

// The fused form for heads sharded over ranks (whole KV heads with their query heads per rank): Hq and Hkv count THIS
// rank's heads, d_qkv is its [B, (Hq + 2 Hkv) * hd] part of the projection, the caches hold its KV heads.  The merged f32
// rows go to columns [col0, col0 + Hq * hd) of every rank's [B, n_total] exchange buffer (the output projection's
// quantiser needs whole rows: pg_quantize_activations_exchange).  `splits` > 0 fixes the number of context slices per
// (sequence, KV head) -- with the single-GPU value (pg_gqa_decode_splits of the unsharded shape) every partial sum is
// formed in the same order as on one GPU and the rows come out bit-identical; 0 lets this rank's shape decide.
// d_work: B * Hq * S * 130 floats for the S in effect.
PG_API int32_t pg_gqa_attention_decode_fused_exchange(pg_ctx *ctx, const float *d_qkv, const int32_t *d_pos, const float *d_cos,
                                                      const float *d_sin, float *d_kcache, float *d_vcache, int64_t B, int64_t Hq,
                                                      int64_t Hkv, int64_t hd, int64_t cap, float *d_work, int32_t splits,
                                                      pg_exchange *ex, int64_t n_total, int64_t col0)
{
    PG_ENTER(ctx);
    PG_REQUIRE(d_cos && d_sin, "gqa_attention_decode_fused_exchange: null rotation tables");
    PG_REQUIRE(ex && ex->connected, "gqa_attention_decode_fused_exchange: the exchange is not connected");
    PG_REQUIRE(col0 >= 0 && col0 + Hq * hd <= n_total && (size_t)B * (size_t)n_total * sizeof(float) <= ex->y_bytes,
               "gqa_attention_decode_fused_exchange: columns outside the exchange buffer");
    const PgPeerOut po = pg_peer_out(ex, n_total, col0);
    return attention_decode(ctx, d_qkv, d_kcache, d_vcache, d_pos, d_cos, d_sin, B, Hq, Hkv, hd, cap, d_work, nullptr, nullptr, nullptr, splits,
                            &po);
}

PG_API int32_t pg_embedding(pg_ctx *ctx, const float *d_table, const int32_t *d_tokens, int64_t B, int64_t dim, float *d_out)
{
    PG_ENTER(ctx);
    PG_REQUIRE(d_table && d_tokens && d_out && dim % 4 == 0, "embedding: bad arguments");
    if (B == 0) return PG_OK;
    return launch_pdl(ctx, embedding_kernel, dim3((unsigned)B), dim3(256), 0, d_table, (const int *)d_tokens, (int)dim, d_out);
}

// tokens[b] = argmax(logits[b, :]) (first maximum); d_pos (nullable) is advanced by one, but never beyond pos_limit
// (pass the KV capacity; 0 = no limit): a decode loop that runs off the end of its cache stops advancing instead of
// writing behind it.
PG_API int32_t pg_argmax_advance(pg_ctx *ctx, const float *d_logits, int64_t B, int64_t V, int32_t *d_tokens, int32_t *d_pos, int64_t pos_limit)
{
    PG_ENTER(ctx);
    PG_REQUIRE(d_logits && d_tokens && V > 0 && V <= 0x7fffffff, "argmax: bad arguments");
    if (B == 0) return PG_OK;
    const int cs = row_cluster(ctx, B, V, 4096);
    return launch_pdl_cluster(ctx, argmax_kernel, dim3((unsigned)(B * cs)), dim3(1024), 0, cs, d_logits, (int)V, (int *)d_tokens, (int *)d_pos,
                              (int)pos_limit, 0, NO_PEER_OUT);
}

// Greedy choice over a vocabulary sharded by column: this rank's [B, V_local] logits cover columns [v0, v0 + V_local).
// Its per-sequence (maximum, index) pair (8 bytes) goes to every rank's exchange buffer ([B][world][2] floats, the
// index as its bit pattern); pg_pick_embed then chooses.
PG_API int32_t pg_argmax_exchange(pg_ctx *ctx, const float *d_logits_local, int64_t B, int64_t V_local, int64_t v0, pg_exchange *ex)
{
    PG_ENTER(ctx);
    PG_REQUIRE(d_logits_local && ex && ex->connected && V_local > 0 && V_local <= 0x7fffffff && v0 >= 0 && v0 + V_local <= 0x7fffffff,
               "argmax_exchange: bad arguments");
    PG_REQUIRE((size_t)B * ex->world * 2 * sizeof(float) <= ex->y_bytes, "argmax_exchange: the exchange buffer is smaller than [B][world][2] floats");
    if (B == 0) return PG_OK;
    const int cs = row_cluster(ctx, B, V_local, 1024);
    return launch_pdl_cluster(ctx, argmax_kernel, dim3((unsigned)(B * cs)), dim3(1024), 0, cs, d_logits_local, (int)V_local, (int *)nullptr,
                              (int *)nullptr, 0, (int)v0, pg_peer_out(ex, (int64_t)ex->world * 2, (int64_t)ex->rank * 2));
}

// Waits (bounded) for every rank's pair, stores tokens[b] = the first maximum over the whole vocabulary, advances
// d_pos (nullable; never beyond pos_limit, 0 = no limit) and, when d_table is given, gathers the tokens' embedding rows
// [B, dim] for the next step.
PG_API int32_t pg_pick_embed(pg_ctx *ctx, pg_exchange *ex, int64_t B, int32_t *d_tokens, int32_t *d_pos, int64_t pos_limit,
                             const float *d_table, int64_t dim, float *d_out)
{
    PG_ENTER(ctx);
    PG_REQUIRE(ex && ex->connected && d_tokens, "pick_embed: null argument or unconnected exchange");
    PG_REQUIRE(!d_table || (d_out && dim > 0 && dim % 4 == 0), "pick_embed: bad embedding arguments");
    if (B == 0) return PG_OK;
    return launch_pdl(ctx, pick_embed_kernel, dim3((unsigned)B), dim3(256), 0, ex->world, (int *)d_tokens, (int *)d_pos,
                      (int)pos_limit, d_table, (int)dim, d_out, pg_peer_wait_of(ctx, ex));
}

}  // extern "C"
