// GQA attention of one new token per sequence against the f32 KV cache, head_dim 128, for 4 or 8
// query heads per KV head (src/attention.rs:141-265: dot * 1/sqrt(hd), softmax, weighted sum of V).
//
// The step reads every cached K and V row once (2 x 512 bytes per position and KV head) and does
// almost no arithmetic, so the kernel is built like the streaming products: keep HBM requests in
// flight and never let the stream drain.
//
//   * One persistent CTA of 12 warps per SM.  A unit of work is (sequence, KV head, slice of the
//     context); there are `S` slices per (sequence, KV head), chosen so that the units about fill
//     the GPU's warps, and a WARP owns a unit.  No block-wide barrier after start-up.
//   * K and V rows of consecutive positions are contiguous in the cache, so a warp streams its
//     slice in batches of P = 32 / G positions with two bulk asynchronous copies per batch (P x 512
//     bytes of K, the same of V) into a private two-slot ring, completion on an mbarrier.
//   * Scores: each lane multiplies its four head-dim elements for the P x G (position, head) pairs,
//     and one 32 x 32 butterfly (31 shuffles) leaves lane i with the complete dot product of pair i.
//   * Online softmax per head (running maximum shared by the lanes of a head, running sum kept per
//     lane and added up once at the end), probabilities handed to all lanes through 128 bytes of
//     shared memory, then the weighted sum of V with the lane's four head-dim elements per head.
//   * The unit writes its unnormalised output with (max, sum); a second small kernel merges the S
//     partials of every (sequence, query head).
//   * FUSED form: the kernel takes the raw output of the fused Q|K|V projection instead of rotated
//     queries and an already appended cache.  Every warp rotates the query heads of its unit itself
//     (RoPE, src/nn.rs:1322-1338: the halves of a head live 16 lanes apart, one shuffle each), and
//     the warp whose slice holds the newest position rotates that token's key, writes key and value
//     to the cache (KVCache::append, src/attention.rs:65-83) and into its ring slot, from where they
//     are used like every other row.  One launch less per layer.
//
// The mbarrier waits are bounded (about a second): on expiry the warp records
// PG_ERR_DEVICE_TIMEOUT in the context's status word and leaves.
#include <math.h>

#include <algorithm>

#include "pg_internal.cuh"

namespace {

constexpr int AT_WARPS = 12;
constexpr int AT_THREADS = AT_WARPS * 32;
constexpr int AT_SLOTS = 2;
constexpr int AT_HD = 128;

__device__ __forceinline__ unsigned long long at_globaltimer()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void at_mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void at_mbar_expect(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool at_mbar_try(uint32_t bar, uint32_t parity)
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
__device__ __forceinline__ bool at_mbar_wait(uint32_t bar, uint32_t parity, int32_t *status, unsigned long long limit_ns)
{
    unsigned long long t0 = 0;
    for (uint32_t it = 1;; ++it) {
        if (at_mbar_try(bar, parity)) return true;
        if ((it & 0xff) == 0) {
            const unsigned long long now = at_globaltimer();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > limit_ns) {
                atomicExch(status, (int32_t)PG_ERR_DEVICE_TIMEOUT);
                return false;
            }
        }
    }
}
__device__ __forceinline__ void at_bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ float4 at_lds128(uint32_t addr)
{
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}

// Slices of the context: `S` per (sequence, KV head), each a whole number of batches.
__host__ __device__ inline int at_chunk(int len, int S, int P) { return (((len + S - 1) / S) + P - 1) / P * P; }

// RoPE of the four elements this lane holds of one head (elements 4 * lane .. 4 * lane + 3): the partner half is 16 lanes away.
// Same operations, in the same order, as rope_kv_append_kernel.
__device__ __forceinline__ float4 at_rope(float4 mine, float4 cs, float4 sn, int lane)
{
    float4 other;
    other.x = __shfl_xor_sync(0xffffffffu, mine.x, 16);
    other.y = __shfl_xor_sync(0xffffffffu, mine.y, 16);
    other.z = __shfl_xor_sync(0xffffffffu, mine.z, 16);
    other.w = __shfl_xor_sync(0xffffffffu, mine.w, 16);
    float4 r;
    if (lane < 16) {   // first half: x0 * c - x1 * s
        r.x = __fsub_rn(__fmul_rn(mine.x, cs.x), __fmul_rn(other.x, sn.x));
        r.y = __fsub_rn(__fmul_rn(mine.y, cs.y), __fmul_rn(other.y, sn.y));
        r.z = __fsub_rn(__fmul_rn(mine.z, cs.z), __fmul_rn(other.z, sn.z));
        r.w = __fsub_rn(__fmul_rn(mine.w, cs.w), __fmul_rn(other.w, sn.w));
    } else {           // second half: x0 * s + x1 * c
        r.x = __fadd_rn(__fmul_rn(other.x, sn.x), __fmul_rn(mine.x, cs.x));
        r.y = __fadd_rn(__fmul_rn(other.y, sn.y), __fmul_rn(mine.y, cs.y));
        r.z = __fadd_rn(__fmul_rn(other.z, sn.z), __fmul_rn(mine.z, cs.z));
        r.w = __fadd_rn(__fmul_rn(other.w, sn.w), __fmul_rn(mine.w, cs.w));
    }
    return r;
}

// G query heads per KV head.  part_o [B*Hq][S][128], part_ml [B*Hq][S][2].
// FUSED: q is the raw [B, (Hq + 2 Hkv) * 128] output of the Q|K|V projection, kc / vc are written at the newest position.
template <int G, bool FUSED>
__global__ void __launch_bounds__(AT_THREADS, 1)
    gqa_decode_stream_kernel(const float *__restrict__ q, float *__restrict__ kc, float *__restrict__ vc,
                             const int *__restrict__ pos_ptr, const float *__restrict__ cos_t, const float *__restrict__ sin_t, int B, int Hq,
                             int Hkv, int cap, int S, float scale, float *__restrict__ part_o, float *__restrict__ part_ml, int32_t *status,
                             unsigned long long limit_ns)
{
    constexpr int P = 32 / G;                 // positions per batch
    constexpr int SLOT = P * AT_HD * 4;       // bytes of K (or V) per batch
    constexpr int WARP_BYTES = AT_SLOTS * 2 * SLOT + 128;
    extern __shared__ __align__(128) unsigned char smem[];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t base = (uint32_t)__cvta_generic_to_shared(smem) + (uint32_t)warp * WARP_BYTES;
    const uint32_t kring = base, vring = base + AT_SLOTS * SLOT, pbuf = base + AT_SLOTS * 2 * SLOT;
    const uint32_t bars = (uint32_t)__cvta_generic_to_shared(smem) + AT_WARPS * WARP_BYTES + (uint32_t)warp * (AT_SLOTS * 8);
    if (lane == 0) {
        for (int i = 0; i < AT_SLOTS; i++) at_mbar_init(bars + 8 * i, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    // the newest K/V row, q and the position come from the preceding kernels
    asm volatile("griddepcontrol.wait;" ::: "memory");

    int len = pg_ld_fresh(pos_ptr) + 1;
    if ((unsigned)(len - 1) >= (unsigned)cap) {
        // the position lies outside the cache (and the rotation tables): record it and treat the context as empty, so
        // that nothing is read or written past an allocation; every unit then reports an empty slice
        if (threadIdx.x == 0) atomicExch(status, (int32_t)PG_ERR_INVALID);
        len = 0;
    }
    float4 rope_c = make_float4(1.f, 1.f, 1.f, 1.f), rope_s = make_float4(0.f, 0.f, 0.f, 0.f);
    if (FUSED && len > 0) {       // the row of the cos / sin tables of the newest position, [max_pos, 64]
        rope_c = __ldg(reinterpret_cast<const float4 *>(cos_t + (int64_t)(len - 1) * (AT_HD / 2)) + (lane & 15));
        rope_s = __ldg(reinterpret_cast<const float4 *>(sin_t + (int64_t)(len - 1) * (AT_HD / 2)) + (lane & 15));
    }
    const int qkv_heads = Hq + 2 * Hkv;
    const int chunk = at_chunk(len, S, P);
    const int units = B * Hkv * S;
    const int my_p = lane / G;             // lane i holds pair (position i / G, head i % G) after the butterfly
    uint32_t fills = 0;                       // ring fills so far: slot = fills % 2, parity = (fills / 2) & 1

    // unit -> (CTA u % grid, warp u / grid): every SM gets work even when the units do not fill the last CTAs' warps
    for (int u = warp * gridDim.x + blockIdx.x; u < units; u += gridDim.x * AT_WARPS) {
        const int pair = u / S, split = u - pair * S;
        const int b = pair / Hkv, kvh = pair - b * Hkv;
        const int t0 = split * chunk, n = min(len, t0 + chunk) - t0;
        float *po = part_o + (((int64_t)b * Hq + kvh * G) * S + split) * AT_HD;   // + h * S * 128
        float *pml = part_ml + (((int64_t)b * Hq + kvh * G) * S + split) * 2;     // + h * S * 2
        if (n <= 0) {
            if (lane < G) {
                pml[(int64_t)lane * S * 2] = -INFINITY;
                pml[(int64_t)lane * S * 2 + 1] = 0.0f;
            }
            continue;
        }
        const int nb = (n + P - 1) / P;
        const char *kbase = reinterpret_cast<const char *>(kc + (((int64_t)b * Hkv + kvh) * cap + t0) * AT_HD);
        const char *vbase = reinterpret_cast<const char *>(vc + (((int64_t)b * Hkv + kvh) * cap + t0) * AT_HD);
        auto issue = [&](int bi, uint32_t f) {
            if (lane == 0) {
                const uint32_t bytes = (uint32_t)min(P, n - bi * P) * (AT_HD * 4);
                const uint32_t bar = bars + (f % AT_SLOTS) * 8;
                at_mbar_expect(bar, 2 * bytes);
                at_bulk_load(kring + (f % AT_SLOTS) * SLOT, kbase + (int64_t)bi * SLOT, bytes, bar);
                at_bulk_load(vring + (f % AT_SLOTS) * SLOT, vbase + (int64_t)bi * SLOT, bytes, bar);
            }
        };
#pragma unroll
        for (int i = 0; i < AT_SLOTS; i++)
            if (i < nb) issue(i, fills + i);

        float4 qv[G];
#pragma unroll
        for (int h = 0; h < G; h++) {
            if (FUSED) {
                const float4 raw = pg_ld_fresh(reinterpret_cast<const float4 *>(q + ((int64_t)b * qkv_heads + kvh * G + h) * AT_HD) + lane);
                qv[h] = at_rope(raw, rope_c, rope_s, lane);
            } else {
                qv[h] = pg_ld_fresh(reinterpret_cast<const float4 *>(q + ((int64_t)b * Hq + kvh * G + h) * AT_HD) + lane);
            }
        }
        // FUSED: this unit appends the newest token's key and value if its slice holds position len - 1
        const bool appends = FUSED && (t0 + n == len);
        float4 k_new = make_float4(0.f, 0.f, 0.f, 0.f), v_new = k_new;
        if (appends) {
            const float4 kraw = pg_ld_fresh(reinterpret_cast<const float4 *>(q + ((int64_t)b * qkv_heads + Hq + kvh) * AT_HD) + lane);
            k_new = at_rope(kraw, rope_c, rope_s, lane);
            v_new = pg_ld_fresh(reinterpret_cast<const float4 *>(q + ((int64_t)b * qkv_heads + Hq + Hkv + kvh) * AT_HD) + lane);
            const int64_t at = (((int64_t)b * Hkv + kvh) * cap + (len - 1)) * AT_HD;
            reinterpret_cast<float4 *>(kc + at)[lane] = k_new;
            reinterpret_cast<float4 *>(vc + at)[lane] = v_new;
        }
        float m_run = -INFINITY, l_run = 0.0f;
        float4 acc[G];
#pragma unroll
        for (int h = 0; h < G; h++) acc[h] = make_float4(0.f, 0.f, 0.f, 0.f);

        for (int bi = 0; bi < nb; bi++, fills++) {
            const uint32_t slot = fills % AT_SLOTS;
            if (!at_mbar_wait(bars + slot * 8, (fills / AT_SLOTS) & 1u, status, limit_ns)) return;
            const int valid = min(P, n - bi * P);
            if (appends && bi == nb - 1) {
                // the bulk copy brought the cache's old bytes for the newest position: put the new row in its place
                const uint32_t off = slot * SLOT + (uint32_t)(valid - 1) * (AT_HD * 4) + lane * 16;
                asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(kring + off), "f"(k_new.x), "f"(k_new.y), "f"(k_new.z), "f"(k_new.w) : "memory");
                asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(vring + off), "f"(v_new.x), "f"(v_new.y), "f"(v_new.z), "f"(v_new.w) : "memory");
                __syncwarp();
            }
            // partial dot products of this lane's four elements: v[p * G + h]
            float v[32];
#pragma unroll
            for (int p = 0; p < P; p++) {
                const float4 kv = at_lds128(kring + slot * SLOT + p * (AT_HD * 4) + lane * 16);
#pragma unroll
                for (int h = 0; h < G; h++) v[p * G + h] = qv[h].x * kv.x + qv[h].y * kv.y + qv[h].z * kv.z + qv[h].w * kv.w;
            }
            // butterfly: lane i ends with the sum over all lanes of v[i]
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) {
                const bool up = (lane & off) != 0;
#pragma unroll
                for (int jx = 0; jx < off; jx++) {
                    const float send = up ? v[jx] : v[jx + off];
                    const float keep = up ? v[jx + off] : v[jx];
                    v[jx] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                }
            }
            const float s = (my_p < valid) ? v[0] * scale : -INFINITY;   // rows past the slice hold stale bytes: masked here, skipped below
            float bm = s;
#pragma unroll
            for (int off = G; off < 32; off <<= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, off));
            const float m_new = fmaxf(m_run, bm);                // finite: the batch has at least one valid position
            const float corr = expf(m_run - m_new);              // 0 on the first batch
            const float pr = expf(s - m_new);                    // 0 for masked pairs
            l_run = fmaf(l_run, corr, pr);
            m_run = m_new;
            asm volatile("st.shared.f32 [%0], %1;" ::"r"(pbuf + lane * 4), "f"(pr) : "memory");
#pragma unroll
            for (int h = 0; h < G; h++) {
                const float c = __shfl_sync(0xffffffffu, corr, h);   // lane h belongs to head h
                acc[h].x *= c;
                acc[h].y *= c;
                acc[h].z *= c;
                acc[h].w *= c;
            }
            __syncwarp();
#pragma unroll
            for (int p = 0; p < P; p++) {
                if (p < valid) {
                    const float4 vv = at_lds128(vring + slot * SLOT + p * (AT_HD * 4) + lane * 16);
                    float pp[G];
#pragma unroll
                    for (int h4 = 0; h4 < G; h4 += 4) {
                        const float4 t4 = at_lds128(pbuf + (p * G + h4) * 4);
                        pp[h4] = t4.x;
                        pp[h4 + 1] = t4.y;
                        pp[h4 + 2] = t4.z;
                        pp[h4 + 3] = t4.w;
                    }
#pragma unroll
                    for (int h = 0; h < G; h++) {
                        acc[h].x = fmaf(pp[h], vv.x, acc[h].x);
                        acc[h].y = fmaf(pp[h], vv.y, acc[h].y);
                        acc[h].z = fmaf(pp[h], vv.z, acc[h].z);
                        acc[h].w = fmaf(pp[h], vv.w, acc[h].w);
                    }
                }
            }
            __syncwarp();                                        // every lane is done with the slot and with pbuf
            if (bi + AT_SLOTS < nb) issue(bi + AT_SLOTS, fills + AT_SLOTS);
        }
        // the lanes of a head add up their sums
        float l = l_run;
#pragma unroll
        for (int off = G; off < 32; off <<= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
        if (lane < G) {
            pml[(int64_t)lane * S * 2] = m_run;
            pml[(int64_t)lane * S * 2 + 1] = l;
        }
#pragma unroll
        for (int h = 0; h < G; h++) reinterpret_cast<float4 *>(po + (int64_t)h * S * AT_HD)[lane] = acc[h];
    }
}

template <int G>
constexpr int at_smem_bytes()
{
    return AT_WARPS * (AT_SLOTS * 2 * (32 / G) * AT_HD * 4 + 128) + AT_WARPS * AT_SLOTS * 8;
}

}  // namespace

// Slices per (sequence, KV head): enough units to give every warp of the GPU one, never shorter than 64 positions.
int pgk_gqa_stream_splits(const pg_ctx *ctx, int64_t B, int64_t Hkv, int64_t cap)
{
    const int64_t pairs = std::max<int64_t>(1, B * Hkv);
    const int64_t warps = (int64_t)ctx->sm_count * AT_WARPS;
    int64_t S = std::max<int64_t>(1, warps / pairs);
    S = std::min<int64_t>(S, std::max<int64_t>(1, cap / 64));
    S = std::min<int64_t>(S, 64);                 // the merge kernel keeps one weight per slice in shared memory
    return (int)S;
}

bool pgk_gqa_stream_supports(int64_t G) { return G == 4 || G == 8; }

int32_t pgk_gqa_decode_stream(pg_ctx *ctx, const float *d_q, float *d_k, float *d_v, const int32_t *d_pos, const float *d_cos,
                              const float *d_sin, int64_t B, int64_t Hq, int64_t Hkv, int64_t cap, int S, float scale, float *part_o,
                              float *part_ml)
{
    // d_cos != NULL: d_q is the raw Q|K|V projection; the kernel applies RoPE and appends the newest key and value
    const bool fused = d_cos != nullptr;
    const int G = (int)(Hq / Hkv);
    const int64_t units = B * Hkv * S;
    PG_REQUIRE(units <= 0x7fffffff, "gqa_attention_decode: too many (sequence, head, slice) units");
    const int grid = (int)std::min<int64_t>(ctx->sm_count, units);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(AT_THREADS);
    cfg.stream = ctx->stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
#define PG_AT_CASE(GG, FF)                                                                                                              \
    {                                                                                                                                   \
        cfg.dynamicSmemBytes = at_smem_bytes<GG>();                                                                                     \
        static std::atomic<uint64_t> smem_set{0};                                                                                       \
        PG_CUDA(pg_max_smem_once(gqa_decode_stream_kernel<GG, FF>, at_smem_bytes<GG>(), ctx->device, smem_set));                        \
        PG_CUDA(cudaLaunchKernelEx(&cfg, gqa_decode_stream_kernel<GG, FF>, d_q, d_k, d_v, (const int *)d_pos, d_cos, d_sin, (int)B, (int)Hq, \
                                   (int)Hkv, (int)cap, S, scale, part_o, part_ml, ctx->d_status, ctx->wait_limit_ns));                  \
    }
    if (G == 4) {
        if (fused) PG_AT_CASE(4, true) else PG_AT_CASE(4, false)
    } else {
        if (fused) PG_AT_CASE(8, true) else PG_AT_CASE(8, false)
    }
#undef PG_AT_CASE
    PG_LAUNCHED();
    return PG_OK;
}
