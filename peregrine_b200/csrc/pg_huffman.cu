// Huffman-coded int8 weights, decoded on the GPU.
//
// The format is the reference's (src/huffman.rs:216-284): one canonical code of at most 12 bits shared by
// `num_streams` bitstreams, bits written MSB first, the last byte of a stream padded with zeros, no
// markers inside a stream.  The reference decodes on the host, one symbol after the other through a
// 4096-entry table indexed by the next 12 bits (src/huffman.rs:254-284) and uploads the bytes
// (to_gpu, src/huffman.rs:430-437).  Here the COMPRESSED bytes cross PCIe and every stream is decoded by
// thousands of threads:
//
//   * a stream is cut into subsequences of 2048 bits; thread i owns the code words that START in
//     subsequence i.  Where its first code word starts is unknown at first (only subsequence 0 starts
//     at bit 0), so the decode is a fixed-point iteration: every thread decodes from its current guess
//     and hands the position where it left its subsequence to its right-hand neighbour, which decodes
//     again if that changed.  Prefix codes resynchronise after a few code words, so the guesses settle
//     in two or three sweeps; the iteration is exact whatever the code (once start[i+1] == end[i] for
//     every i the chain is the sequential one) and bounded by the number of subsequences.
//     A block of 128 threads iterates its 128 subsequences in shared memory; the position handed from
//     one block to the next goes through global memory and a relaunch.
//   * an exclusive scan of the symbols per subsequence gives every thread its place in the output;
//   * a last sweep decodes once more and writes the symbols.
//
// A table entry of length 0 (no code starts with those bits: an incomplete or damaged code) stops the
// sequential decoder's cursor for good, and a stream that ends before its symbols do is decoded from
// zero padding.  Neither can come out of HuffmanTensor::from_quantized; both are decoded the way the
// reference does it, by one thread per stream (decode_serial_kernel), so that results match bit for bit.
#include "pg_internal.cuh"

#include <vector>

namespace {

constexpr int HF_LUT_BITS = 12;                 // MAX_LUT_BITS (src/huffman.rs:13)
constexpr int HF_LUT_SIZE = 1 << HF_LUT_BITS;
constexpr int HF_SUB_BITS = 2048;               // bits per subsequence
constexpr int HF_SUB_WORDS = HF_SUB_BITS / 32;  // 64
constexpr int HF_THREADS = 128;                 // subsequences per block
constexpr int HF_CHUNK_WORDS = HF_THREADS * HF_SUB_WORDS + 2;   // the block's bits plus the 44 a window may run over

struct hf_stream {
    uint64_t byte_off;   // of the stream in the uploaded buffer
    uint64_t bytes;
    uint64_t symbols;
    uint64_t out_off;    // of its first symbol in the output
    uint32_t first_block;
    uint32_t blocks;
};

// word w of the block's chunk lives at w + w/64: one pad word per subsequence, so that threads that are at the
// same depth of their subsequences hit 32 different banks
__device__ __forceinline__ int hf_slot(int w) { return w + (w >> 6); }

// Big-endian words of stream bytes [4*w0, 4*w0 + 4*n) into shared memory, zeros past the end of the stream.
__device__ __forceinline__ void hf_stage(const uint8_t *__restrict__ base, uint64_t bytes, uint64_t w0, uint32_t *s_bits)
{
    const uintptr_t addr = (uintptr_t)base;
    const uint32_t mis = (uint32_t)(addr & 3);
    const uint32_t *aligned = (const uint32_t *)(addr - mis);   // the buffer starts on a word and has 8 bytes of slack at its end
    for (int w = threadIdx.x; w < HF_CHUNK_WORDS; w += HF_THREADS) {
        const uint64_t b = (w0 + (uint64_t)w) * 4;
        uint32_t v = 0;
        if (b < bytes) {
            const uint32_t lo = aligned[b / 4];
            v = mis ? __funnelshift_r(lo, aligned[b / 4 + 1], mis * 8) : lo;    // little-endian: byte 0 of the stream in the low byte
            if (b + 4 > bytes) v &= 0xFFFFFFFFu >> (8 * (uint32_t)(b + 4 - bytes));
            v = __byte_perm(v, 0, 0x0123);                      // first bit of the stream in bit 31
        }
        s_bits[hf_slot(w)] = v;
    }
}

__device__ __forceinline__ uint32_t hf_window(const uint32_t *s_bits, uint32_t pos)
{
    const int w = (int)(pos >> 5);
    return __funnelshift_l(s_bits[hf_slot(w + 1)], s_bits[hf_slot(w)], pos & 31) >> (32 - HF_LUT_BITS);
}

// One sweep of the fixed-point iteration.  start[g]: bit offset, inside subsequence g, of the first code word
// that starts there; count[g]: code words that start there; dirty0[b]: the start of block b's first subsequence
// was changed by the block before it.  *changed counts the hand-overs that crossed a block boundary.
__global__ void __launch_bounds__(HF_THREADS)
    huffman_sync_kernel(const uint8_t *__restrict__ data, const hf_stream *__restrict__ streams, const uint32_t *__restrict__ block_stream,
                        const uint16_t *__restrict__ lut, uint32_t *start, uint32_t *count, uint32_t *dirty0, uint32_t *block_sum,
                        int first_sweep, uint32_t *changed, uint32_t *malformed)
{
    __shared__ uint32_t s_bits[HF_CHUNK_WORDS + HF_CHUNK_WORDS / 64 + 1];
    __shared__ uint16_t s_lut[HF_LUT_SIZE];
    __shared__ uint32_t s_start[HF_THREADS + 1];
    __shared__ uint32_t s_dirty[HF_THREADS + 1];
    __shared__ uint32_t s_red[HF_THREADS / 32];
    __shared__ uint32_t s_flag;

    const uint32_t b = blockIdx.x, t = threadIdx.x;
    if (t == 0) s_flag = first_sweep ? 1u : atomicExch(&dirty0[b], 0u);
    __syncthreads();
    if (!s_flag) return;
    __threadfence();   // the start that came with the flag

    const hf_stream st = streams[block_stream[b]];
    const uint32_t sub0 = (b - st.first_block) * HF_THREADS;               // first subsequence of this block in its stream
    const uint64_t total_bits = st.bytes * 8;
    const uint64_t nsub = (total_bits + HF_SUB_BITS - 1) / HF_SUB_BITS;
    const uint64_t sub = (uint64_t)sub0 + t;
    const bool valid = sub < nsub;
    const size_t g = (size_t)b * HF_THREADS + t;

    for (int i = t; i < HF_LUT_SIZE; i += HF_THREADS) s_lut[i] = lut[i];
    hf_stage(data + st.byte_off, st.bytes, (uint64_t)sub0 * HF_SUB_WORDS, s_bits);
    if (first_sweep) {
        s_start[t] = 0;
        s_dirty[t] = 1;
    } else {
        s_start[t] = pg_ld_fresh(&start[g]);
        s_dirty[t] = (t == 0);
    }
    if (t == 0) s_dirty[HF_THREADS] = 0;
    __syncthreads();

    uint32_t n = first_sweep ? 0 : count[g];
    const uint32_t limit = valid ? (uint32_t)min((uint64_t)HF_SUB_BITS, total_bits - sub * HF_SUB_BITS) : 0;
    for (int sweep = 0; sweep <= HF_THREADS; sweep++) {
        bool handed = false;
        uint32_t next = 0;
        if (valid && s_dirty[t]) {
            uint32_t pos = s_start[t];
            n = 0;
            while (pos < limit) {
                const uint32_t e = s_lut[hf_window(s_bits, t * HF_SUB_BITS + pos)];
                if ((e >> 8) == 0) {   // the sequential decoder would stay here for good
                    atomicOr(malformed, 1u);
                    pos = HF_SUB_BITS;
                    break;
                }
                pos += e >> 8;
                n++;
            }
            next = pos - HF_SUB_BITS;
            handed = sub + 1 < nsub;
        }
        __syncthreads();
        s_dirty[t] = 0;
        __syncthreads();
        bool again = false;
        if (handed) {
            if (t + 1 < HF_THREADS) {
                if (s_start[t + 1] != next) {
                    s_start[t + 1] = next;
                    s_dirty[t + 1] = 1;
                    again = true;
                }
            } else if (pg_ld_fresh(&start[g + 1]) != next || first_sweep) {
                // the next block's first subsequence: through global memory, picked up by the next launch
                start[g + 1] = next;
                __threadfence();
                atomicExch(&dirty0[b + 1], 1u);
                atomicAdd(changed, 1u);
            }
        }
        if (!__syncthreads_or(again)) break;
    }
    // the start of the block's first subsequence belongs to the block before it (to nobody at the head of a stream)
    if (t > 0 || (sub0 == 0 && first_sweep)) start[g] = s_start[t];
    count[g] = valid ? n : 0;
    // symbols of the block, for the scan over blocks
    uint32_t v = valid ? n : 0;
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    if ((t & 31) == 0) s_red[t >> 5] = v;
    __syncthreads();
    if (t == 0) block_sum[b] = s_red[0] + s_red[1] + s_red[2] + s_red[3];
}

// Exclusive scan of block_sum inside every stream (one warp per stream); a stream that holds fewer code words
// than symbols is flagged: the sequential decoder reads it on into the zero padding.
__global__ void huffman_scan_kernel(const hf_stream *__restrict__ streams, int num_streams, const uint32_t *__restrict__ block_sum,
                                    uint64_t *block_off, uint32_t *malformed)
{
    const int s = blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (s >= num_streams) return;
    const hf_stream st = streams[s];
    uint64_t run = 0;
    for (uint32_t i0 = 0; i0 < st.blocks; i0 += 32) {
        const uint32_t i = i0 + lane;
        const uint64_t v = i < st.blocks ? pg_ld_fresh(&block_sum[st.first_block + i]) : 0;
        uint64_t inc = v;
        for (int o = 1; o < 32; o <<= 1) {
            const uint64_t up = __shfl_up_sync(0xFFFFFFFFu, inc, o);
            if (lane >= o) inc += up;
        }
        if (i < st.blocks) block_off[st.first_block + i] = run + inc - v;
        run += __shfl_sync(0xFFFFFFFFu, inc, 31);
    }
    if (lane == 0 && run < st.symbols) atomicOr(malformed, 1u);
}

// The last sweep: decode from the settled starts and write the symbols.
__global__ void __launch_bounds__(HF_THREADS)
    huffman_write_kernel(const uint8_t *__restrict__ data, const hf_stream *__restrict__ streams, const uint32_t *__restrict__ block_stream,
                         const uint16_t *__restrict__ lut, const uint32_t *__restrict__ start, const uint32_t *__restrict__ count,
                         const uint64_t *__restrict__ block_off, int8_t *__restrict__ out)
{
    __shared__ uint32_t s_bits[HF_CHUNK_WORDS + HF_CHUNK_WORDS / 64 + 1];
    __shared__ uint16_t s_lut[HF_LUT_SIZE];
    __shared__ uint32_t s_red[HF_THREADS / 32];

    const uint32_t b = blockIdx.x, t = threadIdx.x;
    const hf_stream st = streams[block_stream[b]];
    const uint32_t sub0 = (b - st.first_block) * HF_THREADS;
    const uint64_t total_bits = st.bytes * 8;
    const uint64_t nsub = (total_bits + HF_SUB_BITS - 1) / HF_SUB_BITS;
    const uint64_t sub = (uint64_t)sub0 + t;
    const bool valid = sub < nsub;
    const size_t g = (size_t)b * HF_THREADS + t;

    for (int i = t; i < HF_LUT_SIZE; i += HF_THREADS) s_lut[i] = lut[i];
    hf_stage(data + st.byte_off, st.bytes, (uint64_t)sub0 * HF_SUB_WORDS, s_bits);

    // exclusive scan of the counts inside the block
    const uint32_t n = pg_ld_fresh(&count[g]);
    uint32_t inc = n;
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t up = __shfl_up_sync(0xFFFFFFFFu, inc, o);
        if ((t & 31) >= o) inc += up;
    }
    if ((t & 31) == 31) s_red[t >> 5] = inc;
    __syncthreads();
    uint32_t before = inc - n;
    for (int w = 0; w < (int)(t >> 5); w++) before += s_red[w];

    if (!valid) return;
    uint64_t idx = pg_ld_fresh(&block_off[b]) + before;         // index of this thread's first symbol in its stream
    if (idx >= st.symbols) return;                              // code words decoded from the padding of the last byte
    const uint32_t limit = (uint32_t)min((uint64_t)HF_SUB_BITS, total_bits - sub * HF_SUB_BITS);
    uint32_t pos = pg_ld_fresh(&start[g]);
    int8_t *dst = out + st.out_off;
    const uint64_t room = st.symbols - idx;
    uint32_t left = (uint32_t)min((uint64_t)n, room);
    // bytes up to the next 4-byte boundary of the output, then words, then the tail
    uint32_t word = 0, have = 0;
    while (pos < limit && left) {
        const uint32_t e = s_lut[hf_window(s_bits, t * HF_SUB_BITS + pos)];
        pos += e >> 8;
        const uint32_t sym = ((e & 0xFFu) - 128u) & 0xFFu;      // table entries hold symbol + 128 (to_gpu_lut, src/huffman.rs:726-737)
        left--;
        if (have == 0 && (((uintptr_t)(dst + idx)) & 3) != 0) {
            dst[idx++] = (int8_t)sym;
            continue;
        }
        word |= sym << (8 * have);
        if (++have == 4) {
            *(uint32_t *)(dst + idx) = word;
            idx += 4;
            word = 0;
            have = 0;
        }
    }
    for (uint32_t i = 0; i < have; i++) dst[idx + i] = (int8_t)(word >> (8 * i));
}

// The reference's loop, one thread per stream (src/huffman.rs:254-284), for streams the parallel decoder flags.
__global__ void huffman_decode_serial_kernel(const uint8_t *__restrict__ data, const hf_stream *__restrict__ streams, int num_streams,
                                             const uint16_t *__restrict__ lut, int8_t *__restrict__ out)
{
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= num_streams) return;
    const hf_stream st = streams[s];
    const uint8_t *bits = data + st.byte_off;
    const uint64_t total_bits = st.bytes * 8;
    uint64_t pos = 0;
    for (uint64_t i = 0; i < st.symbols; i++) {
        uint32_t code = 0;
#pragma unroll
        for (int k = 0; k < 3; k++) {   // 12 bits at any bit offset lie in 3 bytes
            const uint64_t byte = (pos >> 3) + k;
            code = (code << 8) | (byte * 8 < total_bits ? bits[byte] : 0u);
        }
        code = (code >> (12 - (uint32_t)(pos & 7))) & (HF_LUT_SIZE - 1);
        const uint32_t e = lut[code];
        out[st.out_off + i] = (int8_t)(((e & 0xFFu) - 128u) & 0xFFu);
        pos += e >> 8;
    }
}

// canonical_codes + build_decode_lut (src/huffman.rs:155-213) in the packing of to_gpu_lut (src/huffman.rs:726-737).
// Returns false where the reference's table construction would index past its 4096 entries (a panic there).
bool build_lut(const uint8_t *bit_lengths, uint16_t *lut)
{
    for (int i = 0; i < HF_LUT_SIZE; i++) lut[i] = 128;   // (symbol 0, length 0)
    uint32_t per_len[257] = {0}, next[258] = {0};
    int longest = 0;
    for (int s = 0; s < 256; s++) {
        per_len[bit_lengths[s]]++;
        if (bit_lengths[s] > longest) longest = bit_lengths[s];
    }
    per_len[0] = 0;
    uint32_t code = 0;
    for (int len = 1; len <= longest; len++) {
        code = (code + per_len[len - 1]) << 1;
        next[len] = code;
    }
    for (int s = 0; s < 256; s++) {
        const int len = bit_lengths[s];
        if (len == 0) continue;
        const uint32_t c = next[len]++;
        if (len > HF_LUT_BITS) continue;                  // the reference leaves such a symbol out of the table
        const uint32_t base = c << (HF_LUT_BITS - len), span = 1u << (HF_LUT_BITS - len);
        if ((uint64_t)base + span > HF_LUT_SIZE) return false;
        for (uint32_t j = 0; j < span; j++) lut[base + j] = (uint16_t)((len << 8) | s);
    }
    return true;
}

}  // namespace

// Streams back to back in `d_data` (the layout of the serial format, src/serial.rs:320-365) -> symbols back to back in d_out.
int32_t pgk_huffman_decode(pg_ctx *ctx, const uint8_t *bit_lengths, int64_t num_streams, const uint64_t *stream_symbols,
                           const uint64_t *stream_bytes, const uint8_t *d_data, int8_t *d_out)
{
    std::vector<uint16_t> lut(HF_LUT_SIZE);
    PG_REQUIRE(build_lut(bit_lengths, lut.data()), "huffman: the bit lengths do not describe a code of at most 12 bits");
    std::vector<hf_stream> st((size_t)num_streams);
    std::vector<uint32_t> block_stream;
    uint64_t byte_off = 0, out_off = 0;
    for (int64_t s = 0; s < num_streams; s++) {
        hf_stream &h = st[(size_t)s];
        h.byte_off = byte_off;
        h.bytes = stream_bytes[s];
        h.symbols = stream_symbols[s];
        h.out_off = out_off;
        const uint64_t nsub = (h.bytes * 8 + HF_SUB_BITS - 1) / HF_SUB_BITS;
        const uint64_t blocks = (nsub + HF_THREADS - 1) / HF_THREADS;
        PG_REQUIRE(block_stream.size() + blocks < (1ull << 31), "huffman: streams too long");
        h.first_block = (uint32_t)block_stream.size();
        h.blocks = (uint32_t)blocks;
        block_stream.insert(block_stream.end(), (size_t)blocks, (uint32_t)s);
        byte_off += h.bytes;
        out_off += h.symbols;
    }
    if (out_off == 0) return PG_OK;
    const size_t nb = block_stream.size();

    // one allocation: table | streams | block -> stream | start | count | dirty | block sums | block offsets | flags
    size_t off = 0;
    auto take = [&off](size_t bytes) { const size_t at = off; off += (bytes + 255) / 256 * 256; return at; };
    const size_t o_lut = take(HF_LUT_SIZE * 2), o_st = take(st.size() * sizeof(hf_stream)), o_bs = take((nb + 1) * 4),
                 o_start = take((nb * HF_THREADS + 1) * 4), o_count = take(nb * HF_THREADS * 4 + 4), o_dirty = take((nb + 1) * 4),
                 o_sum = take((nb + 1) * 4), o_boff = take((nb + 1) * 8), o_flags = take(8);
    uint8_t *d_work = nullptr;
    cudaError_t e = cudaMalloc((void **)&d_work, off);
    if (e != cudaSuccess) PG_FAIL(e == cudaErrorMemoryAllocation ? PG_ERR_NOMEM : PG_ERR_CUDA, "huffman: %s", cudaGetErrorString(e));
    cudaStream_t q = ctx->stream;
    uint32_t *d_flags = (uint32_t *)(d_work + o_flags);   // [0] hand-overs across blocks in the last sweep, [1] malformed
    const hf_stream *d_st = (const hf_stream *)(d_work + o_st);
    const uint32_t *d_bs = (const uint32_t *)(d_work + o_bs);
    const uint16_t *d_lut = (const uint16_t *)(d_work + o_lut);
    uint32_t flags[2] = {0, 0};
    int32_t rc = PG_OK;
    do {
        e = cudaMemcpyAsync(d_work + o_lut, lut.data(), HF_LUT_SIZE * 2, cudaMemcpyHostToDevice, q);
        if (e == cudaSuccess) e = cudaMemcpyAsync(d_work + o_st, st.data(), st.size() * sizeof(hf_stream), cudaMemcpyHostToDevice, q);
        if (e == cudaSuccess && nb) e = cudaMemcpyAsync(d_work + o_bs, block_stream.data(), nb * 4, cudaMemcpyHostToDevice, q);
        if (e == cudaSuccess) e = cudaMemsetAsync(d_work + o_dirty, 0, (nb + 1) * 4, q);
        if (e == cudaSuccess) e = cudaMemsetAsync(d_work + o_sum, 0, (nb + 1) * 4, q);
        if (e == cudaSuccess) e = cudaMemsetAsync(d_flags, 0, 8, q);
        if (e != cudaSuccess) break;
        bool serial = nb == 0;   // symbols asked of empty streams: all of them come from the padding
        if (nb) {
            // the fixed point: every sweep settles at least one more block, two or three settle all of them on real codes
            for (size_t sweep = 0; sweep <= nb + 1; sweep++) {
                if (sweep) {
                    e = cudaMemsetAsync(d_flags, 0, 4, q);
                    if (e != cudaSuccess) break;
                }
                huffman_sync_kernel<<<(unsigned)nb, HF_THREADS, 0, q>>>(d_data, d_st, d_bs, d_lut, (uint32_t *)(d_work + o_start),
                                                                        (uint32_t *)(d_work + o_count), (uint32_t *)(d_work + o_dirty),
                                                                        (uint32_t *)(d_work + o_sum), sweep == 0, d_flags, d_flags + 1);
                PG_LAUNCHED();
                e = cudaMemcpyAsync(flags, d_flags, 8, cudaMemcpyDeviceToHost, q);
                if (e == cudaSuccess) e = cudaStreamSynchronize(q);
                if (e != cudaSuccess || flags[0] == 0 || flags[1]) break;
            }
            if (e != cudaSuccess) break;
            if (flags[0] != 0 && !flags[1]) {
                rc = PG_ERR_CUDA;
                pg_set_error("huffman: the subsequence starts did not settle");
                break;
            }
            if (!flags[1]) {
                huffman_scan_kernel<<<(unsigned)((num_streams + 3) / 4), 128, 0, q>>>(d_st, (int)num_streams, (const uint32_t *)(d_work + o_sum),
                                                                                     (uint64_t *)(d_work + o_boff), d_flags + 1);
                PG_LAUNCHED();
                e = cudaMemcpyAsync(flags, d_flags, 8, cudaMemcpyDeviceToHost, q);
                if (e == cudaSuccess) e = cudaStreamSynchronize(q);
                if (e != cudaSuccess) break;
            }
            serial = flags[1] != 0;
            if (!serial) {
                huffman_write_kernel<<<(unsigned)nb, HF_THREADS, 0, q>>>(d_data, d_st, d_bs, d_lut, (const uint32_t *)(d_work + o_start),
                                                                         (const uint32_t *)(d_work + o_count),
                                                                         (const uint64_t *)(d_work + o_boff), d_out);
                PG_LAUNCHED();
            }
        }
        if (serial) {
            huffman_decode_serial_kernel<<<(unsigned)((num_streams + 63) / 64), 64, 0, q>>>(d_data, d_st, (int)num_streams, d_lut, d_out);
            PG_LAUNCHED();
        }
        e = cudaStreamSynchronize(q);   // the work buffer goes away below
    } while (0);
    cudaFree(d_work);
    if (e != cudaSuccess) PG_FAIL(PG_ERR_CUDA, "huffman: %s", cudaGetErrorString(e));
    return rc;
}
