// Huffman-coded int8 weights, decoded on the GPU.
//
// The format is the reference's (src/huffman.rs:216-284): one canonical code of at most 12 bits shared by
// `num_streams` bitstreams, bits written MSB first, the last byte of a stream padded with zeros, no
// markers inside a stream.  The reference decodes on the host, one symbol after the other through a
// 4096-entry table indexed by the next 12 bits (src/huffman.rs:254-284) and uploads the bytes
// (to_gpu, src/huffman.rs:430-437).  Here the COMPRESSED bytes cross PCIe and every stream is decoded by
// thousands of threads:
//
//   * a stream is cut into subsequences of 1024 bits; thread i owns the code words that START in
//     subsequence i.  Where its first code word starts is unknown at first (only subsequence 0 starts
//     at bit 0), so the decode is a fixed-point iteration: every thread decodes from its current guess
//     and hands the position where it left its subsequence to its right-hand neighbour, which decodes
//     again if that changed.  Prefix codes resynchronise after a few code words, so the guesses settle
//     in two or three sweeps; the iteration is exact whatever the code (once start[i+1] == end[i] for
//     every i the chain is the sequential one) and bounded by the number of subsequences.
//     A block iterates its 256 subsequences in shared memory; the position handed from
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
constexpr int HF_SUB_BITS = 1024;               // bits per subsequence
constexpr int HF_SUB_WORDS = HF_SUB_BITS / 32;
constexpr int HF_OWN = 256;                     // subsequences a block owns
constexpr int HF_THREADS = 288;                 // slot 0: the subsequence before the block's (a look-behind), slots 1..HF_OWN: its own
constexpr int HF_SLOTS = HF_OWN + 1;
constexpr int HF_CHUNK_WORDS = HF_SLOTS * HF_SUB_WORDS + 4;   // plus the words a window and its prefetch may run over
constexpr uint32_t HF_NONE = 0xFFFFFFFFu;
constexpr int HF_LOOKBACK = 256;                // bits a slot decodes to guess where its neighbour starts

struct hf_stream {
    uint64_t byte_off;   // of the stream in the uploaded buffer
    uint64_t bytes;
    uint64_t symbols;
    uint64_t out_off;    // of its first symbol in the output
    uint32_t first_block;
    uint32_t blocks;
};

// word w of the block's chunk lives at w + w / HF_SUB_WORDS: one pad word per subsequence, so that threads that are
// at the same depth of their subsequences hit 32 different banks
__device__ __forceinline__ int hf_slot(int w) { return w + w / HF_SUB_WORDS; }

// Big-endian words [w0, w0 + HF_CHUNK_WORDS) of a stream into shared memory (w0 may be negative: the look-behind
// of a stream's first block); zeros outside the stream.  Loads go out eight at a time per thread.
__device__ __forceinline__ void hf_stage(const uint8_t *__restrict__ base, uint64_t bytes, int64_t w0, uint32_t *s_bits)
{
    const uintptr_t addr = (uintptr_t)base;
    const uint32_t mis = (uint32_t)(addr & 3);
    const uint32_t *aligned = (const uint32_t *)(addr - mis);   // the buffer starts on a word and has 8 bytes of slack at its end
    constexpr int BATCH = 8;
    for (int w = threadIdx.x; w < HF_CHUNK_WORDS; w += HF_THREADS * BATCH) {
        uint32_t lo[BATCH], hi[BATCH];
#pragma unroll
        for (int k = 0; k < BATCH; k++) {
            const int64_t word = w0 + w + k * HF_THREADS;
            const bool in = w + k * HF_THREADS < HF_CHUNK_WORDS && word >= 0 && (uint64_t)word * 4 < bytes;
            lo[k] = in ? __ldg(aligned + word) : 0u;
            hi[k] = in && mis ? __ldg(aligned + word + 1) : 0u;
        }
#pragma unroll
        for (int k = 0; k < BATCH; k++) {
            const int ww = w + k * HF_THREADS;
            if (ww >= HF_CHUNK_WORDS) break;
            const int64_t word = w0 + ww;
            uint32_t v = 0;
            if (word >= 0 && (uint64_t)word * 4 < bytes) {
                const uint64_t b = (uint64_t)word * 4;
                v = mis ? __funnelshift_r(lo[k], hi[k], mis * 8) : lo[k];   // little-endian: byte 0 of the stream in the low byte
                if (b + 4 > bytes) v &= 0xFFFFFFFFu >> (8 * (uint32_t)(b + 4 - bytes));
                v = __byte_perm(v, 0, 0x0123);                              // first bit of the stream in bit 31
            }
            s_bits[hf_slot(ww)] = v;
        }
    }
}

// A cursor over the staged bits: 64 bits in a register, the word after them already on its way.
struct hf_cursor {
    const uint32_t *bits;
    uint64_t buf;
    uint32_t ahead;
    int word;
    __device__ __forceinline__ void seek(const uint32_t *s_bits, uint32_t bit)
    {
        bits = s_bits;
        word = (int)(bit >> 5);
        buf = ((uint64_t)bits[hf_slot(word)] << 32) | bits[hf_slot(word + 1)];
        ahead = bits[hf_slot(word + 2)];
    }
    // the 12 bits at `bit`, which lies in `word` or one word further
    __device__ __forceinline__ uint32_t window(uint32_t bit)
    {
        if ((int)(bit >> 5) != word) {
            word++;
            buf = (buf << 32) | ahead;
            ahead = bits[hf_slot(word + 2)];
        }
        return (uint32_t)(buf >> (64 - HF_LUT_BITS - (bit & 31))) & (HF_LUT_SIZE - 1);
    }
};

// One sweep of the fixed-point iteration over the subsequence starts.
//   start[g], count[g]   per owned subsequence: bit offset of the first code word that starts in it, code words that start in it
//   used0[b]             the start block b last decoded its first subsequence from
//   handed[b]            where block b's last code word ends, relative to the next block's first subsequence
// Sweep 0 decodes everything: a block guesses the start of its first subsequence from the tail of the subsequence
// before it (slot 0).  Later sweeps only touch blocks whose used0 differs from what the block before them handed
// over; *changed counts the blocks whose own hand-over moved in this sweep.
__global__ void __launch_bounds__(HF_THREADS)
    huffman_sync_kernel(const uint8_t *__restrict__ data, const hf_stream *__restrict__ streams, const uint32_t *__restrict__ block_stream,
                        const uint16_t *__restrict__ lut, uint32_t *start, uint32_t *count, uint32_t *used0, uint32_t *handed,
                        uint32_t *block_sum, int first_sweep, uint32_t *changed, uint32_t *malformed)
{
    __shared__ uint32_t s_bits[HF_CHUNK_WORDS + HF_CHUNK_WORDS / HF_SUB_WORDS + 1];
    __shared__ uint16_t s_lut[HF_LUT_SIZE];
    __shared__ uint32_t s_start[HF_SLOTS + 1];
    __shared__ uint32_t s_dirty[HF_SLOTS + 1];
    __shared__ uint32_t s_red[HF_THREADS / 32];

    const uint32_t b = blockIdx.x, t = threadIdx.x;     // t: slot
    const hf_stream st = streams[block_stream[b]];
    const bool head = b == st.first_block;              // the stream's first block: its first subsequence starts at bit 0
    uint32_t from_left = 0;
    if (!first_sweep) {
        if (head) return;
        // one thread reads (the block before may be writing its hand-over right now), all threads take its view
        if (t == 0) {
            s_start[0] = pg_ld_fresh(&handed[b - 1]);
            s_dirty[0] = s_start[0] != pg_ld_fresh(&used0[b]);
        }
        __syncthreads();
        from_left = s_start[0];
        const bool stale = s_dirty[0] != 0;
        __syncthreads();
        if (!stale) return;
    }
    const int64_t sub0 = (int64_t)(b - st.first_block) * HF_OWN;   // first owned subsequence, in its stream
    const uint64_t total_bits = st.bytes * 8;
    const int64_t nsub = (int64_t)((total_bits + HF_SUB_BITS - 1) / HF_SUB_BITS);
    const int64_t sub = sub0 + (int64_t)t - 1;                      // slot 0 looks behind
    const bool slot = t < HF_SLOTS;
    const bool valid = slot && sub >= 0 && sub < nsub && (t > 0 || first_sweep);
    const size_t g = (size_t)b * HF_OWN + (t - 1);                  // of slots 1..HF_OWN

    for (int i = t; i < HF_LUT_SIZE; i += HF_THREADS) s_lut[i] = lut[i];
    hf_stage(data + st.byte_off, st.bytes, (sub0 - 1) * HF_SUB_WORDS, s_bits);
    if (slot) {
        if (first_sweep) {
            s_start[t] = 0;
            s_dirty[t] = t != 0;                        // slot 0 only takes part in the first guesses
        } else {
            s_start[t] = t == 0 ? 0 : (t == 1 ? from_left : start[g]);
            s_dirty[t] = t == 1;
        }
    }
    if (t == 0) s_dirty[HF_SLOTS] = 0;
    __syncthreads();

    uint32_t n = (first_sweep || !slot || t == 0) ? 0 : count[g];
    uint32_t next = HF_NONE;                            // where this slot's last code word ends, if it was decoded here
    const uint32_t limit = valid ? (uint32_t)min((uint64_t)HF_SUB_BITS, total_bits - (uint64_t)sub * HF_SUB_BITS) : 0;
    if (first_sweep) {
        // First guesses: every slot decodes only the last HF_LOOKBACK bits of its subsequence, from a position that is
        // most likely inside a code word, and tells its right-hand neighbour where it came out.  A prefix code has
        // usually found the code word boundaries again by then, so most slots decode just once below.
        if (valid && sub + 1 < nsub) {
            uint32_t pos = t == 0 ? 0 : HF_SUB_BITS - HF_LOOKBACK;   // slot 0 takes the whole subsequence: a miss there costs a sweep
            hf_cursor cur;
            cur.seek(s_bits, t * HF_SUB_BITS + pos);
            while (pos < HF_SUB_BITS) {
                const uint32_t e = s_lut[cur.window(t * HF_SUB_BITS + pos)];
                if ((e >> 8) == 0) break;
                pos += e >> 8;
            }
            if (pos >= HF_SUB_BITS && t + 1 < HF_SLOTS) s_start[t + 1] = pos - HF_SUB_BITS;
        }
        __syncthreads();
    }
    for (int sweep = 0; sweep <= HF_SLOTS; sweep++) {
        bool hand = false;
        if (valid && s_dirty[t]) {
            uint32_t pos = s_start[t];
            hf_cursor cur;
            cur.seek(s_bits, t * HF_SUB_BITS + pos);
            n = 0;
            while (pos < limit) {
                const uint32_t e = s_lut[cur.window(t * HF_SUB_BITS + pos)];
                if ((e >> 8) == 0) {   // the sequential decoder would stay here for good
                    atomicOr(malformed, 1u);
                    pos = HF_SUB_BITS;
                    break;
                }
                pos += e >> 8;
                n++;
            }
            next = pos - HF_SUB_BITS;
            hand = sub + 1 < nsub;
        }
        __syncthreads();
        if (slot) s_dirty[t] = 0;
        __syncthreads();
        bool again = false;
        if (hand && t + 1 < HF_SLOTS && s_start[t + 1] != next) {
            s_start[t + 1] = next;
            s_dirty[t + 1] = 1;
            again = true;
        }
        if (!__syncthreads_or(again)) break;
    }
    if (t >= 1 && slot) {
        start[g] = s_start[t];
        count[g] = valid ? n : 0;
    }
    if (t == 1) used0[b] = s_start[1];
    if (t == HF_OWN && next != HF_NONE && sub + 1 < nsub) {   // the last owned subsequence was decoded again: its end may have moved
        if (first_sweep || pg_ld_fresh(&handed[b]) != next) {
            handed[b] = next;
            if (!first_sweep) atomicAdd(changed, 1u);
        }
    }
    // symbols of the block, for the scan over blocks
    uint32_t v = (valid && t >= 1) ? n : 0;
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    if ((t & 31) == 0) s_red[t >> 5] = v;
    __syncthreads();
    if (t == 0) {
        uint32_t total = 0;
        for (int w = 0; w < HF_THREADS / 32; w++) total += s_red[w];
        block_sum[b] = total;
    }
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
    __shared__ uint32_t s_bits[HF_CHUNK_WORDS + HF_CHUNK_WORDS / HF_SUB_WORDS + 1];
    __shared__ uint16_t s_lut[HF_LUT_SIZE];
    __shared__ uint32_t s_red[HF_THREADS / 32];

    const uint32_t b = blockIdx.x, t = threadIdx.x;     // here slot t holds owned subsequence t (no look-behind)
    const hf_stream st = streams[block_stream[b]];
    const int64_t sub0 = (int64_t)(b - st.first_block) * HF_OWN;
    const uint64_t total_bits = st.bytes * 8;
    const int64_t nsub = (int64_t)((total_bits + HF_SUB_BITS - 1) / HF_SUB_BITS);
    const int64_t sub = sub0 + t;
    const bool valid = t < HF_OWN && sub < nsub;
    const size_t g = (size_t)b * HF_OWN + t;

    for (int i = t; i < HF_LUT_SIZE; i += HF_THREADS) s_lut[i] = lut[i];
    hf_stage(data + st.byte_off, st.bytes, sub0 * HF_SUB_WORDS, s_bits);

    // exclusive scan of the counts inside the block
    const uint32_t n = t < HF_OWN ? pg_ld_fresh(&count[g]) : 0;
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
    const uint32_t limit = (uint32_t)min((uint64_t)HF_SUB_BITS, total_bits - (uint64_t)sub * HF_SUB_BITS);
    uint32_t pos = pg_ld_fresh(&start[g]);
    int8_t *dst = out + st.out_off;
    uint32_t left = (uint32_t)min((uint64_t)n, st.symbols - idx);
    hf_cursor cur;
    cur.seek(s_bits, t * HF_SUB_BITS + pos);
    // bytes up to the next 4-byte boundary of the output, then words, then the tail
    uint32_t word = 0, have = 0;
    while (pos < limit && left) {
        const uint32_t e = s_lut[cur.window(t * HF_SUB_BITS + pos)];
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

int g_huffman_sweeps = 0;   // sweeps of the last decode (-1: decoded by the sequential kernel)

}  // namespace

// Diagnostic, beside the pg_tune_* knobs: how many sweeps over the subsequence starts the last decode took.
extern "C" PG_API int pg_huffman_last_sweeps(void) { return g_huffman_sweeps; }

// Streams back to back in host memory (the layout of the serial format, src/serial.rs:320-365) -> symbols back to back
// in d_out.  The compressed bytes and the decoder's bookkeeping live in the context's scratch block.
int32_t pgk_huffman_decode(pg_ctx *ctx, const uint8_t *bit_lengths, int64_t num_streams, const uint64_t *stream_symbols,
                           const uint64_t *stream_bytes, const uint8_t *h_data, int8_t *d_out)
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
        const uint64_t blocks = (nsub + HF_OWN - 1) / HF_OWN;
        PG_REQUIRE(block_stream.size() + blocks < (1ull << 31), "huffman: streams too long");
        h.first_block = (uint32_t)block_stream.size();
        h.blocks = (uint32_t)blocks;
        block_stream.insert(block_stream.end(), (size_t)blocks, (uint32_t)s);
        byte_off += h.bytes;
        out_off += h.symbols;
    }
    if (out_off == 0) return PG_OK;
    const size_t nb = block_stream.size();

    // one allocation: table | streams | block -> stream | start | count | used0 | handed | block sums | block offsets | flags
    size_t off = 0;
    auto take = [&off](size_t bytes) { const size_t at = off; off += (bytes + 255) / 256 * 256; return at; };
    const size_t o_lut = take(HF_LUT_SIZE * 2), o_st = take(st.size() * sizeof(hf_stream)), o_bs = take((nb + 1) * 4),
                 o_start = take((nb * HF_OWN + 1) * 4), o_count = take(nb * HF_OWN * 4 + 4), o_used = take((nb + 1) * 4),
                 o_handed = take((nb + 1) * 4), o_sum = take((nb + 1) * 4), o_boff = take((nb + 1) * 8), o_flags = take(8),
                 o_bits = take(byte_off + 16);   // the decoder reads whole words: 8 bytes of slack
    const int32_t reserved = pg_scratch_reserve(ctx, off);
    if (reserved != PG_OK) return reserved;
    uint8_t *d_work = (uint8_t *)ctx->scratch;
    const uint8_t *d_data = d_work + o_bits;
    cudaError_t e = cudaSuccess;
    cudaStream_t q = ctx->stream;
    uint32_t *d_flags = (uint32_t *)(d_work + o_flags);   // [0] hand-overs across blocks in the last sweep, [1] malformed
    const hf_stream *d_st = (const hf_stream *)(d_work + o_st);
    const uint32_t *d_bs = (const uint32_t *)(d_work + o_bs);
    const uint16_t *d_lut = (const uint16_t *)(d_work + o_lut);
    uint32_t flags[2] = {0, 0};
    int32_t rc = PG_OK;
    do {
        if (byte_off) e = cudaMemcpyAsync(d_work + o_bits, h_data, byte_off, cudaMemcpyHostToDevice, q);
        if (e == cudaSuccess) e = cudaMemcpyAsync(d_work + o_lut, lut.data(), HF_LUT_SIZE * 2, cudaMemcpyHostToDevice, q);
        if (e == cudaSuccess) e = cudaMemcpyAsync(d_work + o_st, st.data(), st.size() * sizeof(hf_stream), cudaMemcpyHostToDevice, q);
        if (e == cudaSuccess && nb) e = cudaMemcpyAsync(d_work + o_bs, block_stream.data(), nb * 4, cudaMemcpyHostToDevice, q);
        if (e == cudaSuccess) e = cudaMemsetAsync(d_work + o_used, 0, o_boff - o_used, q);   // used0, handed, block sums
        if (e == cudaSuccess) e = cudaMemsetAsync(d_flags, 0, 8, q);
        if (e != cudaSuccess) break;
        bool serial = nb == 0;   // symbols asked of empty streams: all of them come from the padding
        if (nb) {
            // the fixed point: sweep 0 decodes everything, sweep 1 checks the hand-overs between blocks (and repairs the few
            // that the look-behind guessed wrong); every further sweep settles at least one more block
            for (size_t sweep = 0; sweep <= nb + 2; sweep++) {
                if (sweep > 1) {
                    e = cudaMemsetAsync(d_flags, 0, 4, q);
                    if (e != cudaSuccess) break;
                }
                huffman_sync_kernel<<<(unsigned)nb, HF_THREADS, 0, q>>>(d_data, d_st, d_bs, d_lut, (uint32_t *)(d_work + o_start),
                                                                        (uint32_t *)(d_work + o_count), (uint32_t *)(d_work + o_used),
                                                                        (uint32_t *)(d_work + o_handed), (uint32_t *)(d_work + o_sum),
                                                                        sweep == 0, d_flags, d_flags + 1);
                PG_LAUNCHED();
                if (sweep == 0) {
                    flags[0] = 1;   // the check sweep always runs
                    continue;
                }
                e = cudaMemcpyAsync(flags, d_flags, 8, cudaMemcpyDeviceToHost, q);
                if (e == cudaSuccess) e = cudaStreamSynchronize(q);
                g_huffman_sweeps = (int)sweep + 1;
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
            g_huffman_sweeps = -1;
            huffman_decode_serial_kernel<<<(unsigned)((num_streams + 63) / 64), 64, 0, q>>>(d_data, d_st, (int)num_streams, d_lut, d_out);
            PG_LAUNCHED();
        }
    } while (0);
    if (e != cudaSuccess) PG_FAIL(PG_ERR_CUDA, "huffman: %s", cudaGetErrorString(e));
    return rc;
}
