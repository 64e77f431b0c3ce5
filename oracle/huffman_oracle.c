/*
 * CPU oracle for the Huffman-coded int8 weights of etam103/peregrine.
 *
 * TEST INFRASTRUCTURE ONLY, like peregrine_oracle.c: the checker for the CUDA decoder and for the
 * host-side table builder.  It restates
 *
 *   src/huffman.rs:35-152    HuffmanTable::from_frequencies (two-queue Huffman over the active
 *                            symbols, stable order by frequency, depths clamped to 12 bits AFTER the
 *                            tree is built -- kept as the reference does it, also where that leaves
 *                            a code that is no longer prefix-free)
 *   src/huffman.rs:155-190   canonical_codes
 *   src/huffman.rs:193-213   build_decode_lut (4096 entries; later symbols overwrite earlier ones)
 *   src/huffman.rs:216-251   encode (MSB first, zero padding of the last byte)
 *   src/huffman.rs:254-284   decode (12-bit window, zero padded past the end, LUT lookup)
 *
 * Pinned by the reference's own tests for this module (src/huffman.rs tests, tests/huffman_parity.rs),
 * re-run in tests/test_huffman_cpu.py.
 */
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define PGO_API __attribute__((visibility("default")))
#define NUM_SYMBOLS 256
#define MAX_LUT_BITS 12

typedef struct {
    uint64_t f;
    int node;
} qitem;

/* src/huffman.rs:155-190 */
PGO_API void pgo_huffman_canonical_codes(const uint8_t *bit_lengths, uint32_t *codes)
{
    memset(codes, 0, NUM_SYMBOLS * sizeof(uint32_t));
    int max_len = 0;
    for (int s = 0; s < NUM_SYMBOLS; s++)
        if (bit_lengths[s] > max_len) max_len = bit_lengths[s];
    if (max_len == 0) return;
    uint32_t bl_count[257] = {0}, next_code[257] = {0};
    for (int s = 0; s < NUM_SYMBOLS; s++)
        if (bit_lengths[s] > 0) bl_count[bit_lengths[s]]++;
    uint32_t code = 0;
    for (int bits = 1; bits <= max_len; bits++) {
        code = (code + bl_count[bits - 1]) << 1;
        next_code[bits] = code;
    }
    for (int s = 0; s < NUM_SYMBOLS; s++) {
        const int bl = bit_lengths[s];
        if (bl > 0) codes[s] = next_code[bl]++;
    }
}

/* src/huffman.rs:35-152.  freqs[i] = frequency of symbol (i - 128). */
PGO_API void pgo_huffman_from_frequencies(const uint64_t *freqs, uint8_t *bit_lengths, uint32_t *codes)
{
    memset(bit_lengths, 0, NUM_SYMBOLS);
    memset(codes, 0, NUM_SYMBOLS * sizeof(uint32_t));
    int symbols[NUM_SYMBOLS];
    uint64_t fv[NUM_SYMBOLS];
    int n = 0;
    for (int i = 0; i < NUM_SYMBOLS; i++)
        if (freqs[i] > 0) {
            symbols[n] = i;
            fv[n] = freqs[i];
            n++;
        }
    if (n == 0) return;
    if (n == 1) {
        bit_lengths[symbols[0]] = 1;
        return;
    }
    /* leaves sorted by frequency, stable (Rust's sort_by_key): insertion sort keeps equal keys in index order */
    int order[NUM_SYMBOLS];
    for (int i = 0; i < n; i++) {
        int j = i;
        while (j > 0 && fv[order[j - 1]] > fv[i]) {
            order[j] = order[j - 1];
            j--;
        }
        order[j] = i;
    }
    qitem leaf[NUM_SYMBOLS], inner[NUM_SYMBOLS];
    int lh = 0, lt = n, ih = 0, it = 0;
    for (int i = 0; i < n; i++) {
        leaf[i].f = fv[order[i]];
        leaf[i].node = order[i];
    }
    int parent[2 * NUM_SYMBOLS] = {0};
    int next_node = n;
    for (int step = 0; step < n - 1; step++) {
        qitem pick[2];
        for (int p = 0; p < 2; p++) {
            const int has_leaf = lh < lt, has_inner = ih < it;
            if (has_leaf && has_inner)
                pick[p] = (leaf[lh].f <= inner[ih].f) ? leaf[lh++] : inner[ih++];
            else if (has_leaf)
                pick[p] = leaf[lh++];
            else
                pick[p] = inner[ih++];
        }
        parent[pick[0].node] = next_node;
        parent[pick[1].node] = next_node;
        inner[it].f = pick[0].f + pick[1].f;
        inner[it].node = next_node;
        it++;
        next_node++;
    }
    /* depths; the reference keeps them in u8 and adds 1 per level (a chain of 255 symbols stays below 256) */
    uint8_t depth[2 * NUM_SYMBOLS] = {0};
    const int root = 2 * n - 2;
    depth[root] = 0;
    for (int i = root - 1; i >= 0; i--) depth[i] = (uint8_t)(depth[parent[i]] + 1);
    for (int i = 0; i < n; i++) {
        if (depth[i] > MAX_LUT_BITS) depth[i] = MAX_LUT_BITS;
        bit_lengths[symbols[i]] = depth[i];
    }
    pgo_huffman_canonical_codes(bit_lengths, codes);
}

/* src/huffman.rs:193-213.  lut[code] = (bit_length << 8) | (symbol + 128), the packing of to_gpu_lut (src/huffman.rs:726-737);
 * (length 0, symbol 0) where no code starts with those 12 bits. */
PGO_API void pgo_huffman_build_lut(const uint8_t *bit_lengths, const uint32_t *codes, uint32_t *lut)
{
    for (size_t i = 0; i < (1u << MAX_LUT_BITS); i++) lut[i] = 128u;   /* (symbol 0, length 0): the reference's default entry */
    for (int s = 0; s < NUM_SYMBOLS; s++) {
        const int bl = bit_lengths[s];
        if (bl == 0 || bl > MAX_LUT_BITS) continue;
        const int shift = MAX_LUT_BITS - bl;
        const size_t base = (size_t)codes[s] << shift, count = (size_t)1 << shift;
        /* the reference indexes a Vec of 4096 entries: an over-long prefix would panic there; here it is skipped */
        for (size_t j = 0; j < count && base + j < (1u << MAX_LUT_BITS); j++) lut[base + j] = ((uint32_t)bl << 8) | (uint32_t)s;
    }
}

/* src/huffman.rs:216-251.  Returns the number of bytes written (out must hold at least (sum of lengths + 7) / 8). */
PGO_API size_t pgo_huffman_encode(const uint8_t *bit_lengths, const uint32_t *codes, const int8_t *data, size_t n, uint8_t *out)
{
    size_t nbytes = 0;
    uint8_t cur = 0;
    int fill = 0;
    for (size_t i = 0; i < n; i++) {
        const int idx = (int)data[i] + 128;
        const uint32_t code = codes[idx];
        for (int b = bit_lengths[idx] - 1; b >= 0; b--) {
            cur = (uint8_t)((cur << 1) | ((code >> b) & 1u));
            if (++fill == 8) {
                out[nbytes++] = cur;
                cur = 0;
                fill = 0;
            }
        }
    }
    if (fill > 0) out[nbytes++] = (uint8_t)(cur << (8 - fill));
    return nbytes;
}

/* src/huffman.rs:254-284 */
PGO_API void pgo_huffman_decode(const uint32_t *lut, const uint8_t *bitstream, size_t nbytes, size_t num_symbols, int8_t *out)
{
    const size_t total_bits = nbytes * 8;
    size_t bit_pos = 0;
    for (size_t i = 0; i < num_symbols; i++) {
        size_t avail = total_bits > bit_pos ? total_bits - bit_pos : 0;
        if (avail > MAX_LUT_BITS) avail = MAX_LUT_BITS;
        uint32_t code = 0;
        for (size_t b = 0; b < avail; b++) {
            const size_t p = bit_pos + b;
            code = (code << 1) | ((bitstream[p >> 3] >> (7 - (p & 7))) & 1u);
        }
        code <<= (MAX_LUT_BITS - avail);
        const uint32_t e = lut[code];
        out[i] = (int8_t)((int)(e & 0xFF) - 128);
        bit_pos += e >> 8;
    }
}
