// Host-side parts of libdf11: error text, unit validation and the bit packer.
//
// The packer produces exactly what the reference's pure-Python `encode` produces for
// the same code table (dfloat11/dfloat11_utils.py:118-170): codes appended MSB first,
// `gaps[w]` = bit offset of the first code starting in 8-byte window w,
// `output_positions[b]` = index of the first element whose code starts in 4096-byte
// block b, a last entry equal to the element count, and a final partial byte completed
// with the leading bits of a padding code.  It is a different program: two linear passes
// over the exponents (sizes, then bits) split across threads at element boundaries.
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <thread>
#include <vector>

#include "../../include/df11.h"
#include "df11_common.h"
#include "df11_error.h"

namespace {
thread_local char g_error[512] = "";
}

int df11_fail(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
    return code;
}

extern "C" int df11_version(void) { return 100; /* 0.1.0 */ }

extern "C" const char *df11_last_error(void) { return g_error; }

extern "C" int df11_validate_host(const void *luts_v, int32_t n_luts, int64_t n_bytes, int64_t n_elements,
                                  const void *pos_v, int64_t n_positions, int64_t n_gap_bytes,
                                  int32_t *max_block_elems)
{
    const uint8_t *luts = (const uint8_t *)luts_v;
    const uint32_t *pos = (const uint32_t *)pos_v;
    if (!luts || !pos) return df11_fail(DF11_ERR_BADARG, "null pointer");
    if (n_luts < 2 || n_luts > DF11_MAX_LUTS)
        return df11_fail(DF11_ERR_BADARG, "n_luts = %d, supported range is 2..%d", n_luts, DF11_MAX_LUTS);
    if (n_bytes < 0 || n_elements < 0) return df11_fail(DF11_ERR_BADARG, "negative size");
    const int64_t n_blocks = (n_bytes + DF11_BLOCK_BYTES - 1) / DF11_BLOCK_BYTES;
    if (n_positions != n_blocks + 1)
        return df11_fail(DF11_ERR_CORRUPT, "output_positions has %lld entries, expected %lld",
                         (long long)n_positions, (long long)(n_blocks + 1));
    if (n_gap_bytes != n_blocks * DF11_GAP_BYTES_PER_BLOCK)
        return df11_fail(DF11_ERR_CORRUPT, "gaps has %lld bytes, expected %lld", (long long)n_gap_bytes,
                         (long long)(n_blocks * DF11_GAP_BYTES_PER_BLOCK));
    if (n_elements > 0xFFFFFFFFll) return df11_fail(DF11_ERR_CORRUPT, "element count exceeds 32 bits");
    // every row reachable from the root: pointers in range, leaf symbols have a usable length
    const uint8_t *lens = luts + (size_t)(n_luts - 1) * 256;
    std::vector<int> depth(n_luts, -1);
    std::vector<int> todo(1, 0);
    depth[0] = 0;
    while (!todo.empty()) {
        const int row = todo.back();
        todo.pop_back();
        for (int i = 0; i < 256; ++i) {
            const int e = luts[(size_t)row * 256 + i];
            if (e >= 240 && depth[row] < 3) {
                const int next = 256 - e;
                if (next >= n_luts - 1)
                    return df11_fail(DF11_ERR_CORRUPT, "luts row %d entry %d points to row %d of %d", row, i,
                                     next, n_luts);
                if (depth[next] < 0) {
                    depth[next] = depth[row] + 1;
                    todo.push_back(next);
                }
            } else if (lens[e] == 0 || lens[e] > DF11_MAX_CODE_LEN) {
                return df11_fail(DF11_ERR_CORRUPT, "symbol %d (luts row %d entry %d) has code length %d", e,
                                 row, i, (int)lens[e]);
            }
        }
    }
    int64_t widest = 0;
    if (n_blocks > 0 && pos[0] != 0) return df11_fail(DF11_ERR_CORRUPT, "output_positions[0] = %u", pos[0]);
    for (int64_t b = 0; b < n_blocks; ++b) {
        if (pos[b + 1] < pos[b])
            return df11_fail(DF11_ERR_CORRUPT, "output_positions decreases at block %lld", (long long)b);
        widest = std::max<int64_t>(widest, (int64_t)pos[b + 1] - pos[b]);
    }
    if ((int64_t)pos[n_blocks] != n_elements)
        return df11_fail(DF11_ERR_CORRUPT, "output_positions ends at %u, sign_mantissa has %lld elements",
                         pos[n_blocks], (long long)n_elements);
    if (widest > DF11_MAX_BLOCK_ELEMS)
        return df11_fail(DF11_ERR_CORRUPT, "a format block claims %lld elements (max %d)", (long long)widest,
                         DF11_MAX_BLOCK_ELEMS);
    if (max_block_elems) *max_block_elems = (int32_t)widest;
    return DF11_OK;
}

namespace {

int64_t total_bits(const uint8_t *ex, int64_t i0, int64_t i1, const uint8_t *code_len, bool *missing)
{
    int64_t hist[256] = {0};
    for (int64_t i = i0; i < i1; ++i) ++hist[ex[i]];
    int64_t bits = 0;
    for (int s = 0; s < 256; ++s) {
        if (hist[s] && code_len[s] == 0) *missing = true;
        bits += hist[s] * code_len[s];
    }
    return bits;
}

// Appends codes MSB first.  The writer may start in the middle of a byte whose leading
// bits belong to another thread; that one byte is handed back instead of stored.
struct BitWriter {
    uint8_t *out;
    int64_t byte;          // index of the byte being filled
    uint64_t acc;          // pending bits, right-aligned (leading placeholder bits are 0)
    int n;                 // number of pending bits, < 8 between calls
    int64_t shared_index;  // byte that must not be stored (-1: none)
    uint8_t shared_value;
    void put(uint32_t val, int len)
    {
        acc = (acc << len) | val;
        n += len;
        while (n >= 8) {
            const uint8_t v = (uint8_t)(acc >> (n - 8));
            if (byte == shared_index) shared_value = v; else out[byte] = v;
            ++byte;
            n -= 8;
        }
        acc &= (1ull << n) - 1;
    }
};

struct Chunk {
    int64_t i0, i1;       // element range
    int64_t bit0, bits;   // where element i0 starts, and the chunk's length in bits
    int64_t head_index;   // byte shared with the predecessor (-1: starts on a byte boundary)
    uint8_t head_value;
    int64_t tail_index;   // byte left incomplete at the end (-1: ends on a byte boundary)
    uint8_t tail_value;
    int64_t last_start;   // start bit of the chunk's last element
};

struct Mark {
    int64_t window;
    uint32_t gap;
};

void set_gap(uint8_t *gaps, int64_t window, uint32_t gap)
{
    // 5 bits per window, MSB first (np.packbits order, dfloat11_utils.py:166-170)
    const int64_t bit = window * 5;
    const int64_t j = bit >> 3;
    const int r = (int)(bit & 7);
    const uint32_t v = gap << (11 - r);  // positioned inside a 16-bit big-endian pair
    gaps[j] |= (uint8_t)(v >> 8);
    if (r > 3) gaps[j + 1] |= (uint8_t)v;
}

template <class F>
void run_chunks(int n, F job)
{
    std::vector<std::thread> pool;
    for (int c = 0; c + 1 < n; ++c) pool.emplace_back(job, c);
    job(n - 1);
    for (auto &t : pool) t.join();
}

}  // namespace

extern "C" int64_t df11_encode_size(const void *exponents, int64_t n_elements, const void *code_len)
{
    if (!exponents || !code_len || n_elements < 0) return df11_fail(DF11_ERR_BADARG, "bad argument");
    bool missing = false;
    const int64_t bits = total_bits((const uint8_t *)exponents, 0, n_elements, (const uint8_t *)code_len, &missing);
    if (missing) return df11_fail(DF11_ERR_BADARG, "an exponent value that occurs has no code");
    return (bits + 7) / 8;
}

extern "C" int df11_encode_host(const void *exponents, int64_t n_elements, const void *code_len_v,
                                const void *code_val_v, int32_t pad_len, uint32_t pad_val, void *codes_v,
                                int64_t n_bytes, void *gaps_v, int64_t n_gap_bytes, void *pos_v,
                                int64_t n_positions, int32_t n_threads)
{
    const uint8_t *ex = (const uint8_t *)exponents;
    const uint8_t *code_len = (const uint8_t *)code_len_v;
    const uint32_t *code_val = (const uint32_t *)code_val_v;
    uint8_t *codes = (uint8_t *)codes_v;
    uint8_t *gaps = (uint8_t *)gaps_v;
    uint32_t *pos = (uint32_t *)pos_v;
    if (!ex || !code_len || !code_val || !codes || !gaps || !pos || n_elements < 0)
        return df11_fail(DF11_ERR_BADARG, "bad argument");
    if (n_elements > 0xFFFFFFFFll) return df11_fail(DF11_ERR_BADARG, "element count exceeds 32 bits");
    for (int s = 0; s < 256; ++s)
        if (code_len[s] > DF11_MAX_CODE_LEN)
            return df11_fail(DF11_ERR_BADARG, "code of %d is %d bits", s, (int)code_len[s]);
    if (pad_len < 0 || pad_len > DF11_MAX_CODE_LEN) return df11_fail(DF11_ERR_BADARG, "bad padding code");

    // chunks of at least 64 Ki elements (>= 8 KiB of stream), so two chunk borders never
    // fall into one byte of the stream or of the packed gaps
    const int64_t min_chunk = 65536;
    int64_t want = std::max<int64_t>(1, std::min<int64_t>(n_threads, 256));
    want = std::max<int64_t>(1, std::min<int64_t>(want, n_elements / min_chunk));
    const int64_t per = (n_elements + want - 1) / want;
    const int n_chunks = per > 0 ? (int)((n_elements + per - 1) / per) : 0;
    std::vector<Chunk> chunks(std::max(n_chunks, 1));
    std::vector<char> missing(std::max(n_chunks, 1), 0);

    // pass 1: bits per chunk -> where every chunk starts
    if (n_chunks > 0)
        run_chunks(n_chunks, [&](int c) {
            Chunk &ch = chunks[c];
            ch.i0 = c * per;
            ch.i1 = std::min<int64_t>(n_elements, (c + 1) * per);
            bool m = false;
            ch.bits = total_bits(ex, ch.i0, ch.i1, code_len, &m);
            missing[c] = m;
        });
    int64_t total = 0;
    for (int c = 0; c < n_chunks; ++c) {
        if (missing[c]) return df11_fail(DF11_ERR_BADARG, "an exponent value that occurs has no code");
        chunks[c].bit0 = total;
        total += chunks[c].bits;
    }
    const int64_t want_bytes = (total + 7) / 8;
    const int64_t n_blocks = (want_bytes + DF11_BLOCK_BYTES - 1) / DF11_BLOCK_BYTES;
    if (n_bytes != want_bytes || n_gap_bytes != n_blocks * DF11_GAP_BYTES_PER_BLOCK || n_positions != n_blocks + 1)
        return df11_fail(DF11_ERR_NOSPACE, "buffers must hold %lld stream bytes, %lld gap bytes, %lld positions",
                         (long long)want_bytes, (long long)(n_blocks * DF11_GAP_BYTES_PER_BLOCK),
                         (long long)(n_blocks + 1));
    if (n_gap_bytes > 0) memset(gaps, 0, (size_t)n_gap_bytes);

    // pass 2: each chunk stores the stream bytes it owns alone.  The byte it shares with its
    // predecessor and its own incomplete last byte are returned and combined below, as are
    // the gap entries of the two windows at either end (packed gap bytes are shared too).
    std::vector<std::vector<Mark>> border(std::max(n_chunks, 1));
    if (n_chunks > 0)
        run_chunks(n_chunks, [&](int c) {
            Chunk &ch = chunks[c];
            int64_t bit = ch.bit0;
            int64_t prev_start = ch.i0 > 0 ? bit - code_len[ex[ch.i0 - 1]] : -1;
            ch.head_index = (bit & 7) ? (bit >> 3) : -1;
            BitWriter w{codes, bit >> 3, 0, (int)(bit & 7), ch.head_index, 0};
            const int64_t w_first = bit >> 6;
            const int64_t w_last = (ch.bit0 + ch.bits) >> 6;
            for (int64_t i = ch.i0; i < ch.i1; ++i) {
                const uint32_t s = ex[i];
                if (prev_start < 0 || (prev_start >> 6) != (bit >> 6)) {  // first code starting in its window
                    const int64_t window = bit >> 6;
                    if (window <= w_first + 1 || window >= w_last - 1)
                        border[c].push_back({window, (uint32_t)(bit & 63)});
                    else
                        set_gap(gaps, window, (uint32_t)(bit & 63));
                    if (prev_start < 0 || (prev_start >> 15) != (bit >> 15)) pos[bit >> 15] = (uint32_t)i;
                }
                prev_start = bit;
                w.put(code_val[s], code_len[s]);
                bit += code_len[s];
            }
            ch.head_value = w.shared_value;
            ch.last_start = prev_start;
            if (w.n > 0) {
                if (w.byte == ch.head_index) {  // cannot happen for chunks >= 8 KiB; keep the bits anyway
                    ch.head_value = (uint8_t)(w.acc << (8 - w.n));
                    ch.tail_index = -1;
                } else {
                    ch.tail_index = w.byte;
                    ch.tail_value = (uint8_t)(w.acc << (8 - w.n));
                }
            } else {
                ch.tail_index = -1;
            }
        });
    for (int c = 0; c < n_chunks; ++c) {
        for (const Mark &m : border[c]) set_gap(gaps, m.window, m.gap);
        if (chunks[c].head_index >= 0) {
            const uint8_t carry = (c > 0 && chunks[c - 1].tail_index == chunks[c].head_index) ? chunks[c - 1].tail_value : 0;
            codes[chunks[c].head_index] = (uint8_t)(chunks[c].head_value | carry);
        }
    }
    // the incomplete last byte is completed with the leading bits of the padding code, which
    // also counts as "a code starting here" for the gap / position tables (dfloat11_utils.py:146-160)
    const int rem = (int)(total & 7);
    if (rem) {
        const Chunk &last = chunks[n_chunks - 1];
        if ((last.last_start >> 6) != (total >> 6)) set_gap(gaps, total >> 6, (uint32_t)(total & 63));
        if ((last.last_start >> 15) != (total >> 15)) pos[total >> 15] = (uint32_t)n_elements;
        const int room = 8 - rem;
        uint32_t pad = 0;
        if (pad_len >= room) pad = pad_val >> (pad_len - room);
        else if (pad_len > 0) pad = pad_val << (room - pad_len);
        codes[want_bytes - 1] = (uint8_t)(last.tail_value | (pad & ((1u << room) - 1)));
    }
    pos[n_blocks] = (uint32_t)n_elements;
    return DF11_OK;
}
