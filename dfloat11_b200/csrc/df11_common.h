// Shared definitions of the DF11 decode path: format constants, the multi-symbol
// decode-table entry and the routines that derive it from the on-disk `luts`
// tensor.  Everything here is `__host__ __device__` so that the CUDA kernels and a
// host-side emulation used only by the CPU tests run the very same logic.
//
// Format facts (reference: dfloat11/dfloat11.py:44-49, dfloat11/decode.cu:18):
//   a "window" is 8 bytes of bitstream (one reference thread), a "format block" is
//   512 windows = 4096 bytes (one reference CTA); `output_positions[b]` is the index
//   of the first element whose code starts in format block b; `gaps` holds, 5 bits
//   per window, the bit offset of the first code that starts in that window.
#pragma once
#include <stdint.h>

#ifdef __CUDACC__
#define DF11_HD __host__ __device__ __forceinline__
#else
#define DF11_HD inline
#endif

#define DF11_WINDOW_BYTES 8
#define DF11_WINDOWS_PER_BLOCK 512
#define DF11_BLOCK_BYTES (DF11_WINDOW_BYTES * DF11_WINDOWS_PER_BLOCK)
#define DF11_GAP_BYTES_PER_BLOCK (DF11_WINDOWS_PER_BLOCK * 5 / 8)
#define DF11_MAX_BLOCK_ELEMS (DF11_BLOCK_BYTES * 8)  // shortest possible code is 1 bit
#define DF11_MAX_LUTS 32                             // rows accepted (the format can address 18)
#define DF11_MAX_CODE_LEN 32                         // dfloat11_utils.py:49 keeps codes <= 32 bits

// ---------------------------------------------------------------------------
// Multi-symbol decode table.
//
// Index: the next K bits of the stream.  Entry: up to four consecutive symbols
// that the reference's byte-wise LUT walk (decode.cu:105-118) is certain to
// produce for EVERY stream that starts with those K bits.
//
//   meta (32 bit):  bits 0..5   total bits consumed by the symbols in the entry
//                   bits 8..10  number of symbols, 0 = "escape": the first symbol
//                               cannot be resolved from K bits, do the full walk
//                   bits 16..19 / 20..23 / 24..27  start offset (in bits) of the
//                               2nd / 3rd / 4th symbol, 15 when absent
//   syms (32 bit):  the symbols, first one in the lowest byte
// ---------------------------------------------------------------------------
struct Df11Entry {
    uint32_t meta;
    uint32_t syms;
};

#define DF11_META_NBITS(m) ((m) & 0x3Fu)
#define DF11_META_NSYMS(m) (((m) >> 8) & 7u)
#define DF11_META_ESCAPE 0x0FFF0000u

// Offset of level-u "all equal" flags in the 255-byte agreement table: flag
// (u, blk) says that root-row entries [blk << u, (blk + 1) << u) are all equal.
DF11_HD int df11_agree_offset(int u) { return 256 - (256 >> (u - 1)); }

// Computes one agreement flag by brute force (at most 256 reads; done once per table).
DF11_HD uint8_t df11_agree_flag(const uint8_t *root, int u, int blk)
{
    const int first = blk << u;
    const uint8_t v = root[first];
    uint8_t same = 1;
    for (int i = 1; i < (1 << u); ++i)
        same &= (uint8_t)(root[first + i] == v);
    return same;
}

// The exact per-symbol rule of the reference (decode.cu:105-116) applied to the 32
// bits `x` (MSB first).  `luts` has n_luts rows of 256, the last row holds code
// lengths.  Returns the symbol; *len receives its code length.  *bad is set when the
// tables are unusable here (pointer outside the tensor, length 0 or > 32) -- the
// reference would read out of bounds or never terminate in those cases.
DF11_HD uint32_t df11_walk(const uint8_t *luts, int n_luts, uint32_t x, uint32_t *len, int *bad)
{
    uint32_t e = luts[x >> 24];
#ifdef __CUDA_ARCH__
#pragma unroll
#endif
    for (int shift = 16; shift >= 0; shift -= 8) {
        if (e >= 240u) {
            uint32_t row = 256u - e;
            if (row >= (uint32_t)n_luts) {
                *bad = 1;
                row = 0;
            }
            e = luts[row * 256u + ((x >> shift) & 255u)];
        }
    }
    uint32_t l = luts[(uint32_t)(n_luts - 1) * 256u + e];
    if (l == 0u || l > (uint32_t)DF11_MAX_CODE_LEN) {
        *bad = 1;
        l = 64u;  // leave the window
    }
    *len = l;
    return e;
}

// Builds the entry for K-bit index v.  `agree` is the 255-byte agreement table of the
// root row.  A symbol is taken into the entry only when every completion of the
// unknown trailing bits makes the reference's root lookup return the same non-pointer
// byte, so the entry never differs from the reference's symbol-by-symbol result.
DF11_HD Df11Entry df11_build_entry(const uint8_t *luts, int n_luts, const uint8_t *agree,
                                   uint32_t v, int K)
{
    const uint8_t *lens = luts + (n_luts - 1) * 256;
    const uint32_t left = v << (32 - K);  // index bits, left-aligned
    uint32_t c = 0, nsyms = 0, syms = 0, starts = 0x0FFF0000u;
    for (int j = 0; j < 4; ++j) {
        const int r = K - (int)c;  // index bits still unread
        if (r <= 0)
            break;  // every symbol of an entry starts inside the K index bits
        const int u = r >= 8 ? 0 : 8 - r;  // unknown low bits of this symbol's root byte
        const uint32_t idx = c < 32u ? ((left << c) >> 24) : 0u;
        if (u > 0 && !agree[df11_agree_offset(u) + (int)(idx >> u)])
            break;
        const uint32_t e = luts[idx];
        if (e >= 240u)
            break;  // pointer to a deeper row: needs bits we may not have
        const uint32_t l = lens[e];
        if (l == 0u || l > (uint32_t)DF11_MAX_CODE_LEN)
            break;
        if (j > 0) {
            starts &= ~(0xFu << (12 + 4 * j));
            starts |= c << (12 + 4 * j);
        }
        syms |= e << (8 * j);
        ++nsyms;
        c += l;
        if (c >= 15u)
            break;  // start offsets are stored in 4 bits, 15 meaning "absent" (K <= 14)
    }
    Df11Entry out;
    if (nsyms == 0) {
        out.meta = DF11_META_ESCAPE;
        out.syms = 0;
    } else {
        out.meta = c | (nsyms << 8) | starts;
        out.syms = syms;
    }
    return out;
}

// Number of symbols of a non-escape entry that start before bit offset `lim`
// (lim >= 1; the first symbol starts at 0).
DF11_HD uint32_t df11_owned_syms(uint32_t meta, uint32_t lim)
{
    return 1u + (uint32_t)(((meta >> 16) & 15u) < lim) + (uint32_t)(((meta >> 20) & 15u) < lim) +
           (uint32_t)(((meta >> 24) & 15u) < lim);
}

// 5-bit gap of window t (decode.cu:85-87) without the reference's read past the end.
DF11_HD uint32_t df11_gap(const uint8_t *gaps, int64_t n_gap_bytes, int64_t t)
{
    const int64_t bit = 5 * t;
    const int64_t j = bit >> 3;
    const int r = (int)(bit & 7);
    const uint32_t hi = j < n_gap_bytes ? gaps[j] : 0u;
    const uint32_t lo = (r > 3 && j + 1 < n_gap_bytes) ? gaps[j + 1] : 0u;
    return (((hi << 8) | lo) >> (11 - r)) & 31u;
}

// Two BF16 values from two exponent bytes and two sign/mantissa bytes packed as
// (e1 : sm1 : e0 : sm0), i.e. each half is exponent<<8 | sign<<7 | mantissa.
// decode.cu:207-209 per element:  hi = (sm & 0x80) | (e >> 1),  lo = (e << 7) | (sm & 0x7f).
DF11_HD uint32_t df11_merge_pair(uint32_t w)
{
    return ((w >> 1) & 0x7F807F80u) | ((w << 8) & 0x80008000u) | (w & 0x007F007Fu);
}

// ---------------------------------------------------------------------------
// One window = 8 stream bytes plus 4 bytes of look-ahead, held as three
// big-endian 32-bit words w0:w1:w2.
// ---------------------------------------------------------------------------

// Most significant 32 bits of (hi:lo) << (s mod 32).
DF11_HD uint32_t df11_funnel_l(uint32_t lo, uint32_t hi, uint32_t s)
{
#ifdef __CUDA_ARCH__
    return __funnelshift_l(lo, hi, s);
#else
    s &= 31u;
    return s ? (hi << s) | (lo >> (32u - s)) : hi;
#endif
}

// 32 stream bits starting `pos` bits into the window (pos < 64 for meaningful data;
// larger values stay inside the three registers and return unspecified bits).
DF11_HD uint32_t df11_peek(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t pos)
{
    const bool second = (pos & 32u) != 0u;
    const uint32_t a = second ? w1 : w0;
    const uint32_t b = second ? w2 : w1;
    return df11_funnel_l(b, a, pos);
}

// Counting pass: number of codes that START inside the window's 64 bits (the
// ownership rule of decode.cu:104,129), beginning at bit `gap`.
template <int K>
DF11_HD uint32_t df11_count_window(const Df11Entry *table, const uint8_t *luts, int n_luts,
                                   uint32_t w0, uint32_t w1, uint32_t w2, uint32_t gap, int *bad)
{
    uint32_t pos = gap, cnt = 0;
    // all K index bits inside the window: every symbol of the entry starts before bit 64
    while (pos <= 64u - K) {
        const uint32_t x = df11_peek(w0, w1, w2, pos);
        const uint32_t meta = table[x >> (32 - K)].meta;
        if (DF11_META_NSYMS(meta) == 0u) {
            uint32_t len;
            df11_walk(luts, n_luts, x, &len, bad);
            cnt += 1u;
            pos += len;
        } else {
            cnt += DF11_META_NSYMS(meta);
            pos += DF11_META_NBITS(meta);
        }
    }
    // the last few bits: count only the symbols that start before bit 64
    while (pos < 64u) {
        const uint32_t x = df11_peek(w0, w1, w2, pos);
        const uint32_t meta = table[x >> (32 - K)].meta;
        if (DF11_META_NSYMS(meta) == 0u) {
            uint32_t len;
            df11_walk(luts, n_luts, x, &len, bad);
            cnt += 1u;
            pos += len;
        } else {
            cnt += df11_owned_syms(meta, 64u - pos);
            pos += DF11_META_NBITS(meta);
        }
    }
    return cnt;
}

// Decoding pass: writes the window's exponents to stage[o .. end).  Terminates after
// at most end - o probes whatever the data is.
template <int K>
DF11_HD void df11_decode_window(const Df11Entry *table, const uint8_t *luts, int n_luts, uint32_t w0,
                                uint32_t w1, uint32_t w2, uint32_t gap, uint8_t *stage, int o, int end,
                                int *bad)
{
    uint32_t pos = gap;
    while (o < end) {
        const uint32_t x = df11_peek(w0, w1, w2, pos);
        const Df11Entry e = table[x >> (32 - K)];
        if (DF11_META_NSYMS(e.meta) == 0u) {
            uint32_t len;
            const uint32_t s = df11_walk(luts, n_luts, x, &len, bad);
            stage[o] = (uint8_t)s;
            o += 1;
            pos += len;
        } else {
            // Bytes past the entry's symbol count are rewritten by the same thread's next
            // probe; bytes past `end` belong to the next window and are not touched.
            const int rem = end - o;
            stage[o] = (uint8_t)e.syms;
            if (rem > 1) stage[o + 1] = (uint8_t)(e.syms >> 8);
            if (rem > 2) stage[o + 2] = (uint8_t)(e.syms >> 16);
            if (rem > 3) stage[o + 3] = (uint8_t)(e.syms >> 24);
            o += (int)DF11_META_NSYMS(e.meta);
            pos += DF11_META_NBITS(e.meta);
        }
    }
}
