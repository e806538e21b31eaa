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
// Multi-symbol tables, both indexed by the next K bits of the stream.  An entry
// covers up to four consecutive symbols that the reference's byte-wise LUT walk
// (decode.cu:105-118) is certain to produce for EVERY stream starting with those
// K bits; "escape" means the first symbol cannot be resolved from K bits and the
// full walk must be done for it.
//
//   decode entry (64 bit): .meta = bits consumed | symbols << 8   (escape: 1 << 24)
//                          .syms = the symbols, first one in the lowest byte
//   count entry  (32 bit): bits 0..7  bits consumed              (escape: 128)
//                          bits 8..10 symbols                    (escape: 0)
//                          bits 16..31 start offset of the 1st..4th symbol, 4 bits
//                                     each, 15 when absent      (escape: all 15)
//
// The decoding loops keep "position in window" and "output slot" in ONE register
//   acc = pos | slot << 8
// so that `acc += meta` advances both; the escape value pushes the slot past any
// legal end, which ends the loop without a test inside it.
// ---------------------------------------------------------------------------
struct Df11Entry {
    uint32_t meta;
    uint32_t syms;
};

#define DF11_DEC_ESCAPE (1u << 24)
#define DF11_CNT_ESCAPE 0xFFFF0080u

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

// Builds the entries for K-bit index v (K <= 14).  `agree` is the 255-byte agreement
// table of the root row.  A symbol is taken into the entry only when every completion
// of the unknown trailing bits makes the reference's walk (root row, and one second-level
// row for codes of 9 bits and more) end on the same symbol, and every symbol of an entry
// starts inside the K index bits, so an entry never differs from the reference's
// symbol-by-symbol result.
DF11_HD void df11_build_entry(const uint8_t *luts, int n_luts, const uint8_t *agree, uint32_t v, int K,
                              Df11Entry *dec, uint32_t *cnt)
{
    const uint8_t *lens = luts + (n_luts - 1) * 256;
    const uint32_t left = v << (32 - K);  // index bits, left-aligned
    uint32_t c = 0, nsyms = 0, syms = 0, starts = 0xFFFF0000u;
    for (int j = 0; j < 4; ++j) {
        const int r = K - (int)c;  // index bits still unread
        if (r <= 0)
            break;
        const int u = r >= 8 ? 0 : 8 - r;  // unknown low bits of this symbol's root byte
        const uint32_t idx = (left << c) >> 24;
        if (u > 0 && !agree[df11_agree_offset(u) + (int)(idx >> u)])
            break;
        uint32_t e = luts[idx];
        if (e >= 240u) {
            // pointer to a second-level row, indexed by the next stream byte: usable when the
            // root byte is fully known and every completion of the second byte agrees
            const uint32_t row = 256u - e;
            const int r2 = r - 8;  // known bits of the second byte
            if (u > 0 || r2 <= 0 || row >= (uint32_t)n_luts)
                break;
            const int u2 = r2 >= 8 ? 0 : 8 - r2;
            const uint32_t idx2 = ((left << c) >> 16) & 255u & ~((1u << u2) - 1u);
            const uint8_t *sub = luts + row * 256u;
            e = sub[idx2];
            bool same = true;
            for (uint32_t k = 1; k < (1u << u2); ++k)
                same = same && sub[idx2 + k] == e;
            if (!same || e >= 240u)
                break;  // ambiguous, or a third level: left to the full walk
        }
        const uint32_t l = lens[e];
        if (l == 0u || l > (uint32_t)DF11_MAX_CODE_LEN)
            break;
        starts &= ~(0xFu << (16 + 4 * j));
        starts |= c << (16 + 4 * j);
        syms |= e << (8 * j);
        ++nsyms;
        c += l;
    }
    if (nsyms == 0) {
        dec->meta = DF11_DEC_ESCAPE;
        dec->syms = 0;
        *cnt = DF11_CNT_ESCAPE;
    } else {
        dec->meta = c | (nsyms << 8);
        dec->syms = syms;
        *cnt = c | (nsyms << 8) | starts;
    }
}

// Number of symbols of a count entry that start before bit offset `lim` (1 <= lim <= 15).
DF11_HD uint32_t df11_owned_syms(uint32_t cmeta, uint32_t lim)
{
    return (uint32_t)(((cmeta >> 16) & 15u) < lim) + (uint32_t)(((cmeta >> 20) & 15u) < lim) +
           (uint32_t)(((cmeta >> 24) & 15u) < lim) + (uint32_t)((cmeta >> 28) < lim);
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

// Byte permute with the semantics of CUDA's __byte_perm for selector nibbles 0..7.
DF11_HD uint32_t df11_prmt(uint32_t x, uint32_t y, uint32_t sel)
{
#ifdef __CUDA_ARCH__
    return __byte_perm(x, y, sel);
#else
    const uint64_t both = ((uint64_t)y << 32) | x;
    uint32_t r = 0;
    for (int i = 0; i < 4; ++i)
        r |= (uint32_t)((both >> (8 * ((sel >> (4 * i)) & 7u))) & 0xFFu) << (8 * i);
    return r;
#endif
}

// Four BF16 values from four exponent bytes `e4` and four sign/mantissa bytes `m4`
// (element k in byte k).  Per element, decode.cu:207-209:
//   high byte = (sm & 0x80) | (e >> 1),   low byte = (e << 7) | (sm & 0x7f).
// Both bytes are formed for all four elements at once, then interleaved.
DF11_HD void df11_merge4(uint32_t e4, uint32_t m4, uint32_t *out01, uint32_t *out23)
{
    const uint32_t hi = ((e4 >> 1) & 0x7F7F7F7Fu) | (m4 & 0x80808080u);
    const uint32_t lo = ((e4 << 7) & 0x80808080u) | (m4 & 0x7F7F7F7Fu);
    *out01 = df11_prmt(lo, hi, 0x5140);
    *out23 = df11_prmt(lo, hi, 0x7362);
}

DF11_HD uint16_t df11_merge1(uint32_t e, uint32_t m)
{
    return (uint16_t)(((m & 0x80u) << 8) | (e << 7) | (m & 0x7Fu));
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

// The two window routines are written against a memory policy `M` so that the CUDA
// kernels (32-bit shared-memory addresses, explicit ld/st.shared) and the host
// emulation used by the CPU tests (plain arrays) run the same algorithm:
//   uint32_t  M::cnt(i)        count-table entry i
//   Df11Entry M::dec(i)        decode-table entry i
//   uint32_t  M::lut(i)        byte i of the `luts` tensor (for the escape walk)
//   void      M::put8(addr, v)       stage byte addr = v & 0xFF
//
// df11_walk_m is the exact per-symbol rule of the reference (decode.cu:105-116) applied
// to the 32 bits `x` (MSB first): row 0 is indexed by the first byte, an entry >= 240
// points to row 256 - entry indexed by the next byte (at most four levels), the last row
// holds code lengths.  *bad is set when the tables are unusable (pointer outside the
// tensor, length 0 or > 32) -- the reference would read out of bounds or never terminate.
template <class M>
DF11_HD uint32_t df11_walk_m(const M &m, int n_luts, uint32_t x, uint32_t *len, int *bad)
{
    uint32_t e = m.lut(x >> 24);
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
            e = m.lut(row * 256u + ((x >> shift) & 255u));
        }
    }
    uint32_t l = m.lut((uint32_t)(n_luts - 1) * 256u + e);
    if (l == 0u || l > (uint32_t)DF11_MAX_CODE_LEN) {
        *bad = 1;
        l = 64u;  // leave the window
    }
    *len = l;
    return e;
}

// Counting pass: number of codes that START inside the window's 64 bits (the
// ownership rule of decode.cu:104,129), beginning at bit `gap`.
template <int K, class M>
DF11_HD uint32_t df11_count_window(const M &m, int n_luts, uint32_t w0, uint32_t w1, uint32_t w2,
                                   uint32_t gap, int *bad)
{
    uint32_t acc = gap;  // pos | count << 8   (a caller with nothing to count passes gap = 64)
    for (;;) {
        // all K index bits inside the window: every symbol of an entry starts before bit 64
        while ((acc & 0xFFu) <= 64u - K) {
            const uint32_t x = df11_peek(w0, w1, w2, acc);
            acc += m.cnt(x >> (32 - K)) & 0xFFFFu;
        }
        // the last few bits: count only the symbols that start before bit 64
        while ((acc & 0xFFu) < 64u) {
            const uint32_t x = df11_peek(w0, w1, w2, acc);
            const uint32_t c = m.cnt(x >> (32 - K));
            acc += (c & 0xFFu) + (df11_owned_syms(c, 64u - (acc & 0xFFu)) << 8);
        }
        if ((acc & 0xFFu) < 128u)
            break;
        // an escape entry added 128 to the position: take that one symbol the long way
        acc -= 128u;
        uint32_t len;
        df11_walk_m(m, n_luts, df11_peek(w0, w1, w2, acc), &len, bad);
        acc += len + 256u;
    }
    return acc >> 8;
}

// Decoding pass: writes the window's exponents to stage bytes [o, end).  Terminates after at
// most end - o probes whatever the data is, and writes nothing outside.  Extra policy member:
//   void M::put8(addr, v)    stage byte `addr` = v & 0xFF
// (Collecting the exponents in a 64-bit buffer and storing whole aligned words, single bytes only
// at a window's two ends, was measured: a tenth slower -- the byte stores' bank conflicts cost
// less than the extra shifts.)
template <int K, class M>
DF11_HD void df11_decode_window(const M &m, int n_luts, uint32_t w0, uint32_t w1, uint32_t w2, uint32_t gap,
                                uint32_t o, uint32_t end, int *bad)
{
    uint32_t acc = gap | (o << 8);  // pos | slot << 8
    const uint32_t end_acc = end << 8;
    for (;;) {
        // at least four slots left: store all four bytes of an entry; the ones past its
        // symbol count are rewritten by this thread's next probe
        while (acc + (3u << 8) < end_acc) {
            const Df11Entry e = m.dec(df11_peek(w0, w1, w2, acc) >> (32 - K));
            const uint32_t slot = acc >> 8;
            m.put8(slot, e.syms);
            m.put8(slot + 1u, e.syms >> 8);
            m.put8(slot + 2u, e.syms >> 16);
            m.put8(slot + 3u, e.syms >> 24);
            acc += e.meta;
        }
        // fewer than four left: bytes past `end` belong to the next window
        while (acc < end_acc) {
            const Df11Entry e = m.dec(df11_peek(w0, w1, w2, acc) >> (32 - K));
            const uint32_t slot = acc >> 8, rem = end - slot;
            m.put8(slot, e.syms);
            if (rem > 1u) m.put8(slot + 1u, e.syms >> 8);
            if (rem > 2u) m.put8(slot + 2u, e.syms >> 16);
            acc += e.meta;
        }
        if (!(acc & DF11_DEC_ESCAPE))
            break;
        // an escape entry ended the loop: decode that one symbol with the full walk
        acc -= DF11_DEC_ESCAPE;
        uint32_t len;
        const uint32_t s = df11_walk_m(m, n_luts, df11_peek(w0, w1, w2, acc), &len, bad);
        if (acc < end_acc) m.put8(acc >> 8, s);
        acc += len + 256u;
    }
}

// ---------------------------------------------------------------------------
// Seek points (prepared form).  A one-time pass records, for every group of EPT
// consecutive output elements (EPT = 16 or 32, groups aligned to EPT in the element
// index), the absolute bit position in the stream at which the group's first code
// starts.  A decoding thread then needs nothing but its group number: it reads the
// group's bit position, decodes exactly EPT codes from there and writes EPT BF16
// values -- no shared staging, no scan, no barrier.
//
// Storage: bit position = (hi[g / 32] << 16 | lo[g]) (+ 65536 if lo[g] < lo[32*(g/32)]),
// i.e. 16 bits per group plus 32 bits per 32 groups; the 32 groups of one entry of
// `hi` span at most 31 * 32 * 32 < 65536 bits, so one wrap-around is unambiguous.
// ---------------------------------------------------------------------------

// Walks the codes owned by one window (as df11_count_window does) knowing the output
// index of its first code, and reports every code whose index is a multiple of `ept`:
// emit(group, bit offset inside the window).  Extra policy member: none.
template <int K, class M, class Emit>
DF11_HD void df11_mark_window(const M &m, int n_luts, uint32_t w0, uint32_t w1, uint32_t w2, uint32_t gap,
                              uint64_t first_index, uint32_t ept, Emit emit, int *bad)
{
    uint32_t pos = gap;
    uint64_t idx = first_index;
    while (pos < 64u) {
        const uint32_t x = df11_peek(w0, w1, w2, pos);
        const uint32_t c = m.cnt(x >> (32 - K));
        uint32_t n, nbits, starts;
        if (c == DF11_CNT_ESCAPE) {
            df11_walk_m(m, n_luts, x, &nbits, bad);
            n = 1u;
            starts = 0u;
        } else {
            const uint32_t lim = 64u - pos;
            n = lim >= 15u ? ((c >> 8) & 7u) : df11_owned_syms(c, lim);
            nbits = c & 0xFFu;
            starts = c >> 16;
        }
        const uint32_t k = (uint32_t)(0u - (uint32_t)idx) & (ept - 1u);  // distance to the next multiple
        if (k < n)
            emit((idx + k) / ept, pos + ((starts >> (4u * k)) & 15u));
        idx += n;
        pos += nbits;
    }
}

// ---------------------------------------------------------------------------
// Bit packer arithmetic shared by the GPU packer (df11_encode.cu) and its CPU emulation.
// The stream is a sequence of big-endian 32-bit words; a code of `len` bits (1..32) whose
// first bit is stream bit `bit` lies in word bit >> 5 and possibly the next one.
// ---------------------------------------------------------------------------

// The two big-endian words a code contributes: *hi to word (bit >> 5), *lo to the next (0 when
// the code does not reach it).
DF11_HD void df11_place_code(uint64_t bit, uint32_t len, uint32_t val, uint32_t *hi, uint32_t *lo)
{
    const uint64_t v = (uint64_t)val << (64u - len - (uint32_t)(bit & 31u));
    *hi = (uint32_t)(v >> 32);
    *lo = (uint32_t)v;
}

// A big-endian word as the little-endian machine stores it (what is ORed into memory).
DF11_HD uint32_t df11_bswap32(uint32_t v)
{
    return (v >> 24) | ((v >> 8) & 0xFF00u) | ((v << 8) & 0xFF0000u) | (v << 24);
}

// gaps[window] = g as the bytes to OR into the packed 5-bit array: *byte is the index of the
// first byte, *first / *second what goes into it and into the byte after it (0: nothing).
DF11_HD void df11_gap_field(uint64_t window, uint32_t g, uint64_t *byte, uint32_t *first, uint32_t *second)
{
    const uint64_t bit = 5u * window;
    const uint32_t v = g << (11u - (uint32_t)(bit & 7u));  // the field inside the 16 bits byte:byte+1
    *byte = bit >> 3;
    *first = v >> 8;
    *second = v & 0xFFu;
}

// The bits of the padding code that complete a last byte of which `rem` (1..7) bits are used.
DF11_HD uint32_t df11_pad_bits(uint32_t rem, uint32_t pad_len, uint32_t pad_val)
{
    const uint32_t room = 8u - rem;
    uint32_t pad = 0;
    if (pad_len >= room) pad = pad_val >> (pad_len - room);
    else if (pad_len > 0u) pad = pad_val << (room - pad_len);
    return pad & ((1u << room) - 1u);
}

// Low 32 bits of (hi:lo) >> min(s, 32).
DF11_HD uint32_t df11_funnel_rc(uint32_t lo, uint32_t hi, uint32_t s)
{
#ifdef __CUDA_ARCH__
    return __funnelshift_rc(lo, hi, s);
#else
    if (s >= 32u) return hi;
    return s ? (lo >> s) | (hi << (32u - s)) : lo;
#endif
}

// The exponents a thread has decoded, as a 20-byte shift register x0 (lowest) .. x4: every
// table probe shifts it right by as many bytes as the entry has symbols and enters them at the
// top, first symbol lowest.  After c codes (16 <= c <= 19: the last probe may run up to three
// codes past the sixteenth) code k sits at byte 20 - c + k, so the sixteen wanted bytes are the
// register shifted right by 20 - c bytes, and the c - 16 extra codes stay at the top of x4.
struct Df11ExpShift {
    uint32_t x0, x1, x2, x3, x4;
    DF11_HD void push(uint32_t syms, uint32_t bits)  // bits = 8 * symbols, 0..32
    {
        x0 = df11_funnel_rc(x0, x1, bits);
        x1 = df11_funnel_rc(x1, x2, bits);
        x2 = df11_funnel_rc(x2, x3, bits);
        x3 = df11_funnel_rc(x3, x4, bits);
        x4 = df11_funnel_rc(x4, syms, bits);
    }
    // the sixteen exponents, four per word, lowest byte first; acc as described at DF11_FAST_ESCAPE
    DF11_HD void take(uint32_t acc, uint32_t *e0, uint32_t *e1, uint32_t *e2, uint32_t *e3) const
    {
        const uint32_t bits = 160u - ((acc >> 16) & 0xFFu);  // 8 * (20 - codes done): 8..32
        *e0 = df11_funnel_rc(x0, x1, bits);
        *e1 = df11_funnel_rc(x1, x2, bits);
        *e2 = df11_funnel_rc(x2, x3, bits);
        *e3 = df11_funnel_rc(x3, x4, bits);
    }
};

// Fast-decoder form of a decode-table entry's first word: bits consumed in bits 0..7 (at most
// 31), eight times the number of symbols in bits 16..23; an entry that needs the full walk is
// DF11_FAST_ESCAPE alone.  The running state `acc` of a thread is the sum of the entries it used:
//   bits 0..7   position in the window (64 and more: window used up)
//   bit 15      an escape entry was met
//   bits 16..23 8 * codes done (128 and more: the sixteen codes of this pass are done)
#define DF11_FAST_ESCAPE (1u << 15)
#define DF11_FAST_DONE (128u << 16)
#define DF11_FAST_LEAVE (DF11_FAST_ESCAPE | DF11_FAST_DONE | 64u)

DF11_HD constexpr uint32_t df11_fast_meta(uint32_t meta)
{
    return (meta == DF11_DEC_ESCAPE || (meta & 0xFFu) > 31u) ? DF11_FAST_ESCAPE
                                                             : (meta & 0xFFu) | (((meta >> 8) & 7u) << 19);
}

// Decodes the EPT codes of one group sixteen at a time and hands them over four per word,
// lowest byte first.  The group's first code starts `bit` (0..31) bits into stream word
// `word_index` (32-bit big-endian words; streams up to 16 GiB).  This is the statement of the
// fast kernel's algorithm, instruction for instruction in its arithmetic (the kernel runs the
// inner loop as hand-scheduled device code, df11_decode.cu), and the form the CPU tests run.
// Extra policy members:
//   uint32_t M::word(i)            stream bytes [4i, 4i+4) as a big-endian word, 0 past the end
//   void     M::flush(k, word)     exponents 4k .. 4k+3 of the group
//
// The 96-bit window w0:w1:w2 is kept shifted so that the next code starts at its top bit; a
// group of 16 codes rarely needs more than the 64 positions that gives, so the reload inside
// the loop is the exception, not the rule.
template <int K, int EPT, class M>
DF11_HD void df11_decode_group(const M &m, int n_luts, uint32_t word_index, uint32_t bit, bool active, int *bad)
{
    if (!active) return;
    uint32_t w0, w1, w2;
    auto load = [&]() {
        const uint32_t a = m.word(word_index), b = m.word(word_index + 1u);
        const uint32_t c = m.word(word_index + 2u), d = m.word(word_index + 3u);
        w0 = df11_funnel_l(b, a, bit);
        w1 = df11_funnel_l(c, b, bit);
        w2 = df11_funnel_l(d, c, bit);
    };
    auto shift = [&](uint32_t len) {  // window <<= len, 0 <= len <= 31
        w0 = df11_funnel_l(w1, w0, len);
        w1 = df11_funnel_l(w2, w1, len);
        w2 = len ? w2 << len : w2;
    };
    Df11ExpShift X = {0, 0, 0, 0, 0};
    uint32_t acc = 0;
    for (int part = 0; part < EPT / 16; ++part) {
        if (part > 0) {  // go on where the previous sixteen stopped; codes decoded beyond them are at the top of X
            const uint32_t at = bit + (acc & 0x7Fu);
            word_index += at >> 5;
            bit = at & 31u;
            acc = (acc & ~0xFFu) - DF11_FAST_DONE;
        }
        load();
        for (;;) {
            while ((acc & DF11_FAST_LEAVE) == 0u) {  // the probe loop
                const Df11Entry e = m.dec(w0 >> (32 - K));
                const uint32_t meta = df11_fast_meta(e.meta);
                X.push(e.syms, meta >> 16);
                shift(meta & 31u);
                acc += meta;
            }
            if ((acc & (DF11_FAST_ESCAPE | 64u)) == 0u) break;  // 16 codes done, nothing special
            if (acc & DF11_FAST_ESCAPE) {  // the table could not resolve this code from K bits: full walk
                acc -= DF11_FAST_ESCAPE;
                uint32_t len;
                const uint32_t sym = df11_walk_m(m, n_luts, w0, &len, bad);
                X.push(sym, 8u);
                acc += len | (8u << 16);
                if (len < 32u) {
                    shift(len);
                } else {  // a 32-bit code, or an unusable table (len 64): the reload below follows
                    w0 = w1, w1 = w2, w2 = 0;
                }
            }
            if (acc & DF11_FAST_DONE) break;  // 16 codes done (the position may be past 63)
            if (acc & 64u) {                  // position 64..127: reload the window where the position has got to
                const uint32_t at = bit + (acc & 0x7Fu);
                word_index += at >> 5;
                bit = at & 31u;
                load();
                acc &= ~0xFFu;
            }
        }
        uint32_t e0, e1, e2, e3;
        X.take(acc, &e0, &e1, &e2, &e3);
        m.flush(4u * part + 0u, e0);
        m.flush(4u * part + 1u, e1);
        m.flush(4u * part + 2u, e2);
        m.flush(4u * part + 3u, e3);
    }
}
