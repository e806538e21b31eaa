// Host-side emulation of the CUDA decode kernels' algorithm.  TEST INFRASTRUCTURE ONLY:
// it is compiled by tests/test_emulation.py, never linked into libdf11 and never used by
// the product.  It runs the same table builder, window routines and merge arithmetic
// (dfloat11_b200/csrc/df11_common.h) that the kernels run, with the kernels' block-level
// flow (clamps, alignment phase, 8-element merge groups) restated serially, so that the
// algorithm can be checked against the CPU oracle on a machine without a GPU.
#include <stdint.h>
#include <string.h>

#include <vector>

#include "../../dfloat11_b200/csrc/df11_common.h"
#include "../../include/df11.h"

namespace {

bool g_reverse = false;  // order in which the windows of a block run their decode pass

// Memory policy of the window routines for plain host arrays.
struct HostMem {
    const uint32_t *cnt_t;
    const Df11Entry *dec_t;
    const uint8_t *luts;
    uint8_t *stage;
    uint32_t cnt(uint32_t i) const { return cnt_t[i]; }
    Df11Entry dec(uint32_t i) const { return dec_t[i]; }
    uint32_t lut(uint32_t i) const { return luts[i]; }
    void put8(uint32_t addr, uint32_t v) const { stage[addr] = (uint8_t)v; }
    // seek-point decoder
    const uint8_t *codes = nullptr;
    int64_t n_bytes = 0;
    uint32_t *row = nullptr;
    uint32_t word(uint32_t i) const
    {
        uint32_t v = 0;
        for (int k = 0; k < 4; ++k) {
            const int64_t o = (int64_t)i * 4 + k;
            if (o < n_bytes) v |= (uint32_t)codes[o] << (24 - 8 * k);
        }
        return v;
    }
    void flush(uint32_t k, uint32_t v) const { row[k] = v; }
};

void load_window(const uint8_t *codes, int64_t n_bytes, int64_t t, uint32_t w[3])
{
    w[0] = w[1] = w[2] = 0;
    for (int k = 0; k < 12; ++k) {
        const int64_t i = t * 8 + k;
        const uint32_t byte = i < n_bytes ? codes[i] : 0u;
        w[k >> 2] |= byte << (24 - 8 * (k & 3));
    }
}

template <int K>
void build_tables(const uint8_t *luts, int n_luts, std::vector<Df11Entry> &dec, std::vector<uint32_t> &cnt)
{
    uint8_t agree[256] = {0};
    for (int u = 1; u <= 8; ++u)
        for (int blk = 0; blk < (256 >> u); ++blk) agree[df11_agree_offset(u) + blk] = df11_agree_flag(luts, u, blk);
    dec.resize(1 << K);
    cnt.resize(1 << K);
    for (uint32_t v = 0; v < (1u << K); ++v) df11_build_entry(luts, n_luts, agree, v, K, &dec[v], &cnt[v]);
}

// The prepared form: seek points from the marking pass, then one group per "thread".
template <int K, int EPT>
int run_seek(const uint8_t *luts, int n_luts, const uint8_t *codes, int64_t n_bytes, const uint8_t *sm,
             int64_t n_elements, const uint32_t *pos, const uint8_t *gaps, uint16_t *out, int *status)
{
    const int64_t n_blocks = (n_bytes + DF11_BLOCK_BYTES - 1) / DF11_BLOCK_BYTES;
    const int64_t n_gap_bytes = n_blocks * DF11_GAP_BYTES_PER_BLOCK;
    std::vector<Df11Entry> dec;
    std::vector<uint32_t> cnt;
    build_tables<K>(luts, n_luts, dec, cnt);
    HostMem mem{cnt.data(), dec.data(), luts, nullptr};
    mem.codes = codes;
    mem.n_bytes = n_bytes;
    int bad = 0;

    const uint64_t n_groups = ((uint64_t)n_elements + EPT - 1) / EPT;
    const uint64_t n_chunks = (n_groups + 31) / 32;
    std::vector<uint16_t> lo(n_chunks * 32, 0xDEAD);
    std::vector<uint32_t> hi(n_chunks, 0xDEADBEEF);
    for (int64_t b = 0; b < n_blocks; ++b) {
        uint64_t index = pos[b];
        for (int tid = 0; tid < DF11_WINDOWS_PER_BLOCK; ++tid) {
            const int64_t t = b * DF11_WINDOWS_PER_BLOCK + tid;
            if (t * 8 >= n_bytes) break;
            uint32_t w[3];
            load_window(codes, n_bytes, t, w);
            const uint32_t gap = df11_gap(gaps, n_gap_bytes, t);
            int tbad = 0;
            const uint32_t c = df11_count_window<K>(mem, n_luts, w[0], w[1], w[2], gap, &tbad);
            df11_mark_window<K>(
                mem, n_luts, w[0], w[1], w[2], gap, index, EPT,
                [&](uint64_t group, uint32_t bit_in_window) {
                    if (group >= n_groups) return;
                    const uint64_t bit = (uint64_t)t * 64 + bit_in_window;
                    lo[group] = (uint16_t)bit;
                    if ((group & 31) == 0) hi[group >> 5] = (uint32_t)(bit >> 16);
                },
                &tbad);
            if (tbad) bad |= DF11_STATUS_BAD_TABLE;
            index += c;
        }
    }
    for (uint64_t group = 0; group < n_groups; ++group) {
        const uint64_t chunk = group >> 5;
        const uint32_t l = lo[group], l0 = lo[chunk * 32];
        const uint64_t bitpos = ((uint64_t)hi[chunk] << 16) + l + (l < l0 ? 65536u : 0u);
        uint32_t row[EPT / 4];
        for (int k = 0; k < EPT / 4; ++k) row[k] = 0xEEEEEEEEu;
        mem.row = row;
        int tbad = 0;
        df11_decode_group<K, EPT>(mem, n_luts, (uint32_t)(bitpos >> 5), (uint32_t)bitpos & 31u, true, &tbad);
        if (tbad) bad |= DF11_STATUS_BAD_TABLE;
        const int64_t first = (int64_t)group * EPT;
        if (first + EPT <= n_elements) {
            for (int k = 0; k < EPT / 4; ++k) {
                uint32_t m4, r[2];
                memcpy(&m4, sm + first + 4 * k, 4);
                df11_merge4(row[k], m4, &r[0], &r[1]);
                memcpy(out + first + 4 * k, r, 8);
            }
        } else {
            const uint8_t *bytes = reinterpret_cast<const uint8_t *>(row);
            for (int k = 0; k < EPT && first + k < n_elements; ++k) out[first + k] = df11_merge1(bytes[k], sm[first + k]);
        }
    }
    if (status) *status = bad;
    return 0;
}

template <int K>
int run(const uint8_t *luts, int n_luts, const uint8_t *codes, int64_t n_bytes, const uint8_t *sm,
        int64_t n_elements, const uint32_t *pos, const uint8_t *gaps, uint16_t *out, int max_block_elems,
        int *status)
{
    const int64_t n_blocks = (n_bytes + DF11_BLOCK_BYTES - 1) / DF11_BLOCK_BYTES;
    const int64_t n_gap_bytes = n_blocks * DF11_GAP_BYTES_PER_BLOCK;
    std::vector<Df11Entry> dec;
    std::vector<uint32_t> cnt;
    build_tables<K>(luts, n_luts, dec, cnt);

    int64_t m = max_block_elems > 0 ? max_block_elems : DF11_MAX_BLOCK_ELEMS;
    if (m > DF11_MAX_BLOCK_ELEMS) m = DF11_MAX_BLOCK_ELEMS;
    const int stage_bytes = (int)((m + 15 + 15) / 16 * 16) + 16;
    std::vector<uint8_t> stage(stage_bytes);
    HostMem mem{cnt.data(), dec.data(), luts, stage.data()};
    int bad = 0;

    for (int64_t b = 0; b < n_blocks; ++b) {
        int64_t base = pos[b];
        const int64_t next = pos[b + 1];
        int64_t c = next - base;
        if (c < 0 || next > n_elements) {
            bad |= DF11_STATUS_BAD_POSITIONS;
            c = c < 0 ? 0 : n_elements - base;
            if (c < 0) c = 0;
        }
        const uint32_t phase = (uint32_t)(base & 15);
        if (c + phase > stage_bytes - 16) {
            bad |= DF11_STATUS_TRUNCATED;
            c = stage_bytes - 16 - phase;
        }
        const uint32_t block_cnt = (uint32_t)c;
        memset(stage.data(), 0xEE, stage.size());  // poison: stale bytes must never reach the output

        // the kernel's 512 threads write their windows in no particular order: first every window's
        // slots (count pass + scan), then the decode pass front to back or back to front (g_reverse),
        // so that a window that writes into a neighbour's bytes shows up in one of the two orders
        uint32_t run_sum = 0;
        struct Win { uint32_t w[3], gap, o, end; bool live; } wins[DF11_WINDOWS_PER_BLOCK];
        for (int tid = 0; tid < DF11_WINDOWS_PER_BLOCK; ++tid) {
            Win &x = wins[tid];
            const int64_t t = b * DF11_WINDOWS_PER_BLOCK + tid;
            x.live = t * 8 < n_bytes;
            if (!x.live) continue;
            load_window(codes, n_bytes, t, x.w);
            int tbad = 0;
            x.gap = df11_gap(gaps, n_gap_bytes, t);
            const uint32_t n = df11_count_window<K>(mem, n_luts, x.w[0], x.w[1], x.w[2], x.gap, &tbad);
            uint32_t o = run_sum, end = o + n;
            run_sum += n;
            x.o = (o < block_cnt ? o : block_cnt) + phase;
            x.end = (end < block_cnt ? end : block_cnt) + phase;
            if (tbad) bad |= DF11_STATUS_BAD_TABLE;
        }
        for (int k = 0; k < DF11_WINDOWS_PER_BLOCK; ++k) {
            const Win &x = wins[g_reverse ? DF11_WINDOWS_PER_BLOCK - 1 - k : k];
            if (!x.live) continue;
            int tbad = 0;
            df11_decode_window<K>(mem, n_luts, x.w[0], x.w[1], x.w[2], x.gap, x.o, x.end, &tbad);
            if (tbad) bad |= DF11_STATUS_BAD_TABLE;
        }

        const int64_t gbase = base - phase;
        const uint8_t *sm_blk = sm + gbase;
        uint16_t *out_blk = out + gbase;
        const uint32_t last = phase + block_cnt;
        const uint32_t g_lo = (phase + 7u) >> 3, g_hi = last >> 3;
        for (uint32_t g = g_lo; g < g_hi; ++g) {
            uint32_t ex[2], mm[2], r[4];
            memcpy(ex, stage.data() + 8 * g, 8);
            memcpy(mm, sm_blk + 8 * g, 8);
            df11_merge4(ex[0], mm[0], &r[0], &r[1]);
            df11_merge4(ex[1], mm[1], &r[2], &r[3]);
            memcpy(out_blk + 8 * g, r, 16);
        }
        for (uint32_t tid = 0; tid < 16; ++tid) {
            const uint32_t i = tid < 8u ? 8u * (g_lo - 1u) + tid : 8u * g_hi + (tid - 8u);
            const bool mine = tid < 8u ? ((phase & 7u) != 0u && i >= phase && i < last) : (g_hi >= g_lo && i < last);
            if (mine) out_blk[i] = df11_merge1(stage[i], sm_blk[i]);
        }
    }
    if (status) *status = bad;
    return 0;
}

}  // namespace

extern "C" void df11_emul_window_order(int reverse) { g_reverse = reverse != 0; }

// prepared: 0 = the self-contained two-pass flow, 16 / 32 = seek points every 16 / 32 elements
extern "C" int df11_emul_decode(const uint8_t *luts, int n_luts, const uint8_t *codes, int64_t n_bytes,
                                const uint8_t *sm, int64_t n_elements, const uint32_t *pos,
                                const uint8_t *gaps, uint16_t *out, int K, int prepared, int max_block_elems,
                                int *status)
{
#define DF11_EMUL_CASE(KK)                                                                                          \
    case KK:                                                                                                        \
        if (prepared == 16) return run_seek<KK, 16>(luts, n_luts, codes, n_bytes, sm, n_elements, pos, gaps, out, status); \
        if (prepared == 32) return run_seek<KK, 32>(luts, n_luts, codes, n_bytes, sm, n_elements, pos, gaps, out, status); \
        return run<KK>(luts, n_luts, codes, n_bytes, sm, n_elements, pos, gaps, out, max_block_elems, status);
    switch (K) {
        DF11_EMUL_CASE(9)
        DF11_EMUL_CASE(10)
        DF11_EMUL_CASE(11)
        DF11_EMUL_CASE(12)
        DF11_EMUL_CASE(13)
        DF11_EMUL_CASE(14)
    }
#undef DF11_EMUL_CASE
    return -1;
}

// The two tables for a given K (for statistics and direct inspection in tests).
extern "C" int df11_emul_table(const uint8_t *luts, int n_luts, int K, uint32_t *meta_out, uint32_t *syms_out,
                               uint32_t *cnt_out)
{
    std::vector<Df11Entry> dec;
    std::vector<uint32_t> cnt;
    switch (K) {
    case 9: build_tables<9>(luts, n_luts, dec, cnt); break;
    case 10: build_tables<10>(luts, n_luts, dec, cnt); break;
    case 11: build_tables<11>(luts, n_luts, dec, cnt); break;
    case 12: build_tables<12>(luts, n_luts, dec, cnt); break;
    case 13: build_tables<13>(luts, n_luts, dec, cnt); break;
    case 14: build_tables<14>(luts, n_luts, dec, cnt); break;
    default: return -1;
    }
    for (size_t v = 0; v < dec.size(); ++v) {
        meta_out[v] = dec[v].meta;
        syms_out[v] = dec[v].syms;
        cnt_out[v] = cnt[v];
    }
    return 0;
}

// The GPU bit packer's per-element rules (df11_encode.cu), run one element after the other with
// the same shared arithmetic (df11_place_code, df11_bswap32, df11_gap_field, df11_pad_bits) and
// the same way of writing: ORs into zeroed little-endian 32-bit words.  `codes` must have room
// for n_bytes rounded up to a multiple of 4; `gaps` and `pos` as for df11_encode_host.
extern "C" int df11_emul_pack(const uint8_t *ex, int64_t n, const uint8_t *code_len, const uint32_t *code_val,
                              uint32_t pad_len, uint32_t pad_val, uint8_t *codes, int64_t n_bytes, uint8_t *gaps,
                              int64_t n_gap_bytes, uint32_t *pos, int64_t n_positions)
{
    const int64_t n_blocks = (n_bytes + DF11_BLOCK_BYTES - 1) / DF11_BLOCK_BYTES;
    if (n_gap_bytes != n_blocks * DF11_GAP_BYTES_PER_BLOCK || n_positions != n_blocks + 1) return -1;
    memset(codes, 0, (size_t)((n_bytes + 3) / 4 * 4));
    memset(gaps, 0, (size_t)n_gap_bytes);
    memset(pos, 0, (size_t)n_positions * 4);
    uint32_t *words = reinterpret_cast<uint32_t *>(codes);
    auto or_byte = [](uint8_t *buf, int64_t index, uint32_t value) {
        reinterpret_cast<uint32_t *>(buf)[index >> 2] |= value << (8 * (index & 3));
    };
    auto set_gap = [&](int64_t window, uint32_t g) {
        uint64_t byte;
        uint32_t first, second;
        df11_gap_field((uint64_t)window, g, &byte, &first, &second);
        or_byte(gaps, (int64_t)byte, first);
        if (second) or_byte(gaps, (int64_t)byte + 1, second);
    };
    int64_t bit = 0, prev_start = -1;
    for (int64_t i = 0; i < n; ++i) {
        const uint32_t len = code_len[ex[i]];
        if (len == 0) return -2;
        if (prev_start < 0 || (prev_start >> 6) != (bit >> 6)) {
            set_gap(bit >> 6, (uint32_t)(bit & 63));
            if (prev_start < 0 || (prev_start >> 15) != (bit >> 15)) pos[bit >> 15] = (uint32_t)i;
        }
        uint32_t hi, lo;
        df11_place_code((uint64_t)bit, len, code_val[ex[i]], &hi, &lo);
        words[bit >> 5] |= df11_bswap32(hi);
        if (lo) words[(bit >> 5) + 1] |= df11_bswap32(lo);
        prev_start = bit;
        bit += len;
    }
    const uint32_t rem = (uint32_t)(bit & 7);
    if (rem) {
        if ((prev_start >> 6) != (bit >> 6)) set_gap(bit >> 6, (uint32_t)(bit & 63));
        if ((prev_start >> 15) != (bit >> 15)) pos[bit >> 15] = (uint32_t)n;
        or_byte(codes, n_bytes - 1, df11_pad_bits(rem, pad_len, pad_val));
    }
    pos[n_blocks] = (uint32_t)n;
    return (bit + 7) / 8 == n_bytes ? 0 : -3;
}
