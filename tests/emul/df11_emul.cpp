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

uint32_t byte_perm(uint32_t x, uint32_t y, uint32_t sel)
{
    const uint64_t both = ((uint64_t)y << 32) | x;
    uint32_t r = 0;
    for (int i = 0; i < 4; ++i) {
        const uint32_t n = (sel >> (4 * i)) & 7u;
        r |= (uint32_t)((both >> (8 * n)) & 0xFF) << (8 * i);
    }
    return r;
}

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
int run(const uint8_t *luts, int n_luts, const uint8_t *codes, int64_t n_bytes, const uint8_t *sm,
        int64_t n_elements, const uint32_t *pos, const uint8_t *gaps, uint16_t *out, int prepared,
        int max_block_elems, int *status)
{
    const int64_t n_blocks = (n_bytes + DF11_BLOCK_BYTES - 1) / DF11_BLOCK_BYTES;
    const int64_t n_gap_bytes = n_blocks * DF11_GAP_BYTES_PER_BLOCK;
    uint8_t agree[256] = {0};
    for (int u = 1; u <= 8; ++u)
        for (int blk = 0; blk < (256 >> u); ++blk) agree[df11_agree_offset(u) + blk] = df11_agree_flag(luts, u, blk);
    std::vector<Df11Entry> table(1 << K);
    for (uint32_t v = 0; v < (1u << K); ++v) table[v] = df11_build_entry(luts, n_luts, agree, v, K);

    int64_t m = max_block_elems > 0 ? max_block_elems : DF11_MAX_BLOCK_ELEMS;
    const int stage_bytes = (int)((m + 7 + 15) / 16 * 16) + 16;
    const int stage_cap = stage_bytes - 8;
    std::vector<uint8_t> stage(stage_bytes);
    int bad = 0;

    std::vector<uint16_t> woff;
    if (prepared) {  // the counting launch
        woff.assign(n_blocks * DF11_WINDOWS_PER_BLOCK + 1, 0xFFFF);
        for (int64_t b = 0; b < n_blocks; ++b) {
            uint32_t run_sum = 0;
            for (int tid = 0; tid < DF11_WINDOWS_PER_BLOCK; ++tid) {
                const int64_t t = b * DF11_WINDOWS_PER_BLOCK + tid;
                if (t * 8 >= n_bytes) break;
                uint32_t w[3];
                load_window(codes, n_bytes, t, w);
                int tbad = 0;
                const uint32_t cnt = df11_count_window<K>(table.data(), luts, n_luts, w[0], w[1], w[2],
                                                          df11_gap(gaps, n_gap_bytes, t), &tbad);
                if (tbad) bad |= DF11_STATUS_BAD_TABLE;
                woff[t] = (uint16_t)(run_sum > 65535 ? 65535 : run_sum);
                run_sum += cnt;
            }
        }
    }

    for (int64_t b = 0; b < n_blocks; ++b) {
        int64_t base = pos[b];
        const int64_t next = pos[b + 1];
        int64_t c = next - base;
        if (c < 0 || next > n_elements) {
            bad |= DF11_STATUS_BAD_POSITIONS;
            c = c < 0 ? 0 : n_elements - base;
            if (c < 0) c = 0;
        }
        const int phase = (int)(base & 7);
        if (c + phase > stage_cap) {
            bad |= DF11_STATUS_TRUNCATED;
            c = stage_cap - phase;
        }
        const int block_cnt = (int)c;
        memset(stage.data(), 0xEE, stage.size());  // poison: stale bytes must never reach the output

        uint32_t run_sum = 0;
        for (int tid = 0; tid < DF11_WINDOWS_PER_BLOCK; ++tid) {
            const int64_t t = b * DF11_WINDOWS_PER_BLOCK + tid;
            if (t * 8 >= n_bytes) break;
            uint32_t w[3];
            load_window(codes, n_bytes, t, w);
            const uint32_t gap = df11_gap(gaps, n_gap_bytes, t);
            int o, end, tbad = 0;
            if (prepared) {
                o = woff[t];
                const bool last = tid == DF11_WINDOWS_PER_BLOCK - 1 || (t + 1) * 8 >= n_bytes;
                end = last ? block_cnt : (int)woff[t + 1];
            } else {
                const uint32_t cnt = df11_count_window<K>(table.data(), luts, n_luts, w[0], w[1], w[2], gap, &tbad);
                o = (int)run_sum;
                end = o + (int)cnt;
                run_sum += cnt;
            }
            o = o < block_cnt ? o : block_cnt;
            end = end < block_cnt ? end : block_cnt;
            df11_decode_window<K>(table.data(), luts, n_luts, w[0], w[1], w[2], gap, stage.data(), o + phase,
                                  end + phase, &tbad);
            if (tbad) bad |= DF11_STATUS_BAD_TABLE;
        }

        const int64_t gbase = base - phase;
        const int n_groups = (phase + block_cnt + 7) >> 3;
        for (int g = 0; g < n_groups; ++g) {
            const int64_t G = gbase + 8 * (int64_t)g;
            const int lo = g == 0 ? phase : 0;
            int hi = phase + block_cnt - 8 * g;
            if (hi > 8) hi = 8;
            if (lo == 0 && hi == 8) {
                uint32_t ex[2], mm[2], r[4];
                memcpy(ex, stage.data() + 8 * g, 8);
                memcpy(mm, sm + G, 8);
                r[0] = df11_merge_pair(byte_perm(mm[0], ex[0], 0x5140));
                r[1] = df11_merge_pair(byte_perm(mm[0], ex[0], 0x7362));
                r[2] = df11_merge_pair(byte_perm(mm[1], ex[1], 0x5140));
                r[3] = df11_merge_pair(byte_perm(mm[1], ex[1], 0x7362));
                memcpy(out + G, r, 16);
            } else {
                for (int k = lo; k < hi; ++k) {
                    const uint32_t e = stage[8 * g + k], mv = sm[G + k];
                    out[G + k] = (uint16_t)(((mv & 0x80u) << 8) | (e << 7) | (mv & 0x7Fu));
                }
            }
        }
    }
    if (status) *status = bad;
    return 0;
}

}  // namespace

extern "C" int df11_emul_decode(const uint8_t *luts, int n_luts, const uint8_t *codes, int64_t n_bytes,
                                const uint8_t *sm, int64_t n_elements, const uint32_t *pos,
                                const uint8_t *gaps, uint16_t *out, int K, int prepared, int max_block_elems,
                                int *status)
{
    switch (K) {
    case 9: return run<9>(luts, n_luts, codes, n_bytes, sm, n_elements, pos, gaps, out, prepared, max_block_elems, status);
    case 10: return run<10>(luts, n_luts, codes, n_bytes, sm, n_elements, pos, gaps, out, prepared, max_block_elems, status);
    case 11: return run<11>(luts, n_luts, codes, n_bytes, sm, n_elements, pos, gaps, out, prepared, max_block_elems, status);
    case 12: return run<12>(luts, n_luts, codes, n_bytes, sm, n_elements, pos, gaps, out, prepared, max_block_elems, status);
    case 13: return run<13>(luts, n_luts, codes, n_bytes, sm, n_elements, pos, gaps, out, prepared, max_block_elems, status);
    case 14: return run<14>(luts, n_luts, codes, n_bytes, sm, n_elements, pos, gaps, out, prepared, max_block_elems, status);
    }
    return -1;
}

// Table statistics for a given K: fraction of escape entries and mean symbols per entry.
extern "C" int df11_emul_table(const uint8_t *luts, int n_luts, int K, uint32_t *meta_out, uint32_t *syms_out)
{
    uint8_t agree[256] = {0};
    for (int u = 1; u <= 8; ++u)
        for (int blk = 0; blk < (256 >> u); ++blk) agree[df11_agree_offset(u) + blk] = df11_agree_flag(luts, u, blk);
    for (uint32_t v = 0; v < (1u << K); ++v) {
        const Df11Entry e = df11_build_entry(luts, n_luts, agree, v, K);
        meta_out[v] = e.meta;
        syms_out[v] = e.syms;
    }
    return 0;
}
