/*
 * CPU restatement of the DFloat11 decode rule.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker the CUDA path is compared against; nothing in the
 * shipped library links, loads or calls it.  It is also the timed "CPU
 * baseline" of the benchmark (the reference has no CPU decoder of its own:
 * dfloat11/dfloat11_utils.py only encodes).
 *
 * It restates, as straight scalar C, what one launch of the reference kernel
 * computes (reference file dfloat11/decode.cu):
 *   - 5-bit gap of a window, big-endian bit packing          decode.cu:85-87
 *   - the window's bytes consumed most-significant-bit first  decode.cu:91-100
 *   - hierarchical LUT walk: entry >= 240 points to row 256-entry,
 *     at most four levels; code length from the last row      decode.cu:105-118
 *   - a window owns exactly the codes that START in its 64 bits
 *                                                             decode.cu:104,129
 *   - element rebuild  hi=(sm&0x80)|(e>>1), lo=(e<<7)|(sm&0x7f) decode.cu:207-209
 *   - writes clamped to n_elements                            decode.cu:181,250
 * Bytes of the stream at or past n_bytes read as zero (the reference leaves
 * those registers unset, decode.cu:42-77; whatever they decode to is clamped
 * away).  Unlike the reference, a zero code length is reported as an error
 * instead of looping forever (decode.cu:116-118 shifts by zero), and all
 * sizes are 64-bit.
 *
 * Parity status: pinned against tensors produced by the reference's own
 * encoder (dfloat11_utils.py, imported unmodified) -- see tests/golden/.
 * The reference ships no golden vectors of its own.
 */
#include <stdint.h>
#include <stddef.h>
#include <string.h>
#include <pthread.h>
#include <unistd.h>

#define DF11_WINDOW_BYTES 8      /* bytes_per_thread, dfloat11.py:45 */
#define DF11_WINDOWS_PER_BLOCK 512 /* threads_per_block, dfloat11.py:46 */
#define DF11_BLOCK_BYTES (DF11_WINDOW_BYTES * DF11_WINDOWS_PER_BLOCK)

static inline uint32_t stream_byte(const uint8_t *codes, int64_t n_bytes, int64_t i)
{
    return i < n_bytes ? codes[i] : 0u;
}

/* 32 bits of the stream starting at absolute bit position `bit`, MSB first. */
static inline uint32_t peek32(const uint8_t *codes, int64_t n_bytes, int64_t bit)
{
    int64_t byte = bit >> 3;
    int sh = (int)(bit & 7);
    uint64_t v = 0;
    if (byte + 8 <= n_bytes) { /* fast path: one unaligned 8-byte read, byte-swapped */
        memcpy(&v, codes + byte, 8);
        v = __builtin_bswap64(v);
        return (uint32_t)((v << sh) >> 32);
    }
    for (int k = 0; k < 5; ++k)
        v = (v << 8) | stream_byte(codes, n_bytes, byte + k);
    return (uint32_t)((v >> (8 - sh)) & 0xffffffffu);
}

static inline int window_gap(const uint8_t *gaps, int64_t n_gap_bytes, int64_t t)
{
    int64_t bitpos = 5 * t;
    int64_t j = bitpos >> 3;
    int r = (int)(bitpos & 7);
    uint32_t hi = j < n_gap_bytes ? gaps[j] : 0u;
    /* the second byte only carries gap bits when r > 3; never read past the end */
    uint32_t lo = (r > 3 && j + 1 < n_gap_bytes) ? gaps[j + 1] : 0u;
    return (int)((((hi << 8) | lo) >> (11 - r)) & 31u);
}

/* Decodes format block b.  Returns 0, -1 (zero code length met), or -2 (block
 * did not end on output_positions[b+1] while `strict`). */
static int decode_block(const uint8_t *luts, int n_luts,
                        const uint8_t *codes, int64_t n_bytes,
                        const uint8_t *sm, int64_t n_elements,
                        const uint32_t *pos, const uint8_t *gaps, int64_t n_gap_bytes,
                        uint16_t *out, int64_t b, int64_t n_blocks, int strict)
{
    const uint8_t *lens = luts + 256 * (size_t)(n_luts - 1);
    int64_t o = pos[b];
    for (int64_t t = b * DF11_WINDOWS_PER_BLOCK;
         t < (b + 1) * DF11_WINDOWS_PER_BLOCK && t * DF11_WINDOW_BYTES < n_bytes; ++t) {
        int64_t base = t * 64;
        int p = window_gap(gaps, n_gap_bytes, t);
        while (p < 64) {
            uint32_t x = peek32(codes, n_bytes, base + p);
            uint32_t e = luts[x >> 24];
            if (e >= 240) {
                e = luts[256 * (256 - e) + ((x >> 16) & 255)];
                if (e >= 240) {
                    e = luts[256 * (256 - e) + ((x >> 8) & 255)];
                    if (e >= 240)
                        e = luts[256 * (256 - e) + (x & 255)];
                }
            }
            if (o < n_elements) {
                uint32_t m = sm[o];
                out[o] = (uint16_t)(((m & 0x80u) << 8) | (e << 7) | (m & 0x7fu));
            }
            ++o;
            int len = lens[e];
            if (len == 0)
                return -1;
            p += len;
        }
    }
    if (strict && b + 1 < n_blocks && o != (int64_t)pos[b + 1])
        return -2;
    return 0;
}

struct span_job {
    const uint8_t *luts; int n_luts;
    const uint8_t *codes; int64_t n_bytes;
    const uint8_t *sm; int64_t n_elements;
    const uint32_t *pos; const uint8_t *gaps; int64_t n_gap_bytes;
    uint16_t *out; int64_t b0, b1, n_blocks; int strict; int status;
};

static void *span_main(void *arg)
{
    struct span_job *j = (struct span_job *)arg;
    for (int64_t b = j->b0; b < j->b1; ++b) {
        int rc = decode_block(j->luts, j->n_luts, j->codes, j->n_bytes, j->sm, j->n_elements,
                              j->pos, j->gaps, j->n_gap_bytes, j->out, b, j->n_blocks, j->strict);
        if (rc != 0) {
            j->status = rc;
            break;
        }
    }
    return NULL;
}

/*
 * Whole-unit decode.  All pointers are host pointers.
 *   luts              [n_luts*256]   rows 0..n_luts-2 decode tables, last row code lengths
 *   codes             [n_bytes]      Huffman bitstream
 *   sign_mantissa     [n_elements]
 *   output_positions  [n_blocks+1]   n_blocks = ceil(n_bytes / 4096)
 *   gaps              [n_gap_bytes]  5 bits per window
 *   out               [n_elements]   BF16 bit patterns
 *   n_threads         <=1: serial; >1: contiguous runs of format blocks on that many threads
 *   strict            non-zero: also verify every block ends on the next output position
 * Returns 0 on success, a negative code otherwise.
 */
int df11_oracle_decode(const uint8_t *luts, int n_luts,
                       const uint8_t *codes, int64_t n_bytes,
                       const uint8_t *sign_mantissa, int64_t n_elements,
                       const uint32_t *output_positions,
                       const uint8_t *gaps, int64_t n_gap_bytes,
                       uint16_t *out, int n_threads, int strict)
{
    if (n_luts < 2 || n_bytes < 0 || n_elements < 0)
        return -3;
    int64_t n_blocks = (n_bytes + DF11_BLOCK_BYTES - 1) / DF11_BLOCK_BYTES;
    if (n_threads < 1)
        n_threads = 1;
    if (n_threads > 256)
        n_threads = 256;
    if ((int64_t)n_threads > n_blocks)
        n_threads = n_blocks > 0 ? (int)n_blocks : 1;
    struct span_job jobs[256];
    pthread_t tids[256];
    int64_t per = (n_blocks + n_threads - 1) / n_threads;
    for (int i = 0; i < n_threads; ++i) {
        struct span_job j = {luts, n_luts, codes, n_bytes, sign_mantissa, n_elements,
                             output_positions, gaps, n_gap_bytes, out,
                             i * per, (i + 1) * per < n_blocks ? (i + 1) * per : n_blocks,
                             n_blocks, strict, 0};
        jobs[i] = j;
    }
    if (n_threads == 1) {
        span_main(&jobs[0]);
        return jobs[0].status;
    }
    int started = 0;
    for (int i = 0; i < n_threads; ++i) {
        if (pthread_create(&tids[i], NULL, span_main, &jobs[i]) != 0)
            break;
        ++started;
    }
    for (int i = started; i < n_threads; ++i)
        span_main(&jobs[i]); /* could not start a thread: run its share here */
    int status = 0;
    for (int i = 0; i < started; ++i)
        pthread_join(tids[i], NULL);
    for (int i = 0; i < n_threads; ++i)
        if (jobs[i].status != 0)
            status = jobs[i].status;
    return status;
}

/* Number of host cores the process may use. */
int df11_oracle_max_threads(void)
{
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}
