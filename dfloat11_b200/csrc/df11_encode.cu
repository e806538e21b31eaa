// DF11 bit packer on the GPU: exponent bytes + code table -> `encoded_exponent`, `gaps`,
// `output_positions`, byte for byte what the reference's pure-Python `encode` produces for the
// same code table (dfloat11/dfloat11_utils.py:118-170) and what df11_encode_host produces
// (df11_host.cpp): codes appended MSB first, gaps[w] = bit offset of the first code starting in
// 8-byte window w, output_positions[b] = index of the first element whose code starts in
// 4096-byte block b, a last entry equal to the element count, and a final partial byte completed
// with the leading bits of a padding code.
//
// Three kernels.  count: bits per chunk of 4096 elements.  scan: one CTA turns the chunk sizes
// into chunk start bits and the total (the host reads the total to size the outputs).  pack: one
// CTA per chunk scans its 4096 code lengths, then every thread ORs its 16 codes into the zeroed
// stream (byte-swapped 32-bit atomics, so the stream is big-endian without a second pass) and
// records the gap / position entries of the codes that are first in their window / block.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/df11.h"
#include "df11_common.h"
#include "df11_error.h"

namespace {

constexpr int kEncThreads = 256;
constexpr int kEncPerThread = 16;
constexpr int kEncChunk = kEncThreads * kEncPerThread;  // elements per CTA

struct EncTables {
    uint8_t len[256];
    uint32_t val[256];
};

__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t v, uint32_t *warp_sums, uint32_t *total)
{
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    uint32_t incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const uint32_t n = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= (uint32_t)d) incl += n;
    }
    if (lane == 31u) warp_sums[warp] = incl;
    __syncthreads();
    uint32_t before = 0, all = 0;
    for (uint32_t k = 0; k < kEncThreads / 32; ++k) {
        const uint32_t s = warp_sums[k];
        if (k < warp) before += s;
        all += s;
    }
    if (total) *total = all;
    return before + incl - v;
}

// bits of every chunk; an exponent value that occurs but has no code sets the status word
__global__ void __launch_bounds__(kEncThreads) df11_enc_count_kernel(const uint8_t *ex, int64_t n, EncTables t,
                                                                     uint32_t *chunk_bits, int *status)
{
    __shared__ uint32_t warp_sums[kEncThreads / 32];
    const int64_t base = (int64_t)blockIdx.x * kEncChunk + (int64_t)threadIdx.x * kEncPerThread;
    uint32_t bits = 0;
    bool missing = false;
    for (int k = 0; k < kEncPerThread; ++k) {
        const int64_t i = base + k;
        if (i < n) {
            const uint32_t l = t.len[__ldg(ex + i)];
            missing |= l == 0u;
            bits += l;
        }
    }
    uint32_t total;
    block_exclusive_scan(bits, warp_sums, &total);
    if (threadIdx.x == 0) chunk_bits[blockIdx.x] = total;
    if (missing && status) atomicOr(status, DF11_STATUS_BAD_TABLE);
}

// one CTA: exclusive scan of the chunk sizes -> chunk start bits (64-bit) and the total
__global__ void __launch_bounds__(1024) df11_enc_scan_kernel(const uint32_t *chunk_bits, int64_t n_chunks,
                                                              unsigned long long *chunk_start,
                                                              unsigned long long *total_bits)
{
    __shared__ unsigned long long sums[1024];
    const int64_t per = (n_chunks + 1023) / 1024;
    const int64_t c0 = (int64_t)threadIdx.x * per, c1 = c0 + per < n_chunks ? c0 + per : n_chunks;
    unsigned long long mine = 0;
    for (int64_t c = c0; c < c1; ++c) mine += chunk_bits[c];
    sums[threadIdx.x] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long run = 0;
        for (int k = 0; k < 1024; ++k) {
            const unsigned long long s = sums[k];
            sums[k] = run;
            run += s;
        }
        *total_bits = run;
    }
    __syncthreads();
    unsigned long long run = sums[threadIdx.x];
    for (int64_t c = c0; c < c1; ++c) {
        chunk_start[c] = run;
        run += chunk_bits[c];
    }
}

// OR `value` into byte `index` of a zeroed, 4-byte aligned buffer
__device__ __forceinline__ void or_byte(uint8_t *buf, int64_t index, uint32_t value)
{
    atomicOr(reinterpret_cast<uint32_t *>(buf) + (index >> 2), value << (8 * (index & 3)));
}

// gaps[w] = g: a 5-bit field at bit 5w of the packed array, most significant bit first
__device__ __forceinline__ void set_gap(uint8_t *gaps, int64_t window, uint32_t g)
{
    uint64_t byte;
    uint32_t first, second;
    df11_gap_field((uint64_t)window, g, &byte, &first, &second);
    or_byte(gaps, (int64_t)byte, first);
    if (second) or_byte(gaps, (int64_t)byte + 1, second);
}

__global__ void __launch_bounds__(kEncThreads) df11_enc_pack_kernel(const uint8_t *ex, int64_t n, EncTables t,
                                                                    const unsigned long long *chunk_start,
                                                                    uint32_t pad_len, uint32_t pad_val, uint8_t *codes,
                                                                    int64_t n_bytes, uint8_t *gaps, uint32_t *pos,
                                                                    int64_t n_blocks)
{
    __shared__ uint32_t warp_sums[kEncThreads / 32];
    const int64_t first = (int64_t)blockIdx.x * kEncChunk + (int64_t)threadIdx.x * kEncPerThread;
    uint32_t sym[kEncPerThread];
    uint32_t bits = 0;
#pragma unroll
    for (int k = 0; k < kEncPerThread; ++k) {
        const int64_t i = first + k;
        sym[k] = i < n ? (uint32_t)__ldg(ex + i) : 256u;
        bits += sym[k] < 256u ? t.len[sym[k]] : 0u;
    }
    const uint32_t before = block_exclusive_scan(bits, warp_sums, nullptr);
    if (first >= n) return;
    int64_t bit = (int64_t)chunk_start[blockIdx.x] + before;
    // where the previous element's code starts (decides whether mine is first in its window / block)
    int64_t prev_start = first > 0 ? bit - t.len[__ldg(ex + first - 1)] : -1;
    uint32_t *words = reinterpret_cast<uint32_t *>(codes);
#pragma unroll
    for (int k = 0; k < kEncPerThread; ++k) {
        if (sym[k] >= 256u) break;
        const int64_t i = first + k;
        const uint32_t len = t.len[sym[k]];
        if (prev_start < 0 || (prev_start >> 6) != (bit >> 6)) {
            set_gap(gaps, bit >> 6, (uint32_t)(bit & 63));
            if (prev_start < 0 || (prev_start >> 15) != (bit >> 15)) pos[bit >> 15] = (uint32_t)i;
        }
        if (len > 0u) {
            // the code, MSB first, inside the 64 bits of big-endian words (bit >> 5) and the next one
            uint32_t hi, lo;
            df11_place_code((uint64_t)bit, len, t.val[sym[k]], &hi, &lo);
            const int64_t w = bit >> 5;
            atomicOr(words + w, df11_bswap32(hi));
            if (lo) atomicOr(words + w + 1, df11_bswap32(lo));
        }
        prev_start = bit;
        bit += len;
        if (i == n - 1) {
            // the incomplete last byte is completed with the leading bits of the padding code, which
            // also counts as a code starting there for the gap / position tables
            const uint32_t rem = (uint32_t)(bit & 7);
            if (rem) {
                if ((prev_start >> 6) != (bit >> 6)) set_gap(gaps, bit >> 6, (uint32_t)(bit & 63));
                if ((prev_start >> 15) != (bit >> 15)) pos[bit >> 15] = (uint32_t)n;
                or_byte(codes, n_bytes - 1, df11_pad_bits(rem, pad_len, pad_val));
            }
            pos[n_blocks] = (uint32_t)n;
        }
    }
}

int fill_tables(const void *code_len, const void *code_val, EncTables *t)
{
    if (!code_len || !code_val) return df11_fail(DF11_ERR_BADARG, "null code table");
    const uint8_t *l = (const uint8_t *)code_len;
    const uint32_t *v = (const uint32_t *)code_val;
    for (int s = 0; s < 256; ++s) {
        if (l[s] > DF11_MAX_CODE_LEN) return df11_fail(DF11_ERR_BADARG, "code of %d is %d bits", s, (int)l[s]);
        t->len[s] = l[s];
        t->val[s] = v[s];
    }
    return DF11_OK;
}

struct EncDeviceGuard {
    int prev = -1;
    bool ok = false;
    explicit EncDeviceGuard(int device)
    {
        ok = cudaGetDevice(&prev) == cudaSuccess && cudaSetDevice(device) == cudaSuccess;
    }
    ~EncDeviceGuard()
    {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

int64_t enc_chunks(int64_t n) { return (n + kEncChunk - 1) / kEncChunk; }

}  // namespace

extern "C" int64_t df11_encode_device_workspace_bytes(int64_t n_elements)
{
    if (n_elements < 0 || n_elements > 0xFFFFFFFFll) return df11_fail(DF11_ERR_BADARG, "element count out of range");
    const int64_t c = enc_chunks(n_elements) + 1;
    return c * 4 /* chunk sizes */ + ((c * 4 + 7) / 8) * 8 - c * 4 /* align */ + c * 8 /* chunk starts */ + 8 /* total */;
}

namespace {
struct EncWorkspace {
    uint32_t *chunk_bits;
    unsigned long long *chunk_start, *total;
};
EncWorkspace carve(void *workspace, int64_t n_elements)
{
    const int64_t c = enc_chunks(n_elements) + 1;
    EncWorkspace w;
    w.chunk_bits = (uint32_t *)workspace;
    w.chunk_start = (unsigned long long *)((uint8_t *)workspace + ((c * 4 + 7) / 8) * 8);
    w.total = w.chunk_start + c;
    return w;
}
}  // namespace

// Step 1: sizes.  Queues the count and scan kernels and copies the total number of stream bits
// to *total_bits_host (pinned or pageable host memory); the caller synchronises the stream
// before reading it.  `code_len` / `code_val` are HOST arrays of 256 entries.
extern "C" int df11_encode_device_count(const void *exponents, int64_t n_elements, const void *code_len,
                                        const void *code_val, void *workspace, int64_t workspace_bytes,
                                        void *total_bits_host, void *status, int32_t device, void *stream)
{
    if (!exponents || !workspace || !total_bits_host || n_elements <= 0 || n_elements > 0xFFFFFFFFll)
        return df11_fail(DF11_ERR_BADARG, "bad argument");
    if (workspace_bytes < df11_encode_device_workspace_bytes(n_elements) || ((uintptr_t)workspace & 7))
        return df11_fail(DF11_ERR_NOSPACE, "workspace must be 8-byte aligned and hold %lld bytes",
                         (long long)df11_encode_device_workspace_bytes(n_elements));
    EncTables t;
    int rc = fill_tables(code_len, code_val, &t);
    if (rc != DF11_OK) return rc;
    EncDeviceGuard guard(device);
    if (!guard.ok) return df11_fail(DF11_ERR_CUDA, "cudaSetDevice(%d) failed", device);
    const EncWorkspace w = carve(workspace, n_elements);
    const int64_t chunks = enc_chunks(n_elements);
    cudaStream_t s = (cudaStream_t)stream;
    df11_enc_count_kernel<<<(unsigned)chunks, kEncThreads, 0, s>>>((const uint8_t *)exponents, n_elements, t,
                                                                  w.chunk_bits, (int *)status);
    df11_enc_scan_kernel<<<1, 1024, 0, s>>>(w.chunk_bits, chunks, w.chunk_start, w.total);
    cudaError_t e = cudaMemcpyAsync(total_bits_host, w.total, 8, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return df11_fail(DF11_ERR_CUDA, "encoder launch failed: %s", cudaGetErrorString(e));
    return DF11_OK;
}

// Step 2: the stream and its tables, into caller-owned device buffers sized from step 1's total:
// `codes` 4-byte aligned with room for n_bytes rounded up to a multiple of 4; `gaps`
// 320 * n_blocks bytes, 4-byte aligned; `positions` n_blocks + 1 words.  The workspace must
// still hold what step 1 left there.
extern "C" int df11_encode_device_pack(const void *exponents, int64_t n_elements, const void *code_len,
                                       const void *code_val, int32_t pad_len, uint32_t pad_val, void *workspace,
                                       void *codes, int64_t n_bytes, void *gaps, int64_t n_gap_bytes,
                                       void *positions, int64_t n_positions, int32_t device, void *stream)
{
    if (!exponents || !workspace || !codes || !gaps || !positions || n_elements <= 0 || n_elements > 0xFFFFFFFFll)
        return df11_fail(DF11_ERR_BADARG, "bad argument");
    if (((uintptr_t)codes & 3) || ((uintptr_t)gaps & 3) || ((uintptr_t)positions & 3))
        return df11_fail(DF11_ERR_BADARG, "codes, gaps and positions must be 4-byte aligned");
    if (pad_len < 0 || pad_len > DF11_MAX_CODE_LEN) return df11_fail(DF11_ERR_BADARG, "bad padding code");
    const int64_t n_blocks = (n_bytes + DF11_BLOCK_BYTES - 1) / DF11_BLOCK_BYTES;
    if (n_bytes <= 0 || n_gap_bytes != n_blocks * DF11_GAP_BYTES_PER_BLOCK || n_positions != n_blocks + 1)
        return df11_fail(DF11_ERR_NOSPACE, "buffers must hold %lld gap bytes and %lld positions for %lld stream bytes",
                         (long long)(n_blocks * DF11_GAP_BYTES_PER_BLOCK), (long long)(n_blocks + 1),
                         (long long)n_bytes);
    EncTables t;
    int rc = fill_tables(code_len, code_val, &t);
    if (rc != DF11_OK) return rc;
    EncDeviceGuard guard(device);
    if (!guard.ok) return df11_fail(DF11_ERR_CUDA, "cudaSetDevice(%d) failed", device);
    const EncWorkspace w = carve(workspace, n_elements);
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(codes, 0, (size_t)((n_bytes + 3) / 4 * 4), s);
    if (e == cudaSuccess) e = cudaMemsetAsync(gaps, 0, (size_t)n_gap_bytes, s);
    if (e == cudaSuccess) e = cudaMemsetAsync(positions, 0, (size_t)n_positions * 4, s);
    if (e != cudaSuccess) return df11_fail(DF11_ERR_CUDA, "cudaMemsetAsync failed: %s", cudaGetErrorString(e));
    df11_enc_pack_kernel<<<(unsigned)enc_chunks(n_elements), kEncThreads, 0, s>>>(
        (const uint8_t *)exponents, n_elements, t, w.chunk_start, (uint32_t)pad_len, pad_val, (uint8_t *)codes,
        n_bytes, (uint8_t *)gaps, (uint32_t *)positions, n_blocks);
    e = cudaGetLastError();
    if (e != cudaSuccess) return df11_fail(DF11_ERR_CUDA, "encoder launch failed: %s", cudaGetErrorString(e));
    return DF11_OK;
}
