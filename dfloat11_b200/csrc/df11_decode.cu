// DF11 -> BF16 decompression kernels for B200 (sm_100a) and their C entry points.
//
// What one launch computes is fixed by the reference kernel dfloat11/decode.cu:25-253
// (see df11_common.h for the format); how it is computed is not taken from it:
//
//   * persistent CTAs: grid = SMs x resident CTAs, each CTA walks format blocks
//     b, b + grid, ... and builds its lookup tables in shared memory once;
//   * a 2^K-entry multi-symbol table (up to four exponents per probe, derived from
//     `luts`) replaces the reference's 2-5 dependent global loads per symbol;
//   * a window (8 stream bytes + 4 look-ahead) lives in three registers, loaded
//     with one 8-byte and one 4-byte coalesced load;
//   * output slots come from a warp-shuffle scan (2 barriers per block, not 18),
//     or -- in the prepared form -- from per-window offsets computed once per unit;
//   * decoded exponents are staged as bytes in shared memory and merged with the
//     sign/mantissa bytes eight elements at a time: one 8-byte load, one 16-byte
//     fully coalesced store per thread;
//   * every loop is bounded and every index is clamped: inconsistent tensors set a
//     status bit instead of hanging (decode.cu:116-118 can spin forever).
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "../../include/df11.h"
#include "df11_common.h"
#include "df11_error.h"

namespace {

constexpr int kThreads = 512;  // one window per thread, one format block per CTA pass
constexpr int kWarps = kThreads / 32;
constexpr int kTableBits = 11;  // K: index width of the multi-symbol table

enum Mode { kTwoPass = 0, kCount = 1, kPrepared = 2 };

struct Params {
    const uint8_t *luts;
    const uint8_t *codes;
    const uint8_t *sm;
    const uint32_t *pos;
    const uint8_t *gaps;
    uint16_t *out;
    const Df11Entry *table_g;  // prebuilt table in global memory, or null: build it here
    uint16_t *woff;            // per-window element offset inside its format block
    int *status;
    int64_t n_bytes;
    int64_t n_elements;
    int64_t n_blocks;
    int64_t n_gap_bytes;
    int n_luts;
    int stage_cap;  // elements the shared staging area can hold (including phase)
    int codes_aligned;
    int io_aligned;
};

__device__ __forceinline__ void load_window(const Params &p, int64_t t, uint32_t &w0, uint32_t &w1,
                                            uint32_t &w2)
{
    const int64_t off = t * DF11_WINDOW_BYTES;
    if (p.codes_aligned && off + 12 <= p.n_bytes) {
        const uint2 v = __ldg(reinterpret_cast<const uint2 *>(p.codes + off));
        const uint32_t x = __ldg(reinterpret_cast<const uint32_t *>(p.codes + off + 8));
        w0 = __byte_perm(v.x, 0, 0x0123);
        w1 = __byte_perm(v.y, 0, 0x0123);
        w2 = __byte_perm(x, 0, 0x0123);
    } else {
        uint32_t w[3] = {0, 0, 0};
#pragma unroll
        for (int k = 0; k < 12; ++k) {
            const int64_t i = off + k;
            const uint32_t byte = i < p.n_bytes ? (uint32_t)__ldg(p.codes + i) : 0u;
            w[k >> 2] |= byte << (24 - 8 * (k & 3));
        }
        w0 = w[0], w1 = w[1], w2 = w[2];
    }
}

__device__ __forceinline__ uint16_t merge_one(uint32_t e, uint32_t m)
{
    return (uint16_t)(((m & 0x80u) << 8) | (e << 7) | (m & 0x7Fu));
}

template <int K, int MODE>
__global__ void __launch_bounds__(kThreads, 4) df11_kernel(const Params p)
{
    extern __shared__ __align__(16) uint8_t smem[];
    Df11Entry *table = reinterpret_cast<Df11Entry *>(smem);
    uint8_t *luts_s = smem + (sizeof(Df11Entry) << K);
    uint8_t *agree = luts_s + p.n_luts * 256;
    uint32_t *wsum = reinterpret_cast<uint32_t *>(agree + 256);
    uint8_t *stage = reinterpret_cast<uint8_t *>(wsum + 32);

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    int bad = 0;

    // ---- once per CTA: tables into shared memory -------------------------------------
    for (int i = tid; i < p.n_luts * 256; i += kThreads) luts_s[i] = __ldg(p.luts + i);
    __syncthreads();
    if (p.table_g != nullptr) {
        const uint4 *src = reinterpret_cast<const uint4 *>(p.table_g);
        uint4 *dst = reinterpret_cast<uint4 *>(table);
        for (int i = tid; i < (1 << K) / 2; i += kThreads) dst[i] = __ldg(src + i);
    } else {
        for (int task = tid; task < 255; task += kThreads) {
            int u = 1;
            while (task >= df11_agree_offset(u + 1) && u < 8) ++u;
            agree[task] = df11_agree_flag(luts_s, u, task - df11_agree_offset(u));
        }
        __syncthreads();
        for (int v = tid; v < (1 << K); v += kThreads)
            table[v] = df11_build_entry(luts_s, p.n_luts, agree, (uint32_t)v, K);
    }
    __syncthreads();

    // ---- format blocks -----------------------------------------------------------------
    for (int64_t b = blockIdx.x; b < p.n_blocks; b += gridDim.x) {
        const int64_t t = b * DF11_WINDOWS_PER_BLOCK + tid;  // my window
        const bool live = t * DF11_WINDOW_BYTES < p.n_bytes;

        int64_t base = 0;
        int block_cnt = 0, phase = 0;
        if (MODE != kCount) {
            base = (int64_t)p.pos[b];
            const int64_t next = (int64_t)p.pos[b + 1];
            int64_t c = next - base;
            if (c < 0 || next > p.n_elements) {
                bad |= DF11_STATUS_BAD_POSITIONS;
                c = c < 0 ? 0 : p.n_elements - base;
                if (c < 0) c = 0;
            }
            phase = (int)(base & 7);
            if (c + phase > p.stage_cap) {
                bad |= DF11_STATUS_TRUNCATED;
                c = p.stage_cap - phase;
            }
            block_cnt = (int)c;
        }

        uint32_t w0 = 0, w1 = 0, w2 = 0, gap = 0;
        if (live) {
            load_window(p, t, w0, w1, w2);
            gap = df11_gap(p.gaps, p.n_gap_bytes, t);
        }

        int o = 0, end = 0;
        if (MODE == kPrepared) {
            if (live) {
                o = (int)p.woff[t];
                const bool last = tid == DF11_WINDOWS_PER_BLOCK - 1 ||
                                  (t + 1) * DF11_WINDOW_BYTES >= p.n_bytes;
                end = last ? block_cnt : (int)p.woff[t + 1];
            }
        } else {
            int tbad = 0;
            const uint32_t cnt =
                live ? df11_count_window<K>(table, luts_s, p.n_luts, w0, w1, w2, gap, &tbad) : 0u;
            if (tbad) bad |= DF11_STATUS_BAD_TABLE;
            // block-wide exclusive scan: shuffles inside a warp, one hop through shared memory
            uint32_t incl = cnt;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const uint32_t n = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl += n;
            }
            if (lane == 31) wsum[warp] = incl;
            __syncthreads();
            uint32_t ws = lane < kWarps ? wsum[lane] : 0u;
#pragma unroll
            for (int d = 1; d < kWarps; d <<= 1) {
                const uint32_t n = __shfl_up_sync(0xffffffffu, ws, d);
                if (lane >= d) ws += n;
            }
            const uint32_t before = __shfl_sync(0xffffffffu, ws, warp > 0 ? warp - 1 : 0);
            o = (int)((warp > 0 ? before : 0u) + incl - cnt);
            end = o + (int)cnt;
            if (MODE == kCount) {
                if (live) p.woff[t] = (uint16_t)(o > 65535 ? 65535 : o);
                __syncthreads();  // wsum is reused by the next block
                continue;
            }
        }

        // clamp to what this block may write, then shift by the block's alignment phase
        o = o < block_cnt ? o : block_cnt;
        end = end < block_cnt ? end : block_cnt;
        {
            int tbad = 0;
            df11_decode_window<K>(table, luts_s, p.n_luts, w0, w1, w2, gap, stage, o + phase,
                                  end + phase, &tbad);
            if (tbad) bad |= DF11_STATUS_BAD_TABLE;
        }
        __syncthreads();

        // ---- merge with sign/mantissa, eight elements per thread step ------------------
        const int64_t gbase = base - phase;  // multiple of 8
        const int n_groups = (phase + block_cnt + 7) >> 3;
        for (int g = tid; g < n_groups; g += kThreads) {
            const int64_t G = gbase + 8 * (int64_t)g;
            const int lo = g == 0 ? phase : 0;
            const int hi = min(phase + block_cnt - 8 * g, 8);
            if (lo == 0 && hi == 8 && p.io_aligned) {
                const uint2 ex = *reinterpret_cast<const uint2 *>(stage + 8 * g);
                const uint2 m = __ldg(reinterpret_cast<const uint2 *>(p.sm + G));
                uint4 r;
                r.x = df11_merge_pair(__byte_perm(m.x, ex.x, 0x5140));
                r.y = df11_merge_pair(__byte_perm(m.x, ex.x, 0x7362));
                r.z = df11_merge_pair(__byte_perm(m.y, ex.y, 0x5140));
                r.w = df11_merge_pair(__byte_perm(m.y, ex.y, 0x7362));
                *reinterpret_cast<uint4 *>(p.out + G) = r;
            } else {
                for (int k = lo; k < hi; ++k)
                    p.out[G + k] = merge_one(stage[8 * g + k], __ldg(p.sm + G + k));
            }
        }
        __syncthreads();  // staging and wsum are reused by the next block
    }

    if (bad && p.status != nullptr) atomicOr(p.status, bad);
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------

struct DeviceInfo {
    bool ready = false;
    int sm_count = 0;
    int max_smem_optin = 0;
};
std::mutex g_mutex;
DeviceInfo g_devices[64];
bool g_attr_set[64][3] = {};

struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int device)
    {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != device && cudaSetDevice(device) != cudaSuccess) ok = false;
    }
    ~DeviceGuard()
    {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

int device_info(int device, DeviceInfo *out)
{
    if (device < 0 || device >= 64) return df11_fail(DF11_ERR_BADARG, "device index %d out of range", device);
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceInfo &d = g_devices[device];
    if (!d.ready) {
        cudaError_t e = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, device);
        if (e == cudaSuccess)
            e = cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
        if (e != cudaSuccess) return df11_fail(DF11_ERR_CUDA, "device query failed: %s", cudaGetErrorString(e));
        d.ready = true;
    }
    *out = d;
    return DF11_OK;
}

size_t smem_bytes(int n_luts, int stage_bytes)
{
    return (sizeof(Df11Entry) << kTableBits) + (size_t)n_luts * 256 + 256 + 32 * 4 + (size_t)stage_bytes;
}

template <int MODE>
int launch(Params p, int stage_bytes, int device, cudaStream_t stream)
{
    DeviceInfo info;
    int rc = device_info(device, &info);
    if (rc != DF11_OK) return rc;
    DeviceGuard guard(device);
    if (!guard.ok) return df11_fail(DF11_ERR_CUDA, "cudaSetDevice(%d) failed", device);

    const size_t smem = smem_bytes(p.n_luts, stage_bytes);
    if (smem > (size_t)info.max_smem_optin)
        return df11_fail(DF11_ERR_BADARG, "needs %zu bytes of shared memory, device allows %d", smem,
                         info.max_smem_optin);
    auto kernel = df11_kernel<kTableBits, MODE>;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (!g_attr_set[device][MODE]) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 info.max_smem_optin);
            if (e != cudaSuccess)
                return df11_fail(DF11_ERR_CUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
            g_attr_set[device][MODE] = true;
        }
    }
    int per_sm = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, smem);
    if (e != cudaSuccess || per_sm < 1)
        return df11_fail(DF11_ERR_CUDA, "occupancy query failed (%s, %d CTAs/SM)", cudaGetErrorString(e), per_sm);
    int64_t grid = (int64_t)info.sm_count * per_sm;
    if (grid > p.n_blocks) grid = p.n_blocks;
    kernel<<<(unsigned)grid, kThreads, smem, stream>>>(p);
    e = cudaGetLastError();
    if (e != cudaSuccess) return df11_fail(DF11_ERR_CUDA, "kernel launch failed: %s", cudaGetErrorString(e));
    return DF11_OK;
}

int check_common(const void *luts, const void *codes, const void *pos, const void *gaps, int32_t n_luts,
                 int64_t n_bytes, int64_t n_elements)
{
    if (!luts || !codes || !pos || !gaps) return df11_fail(DF11_ERR_BADARG, "null tensor pointer");
    if (n_luts < 2 || n_luts > DF11_MAX_LUTS)
        return df11_fail(DF11_ERR_BADARG, "n_luts = %d, supported range is 2..%d", n_luts, DF11_MAX_LUTS);
    if (n_bytes < 0 || n_elements < 0) return df11_fail(DF11_ERR_BADARG, "negative size");
    if (n_elements > 0xFFFFFFFFll)
        return df11_fail(DF11_ERR_BADARG, "n_elements = %lld does not fit the format's 32-bit output positions",
                         (long long)n_elements);
    return DF11_OK;
}

int stage_bytes_for(int32_t max_block_elems, int *cap)
{
    int64_t m = max_block_elems > 0 ? max_block_elems : DF11_MAX_BLOCK_ELEMS;
    if (m > DF11_MAX_BLOCK_ELEMS) m = DF11_MAX_BLOCK_ELEMS;
    const int bytes = (int)((m + 7 + 15) / 16 * 16) + 16;  // phase (<= 7) + elements, padded
    *cap = bytes - 8;
    return bytes;
}

constexpr int64_t kAuxTableBytes = (int64_t)sizeof(Df11Entry) << kTableBits;

__global__ void df11_table_kernel(const uint8_t *luts, int n_luts, Df11Entry *table)
{
    __shared__ uint8_t luts_s[DF11_MAX_LUTS * 256];
    __shared__ uint8_t agree[256];
    for (int i = threadIdx.x; i < n_luts * 256; i += blockDim.x) luts_s[i] = luts[i];
    __syncthreads();
    for (int task = threadIdx.x; task < 255; task += blockDim.x) {
        int u = 1;
        while (task >= df11_agree_offset(u + 1) && u < 8) ++u;
        agree[task] = df11_agree_flag(luts_s, u, task - df11_agree_offset(u));
    }
    __syncthreads();
    for (int v = threadIdx.x; v < (1 << kTableBits); v += blockDim.x)
        table[v] = df11_build_entry(luts_s, n_luts, agree, (uint32_t)v, kTableBits);
}

}  // namespace

extern "C" int df11_decode(const void *luts, const void *codes, const void *sign_mantissa,
                           const void *output_positions, const void *gaps, void *out_bf16, int32_t n_luts,
                           int64_t n_bytes, int64_t n_elements, int32_t max_block_elems, void *status,
                           int32_t device, void *stream)
{
    int rc = check_common(luts, codes, output_positions, gaps, n_luts, n_bytes, n_elements);
    if (rc != DF11_OK) return rc;
    if (n_bytes == 0 || n_elements == 0) return DF11_OK;
    if (!sign_mantissa || !out_bf16) return df11_fail(DF11_ERR_BADARG, "null tensor pointer");
    Params p = {};
    p.luts = (const uint8_t *)luts;
    p.codes = (const uint8_t *)codes;
    p.sm = (const uint8_t *)sign_mantissa;
    p.pos = (const uint32_t *)output_positions;
    p.gaps = (const uint8_t *)gaps;
    p.out = (uint16_t *)out_bf16;
    p.status = (int *)status;
    p.n_bytes = n_bytes;
    p.n_elements = n_elements;
    p.n_blocks = (n_bytes + DF11_BLOCK_BYTES - 1) / DF11_BLOCK_BYTES;
    p.n_gap_bytes = p.n_blocks * DF11_GAP_BYTES_PER_BLOCK;
    p.n_luts = n_luts;
    const int stage_bytes = stage_bytes_for(max_block_elems, &p.stage_cap);
    p.codes_aligned = ((uintptr_t)codes & 7) == 0;
    p.io_aligned = ((uintptr_t)sign_mantissa & 7) == 0 && ((uintptr_t)out_bf16 & 15) == 0;
    return launch<kTwoPass>(p, stage_bytes, device, (cudaStream_t)stream);
}

extern "C" int64_t df11_aux_bytes(int64_t n_bytes)
{
    if (n_bytes < 0) return df11_fail(DF11_ERR_BADARG, "negative size");
    const int64_t n_blocks = (n_bytes + DF11_BLOCK_BYTES - 1) / DF11_BLOCK_BYTES;
    // table, then one uint16 per window (+1 so that woff[t + 1] is always readable), padded
    return kAuxTableBytes + ((n_blocks * DF11_WINDOWS_PER_BLOCK + 1) * 2 + 15) / 16 * 16;
}

extern "C" int df11_prepare(const void *luts, const void *codes, const void *output_positions,
                            const void *gaps, void *aux, int64_t aux_bytes, int32_t n_luts, int64_t n_bytes,
                            int64_t n_elements, void *status, int32_t device, void *stream)
{
    int rc = check_common(luts, codes, output_positions, gaps, n_luts, n_bytes, n_elements);
    if (rc != DF11_OK) return rc;
    if (!aux || ((uintptr_t)aux & 15)) return df11_fail(DF11_ERR_BADARG, "aux buffer is null or not 16-byte aligned");
    if (aux_bytes < df11_aux_bytes(n_bytes))
        return df11_fail(DF11_ERR_NOSPACE, "aux buffer holds %lld bytes, %lld needed", (long long)aux_bytes,
                         (long long)df11_aux_bytes(n_bytes));
    {
        DeviceGuard guard(device);
        if (!guard.ok) return df11_fail(DF11_ERR_CUDA, "cudaSetDevice(%d) failed", device);
        df11_table_kernel<<<1, 512, 0, (cudaStream_t)stream>>>((const uint8_t *)luts, n_luts, (Df11Entry *)aux);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return df11_fail(DF11_ERR_CUDA, "kernel launch failed: %s", cudaGetErrorString(e));
    }
    if (n_bytes == 0) return DF11_OK;
    Params p = {};
    p.luts = (const uint8_t *)luts;
    p.codes = (const uint8_t *)codes;
    p.pos = (const uint32_t *)output_positions;
    p.gaps = (const uint8_t *)gaps;
    p.table_g = (const Df11Entry *)aux;  // written by the launch above, same stream
    p.woff = (uint16_t *)((uint8_t *)aux + kAuxTableBytes);
    p.status = (int *)status;
    p.n_bytes = n_bytes;
    p.n_elements = n_elements;
    p.n_blocks = (n_bytes + DF11_BLOCK_BYTES - 1) / DF11_BLOCK_BYTES;
    p.n_gap_bytes = p.n_blocks * DF11_GAP_BYTES_PER_BLOCK;
    p.n_luts = n_luts;
    p.stage_cap = 0;
    p.codes_aligned = ((uintptr_t)codes & 7) == 0;
    return launch<kCount>(p, 16, device, (cudaStream_t)stream);
}

extern "C" int df11_decode_prepared(const void *luts, const void *codes, const void *sign_mantissa,
                                    const void *output_positions, const void *gaps, const void *aux,
                                    void *out_bf16, int32_t n_luts, int64_t n_bytes, int64_t n_elements,
                                    int32_t max_block_elems, void *status, int32_t device, void *stream)
{
    int rc = check_common(luts, codes, output_positions, gaps, n_luts, n_bytes, n_elements);
    if (rc != DF11_OK) return rc;
    if (n_bytes == 0 || n_elements == 0) return DF11_OK;
    if (!sign_mantissa || !out_bf16 || !aux || ((uintptr_t)aux & 15))
        return df11_fail(DF11_ERR_BADARG, "null tensor pointer or misaligned aux buffer");
    Params p = {};
    p.luts = (const uint8_t *)luts;
    p.codes = (const uint8_t *)codes;
    p.sm = (const uint8_t *)sign_mantissa;
    p.pos = (const uint32_t *)output_positions;
    p.gaps = (const uint8_t *)gaps;
    p.out = (uint16_t *)out_bf16;
    p.table_g = (const Df11Entry *)aux;
    p.woff = (uint16_t *)((uint8_t *)aux + kAuxTableBytes);
    p.status = (int *)status;
    p.n_bytes = n_bytes;
    p.n_elements = n_elements;
    p.n_blocks = (n_bytes + DF11_BLOCK_BYTES - 1) / DF11_BLOCK_BYTES;
    p.n_gap_bytes = p.n_blocks * DF11_GAP_BYTES_PER_BLOCK;
    p.n_luts = n_luts;
    const int stage_bytes = stage_bytes_for(max_block_elems, &p.stage_cap);
    p.codes_aligned = ((uintptr_t)codes & 7) == 0;
    p.io_aligned = ((uintptr_t)sign_mantissa & 7) == 0 && ((uintptr_t)out_bf16 & 15) == 0;
    return launch<kPrepared>(p, stage_bytes, device, (cudaStream_t)stream);
}
