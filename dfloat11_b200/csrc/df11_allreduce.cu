// One-shot all-reduce of a small BF16 activation tensor over NVLink peer memory, for the
// partitioned (tensor-parallel) mode: after every row-parallel layer the ranks' partial outputs
// ([batch, hidden] BF16: 32 KB at batch 1 for hidden 16384) are summed.  At that size a
// collective is pure latency; this kernel does it in one launch with plain peer loads and
// stores -- no library call, no multicast object, no TMA:
//
//   1. every rank copies its slice into its own buffer in symmetric memory (local stores),
//   2. tells every peer so (one flag per rank, CTA and call parity, written into the PEER's flag
//      area with a system-scope release store),
//   3. waits until all ranks' flags for this call have arrived in its own flag area (bounded),
//   4. reads every rank's slice (peer loads over NVLink), adds them in rank order in fp32 and
//      rounds once to BF16: the same bits on every rank, run to run.
//
// The call number lives in device memory and is advanced by the kernel itself, so a launch
// recorded in a CUDA graph can be replayed.  Buffers alternate between two halves by call
// parity: a rank can only be one call ahead of a peer (it needs the peer's flag of call s to
// finish call s), so the half written in call s + 2 is no longer being read.
//
// Tensors of up to 64 KB on 1, 2, 4 or 8 ranks take a second, faster form with no flags and no
// fences, and no barrier before the result is written (`df11_allreduce_ll_kernel`): every rank PUSHES its slice into every rank's
// buffer as 8-byte pairs {4 bytes of data, call tag}; an 8-byte store arrives whole, so a pair
// whose tag is this call's tag is this call's data.  A thread writes the pairs of its own 16
// bytes to all ranks, polls the pairs of all ranks for the same 16 bytes in its own buffer
// (bounded), sums them in rank order and writes the result: one NVLink crossing instead of
// fence + flag round trip + data round trip.  (The same idea as the low-latency protocol of
// collective libraries; written here from its published description.)
// The reference has no counterpart: its only multi-GPU form places whole layers on different
// devices (dfloat11/dfloat11.py:455-460).
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/df11.h"
#include "df11_error.h"

namespace {

constexpr int kMaxRanks = 8;
constexpr int kMaxCtas = 32;
constexpr int kThreads = 512;
constexpr uint64_t kWaitNs = 2000ull * 1000 * 1000;  // a peer that has not shown up after two seconds is not coming
// A wait ends when its time is up; and, whatever the clock says, after a number of polls that
// grows with that time (a poll takes some hundred nanoseconds at the very least).  Once a call has
// given up (DF11_STATUS_TIMEOUT in the caller's status word), the calls after it do not wait
// again: a forward pass with hundreds of all-reduces then ends at once, with the status set,
// instead of waiting that time hundreds of times.
__device__ __forceinline__ uint64_t poll_limit(uint64_t wait_ns, const int *status)
{
    if (status != nullptr && (*reinterpret_cast<const volatile int *>(status) & DF11_STATUS_TIMEOUT)) return 1;
    return wait_ns / 128u + 4096u;
}
constexpr size_t kFlagBytes = (size_t)2 * kMaxCtas * kMaxRanks * sizeof(uint32_t);
// pushed form: after the flags, two halves (call parity) of [rank][vector] cells of 32 bytes
// (16 bytes of data as four {data, tag} pairs)
constexpr int kLlThreads = 128;
constexpr uint32_t kLlSlotVecs = 4096;                                   // 64 KB of data per rank and call
constexpr size_t kLlHalfBytes = (size_t)kMaxRanks * kLlSlotVecs * 32;    // 1 MiB
// counters of one rank: [0] call number of the flag form, [1] its CTAs done, [2 + c] the number of
// pushed calls CTA c has taken part in (a cell is only ever touched by the CTA with its number,
// so each CTA can keep its own count: no atomic, no fence at the end of the kernel)
constexpr int kLlCtas = kLlSlotVecs / kLlThreads;
constexpr int kCounterWords = 64;
static_assert(2 + kLlCtas <= kCounterWords, "counter block too small");

struct Peers {
    uint8_t *data[kMaxRanks];    // each rank's buffer: two halves of slot_bytes
    uint32_t *flags[kMaxRanks];  // each rank's flag area: [2][kMaxCtas][kMaxRanks]
};

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_volatile16(const void *p)
{
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void st_volatile16(void *p, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint64_t global_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ uint32_t bf16x2_from_floats(float lo, float hi)  // round to nearest even; NaN stays NaN
{
    auto one = [](float f) -> uint32_t {
        uint32_t u = __float_as_uint(f);
        if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (u >> 16) | 0x40u;
        u += 0x7FFFu + ((u >> 16) & 1u);
        return u >> 16;
    };
    return one(lo) | (one(hi) << 16);
}

// WORLD > 0: the number of ranks is known at compile time, the loads of all ranks' vectors are
// issued together (one NVLink round trip instead of one per rank); WORLD = 0: any number up to 8.
// `cta` of `n_ctas`: this CTA's place among the CTAs that work for `rank` (the whole grid in the
// real launch; one row of the grid when one launch plays all ranks, see the self-test below).
template <int WORLD>
__device__ __forceinline__ void flag_form(const Peers &peers, uint32_t *counters, int rank, int world_arg,
                                          const uint4 *in, uint4 *out, uint32_t n_vec, uint32_t vec_per_cta,
                                          uint32_t slot_bytes, uint64_t wait_ns, int *status, uint32_t cta,
                                          uint32_t n_ctas)
{
    const int world = WORLD > 0 ? WORLD : world_arg;
    const uint32_t tid = threadIdx.x;
    const uint32_t call = *reinterpret_cast<volatile uint32_t *>(counters);  // advanced by the last CTA to finish
    const uint32_t tag = call + 1u != 0u ? call + 1u : 1u;  // never 0: the flag areas start zeroed
    const uint64_t polls = poll_limit(wait_ns, status);     // read early: its latency hides behind the copy below
    const uint32_t half = call & 1u;
    const uint32_t v0 = cta * vec_per_cta, v1 = min(n_vec, v0 + vec_per_cta);
    const uint32_t flag_index = (half * kMaxCtas + cta) * kMaxRanks;

    // 1. my slice into my own half
    uint4 *mine = reinterpret_cast<uint4 *>(peers.data[rank] + (size_t)half * slot_bytes);
    for (uint32_t v = v0 + tid; v < v1; v += kThreads) mine[v] = in[v];
    __threadfence_system();
    __syncthreads();
    // 2. tell every rank (myself included), 3. wait for every rank
    bool ok = true;
    if (tid < (uint32_t)world) {
        st_release_sys(peers.flags[tid] + flag_index + rank, tag);
        const uint32_t *theirs = peers.flags[rank] + flag_index + tid;
        const uint64_t t0 = global_ns();
        ok = false;
        for (uint64_t it = 0; it < polls; ++it) {
            if (ld_acquire_sys(theirs) == tag) {
                ok = true;
                break;
            }
            if ((it & 63u) == 63u && global_ns() - t0 > wait_ns) break;
        }
    }
    const int all_ok = __syncthreads_and(ok ? 1 : 0);
    // 4. sum in rank order
    if (all_ok) {
        auto add = [](float *acc, const uint4 &x) {
            const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                acc[2 * k] += __uint_as_float(w[k] << 16);
                acc[2 * k + 1] += __uint_as_float(w[k] & 0xFFFF0000u);
            }
        };
        for (uint32_t v = v0 + tid; v < v1; v += kThreads) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            const size_t offset = (size_t)half * slot_bytes + (size_t)v * 16;
            if (WORLD > 0) {
                uint4 x[WORLD > 0 ? WORLD : 1];
#pragma unroll
                for (int r = 0; r < WORLD; ++r) x[r] = ld_volatile16(peers.data[r] + offset);  // all in flight together
#pragma unroll
                for (int r = 0; r < WORLD; ++r) add(acc, x[r]);
            } else {
                for (int r = 0; r < world; ++r) add(acc, ld_volatile16(peers.data[r] + offset));
            }
            out[v] = make_uint4(bf16x2_from_floats(acc[0], acc[1]), bf16x2_from_floats(acc[2], acc[3]),
                                bf16x2_from_floats(acc[4], acc[5]), bf16x2_from_floats(acc[6], acc[7]));
        }
    } else if (tid == 0 && status != nullptr) {
        atomicOr(status, DF11_STATUS_TIMEOUT);  // the output is left as it was; the host reads the status
    }
    // the last CTA to get here advances the call number (every CTA has read it by then)
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(counters + 1, 1u) == n_ctas - 1u) {
            counters[1] = 0u;
            __threadfence();
            *reinterpret_cast<volatile uint32_t *>(counters) = call + 1u;
        }
    }
}

template <int WORLD>
__global__ void __launch_bounds__(kThreads) df11_allreduce_kernel(const Peers peers, uint32_t *counters, int rank,
                                                                  int world_arg, const uint4 *in, uint4 *out,
                                                                  uint32_t n_vec, uint32_t vec_per_cta,
                                                                  uint32_t slot_bytes, uint64_t wait_ns, int *status)
{
    flag_form<WORLD>(peers, counters, rank, world_arg, in, out, n_vec, vec_per_cta, slot_bytes, wait_ns, status,
                     blockIdx.x, gridDim.x);
}

// The pushed form: one 16-byte vector per thread, no shared state between threads.
template <int WORLD>
__device__ __forceinline__ void pushed_form(const Peers &peers, const uint8_t *own, uint32_t *counters, int rank,
                                            const uint4 *in, uint4 *out, uint32_t n_vec, uint64_t wait_ns,
                                            int *status, uint32_t cta, uint32_t n_ctas)
{
    uint32_t *sequence = counters + 2 + cta;  // pushed calls this CTA has seen: the same on every rank
    const uint32_t call = *reinterpret_cast<volatile uint32_t *>(sequence);
    const uint64_t polls = poll_limit(wait_ns, status);  // read early: its latency hides behind the loads below
    uint32_t tag = call + 1u;  // never 0: the buffers start zeroed
    if (tag == 0u) tag = 1u;   // (the neighbouring calls' tags in the same half are 0xFFFFFFFF and 2)
    const uint32_t v = cta * kLlThreads + threadIdx.x;
    const size_t half = kFlagBytes + (size_t)(call & 1u) * kLlHalfBytes;
    bool ok = true;
    if (v < n_vec) {
        const uint4 x = in[v];
        const size_t mine = half + ((size_t)rank * kLlSlotVecs + v) * 32;
#pragma unroll
        for (int r = 0; r < WORLD; ++r) {
            uint8_t *cell = reinterpret_cast<uint8_t *>(peers.flags[r]) + mine;
            st_volatile16(cell, x.x, tag, x.y, tag);
            st_volatile16(cell + 16, x.z, tag, x.w, tag);
        }
        const uint8_t *cells = own + half + (size_t)v * 32;  // this rank's own area (= peers.flags[rank])
        uint4 a[WORLD], b[WORLD];
        const uint64_t t0 = global_ns();
        ok = false;
        for (uint64_t it = 0; it < polls; ++it) {
            bool all = true;
#pragma unroll
            for (int r = 0; r < WORLD; ++r) {
                a[r] = ld_volatile16(cells + (size_t)r * kLlSlotVecs * 32);
                b[r] = ld_volatile16(cells + (size_t)r * kLlSlotVecs * 32 + 16);
                all &= a[r].y == tag && a[r].w == tag && b[r].y == tag && b[r].w == tag;
            }
            if (all) {
                ok = true;
                break;
            }
            if ((it & 63u) == 63u && global_ns() - t0 > wait_ns) break;
        }
        if (ok) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int r = 0; r < WORLD; ++r) {  // rank order, fp32
                const uint32_t w[4] = {a[r].x, a[r].z, b[r].x, b[r].z};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    acc[2 * k] += __uint_as_float(w[k] << 16);
                    acc[2 * k + 1] += __uint_as_float(w[k] & 0xFFFF0000u);
                }
            }
            out[v] = make_uint4(bf16x2_from_floats(acc[0], acc[1]), bf16x2_from_floats(acc[2], acc[3]),
                                bf16x2_from_floats(acc[4], acc[5]), bf16x2_from_floats(acc[6], acc[7]));
        }
    }
    const int all_ok = __syncthreads_and(ok ? 1 : 0);  // every thread has read the count by now
    if (threadIdx.x == 0) {
        if (!all_ok && status != nullptr) atomicOr(status, DF11_STATUS_TIMEOUT);
        *sequence = call + 1u;  // seen by the next launch on this stream
    }
    (void)n_ctas;
}

template <int WORLD>
__global__ void __launch_bounds__(kLlThreads) df11_allreduce_ll_kernel(const Peers peers, const uint8_t *own,
                                                                       uint32_t *counters, int rank, const uint4 *in,
                                                                       uint4 *out, uint32_t n_vec,
                                                                       uint64_t wait_ns, int *status)
{
    pushed_form<WORLD>(peers, own, counters, rank, in, out, n_vec, wait_ns, status, blockIdx.x, gridDim.x);
}

// All ranks played by ONE launch on one GPU (row y of the grid is rank y; a cooperative launch, so
// that every CTA is resident while the rows wait for one another): the same code as above on
// `world` buffers, flag areas, counters, inputs and outputs laid out one after another.
struct Emulated {
    uint8_t *data, *flags;       // [world] buffers of 2 * slot_bytes, [world] flag areas
    uint32_t *counters;          // [world][kCounterWords]
    const uint4 *in;             // [world][n_vec]
    uint4 *out;                  // [world][n_vec]
};

template <int WORLD, bool PUSHED>
__global__ void __launch_bounds__(PUSHED ? kLlThreads : kThreads) df11_allreduce_emulated_kernel(
    const Emulated e, uint32_t n_vec, uint32_t vec_per_cta, uint32_t slot_bytes, uint64_t wait_ns, int *status)
{
    const int rank = blockIdx.y;
    Peers peers = {};
#pragma unroll
    for (int r = 0; r < WORLD; ++r) {
        peers.data[r] = e.data + (size_t)r * 2 * slot_bytes;
        peers.flags[r] = reinterpret_cast<uint32_t *>(e.flags + (size_t)r * (kFlagBytes + 2 * kLlHalfBytes));
    }
    uint32_t *counters = e.counters + kCounterWords * rank;
    const uint4 *in = e.in + (size_t)rank * n_vec;
    uint4 *out = e.out + (size_t)rank * n_vec;
    // 2, 4 and 8 ranks: the specialised kernels of the real launch; any other number: the general one
    constexpr int kSpecial = (WORLD == 2 || WORLD == 4 || WORLD == 8) ? WORLD : 0;
    if (PUSHED)
        pushed_form<WORLD>(peers, e.flags + (size_t)rank * (kFlagBytes + 2 * kLlHalfBytes), counters, rank, in, out,
                           n_vec, wait_ns, status, blockIdx.x, gridDim.x);
    else
        flag_form<kSpecial>(peers, counters, rank, WORLD, in, out, n_vec, vec_per_cta, slot_bytes, wait_ns, status,
                            blockIdx.x, gridDim.x);
}

template <int WORLD>
cudaError_t launch_emulated(const Emulated &e, uint32_t n_vec, uint32_t slot_bytes, uint64_t wait_ns, int *status,
                            cudaStream_t stream)
{
    const bool pushed = n_vec <= kLlSlotVecs && (WORLD == 2 || WORLD == 4 || WORLD == 8);  // as the real launch chooses
    uint32_t ctas, per = 0;
    if (pushed) {
        ctas = (n_vec + kLlThreads - 1) / kLlThreads;
    } else {
        ctas = (n_vec + (uint32_t)kThreads - 1u) / (uint32_t)kThreads;
        if (ctas > (uint32_t)kMaxCtas) ctas = kMaxCtas;
        per = (n_vec + ctas - 1u) / ctas;
    }
    Emulated ee = e;
    void *args[] = {&ee, &n_vec, &per, &slot_bytes, &wait_ns, &status};
    const void *fn = pushed ? (const void *)df11_allreduce_emulated_kernel<WORLD, true>
                            : (const void *)df11_allreduce_emulated_kernel<WORLD, false>;
    return cudaLaunchCooperativeKernel(fn, dim3(ctas, WORLD), dim3(pushed ? kLlThreads : kThreads), args, 0, stream);
}

}  // namespace

extern "C" int df11_selftest_allreduce_one_gpu(int32_t world, void *data, void *flags, void *counters,
                                               const void *in_bf16, void *out_bf16, int64_t n_elements,
                                               int64_t slot_bytes, int64_t wait_ms, void *status, int32_t device,
                                               void *stream)
{
    if (!data || !flags || !counters || !in_bf16 || !out_bf16) return df11_fail(DF11_ERR_BADARG, "null pointer");
    if (world != 2 && world != 3 && world != 4 && world != 8)
        return df11_fail(DF11_ERR_BADARG, "world must be 2, 3, 4 or 8");
    if (n_elements <= 0 || n_elements % 8 || n_elements * 2 > slot_bytes || slot_bytes % 16 || slot_bytes > 0x7FFFFFFF)
        return df11_fail(DF11_ERR_BADARG, "n_elements must be a positive multiple of 8 that fits slot_bytes");
    if (((uintptr_t)data | (uintptr_t)flags | (uintptr_t)in_bf16 | (uintptr_t)out_bf16) & 15)
        return df11_fail(DF11_ERR_BADARG, "buffers must be 16-byte aligned");
    int prev = -1;
    cudaGetDevice(&prev);
    if (prev != device && cudaSetDevice(device) != cudaSuccess)
        return df11_fail(DF11_ERR_CUDA, "cudaSetDevice(%d) failed", device);
    int cooperative = 0;
    cudaDeviceGetAttribute(&cooperative, cudaDevAttrCooperativeLaunch, device);
    cudaError_t err = cudaErrorNotSupported;
    if (cooperative) {
        Emulated e = {(uint8_t *)data, (uint8_t *)flags, (uint32_t *)counters, (const uint4 *)in_bf16, (uint4 *)out_bf16};
        const uint32_t n_vec = (uint32_t)(n_elements / 8);
        const uint64_t wait_ns = wait_ms > 0 ? (uint64_t)wait_ms * 1000000ull : 200ull * 1000 * 1000;
        err = world == 3 ? launch_emulated<3>(e, n_vec, (uint32_t)slot_bytes, wait_ns, (int *)status, (cudaStream_t)stream)
            : world == 2 ? launch_emulated<2>(e, n_vec, (uint32_t)slot_bytes, wait_ns, (int *)status, (cudaStream_t)stream)
            : world == 4 ? launch_emulated<4>(e, n_vec, (uint32_t)slot_bytes, wait_ns, (int *)status, (cudaStream_t)stream)
                         : launch_emulated<8>(e, n_vec, (uint32_t)slot_bytes, wait_ns, (int *)status, (cudaStream_t)stream);
    }
    if (prev >= 0 && prev != device) cudaSetDevice(prev);
    if (err != cudaSuccess) return df11_fail(DF11_ERR_CUDA, "cooperative launch failed: %s", cudaGetErrorString(err));
    return DF11_OK;
}

extern "C" int64_t df11_allreduce_flag_bytes(void) { return (int64_t)(kFlagBytes + 2 * kLlHalfBytes); }
extern "C" int64_t df11_allreduce_counter_bytes(void) { return (int64_t)kCounterWords * sizeof(uint32_t); }

extern "C" int df11_allreduce_bf16(const uint64_t *peer_data, const uint64_t *peer_flags, void *counters, int32_t rank,
                                   int32_t world, const void *in_bf16, void *out_bf16, int64_t n_elements,
                                   int64_t slot_bytes, int64_t wait_ms, void *status, int32_t device, void *stream)
{
    if (!peer_data || !peer_flags || !counters || !in_bf16 || !out_bf16)
        return df11_fail(DF11_ERR_BADARG, "null pointer");
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world)
        return df11_fail(DF11_ERR_BADARG, "rank %d of %d: up to %d ranks", rank, world, kMaxRanks);
    if (n_elements < 0 || n_elements % 8) return df11_fail(DF11_ERR_BADARG, "n_elements must be a multiple of 8");
    if (n_elements * 2 > slot_bytes || slot_bytes % 16 || slot_bytes > 0x7FFFFFFF)
        return df11_fail(DF11_ERR_NOSPACE, "%lld elements do not fit a buffer half of %lld bytes", (long long)n_elements,
                         (long long)slot_bytes);
    if (((uintptr_t)in_bf16 & 15) || ((uintptr_t)out_bf16 & 15) || ((uintptr_t)counters & 3))
        return df11_fail(DF11_ERR_BADARG, "in / out must be 16-byte aligned");
    if (n_elements == 0) return DF11_OK;
    Peers peers = {};
    for (int r = 0; r < world; ++r) {
        if (!peer_data[r] || !peer_flags[r] || (peer_data[r] & 15) || (peer_flags[r] & 3))
            return df11_fail(DF11_ERR_BADARG, "peer pointer %d is null or misaligned", r);
        peers.data[r] = reinterpret_cast<uint8_t *>(peer_data[r]);
        peers.flags[r] = reinterpret_cast<uint32_t *>(peer_flags[r]);
    }
    int prev = -1;
    cudaGetDevice(&prev);
    if (prev != device && cudaSetDevice(device) != cudaSuccess)
        return df11_fail(DF11_ERR_CUDA, "cudaSetDevice(%d) failed", device);
    const uint32_t n_vec = (uint32_t)(n_elements / 8);
    const uint64_t wait_ns = wait_ms > 0 ? (uint64_t)wait_ms * 1000000ull : kWaitNs;
    if (n_vec <= kLlSlotVecs && (world == 1 || world == 2 || world == 4 || world == 8)) {
        auto kernel = world == 1 ? df11_allreduce_ll_kernel<1> : world == 2 ? df11_allreduce_ll_kernel<2>
                    : world == 4 ? df11_allreduce_ll_kernel<4> : df11_allreduce_ll_kernel<8>;
        kernel<<<(n_vec + kLlThreads - 1) / kLlThreads, kLlThreads, 0, (cudaStream_t)stream>>>(
            peers, reinterpret_cast<const uint8_t *>(peers.flags[rank]), (uint32_t *)counters, rank, (const uint4 *)in_bf16,
            (uint4 *)out_bf16, n_vec, wait_ns, (int *)status);
        const cudaError_t e = cudaGetLastError();
        if (prev >= 0 && prev != device) cudaSetDevice(prev);
        if (e != cudaSuccess) return df11_fail(DF11_ERR_CUDA, "kernel launch failed: %s", cudaGetErrorString(e));
        return DF11_OK;
    }
    uint32_t ctas = (n_vec + (uint32_t)kThreads - 1u) / (uint32_t)kThreads;  // one vector per thread
    if (ctas > (uint32_t)kMaxCtas) ctas = kMaxCtas;
    if (ctas < 1u) ctas = 1u;
    const uint32_t per = (n_vec + ctas - 1u) / ctas;
    auto kernel = world == 2 ? df11_allreduce_kernel<2> : world == 4 ? df11_allreduce_kernel<4>
                : world == 8 ? df11_allreduce_kernel<8> : df11_allreduce_kernel<0>;
    kernel<<<ctas, kThreads, 0, (cudaStream_t)stream>>>(peers, (uint32_t *)counters, rank, world,
                                                        (const uint4 *)in_bf16, (uint4 *)out_bf16, n_vec, per,
                                                        (uint32_t)slot_bytes, wait_ns, (int *)status);
    const cudaError_t e = cudaGetLastError();
    if (prev >= 0 && prev != device) cudaSetDevice(prev);
    if (e != cudaSuccess) return df11_fail(DF11_ERR_CUDA, "kernel launch failed: %s", cudaGetErrorString(e));
    return DF11_OK;
}
