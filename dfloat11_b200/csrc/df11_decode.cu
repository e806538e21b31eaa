// DF11 -> BF16 decompression kernels for B200 (sm_100a) and their C entry points.
//
// What one launch computes is fixed by the reference kernel dfloat11/decode.cu:25-253
// (see df11_common.h for the format); how it is computed is not taken from it.
//
// Two decoders live here.
//
// df11_fast_kernel (behind df11_decode_prepared): a one-time pass over a unit
// (df11_sync_kernel, behind df11_prepare) records a seek point -- the stream bit position
// -- for every group of 16 or 32 consecutive output elements.  Afterwards a thread needs
// only its group number: it reads the seek point, pulls the stream words it needs through
// L1 (neighbouring threads read neighbouring words), decodes exactly one group with a
// 2^K-entry multi-symbol table held in shared memory (up to four exponents per probe), merges
// the exponents with one 16-byte load of sign/mantissa bytes and writes 16-byte stores.  No
// staging of exponents, no scan, no barrier in the steady state; all global accesses of a
// warp are contiguous.
//
// df11_decode_kernel (behind df11_decode): needs nothing but the six DF11 tensors.
// Persistent CTAs walk the format blocks; every global read is a TMA bulk copy
// (cp.async.bulk with mbarrier completion, each CTA fetching for itself): the next block's bitstream and
// gap bytes arrive in a double buffer while the current block is decoded, and the block's
// sign/mantissa bytes arrive while its exponents are decoded.  One window per thread in
// three registers; output slots from a counting pass and a warp-shuffle scan (2 barriers
// per block instead of the reference's 18); exponents staged as bytes in shared memory and
// merged eight elements at a time with 16-byte coalesced stores.
//
// In both, every loop and every wait is bounded and every index is clamped: inconsistent
// tensors set a status bit instead of hanging (decode.cu:116-118 can spin forever).
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <mutex>

#include "../../include/df11.h"
#include "df11_common.h"
#include "df11_error.h"

namespace {

constexpr int kThreads = 512;  // one window per thread, one format block per CTA pass
constexpr int kWarps = kThreads / 32;
#ifndef DF11_TABLE_BITS
#define DF11_TABLE_BITS 11
#endif
#ifndef DF11_FAST_TABLE_BITS
#define DF11_FAST_TABLE_BITS 12
#endif
#ifndef DF11_FAST_MIN_CTAS
#define DF11_FAST_MIN_CTAS 2
#endif
#ifndef DF11_GEMV_THREADS
#define DF11_GEMV_THREADS 1024
#endif
#ifndef DF11_GEMV_MIN_CTAS
#define DF11_GEMV_MIN_CTAS 1
#endif
constexpr int kTableBits = DF11_TABLE_BITS;           // K of the self-contained decoder and the seek-point pass
constexpr int kFastTableBits = DF11_FAST_TABLE_BITS;  // K of the fast decoder (its table is larger, its CTAs smaller)

constexpr int kCodesBufBytes = DF11_BLOCK_BYTES + 16;      // block + look-ahead, multiple of 16
constexpr int kInBufBytes = kCodesBufBytes + DF11_GAP_BYTES_PER_BLOCK;  // stream bytes, then gap bytes
// Bounded waits for bulk copies.  A copy of a few KB lands within microseconds; a wait gives up
// after kWaitNs of wall time (and after kWaitPolls polls whatever the clock says).  A CTA that gave
// up leaves its loop, waits once more, kDrainNs at most, for the copies it still has in flight into
// its own shared memory, and returns.
constexpr uint32_t kWaitPolls = 1u << 20;
constexpr uint64_t kWaitNs = 50ull * 1000 * 1000;
constexpr uint64_t kDrainNs = 200ull * 1000 * 1000;
// Two CTAs of 512 threads per SM: with 32-byte stores, two copies of the decode table per SM beat
// four (measured on one Llama-8B block: 256 x 4 5 388 GB/s, 512 x 2 5 491, 1024 x 1 with a 2^14-entry
// table 5 487, 512 x 2 with 2^13 entries 5 451).
#ifndef DF11_FAST_THREADS
#define DF11_FAST_THREADS 512
#endif
constexpr int kFastThreads = DF11_FAST_THREADS;
// The fused product runs one CTA of 1024 threads per SM: its launches are short, and one copy of
// the decode table per SM instead of four shortens every one of them.
constexpr int kGemvThreads = DF11_GEMV_THREADS;

struct Params {
    const uint8_t *luts;
    const uint8_t *codes;
    const uint8_t *sm;
    const uint32_t *pos;
    const uint8_t *gaps;
    uint16_t *out;
    const Df11Entry *table_g;  // prebuilt decode table in global memory (prepared form)
    uint32_t *sync_hi;         // seek points: high part, one per 32 groups
    uint16_t *sync_lo;         // seek points: low 16 bits, one per group
    int *status;
    int64_t n_bytes;
    int64_t n_elements;
    int64_t n_blocks;
    int64_t n_chunks;          // ceil(number of groups / 32)
    const int64_t *rows;       // row-wise decode: the rows to produce, else null
    uint32_t chunks_per_row;   // row-wise decode: 512-element chunks per row
    uint32_t n_tasks;          // row-wise decode: rows wanted * chunks_per_row
    uint32_t n_rows_total;     // row-wise decode: rows the unit holds
    uint32_t chunk_first;      // range decode: first chunk to produce (its output starts at `out`), else 0
    uint32_t chunk_count;      // range decode: chunks to produce; 0 = the whole unit
    int n_luts;
    int ept;          // elements per seek point (16 or 32)
    int stage_bytes;  // shared staging area (and sign/mantissa tile), multiple of 16
    int codes_aligned;  // bit 0: codes 16-byte aligned, bit 1: gaps 16-byte aligned (bulk copies allowed),
                        // bit 2: codes 4-byte aligned (word loads allowed)
    int sm_aligned;     // bit 0: sign_mantissa 16-byte aligned (bulk copies / 16-byte loads allowed), bit 1: 32-byte
    int out_aligned;    // bit 0: out 16-byte aligned (vector stores allowed), bit 1: 32-byte (256-bit stores)
    // self-test of the bounded waits (df11_selftest_wait_timeout): the producer announces the
    // bytes of format block `drop_block`'s input copy but never issues it, and waits are cut to
    // `wait_ns`.  0 / -1 in every ordinary launch.
    int64_t drop_block;
    uint64_t wait_ns;
};

// ---- shared-memory accessors: explicit 32-bit shared addresses ---------------------------
__device__ __forceinline__ uint32_t lds32(uint32_t a)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a)
{
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds8(uint32_t a)
{
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
template <int OFF>
__device__ __forceinline__ void sts8(uint32_t a, uint32_t v)
{
    asm volatile("st.shared.u8 [%0+%2], %1;" ::"r"(a), "r"(v), "n"(OFF) : "memory");
}

// ---- 256-bit global accesses (one instruction for 32 bytes per lane; address 32-byte aligned):
// half the load/store instructions and memory-pipe wavefronts of two 16-byte accesses.
__device__ __forceinline__ void stg256(void *dst, const uint4 &a, const uint4 &b)
{
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "r"(a.x), "r"(a.y), "r"(a.z),
                 "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w)
                 : "memory");
}
__device__ __forceinline__ void ldg256(const void *src, uint4 &a, uint4 &b)
{
    asm volatile("ld.global.nc.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w), "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w)
                 : "l"(src));
}

// ---- programmatic dependent launch: a kernel launched with the stream-serialization attribute
// may start before the kernel ahead of it in the stream has ended; it must not touch that
// kernel's results before grid_dependency_wait().  Both are no-ops in an ordinary launch.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- TMA bulk copy global -> shared with mbarrier completion, one CTA as target ---------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// src and dst 16-byte aligned, bytes a non-zero multiple of 16
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0u;
}
__device__ __forceinline__ uint64_t global_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Waits for the given phase of an mbarrier; gives up after `limit_ns` nanoseconds or kWaitPolls
// polls, whichever comes first.  The clock is only read when the first poll fails.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, uint64_t limit_ns)
{
    const uint64_t t0 = global_ns();
    for (uint32_t it = 0; it < kWaitPolls; ++it) {
        if (mbar_try(bar, parity)) return true;
        if (global_ns() - t0 > limit_ns) break;
    }
    return false;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint64_t limit_ns)
{
    if (mbar_try(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, limit_ns);
}

// Memory policy of the window routines (df11_common.h) for the kernels: every table probe is
// one ld.shared, every staged exponent one st.shared.u8.
struct SmemPolicy {
    uint32_t dec_addr, cnt_addr, stage_addr, luts_addr;
    __device__ __forceinline__ uint32_t cnt(uint32_t i) const { return lds32(cnt_addr + i * 4u); }
    __device__ __forceinline__ Df11Entry dec(uint32_t i) const
    {
        const uint2 v = lds64(dec_addr + i * 8u);
        Df11Entry e;
        e.meta = v.x;
        e.syms = v.y;
        return e;
    }
    __device__ __forceinline__ uint32_t lut(uint32_t i) const { return lds8(luts_addr + i); }
    __device__ __forceinline__ void put8(uint32_t addr, uint32_t v) const { sts8<0>(stage_addr + addr, v); }
};

// Window words read straight from global memory, for blocks at the end of the stream (bytes
// past the end read as 0) and for streams that are not 16-byte aligned.
__device__ __noinline__ uint3 load_window_slow(const uint8_t *codes, int64_t n_bytes, int64_t off)
{
    uint32_t w[3] = {0, 0, 0};
#pragma unroll
    for (int k = 0; k < 12; ++k) {
        const int64_t i = off + k;
        const uint32_t byte = i < n_bytes ? (uint32_t)__ldg(codes + i) : 0u;
        w[k >> 2] |= byte << (24 - 8 * (k & 3));
    }
    return make_uint3(w[0], w[1], w[2]);
}

// 5-bit gap of window `w` of a block from the block's 320 gap bytes (decode.cu:85-87); the
// second byte is read only when the field straddles a byte boundary.
template <class F>
__device__ __forceinline__ uint32_t block_gap(F byte_at, uint32_t w)
{
    const uint32_t bit = 5u * w, j = bit >> 3, r = bit & 7u;
    const uint32_t hi = byte_at(j);
    const uint32_t lo = byte_at(r > 3u ? j + 1u : j);
    return (((hi << 8) | lo) >> (11u - r)) & 31u;
}

__device__ __forceinline__ void build_tables_smem(const Params &p, uint8_t *luts_s, uint8_t *agree, Df11Entry *dec,
                                                  uint32_t *cnt, int K, uint32_t tid)
{
    for (int task = tid; task < 255; task += kThreads) {
        int u = 1;
        while (task >= df11_agree_offset(u + 1) && u < 8) ++u;
        agree[task] = df11_agree_flag(luts_s, u, task - df11_agree_offset(u));
    }
    __syncthreads();
    for (int v = tid; v < (1 << K); v += kThreads) {
        Df11Entry e;
        uint32_t c;
        df11_build_entry(luts_s, p.n_luts, agree, (uint32_t)v, K, &e, &c);
        if (dec) dec[v] = e;
        if (cnt) cnt[v] = c;
    }
}

// Block-wide exclusive scan of one value per thread; returns the exclusive prefix.
__device__ __forceinline__ uint32_t block_scan(uint32_t v, uint32_t *wsum, uint32_t lane, uint32_t warp)
{
    uint32_t incl = v;
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
    return (warp > 0 ? before : 0u) + incl - v;
}

// ---------------------------------------------------------------------------------------
// Seek-point kernel (once per unit, behind df11_prepare).  One window per thread: count the
// window's codes, scan the counts inside the format block, then walk the window again knowing
// the output index of its first code and record the bit position of every code whose index
// is a multiple of EPT.
// ---------------------------------------------------------------------------------------
template <int K>
__global__ void __launch_bounds__(kThreads, 3) df11_sync_kernel(const Params p)
{
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t smem_addr = (uint32_t)__cvta_generic_to_shared(smem);
    uint8_t *luts_s = smem + (4u << K);
    uint8_t *agree = luts_s + p.n_luts * 256;
    uint32_t *wsum = reinterpret_cast<uint32_t *>(agree + 256);
    SmemPolicy mem;
    mem.dec_addr = 0;
    mem.cnt_addr = smem_addr;
    mem.stage_addr = 0;
    mem.luts_addr = smem_addr + (4u << K);

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    int bad = 0;
    for (int i = tid; i < p.n_luts * 256; i += kThreads) luts_s[i] = __ldg(p.luts + i);
    __syncthreads();
    build_tables_smem(p, luts_s, agree, nullptr, reinterpret_cast<uint32_t *>(smem), K, tid);
    __syncthreads();

    const uint32_t ept = (uint32_t)p.ept;
    const uint64_t n_groups = ((uint64_t)p.n_elements + ept - 1) / ept;
    for (int64_t b = blockIdx.x; b < p.n_blocks; b += gridDim.x) {
        const int64_t off = b * DF11_BLOCK_BYTES + (int64_t)tid * DF11_WINDOW_BYTES;
        const uint8_t *g = p.gaps + b * DF11_GAP_BYTES_PER_BLOCK;
        const uint32_t gap = block_gap([&](uint32_t j) { return (uint32_t)__ldg(g + j); }, tid);
        const bool live = off < p.n_bytes;
        uint3 w = make_uint3(0, 0, 0);
        uint32_t cnt = 0;
        int tbad = 0;
        if (live) {
            if ((p.codes_aligned & 1) && off + 12 <= p.n_bytes) {
                const uint2 v = __ldg(reinterpret_cast<const uint2 *>(p.codes + off));
                const uint32_t x = __ldg(reinterpret_cast<const uint32_t *>(p.codes + off + 8));
                w = make_uint3(__byte_perm(v.x, 0, 0x0123), __byte_perm(v.y, 0, 0x0123), __byte_perm(x, 0, 0x0123));
            } else {
                w = load_window_slow(p.codes, p.n_bytes, off);
            }
        }
        cnt = df11_count_window<K>(mem, p.n_luts, w.x, w.y, w.z, live ? gap : 64u, &tbad);
        const uint32_t o = block_scan(cnt, wsum, lane, warp);
        if (live) {
            const uint64_t first = (uint64_t)__ldg(p.pos + b) + o;
            const uint64_t window_bit = (uint64_t)off * 8u;
            df11_mark_window<K>(
                mem, p.n_luts, w.x, w.y, w.z, gap, first, ept,
                [&](uint64_t group, uint32_t bit_in_window) {
                    if (group >= n_groups) return;  // padding decoded past the last element
                    const uint64_t bit = window_bit + bit_in_window;
                    p.sync_lo[group] = (uint16_t)bit;
                    if ((group & 31u) == 0) p.sync_hi[group >> 5] = (uint32_t)(bit >> 16);
                },
                &tbad);
        }
        if (tbad) bad |= DF11_STATUS_BAD_TABLE;
        __syncthreads();  // wsum is reused by the next block
    }
    if (bad && p.status != nullptr) atomicOr(p.status, bad);
}

struct FastTables {
    uint32_t dec_addr, luts_addr;
    __device__ __forceinline__ uint32_t lut(uint32_t i) const { return lds8(luts_addr + i); }
};

// The exponent shift register (Df11ExpShift), the fast entry format (df11_fast_meta) and the
// meaning of the running state `acc` are defined in df11_common.h, where the CPU tests run the
// same arithmetic.
using ExpShift = Df11ExpShift;
constexpr uint32_t kFastEscape = DF11_FAST_ESCAPE;
constexpr uint32_t kFastDone = DF11_FAST_DONE;
constexpr uint32_t kFastLeave = DF11_FAST_LEAVE;
__host__ __device__ constexpr uint32_t fast_meta(uint32_t meta) { return df11_fast_meta(meta); }

// The probe loop of the fast decoder (the device form of df11_decode_group's inner loop,
// df11_common.h, for 16 codes).  The 96-bit window w0:w1:w2 is kept shifted so that the next
// code starts at its top bit.  One pass: index the table with the top K bits, shift the
// entry's symbols into the exponent register, shift the window by the bits consumed.  The
// window shifts take their amount modulo 32 from the entry word itself; the register shift
// clamps at 32, which is what four symbols need.  Table index, address and the symbol count
// are formed with multiply instructions to keep them off the integer ALU pipe, which is the
// busiest unit of this kernel.
template <int K>
__device__ __forceinline__ void probe_loop(uint32_t &acc, ExpShift &X, uint32_t &w0, uint32_t &w1, uint32_t &w2,
                                           uint32_t dec_addr)
{
    asm volatile(
        "{\n\t"
        ".reg .pred pl;\n\t"
        ".reg .b32 t, i, m, s, n8;\n\t"
        "DF11_PROBE:\n\t"
        "mul.hi.u32 i, %6, %10;\n\t"             // top K bits of the window
        "mad.lo.u32 i, i, 8, %9;\n\t"
        "ld.shared.v2.u32 {m, s}, [i];\n\t"
        "mul.hi.u32 n8, m, 65536;\n\t"           // 8 * symbols of the entry
        "shf.r.clamp.b32 %1, %1, %2, n8;\n\t"
        "shf.r.clamp.b32 %2, %2, %3, n8;\n\t"
        "shf.r.clamp.b32 %3, %3, %4, n8;\n\t"
        "shf.r.clamp.b32 %4, %4, %5, n8;\n\t"
        "shf.r.clamp.b32 %5, %5, s, n8;\n\t"
        "shf.l.wrap.b32 %6, %7, %6, m;\n\t"      // window <<= bits consumed
        "shf.l.wrap.b32 %7, %8, %7, m;\n\t"
        "shf.l.wrap.b32 %8, 0, %8, m;\n\t"
        "add.u32 %0, %0, m;\n\t"
        "and.b32 t, %0, %11;\n\t"
        "setp.eq.u32 pl, t, 0;\n\t"
        "@pl bra DF11_PROBE;\n\t"
        "}"
        : "+r"(acc), "+r"(X.x0), "+r"(X.x1), "+r"(X.x2), "+r"(X.x3), "+r"(X.x4), "+r"(w0), "+r"(w1), "+r"(w2)
        : "r"(dec_addr), "n"(1 << K), "n"(kFastLeave));
}

// Four raw stream words starting at word `wi`, byte by byte: for the end of the stream (bytes past
// it read as 0) and for any word index, however wrong.
__device__ __noinline__ uint4 stream_words_slow(const uint8_t *codes, int64_t n_bytes, uint32_t wi)
{
    uint32_t v[4] = {0, 0, 0, 0};
    const int64_t off = (int64_t)wi * 4;
    for (int k = 0; k < 16; ++k)
        if (off + k < n_bytes) v[k >> 2] |= (uint32_t)__ldg(codes + off + k) << (8 * (k & 3));
    return make_uint4(v[0], v[1], v[2], v[3]);
}

// The 96-bit window four raw words give once byte-swapped and shifted left by `bit`.
__device__ __forceinline__ void stream_window(const uint4 &r, uint32_t bit, uint32_t &w0, uint32_t &w1, uint32_t &w2)
{
    const uint32_t a = __byte_perm(r.x, 0, 0x0123), b = __byte_perm(r.y, 0, 0x0123);
    const uint32_t c = __byte_perm(r.z, 0, 0x0123), d = __byte_perm(r.w, 0, 0x0123);
    w0 = __funnelshift_l(b, a, bit);
    w1 = __funnelshift_l(c, b, bit);
    w2 = __funnelshift_l(d, c, bit);
}

// The inner loop of the fast decoder for tasks that are known to be whole chunks of 32 * EPT
// elements of aligned tensors (a seek point every EPT = 16 or 32 elements).  This warp runs
// `n_seq` tasks, numbered 0 .. n_seq-1 in the order it runs them; task j is chunk `chunk_of(j)`.
// For every sixteen elements of this lane's group the sink gets the task's number, which
// sixteen of the group they are (`part`, 0 or 1), their exponents (four per word, lowest byte
// first) and their sign/mantissa bytes.  With EPT = 32 the second half of a group goes on where
// the first stopped: its stream words were loaded by neighbouring lanes a moment ago, so the
// reload in the middle of a task is served by L1.
//
// Three stages run ahead of each other: the seek point of the task after the next is being
// loaded while the stream words and sign/mantissa bytes of the next task are being loaded
// while the current task is decoded.  Task numbers fetched ahead are clamped to the last
// task instead of being branched around, and the loop is unrolled twice so that the two
// input sets swap roles without register moves.
//
// CHECKED = false: the caller guarantees that at least 16 whole stream words follow the
// start of every task's last group (true for every chunk but the last two of a unit), so a
// word index is only clamped: a foreign auxiliary buffer gives wrong output, never a fault.
// CHECKED = true: any chunk of the unit; word loads near the end of the stream go byte by byte.
template <int K, int EPT, bool CHECKED, class ChunkOf, class Sink>
__device__ __forceinline__ void lean_tasks(const Params &p, const FastTables &tab, uint32_t lane, uint32_t n_seq,
                                           ChunkOf &&chunk_of, uint32_t n_words, int &bad, Sink &&sink)
{
    if (n_seq == 0u) return;
    const uint32_t *codes32 = reinterpret_cast<const uint32_t *>(p.codes);
    const uint32_t last_task = n_seq - 1u;
    const uint32_t last_wi = n_words - 4u;  // callers make sure of n_words >= 4
    struct Inputs {
        uint32_t wi, bit;
        uint4 words, sm[EPT / 16];
    };
    auto words_at = [&](uint32_t wi) -> uint4 {
        if (CHECKED && wi > last_wi) return stream_words_slow(p.codes, p.n_bytes, wi);
        const uint32_t *src = codes32 + wi;
        return make_uint4(__ldg(src), __ldg(src + 1), __ldg(src + 2), __ldg(src + 3));
    };
    uint32_t lo_n, hi_n;  // seek point of the task after the next
    auto fetch_seek = [&](uint32_t t) {
        const uint32_t chunk = chunk_of(min(t, last_task));
        lo_n = (uint32_t)__ldg(p.sync_lo + chunk * 32u + lane);
        hi_n = __ldg(p.sync_hi + chunk);
    };
    auto fetch_inputs = [&](uint32_t t, Inputs &in) {  // uses the seek point fetched for task t
        const uint32_t chunk = chunk_of(min(t, last_task));
        uint32_t lo = lo_n;
        const uint32_t lo0 = __shfl_sync(0xffffffffu, lo, 0);
        if (lo < lo0) lo += 65536u;
        in.wi = (hi_n << 11) + (lo >> 5);
        if (!CHECKED) in.wi = min(in.wi, last_wi);
        in.bit = lo & 31u;
        in.words = words_at(in.wi);
        const uint4 *sm16 = reinterpret_cast<const uint4 *>(p.sm) + (chunk * 32u + lane) * (EPT / 16);
        if (EPT == 32 && (p.sm_aligned & 2)) {
            ldg256(sm16, in.sm[0], in.sm[EPT / 16 - 1]);
        } else {
#pragma unroll
            for (int part = 0; part < EPT / 16; ++part) in.sm[part] = __ldg(sm16 + part);
        }
    };
    ExpShift X = {0, 0, 0, 0, 0};
    auto run_task = [&](uint32_t t, const Inputs &cur, Inputs &nxt) {
        fetch_inputs(t + 1u, nxt);
        fetch_seek(t + 2u);
        uint32_t wi = cur.wi, bit = cur.bit, acc = 0, w0, w1, w2;
        stream_window(cur.words, bit, w0, w1, w2);
#pragma unroll
        for (int part = 0; part < EPT / 16; ++part) {
            if (part > 0) {  // go on where the first sixteen stopped; codes decoded beyond them are at the top of X
                const uint32_t at = bit + (acc & 0x7Fu);
                wi += at >> 5;
                if (!CHECKED) wi = min(wi, last_wi);
                bit = at & 31u;
                acc = (acc & ~0xFFu) - kFastDone;
                stream_window(words_at(wi), bit, w0, w1, w2);
            }
            for (;;) {
                probe_loop<K>(acc, X, w0, w1, w2, tab.dec_addr);
                if (acc & kFastDone) break;  // the usual exit
                if (acc & kFastEscape) {     // full walk for one symbol
                    acc -= kFastEscape;
                    uint32_t len;
                    int tbad = 0;
                    const uint32_t sym = df11_walk_m(tab, p.n_luts, w0, &len, &tbad);
                    if (tbad) bad |= DF11_STATUS_BAD_TABLE;
                    X.push(sym, 8u);
                    acc += len | (8u << 16);
                    if (len < 32u) {
                        w0 = __funnelshift_l(w1, w0, len);
                        w1 = __funnelshift_l(w2, w1, len);
                        w2 <<= len;
                    } else {
                        w0 = w1, w1 = w2, w2 = 0;
                    }
                    if (acc & kFastDone) break;
                }
                if (acc & 64u) {  // position 64..127: reload the window where the position has got to
                    const uint32_t at = bit + (acc & 0x7Fu);
                    wi += at >> 5;
                    if (!CHECKED) wi = min(wi, last_wi);
                    bit = at & 31u;
                    stream_window(words_at(wi), bit, w0, w1, w2);
                    acc &= ~0xFFu;
                }
            }
            uint32_t e0, e1, e2, e3;
            X.take(acc, &e0, &e1, &e2, &e3);
            sink(t, (uint32_t)part, e0, e1, e2, e3, cur.sm[part]);
        }
    };
    Inputs a, b;
    fetch_seek(0u);
    fetch_inputs(0u, a);
    fetch_seek(1u);
    for (uint32_t j = 0;;) {
        run_task(j, a, b);
        if (++j >= n_seq) break;
        run_task(j, b, a);
        if (++j >= n_seq) break;
    }
}

// ---------------------------------------------------------------------------------------
// Fast decoder (behind df11_decode_prepared).  A warp handles 32 consecutive groups, i.e. one
// contiguous run of 32*EPT outputs; a thread decodes its group 16 codes at a time.
// Shared memory: the decode table and `luts` (for the rare full walk).
// ---------------------------------------------------------------------------------------
template <int K, int EPT, bool ROWS>
__global__ void __launch_bounds__(kFastThreads, DF11_FAST_MIN_CTAS) df11_fast_kernel(const Params p)
{
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t smem_addr = (uint32_t)__cvta_generic_to_shared(smem);
    constexpr uint32_t luts_off = 8u << K;
    const uint32_t tid = threadIdx.x, lane = tid & 31u;

    {   // once per CTA: decode table (built by df11_prepare) and luts into shared memory
        const uint4 *src = reinterpret_cast<const uint4 *>(p.table_g);
        uint4 *dst = reinterpret_cast<uint4 *>(smem);
        for (int i = tid; i < (1 << K) / 2; i += kFastThreads) dst[i] = __ldg(src + i);
        for (int i = tid; i < p.n_luts * 256; i += kFastThreads) smem[luts_off + i] = __ldg(p.luts + i);
    }
    __syncthreads();

    FastTables tab;
    tab.dec_addr = smem_addr;
    tab.luts_addr = smem_addr + luts_off;
    const uint32_t *codes32 = reinterpret_cast<const uint32_t *>(p.codes);
    // words that can be loaded whole; 0 sends every word of an unaligned stream the slow way
    const uint32_t n_words = (p.codes_aligned & 4) ? (uint32_t)(p.n_bytes >> 2) : 0u;
    const uint32_t n_whole = n_words > 3u ? n_words - 3u : 0u;  // word indices with three whole words after them
    const bool vec = (p.sm_aligned & 1) && (p.out_aligned & 1);  // 16-byte loads and stores allowed
    const bool wide = (p.out_aligned & 2) != 0;                  // 32-byte stores allowed
    int bad = 0;

    // Four raw stream words starting at word `wi` (bytes past the end read as 0), and the 96-bit
    // window they give once byte-swapped and shifted left by `bit`.
    auto load_words_slow = [&](uint32_t wi, uint4 &r) {  // end of the stream, or an unaligned stream
        uint32_t v[4] = {0, 0, 0, 0};
        const int64_t off = (int64_t)wi * 4;
        for (int k = 0; k < 16; ++k)
            if (off + k < p.n_bytes) v[k >> 2] |= (uint32_t)__ldg(p.codes + off + k) << (8 * (k & 3));
        r = make_uint4(v[0], v[1], v[2], v[3]);
    };
    auto load_words = [&](uint32_t wi, uint4 &r) {
        if (wi < n_whole) {  // the common case: four whole words, one bounds check
            const uint32_t *src = codes32 + wi;
            r = make_uint4(__ldg(src), __ldg(src + 1), __ldg(src + 2), __ldg(src + 3));
        } else {
            load_words_slow(wi, r);
        }
    };
    auto make_window = [&](const uint4 &r, uint32_t bit, uint32_t &w0, uint32_t &w1, uint32_t &w2) {
        const uint32_t a = __byte_perm(r.x, 0, 0x0123), b = __byte_perm(r.y, 0, 0x0123);
        const uint32_t c = __byte_perm(r.z, 0, 0x0123), d = __byte_perm(r.w, 0, 0x0123);
        w0 = __funnelshift_l(b, a, bit);
        w1 = __funnelshift_l(c, b, bit);
        w2 = __funnelshift_l(d, c, bit);
    };

    // A task is one chunk of 32 groups.  Whole-unit decode: task t is chunk t and writes where it
    // reads.  Range decode (chunk_count > 0): task t is chunk chunk_first + t and writes to the t-th
    // chunk of the output.  Row-wise decode (ROWS): task t is chunk t % chunks_per_row of row
    // rows[t / chunks_per_row] and writes to the t-th chunk of the output.
    const uint32_t n_tasks = ROWS ? p.n_tasks : (p.chunk_count ? p.chunk_count : (uint32_t)p.n_chunks);
    const uint32_t n_elements = (uint32_t)p.n_elements;  // the host side rejects units too close to 2^32
    const uint32_t warps = gridDim.x * (kFastThreads / 32);
    auto chunk_of = [&](uint32_t task) -> uint32_t {
        if (!ROWS) return task + p.chunk_first;
        const uint32_t r = task / p.chunks_per_row;
        int64_t row = __ldg(p.rows + r);
        if (row < 0 || row >= (int64_t)p.n_rows_total) {
            bad |= DF11_STATUS_BAD_POSITIONS;  // an index outside the table: decode row 0 instead
            row = 0;
        }
        return (uint32_t)row * p.chunks_per_row + (task - r * p.chunks_per_row);
    };

    // What a task needs before it can run: where its first code starts, the stream words
    // there and its first sixteen sign/mantissa bytes.  Loaded one task ahead.
    struct Inputs {
        uint32_t wi, bit, chunk;
        uint4 words, sm;
    };
    // Stage 1 of the pipeline: the raw seek point of a chunk (16 low bits per group, the high
    // part once per 32 groups).  Stage 2: stream word / bit of every lane, then the loads.
    auto load_seek = [&](uint32_t chunk, uint32_t &lo, uint32_t &hi) {
        lo = (uint32_t)__ldg(p.sync_lo + chunk * 32u + lane);  // padded to 32 per chunk: always readable
        hi = __ldg(p.sync_hi + chunk);
    };
    auto issue_inputs = [&](uint32_t chunk, uint32_t lo, uint32_t hi, Inputs &in) {
        const uint32_t lo0 = __shfl_sync(0xffffffffu, lo, 0);
        if (lo < lo0) lo += 65536u;
        in.wi = (hi << 11) + (lo >> 5);  // (hi << 16 | lo) >> 5
        in.bit = lo & 31u;
        in.chunk = chunk;
        const uint32_t first = (chunk * 32u + lane) * EPT;
        if (first < n_elements) {
            load_words(in.wi, in.words);
            if (vec && n_elements - first >= 16u) in.sm = __ldg(reinterpret_cast<const uint4 *>(p.sm + first));
        }
    };

    uint32_t task = blockIdx.x * (kFastThreads / 32) + (tid >> 5);

    // Whole-unit and range decode of aligned tensors: every chunk but the last two of the unit takes
    // the lean loop (such a chunk is full, and at least 512 further codes, 16 stream words or more,
    // follow it).
    if (!ROWS && vec && n_words >= 4u && p.n_chunks > 2 && p.chunk_first + 2u < (uint32_t)p.n_chunks) {
        const uint32_t n_lean = min(n_tasks, (uint32_t)p.n_chunks - 2u - p.chunk_first);
        const uint32_t mine = task < n_lean ? (n_lean - 1u - task) / warps + 1u : 0u;  // this warp's lean tasks
        const uint32_t task0 = task, chunk0 = task + p.chunk_first;
        lean_tasks<K, EPT, false>(
            p, tab, lane, mine, [&](uint32_t j) { return chunk0 + j * warps; }, n_words, bad,
            [&](uint32_t j, uint32_t part, uint32_t e0, uint32_t e1, uint32_t e2, uint32_t e3, const uint4 &m) {
                uint4 r0, r1;
                df11_merge4(e0, m.x, &r0.x, &r0.y);
                df11_merge4(e1, m.y, &r0.z, &r0.w);
                df11_merge4(e2, m.z, &r1.x, &r1.y);
                df11_merge4(e3, m.w, &r1.z, &r1.w);
                uint4 *dst = reinterpret_cast<uint4 *>(p.out) +
                             ((task0 + j * warps) * 32u + lane) * (EPT / 8) + 2u * part;
                if (wide) {
                    stg256(dst, r0, r1);
                } else {
                    dst[0] = r0;
                    dst[1] = r1;
                }
            });
        task += mine * warps;  // this warp's first task after them
    }

    // General loop: what the lean loop left (the last chunks), row-wise decode, unaligned tensors.
    Inputs cur = {0, 0, 0, make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
    uint32_t lo_next = 0, hi_next = 0, chunk_next = 0;
    if (task < n_tasks) {
        uint32_t lo, hi;
        const uint32_t chunk = chunk_of(task);
        load_seek(chunk, lo, hi);
        issue_inputs(chunk, lo, hi, cur);
        if (task + warps < n_tasks) {
            chunk_next = chunk_of(task + warps);
            load_seek(chunk_next, lo_next, hi_next);
        }
    }
    for (; task < n_tasks; task += warps) {
        // keep the pipeline full: inputs of the next task, seek point of the one after it
        Inputs nxt = {0, 0, 0, make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
        if (task + warps < n_tasks) {
            issue_inputs(chunk_next, lo_next, hi_next, nxt);
            if (task + 2u * warps < n_tasks) {
                chunk_next = chunk_of(task + 2u * warps);
                load_seek(chunk_next, lo_next, hi_next);
            }
        }

        uint32_t first = (cur.chunk * 32u + lane) * EPT;  // the element my next code decodes to
        // where it goes: its own place, or (row-wise) the matching place of the gathered output
        const uint32_t shift = (task * 32u + lane) * EPT - first;  // 0 for whole-unit decode
        uint32_t wi = cur.wi, bit = cur.bit;
        uint32_t acc = 0;  // see kFastEscape
        ExpShift X = {0, 0, 0, 0, 0};
#pragma unroll
        for (int part = 0; part < EPT / 16; ++part, first += 16u) {
            if (first >= n_elements) break;
            const bool whole = n_elements - first >= 16u;
            uint4 m = cur.sm;
            // 96-bit window whose top bit is my next code.  A later part continues where the
            // previous one stopped: codes it decoded beyond its sixteenth are at the top of X.
            uint32_t w0, w1, w2;
            if (part == 0) {
                make_window(cur.words, bit, w0, w1, w2);
            } else {
                if (whole && vec) m = __ldg(reinterpret_cast<const uint4 *>(p.sm + first));
                const uint32_t at = bit + (acc & 0x7Fu);
                wi += at >> 5;
                bit = at & 31u;
                acc = (acc & ~0xFFu) - kFastDone;
                uint4 r;
                load_words(wi, r);
                make_window(r, bit, w0, w1, w2);
            }
            for (;;) {
                if ((acc & kFastLeave) == 0u) probe_loop<K>(acc, X, w0, w1, w2, tab.dec_addr);
                if ((acc & (kFastEscape | 64u)) == 0u) break;  // 16 codes done, nothing special
                if (acc & kFastEscape) {
                    // the table could not resolve this code from K bits: full walk for one symbol
                    acc -= kFastEscape;
                    uint32_t len;
                    int tbad = 0;
                    const uint32_t sym = df11_walk_m(tab, p.n_luts, w0, &len, &tbad);
                    if (tbad) bad |= DF11_STATUS_BAD_TABLE;
                    X.push(sym, 8u);
                    acc += len | (8u << 16);
                    if (len < 32u) {  // window <<= len
                        w0 = __funnelshift_l(w1, w0, len);
                        w1 = __funnelshift_l(w2, w1, len);
                        w2 <<= len;
                    } else {          // a 32-bit code, or an unusable table (len 64): the reload below follows
                        w0 = w1, w1 = w2, w2 = 0;
                    }
                }
                if (acc & kFastDone) break;  // 16 codes done (the position may be past 63)
                if (acc & 64u) {
                    // position 64..127: reload the window at the code the position has reached
                    const uint32_t at = bit + (acc & 0x7Fu);
                    wi += at >> 5;
                    bit = at & 31u;
                    uint4 r;
                    load_words(wi, r);
                    make_window(r, bit, w0, w1, w2);
                    acc &= ~0xFFu;
                }
            }

            uint32_t e0, e1, e2, e3;
            X.take(acc, &e0, &e1, &e2, &e3);
            if (whole && vec) {
                uint4 r0, r1;
                df11_merge4(e0, m.x, &r0.x, &r0.y);
                df11_merge4(e1, m.y, &r0.z, &r0.w);
                df11_merge4(e2, m.z, &r1.x, &r1.y);
                df11_merge4(e3, m.w, &r1.z, &r1.w);
                uint4 *dst = reinterpret_cast<uint4 *>(p.out + (first + shift));
                dst[0] = r0;
                dst[1] = r1;
            } else {  // the last, partial piece of the unit, or unaligned tensors
                const uint32_t e[4] = {e0, e1, e2, e3};
                for (uint32_t k = 0; k < 16u && first + k < n_elements; ++k)
                    p.out[first + shift + k] =
                        df11_merge1((e[k >> 2] >> (8u * (k & 3u))) & 255u, __ldg(p.sm + first + k));
            }
        }
        cur = nxt;
    }
    if (bad && p.status != nullptr) atomicOr(p.status, bad);
}

// ---------------------------------------------------------------------------------------
// Decode fused with a matrix-vector product (behind df11_gemv_prepared): y = W x for one
// [n_rows, in_features] matrix that lies inside a unit, for up to four activation vectors,
// without ever writing W.  Batch-1 generation is bound by memory traffic: decode-then-GEMV
// reads the compressed weights, writes 2 bytes per weight and reads them again; this reads
// the compressed weights only.
//
// A work item is a run of consecutive 512-element chunks of one row (1, 2, 4 or 8 of them,
// chosen per launch: as long as the items still spread evenly over the warps); items go
// round the warps, so the work is balanced whatever the matrix shape.  A lane multiplies its
// sixteen decoded weights with the sixteen activations of the same columns (bf16 x bf16
// products are exact in fp32; fp32 accumulation) and keeps the sum over the run; at the end
// of a run the warp adds its 32 lanes up.  A run that is a whole row is the output: bias,
// one rounding to bf16, stored.  Otherwise the run's sum is stored and a second, small
// kernel adds each row's sums in order.  Either way the result does not depend on timing.
// ---------------------------------------------------------------------------------------
struct GemvArgs {
    const uint16_t *x;     // [m][in_features] bf16
    uint16_t *y;           // [m][n_rows] bf16
    const uint16_t *bias;  // [n_rows] bf16, or null
    float *partial;        // [m][runs per row][n_rows]
    uint32_t first_chunk, chunks_per_row, n_rows;
    uint32_t run_log;      // a work item is 1 << run_log consecutive chunks of a row
};

__device__ __forceinline__ float bf16_dot2(uint32_t w, uint32_t x, float acc)
{
    asm("{\n\t"
        ".reg .b16 wl, wh, xl, xh;\n\t"
        "mov.b32 {wl, wh}, %1;\n\t"
        "mov.b32 {xl, xh}, %2;\n\t"
        "fma.rn.f32.bf16 %0, wl, xl, %0;\n\t"
        "fma.rn.f32.bf16 %0, wh, xh, %0;\n\t"
        "}"
        : "+f"(acc)
        : "r"(w), "r"(x));
    return acc;
}

__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }

__device__ __forceinline__ uint16_t float_to_bf16_bits(float f)  // round to nearest even; NaN stays NaN
{
    uint32_t u = __float_as_uint(f);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40u);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

template <int K, int EPT, int M, bool CHECKED>
__global__ void __launch_bounds__(kGemvThreads, DF11_GEMV_MIN_CTAS) df11_gemv_kernel(const Params p, const GemvArgs g)
{
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t smem_addr = (uint32_t)__cvta_generic_to_shared(smem);
    constexpr uint32_t luts_off = 8u << K;
    const uint32_t tid = threadIdx.x, lane = tid & 31u;
    {
        const uint4 *src = reinterpret_cast<const uint4 *>(p.table_g);
        uint4 *dst = reinterpret_cast<uint4 *>(smem);
        for (int i = tid; i < (1 << K) / 2; i += kGemvThreads) dst[i] = __ldg(src + i);
        for (int i = tid; i < p.n_luts * 256; i += kGemvThreads) smem[luts_off + i] = __ldg(p.luts + i);
    }
    __syncthreads();
    // Tables, seek points, stream and sign/mantissa bytes belong to the unit and may be read while
    // the kernel ahead in the stream still runs; the activations are its result, and the scratch
    // and the output may still be in use by it: the sink waits before it touches any of them.
    grid_launch_dependents();
    bool waited = false;
    FastTables tab;
    tab.dec_addr = smem_addr;
    tab.luts_addr = smem_addr + luts_off;

    // Work items are runs of `run` consecutive chunks of one row (run = 1 << run_log divides
    // chunks_per_row); items go round the warps.  A lane keeps its products of a run in a
    // register, so the warp adds its 32 lanes up once per run, not once per chunk.
    const uint32_t n_words = (uint32_t)(p.n_bytes >> 2);
    const uint32_t warps = gridDim.x * (kGemvThreads / 32);
    const uint32_t gw = blockIdx.x * (kGemvThreads / 32) + (tid >> 5);
    const uint32_t cpr = g.chunks_per_row, run_log = g.run_log, run = 1u << run_log;
    const uint32_t parts = cpr >> run_log;  // runs per row
    const uint32_t n_items = g.n_rows * parts;
    const uint32_t my_items = gw < n_items ? (n_items - 1u - gw) / warps + 1u : 0u;
    constexpr uint32_t chunk_elems = 32u * EPT;
    const uint32_t in_features = cpr * chunk_elems;
    const uint32_t step_rows = warps / parts, step_parts = warps - step_rows * parts;
    uint32_t row = gw / parts, part = gw - row * parts;  // of the item the sink is in
    int bad = 0;
    float sum[M];
#pragma unroll
    for (int m = 0; m < M; ++m) sum[m] = 0.f;

    lean_tasks<K, EPT, CHECKED>(
        p, tab, lane, my_items << run_log,
        [&](uint32_t j) { return g.first_chunk + ((gw + (j >> run_log) * warps) << run_log) + (j & (run - 1u)); },
        n_words, bad,
        [&](uint32_t j, uint32_t half, uint32_t e0, uint32_t e1, uint32_t e2, uint32_t e3, const uint4 &sm) {
            if (!waited) {
                grid_dependency_wait();
                waited = true;
            }
            uint32_t w[8];
            df11_merge4(e0, sm.x, &w[0], &w[1]);
            df11_merge4(e1, sm.y, &w[2], &w[3]);
            df11_merge4(e2, sm.z, &w[4], &w[5]);
            df11_merge4(e3, sm.w, &w[6], &w[7]);
            const uint32_t sub = j & (run - 1u);
            const uint32_t column = ((part << run_log) + sub) * chunk_elems + EPT * lane + 16u * half;
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const uint4 *xp = reinterpret_cast<const uint4 *>(g.x + (size_t)m * in_features + column);
                const uint4 xa = __ldg(xp), xb = __ldg(xp + 1);
                float s0 = sum[m], s1 = 0.f;
                s0 = bf16_dot2(w[0], xa.x, s0);
                s1 = bf16_dot2(w[1], xa.y, s1);
                s0 = bf16_dot2(w[2], xa.z, s0);
                s1 = bf16_dot2(w[3], xa.w, s1);
                s0 = bf16_dot2(w[4], xb.x, s0);
                s1 = bf16_dot2(w[5], xb.y, s1);
                s0 = bf16_dot2(w[6], xb.z, s0);
                s1 = bf16_dot2(w[7], xb.w, s1);
                sum[m] = s0 + s1;
            }
            if (half != EPT / 16 - 1 || sub != run - 1u) return;
            // end of the run: add the lanes up; a run that is a whole row gives the output itself
#pragma unroll
            for (int m = 0; m < M; ++m) {
                float t = sum[m];
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) t += __shfl_xor_sync(0xffffffffu, t, d);
                if (lane == 0) {
                    if (parts == 1u) {
                        if (g.bias) t += bf16_bits_to_float(g.bias[row]);
                        g.y[(size_t)m * g.n_rows + row] = float_to_bf16_bits(t);
                    } else {
                        g.partial[((size_t)m * parts + part) * g.n_rows + row] = t;
                    }
                }
                sum[m] = 0.f;
            }
            row += step_rows;
            part += step_parts;
            if (part >= parts) part -= parts, ++row;
        });
    if (bad && p.status != nullptr) atomicOr(p.status, bad);
}

// One thread per output: the row's partial sums in order, bias, one rounding to bf16.
__global__ void __launch_bounds__(256) df11_gemv_finish_kernel(const GemvArgs g, int m_count)
{
    grid_dependency_wait();
    const uint32_t i = blockIdx.x * 256u + threadIdx.x;
    if (i >= g.n_rows * (uint32_t)m_count) return;
    const uint32_t m = i / g.n_rows, row = i - m * g.n_rows;
    const uint32_t parts = g.chunks_per_row >> g.run_log;
    const float *part = g.partial + (size_t)m * parts * g.n_rows + row;
    float total = 0.f;
    for (uint32_t k = 0; k < parts; ++k) total += part[(size_t)k * g.n_rows];
    if (g.bias) total += bf16_bits_to_float(g.bias[row]);
    g.y[i] = float_to_bf16_bits(total);
}

// ---------------------------------------------------------------------------------------
// Self-contained decode kernel (behind df11_decode): count pass + scan + decode pass per block.
//
// Shared memory (byte offsets from the dynamic shared base):
//   [0, 8<<K)               decode table
//   [.., +4<<K)             count table
//   2 input buffers         each: 4112 stream bytes, then the block's 320 gap bytes
//   stage                   exponent bytes of the current block
//   tile                    sign/mantissa bytes of the current block
//   3 mbarriers, luts, agree, wsum
// ---------------------------------------------------------------------------------------
template <int K>
struct Layout {
    static constexpr uint32_t dec = 0;
    static constexpr uint32_t cnt = 8u << K;
    static constexpr uint32_t in0 = cnt + (4u << K);
    static constexpr uint32_t stage = in0 + 2u * kInBufBytes;
};

template <int K>
__global__ void __launch_bounds__(kThreads, 3) df11_decode_kernel(const Params p)
{
    extern __shared__ __align__(16) uint8_t smem[];
    using L = Layout<K>;
    const uint32_t smem_addr = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t tile_off = L::stage + p.stage_bytes;
    const uint32_t bars_off = tile_off + p.stage_bytes;
    uint8_t *luts_s = smem + bars_off + 32;
    uint8_t *agree = luts_s + p.n_luts * 256;
    uint32_t *wsum = reinterpret_cast<uint32_t *>(agree + 256);

    SmemPolicy mem;
    mem.dec_addr = smem_addr + L::dec;
    mem.cnt_addr = smem_addr + L::cnt;
    mem.stage_addr = smem_addr + L::stage;
    mem.luts_addr = smem_addr + bars_off + 32;
    const uint32_t tile_addr = smem_addr + tile_off;
    const uint32_t bar_in = smem_addr + bars_off;       // two barriers, 8 bytes apart
    const uint32_t bar_sm = smem_addr + bars_off + 16;

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    int bad = 0;

    // ---- once per CTA --------------------------------------------------------------------
    if (tid == 0) {
        mbar_init(bar_in, 1);
        mbar_init(bar_in + 8, 1);
        mbar_init(bar_sm, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = tid; i < p.n_luts * 256; i += kThreads) luts_s[i] = __ldg(p.luts + i);
    __syncthreads();
    build_tables_smem(p, luts_s, agree, reinterpret_cast<Df11Entry *>(smem + L::dec),
                      reinterpret_cast<uint32_t *>(smem + L::cnt), K, tid);
    __syncthreads();

    // A block's stream bytes come by bulk copy when all 4112 of them exist and are aligned.
    auto streamed = [&](int64_t b) {
        return (p.codes_aligned & 1) && (b + 1) * (int64_t)DF11_BLOCK_BYTES + 16 <= p.n_bytes;
    };
    // Producer (thread 0): bulk copies of block b's inputs into input buffer `buf`.
    const bool side_streamed = (p.codes_aligned & 2) != 0;  // gap bytes by bulk copy when aligned
    auto issue_inputs = [&](int64_t b, uint32_t buf) {
        const uint32_t dst = smem_addr + L::in0 + buf * kInBufBytes;
        const uint32_t bar = bar_in + 8 * buf;
        const bool with_codes = streamed(b);
        const uint32_t total = (with_codes ? kCodesBufBytes : 0) + (side_streamed ? DF11_GAP_BYTES_PER_BLOCK : 0);
        if (total == 0) {
            mbar_arrive(bar);
            return;
        }
        mbar_expect_tx(bar, total);
        if (b == p.drop_block) return;  // self-test: bytes announced, nothing issued, nothing in flight
        if (with_codes) bulk_g2s(dst, p.codes + b * DF11_BLOCK_BYTES, kCodesBufBytes, bar);
        if (side_streamed)
            bulk_g2s(dst + kCodesBufBytes, p.gaps + b * DF11_GAP_BYTES_PER_BLOCK, DF11_GAP_BYTES_PER_BLOCK, bar);
    };
    const uint64_t wait_ns = p.wait_ns ? p.wait_ns : kWaitNs;
    uint32_t n_in[2] = {0, 0}, n_sm = 0;  // copies announced per barrier so far (uniform over the CTA)

    if ((int64_t)blockIdx.x < p.n_blocks) {
        if (tid == 0) issue_inputs(blockIdx.x, 0);
        ++n_in[0];
    }

    uint32_t it = 0;
    for (int64_t b = blockIdx.x; b < p.n_blocks; b += gridDim.x, ++it) {
        const uint32_t cur = it & 1u;
        const uint32_t in_addr = smem_addr + L::in0 + cur * kInBufBytes;

        // next block's inputs start flowing into the other buffer (all its readers passed
        // the barrier that ended the previous iteration)
        if (b + gridDim.x < p.n_blocks) {
            if (tid == 0) issue_inputs(b + gridDim.x, cur ^ 1u);
            ++n_in[cur ^ 1u];
        }

        // A wait that runs out: this thread goes through the block on whatever its buffer holds
        // (every index below is clamped) and the CTA leaves the loop at the block's last barrier.
        if (!mbar_wait(bar_in + 8 * cur, (it >> 1) & 1u, wait_ns)) bad |= DF11_STATUS_TIMEOUT;

        // ---- block bookkeeping (uniform) ---------------------------------------------------
        const int64_t base = (int64_t)__ldg(p.pos + b);
        const int64_t next = (int64_t)__ldg(p.pos + b + 1);
        int64_t c = next - base;
        if (c < 0 || next > p.n_elements) {
            bad |= DF11_STATUS_BAD_POSITIONS;
            c = c < 0 ? 0 : p.n_elements - base;
            if (c < 0) c = 0;
        }
        const uint32_t phase = (uint32_t)(base & 15);
        if (c + phase > p.stage_bytes - 16) {
            bad |= DF11_STATUS_TRUNCATED;
            c = p.stage_bytes - 16 - phase;
        }
        const uint32_t block_cnt = (uint32_t)c;
        const uint32_t last = phase + block_cnt;  // one past the last staging byte in use
        const int64_t gbase = base - phase;       // multiple of 16
        const uint8_t *sm_blk = p.sm + gbase;

        // ---- sign/mantissa tile of this block: bulk copy, overlapped with the decode --------
        // Whole 16-byte pieces that lie inside the tensor come by TMA; a ragged end (only at
        // the very end of the unit) or an unaligned tensor is fetched with plain loads.
        uint32_t tma_bytes = 0;
        if (p.sm_aligned && block_cnt > 0) {  // then base < n_elements, so `avail` is not negative
            const int64_t avail = (p.n_elements - gbase) & ~(int64_t)15;
            const uint32_t want = (last + 15u) & ~15u;
            tma_bytes = (int64_t)want <= avail ? want : (uint32_t)avail;
        }
        if (tid == 0) {
            if (tma_bytes) {
                mbar_expect_tx(bar_sm, tma_bytes);
                bulk_g2s(tile_addr, sm_blk, tma_bytes, bar_sm);
            } else {
                mbar_arrive(bar_sm);
            }
        }
        ++n_sm;
        for (uint32_t i = max(tma_bytes, phase) + tid; i < last; i += kThreads)
            smem[tile_off + i] = __ldg(sm_blk + i);

        // ---- my window ------------------------------------------------------------------------
        uint32_t w0 = 0, w1 = 0, w2 = 0;
        bool live = true;
        if (streamed(b)) {
            const uint2 v = lds64(in_addr + 8u * tid);
            w0 = __byte_perm(v.x, 0, 0x0123);
            w1 = __byte_perm(v.y, 0, 0x0123);
            w2 = __byte_perm(lds32(in_addr + 8u * tid + 8u), 0, 0x0123);
        } else {
            const int64_t off = b * DF11_BLOCK_BYTES + (int64_t)tid * DF11_WINDOW_BYTES;
            live = off < p.n_bytes;
            if (live) {
                const uint3 v = load_window_slow(p.codes, p.n_bytes, off);
                w0 = v.x, w1 = v.y, w2 = v.z;
            }
        }

        uint32_t gap;
        if (side_streamed) {
            gap = block_gap([&](uint32_t j) { return lds8(in_addr + kCodesBufBytes + j); }, tid);
        } else {
            const uint8_t *g = p.gaps + b * DF11_GAP_BYTES_PER_BLOCK;
            gap = block_gap([&](uint32_t j) { return (uint32_t)__ldg(g + j); }, tid);
        }
        int cbad = 0;
        const uint32_t cnt = df11_count_window<K>(mem, p.n_luts, w0, w1, w2, live ? gap : 64u, &cbad);
        if (cbad) bad |= DF11_STATUS_BAD_TABLE;
        uint32_t o = block_scan(cnt, wsum, lane, warp);
        uint32_t end = o + cnt;

        // clamp to what this block may write, then shift by the block's alignment phase
        o = min(o, block_cnt) + phase;
        end = min(end, block_cnt) + phase;
        {
            int tbad = 0;
            df11_decode_window<K>(mem, p.n_luts, w0, w1, w2, gap, o, end, &tbad);
            if (tbad) bad |= DF11_STATUS_BAD_TABLE;
        }
        __syncthreads();
        if (!mbar_wait(bar_sm, it & 1u, (bad & DF11_STATUS_TIMEOUT) ? 0ull : wait_ns)) bad |= DF11_STATUS_TIMEOUT;

        // ---- merge with sign/mantissa ------------------------------------------------------------
        // Groups of eight elements aligned to eight in the output: group g covers staging and tile
        // bytes [8g, 8g+8).  Complete groups: two 8-byte shared loads, one 16-byte global store.
        uint16_t *out_blk = p.out + gbase;
        if (p.out_aligned) {
            const uint32_t g_lo = (phase + 7u) >> 3, g_hi = last >> 3;
            for (uint32_t g = g_lo + tid; g < g_hi; g += kThreads) {
                const uint2 ex = lds64(mem.stage_addr + 8u * g);
                const uint2 m = lds64(tile_addr + 8u * g);
                uint4 r;
                df11_merge4(ex.x, m.x, &r.x, &r.y);
                df11_merge4(ex.y, m.y, &r.z, &r.w);
                reinterpret_cast<uint4 *>(out_blk)[g] = r;
            }
            // elements of the (at most two) incomplete groups at either end, one per thread
            if (tid < 16u) {
                const uint32_t i = tid < 8u ? 8u * (g_lo - 1u) + tid : 8u * g_hi + (tid - 8u);
                const bool mine = tid < 8u ? ((phase & 7u) != 0u && i >= phase && i < last)
                                           : (g_hi >= g_lo && i < last);
                if (mine) out_blk[i] = df11_merge1(lds8(mem.stage_addr + i), lds8(tile_addr + i));
            }
        } else {
            for (uint32_t i = phase + tid; i < last; i += kThreads)
                out_blk[i] = df11_merge1(lds8(mem.stage_addr + i), lds8(tile_addr + i));
        }
        // staging, tile, wsum and this input buffer are reused; and if any thread's wait ran out the
        // CTA stops here: its remaining blocks stay undecoded, the status word says so
        if (__syncthreads_or(bad & DF11_STATUS_TIMEOUT)) break;
    }

    // Never retire with a copy still on its way into this CTA's shared memory: the thread that
    // issued the copies waits (bounded) for the last phase announced on each barrier.  After a
    // normal run all of them completed long ago and this costs three polls.
    if (tid == 0) {
        const uint64_t drain_ns = p.wait_ns ? p.wait_ns : kDrainNs;
        bool drained = true;
        if (n_in[0]) drained &= mbar_wait(bar_in, (n_in[0] - 1u) & 1u, drain_ns);
        if (n_in[1]) drained &= mbar_wait(bar_in + 8, (n_in[1] - 1u) & 1u, drain_ns);
        if (n_sm) drained &= mbar_wait(bar_sm, (n_sm - 1u) & 1u, drain_ns);
        if (!drained) bad |= DF11_STATUS_TIMEOUT;
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
bool g_attr_set[64][24] = {};

struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int device)
    {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != device) {
            changed = true;
            if (cudaSetDevice(device) != cudaSuccess) ok = false;
        }
    }
    ~DeviceGuard()
    {
        if (prev >= 0 && changed) cudaSetDevice(prev);
    }
    bool changed = false;
};

// CTAs per SM of a kernel for a given shared-memory size, asked once per device and kernel slot
// (and again when the size changes): the query costs more host time than the launch itself.
struct OccupancyCache {
    size_t smem = ~(size_t)0;
    int per_sm = 0;
};
OccupancyCache g_occupancy[64][24];

template <class Kernel>
int ctas_per_sm(Kernel kernel, int device, int slot, int threads, size_t smem, int *per_sm)
{
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (g_occupancy[device][slot].smem == smem) {
            *per_sm = g_occupancy[device][slot].per_sm;
            return DF11_OK;
        }
    }
    int n = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, smem);
    if (e != cudaSuccess || n < 1)
        return df11_fail(DF11_ERR_CUDA, "occupancy query failed (%s, %d CTAs/SM)", cudaGetErrorString(e), n);
    std::lock_guard<std::mutex> lock(g_mutex);
    g_occupancy[device][slot].smem = smem;
    g_occupancy[device][slot].per_sm = n;
    *per_sm = n;
    return DF11_OK;
}

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

template <class Kernel>
int launch(Kernel kernel, int threads, int slot, size_t smem, int64_t work_items, const Params &p, int device,
           cudaStream_t stream, int max_ctas_per_sm = 0)
{
    DeviceInfo info;
    int rc = device_info(device, &info);
    if (rc != DF11_OK) return rc;
    DeviceGuard guard(device);
    if (!guard.ok) return df11_fail(DF11_ERR_CUDA, "cudaSetDevice(%d) failed", device);
    if (smem > (size_t)info.max_smem_optin)
        return df11_fail(DF11_ERR_BADARG, "needs %zu bytes of shared memory, device allows %d", smem,
                         info.max_smem_optin);
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (!g_attr_set[device][slot]) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 info.max_smem_optin);
            if (e != cudaSuccess)
                return df11_fail(DF11_ERR_CUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
            g_attr_set[device][slot] = true;
        }
    }
    int per_sm = 0;
    rc = ctas_per_sm(kernel, device, slot, threads, smem, &per_sm);
    if (rc != DF11_OK) return rc;
    cudaError_t e;
    if (max_ctas_per_sm > 0 && per_sm > max_ctas_per_sm) per_sm = max_ctas_per_sm;  // leave room for other kernels
    int64_t grid = (int64_t)info.sm_count * per_sm;
    if (grid > work_items) grid = work_items;
    if (grid < 1) grid = 1;
    kernel<<<(unsigned)grid, threads, smem, stream>>>(p);
    e = cudaGetLastError();
    if (e != cudaSuccess) return df11_fail(DF11_ERR_CUDA, "kernel launch failed: %s", cudaGetErrorString(e));
    return DF11_OK;
}

// The same for the fused product kernels, which take a second argument block.
template <class Kernel>
int launch_gemv(Kernel kernel, int slot, int m_count, size_t smem, int64_t work_items, const Params &p,
                const GemvArgs &g, int device, cudaStream_t stream)
{
    DeviceInfo info;
    int rc = device_info(device, &info);
    if (rc != DF11_OK) return rc;
    DeviceGuard guard(device);
    if (!guard.ok) return df11_fail(DF11_ERR_CUDA, "cudaSetDevice(%d) failed", device);
    if (smem > (size_t)info.max_smem_optin)
        return df11_fail(DF11_ERR_BADARG, "needs %zu bytes of shared memory, device allows %d", smem,
                         info.max_smem_optin);
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (!g_attr_set[device][slot]) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 info.max_smem_optin);
            if (e != cudaSuccess)
                return df11_fail(DF11_ERR_CUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
            g_attr_set[device][slot] = true;
        }
    }
    int per_sm = 0;
    rc = ctas_per_sm(kernel, device, slot, kGemvThreads, smem, &per_sm);
    if (rc != DF11_OK) return rc;
    cudaError_t e;
    int64_t grid = (int64_t)info.sm_count * per_sm;
    if (grid > work_items) grid = work_items;
    if (grid < 1) grid = 1;
    // Longest run (8, 4, 2, 1 chunks, dividing the row) that keeps the warps busy: either there
    // are no more items than resident warps (then the grid shrinks to one item per warp: no
    // partly filled last round), or the items fill the warps' rounds to 85 %.
    GemvArgs args = g;
    const int64_t warps = grid * (kGemvThreads / 32);
    args.run_log = 0;
    for (int log = 3; log >= 0; --log) {
        if (g.chunks_per_row % (1u << log)) continue;
        const int64_t items = (int64_t)g.n_rows * (g.chunks_per_row >> log);
        if (items <= warps) {
            args.run_log = (uint32_t)log;
            grid = (items + kGemvThreads / 32 - 1) / (kGemvThreads / 32);
            break;
        }
        const int64_t rounds = (items + warps - 1) / warps;
        if (log == 0 || items * 100 >= rounds * warps * 85) {
            args.run_log = (uint32_t)log;
            break;
        }
    }
    // Both kernels may start while the kernel ahead of them in the stream drains: the first
    // loads its tables meanwhile, the second is in place when the first ends.
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kGemvThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, kernel, p, args);
    if (e == cudaSuccess && (g.chunks_per_row >> args.run_log) > 1u) {
        const unsigned outputs = g.n_rows * (unsigned)m_count;
        cfg.gridDim = dim3((outputs + 255u) / 256u);
        cfg.blockDim = dim3(256);
        cfg.dynamicSmemBytes = 0;
        e = cudaLaunchKernelEx(&cfg, df11_gemv_finish_kernel, args, m_count);
    }
    if (e != cudaSuccess) return df11_fail(DF11_ERR_CUDA, "kernel launch failed: %s", cudaGetErrorString(e));
    return DF11_OK;
}

size_t small_tables_bytes(int n_luts) { return (size_t)n_luts * 256 + 256 + 32 * 4; }

int launch_decode(const Params &p, int device, cudaStream_t stream)
{
    const size_t smem = Layout<kTableBits>::stage + 2 * (size_t)p.stage_bytes + 32 + small_tables_bytes(p.n_luts);
    return launch(df11_decode_kernel<kTableBits>, kThreads, 0, smem, p.n_blocks, p, device, stream);
}

// Elements per seek point of the prepared form, process-wide: DF11_EPT in the environment (16 or
// 32) when the library is first used, else DF11_DEFAULT_EPT; df11_seek_interval() changes it.
#ifndef DF11_DEFAULT_EPT
#define DF11_DEFAULT_EPT 16
#endif
std::atomic<int> g_ept{0};
int elements_per_seek_point()
{
    int ept = g_ept.load(std::memory_order_relaxed);
    if (ept == 0) {
        const char *e = getenv("DF11_EPT");
        const int v = e ? atoi(e) : 0;
        ept = (v == 16 || v == 32) ? v : DF11_DEFAULT_EPT;
        g_ept.store(ept, std::memory_order_relaxed);
    }
    return ept;
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

// Shared staging: alignment phase (<= 15) + elements of the widest block, rounded up to whole
// 16-byte pieces, plus the 16 bytes the kernel keeps as a margin.
int stage_bytes_for(int32_t max_block_elems)
{
    int64_t m = max_block_elems > 0 ? max_block_elems : DF11_MAX_BLOCK_ELEMS;
    if (m > DF11_MAX_BLOCK_ELEMS) m = DF11_MAX_BLOCK_ELEMS;
    return (int)((m + 15 + 15) / 16 * 16) + 16;
}

constexpr int64_t kAuxTableBytes = (int64_t)sizeof(Df11Entry) << kFastTableBits;

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
    for (int v = threadIdx.x; v < (1 << kFastTableBits); v += blockDim.x) {
        Df11Entry e;
        uint32_t c;
        df11_build_entry(luts_s, n_luts, agree, (uint32_t)v, kFastTableBits, &e, &c);
        e.meta = fast_meta(e.meta);  // the prepared form's table is read by df11_fast_kernel only
        table[v] = e;
    }
}

Params base_params(const void *luts, const void *codes, const void *pos, const void *gaps, int32_t n_luts,
                   int64_t n_bytes, int64_t n_elements, void *status)
{
    Params p = {};
    p.luts = (const uint8_t *)luts;
    p.codes = (const uint8_t *)codes;
    p.pos = (const uint32_t *)pos;
    p.gaps = (const uint8_t *)gaps;
    p.status = (int *)status;
    p.n_bytes = n_bytes;
    p.n_elements = n_elements;
    p.n_blocks = (n_bytes + DF11_BLOCK_BYTES - 1) / DF11_BLOCK_BYTES;
    p.n_luts = n_luts;
    p.stage_bytes = 16;
    p.drop_block = -1;
    p.codes_aligned = (((uintptr_t)codes & 15) == 0 ? 1 : 0) | (((uintptr_t)gaps & 15) == 0 ? 2 : 0) |
                      (((uintptr_t)codes & 3) == 0 ? 4 : 0);
    return p;
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
    Params p = base_params(luts, codes, output_positions, gaps, n_luts, n_bytes, n_elements, status);
    p.sm = (const uint8_t *)sign_mantissa;
    p.out = (uint16_t *)out_bf16;
    p.stage_bytes = stage_bytes_for(max_block_elems);
    p.sm_aligned = (((uintptr_t)sign_mantissa & 15) == 0 ? 1 : 0) | (((uintptr_t)sign_mantissa & 31) == 0 ? 2 : 0);
    p.out_aligned = (((uintptr_t)out_bf16 & 15) == 0 ? 1 : 0) | (((uintptr_t)out_bf16 & 31) == 0 ? 2 : 0);
    return launch_decode(p, device, (cudaStream_t)stream);
}

extern "C" int df11_selftest_wait_timeout(const void *luts, const void *codes, const void *sign_mantissa,
                                          const void *output_positions, const void *gaps, void *out_bf16,
                                          int32_t n_luts, int64_t n_bytes, int64_t n_elements,
                                          int32_t max_block_elems, int64_t drop_block, void *status, int32_t device,
                                          void *stream)
{
    int rc = check_common(luts, codes, output_positions, gaps, n_luts, n_bytes, n_elements);
    if (rc != DF11_OK) return rc;
    if (!sign_mantissa || !out_bf16 || n_bytes == 0 || n_elements == 0)
        return df11_fail(DF11_ERR_BADARG, "the self-test needs a non-empty unit");
    Params p = base_params(luts, codes, output_positions, gaps, n_luts, n_bytes, n_elements, status);
    if (drop_block < 0 || drop_block >= p.n_blocks)
        return df11_fail(DF11_ERR_BADARG, "drop_block = %lld, the unit has %lld format blocks", (long long)drop_block,
                         (long long)p.n_blocks);
    p.sm = (const uint8_t *)sign_mantissa;
    p.out = (uint16_t *)out_bf16;
    p.stage_bytes = stage_bytes_for(max_block_elems);
    p.sm_aligned = (((uintptr_t)sign_mantissa & 15) == 0 ? 1 : 0) | (((uintptr_t)sign_mantissa & 31) == 0 ? 2 : 0);
    p.out_aligned = (((uintptr_t)out_bf16 & 15) == 0 ? 1 : 0) | (((uintptr_t)out_bf16 & 31) == 0 ? 2 : 0);
    if (!(p.codes_aligned & 1) && !(p.codes_aligned & 2))
        return df11_fail(DF11_ERR_BADARG, "the self-test needs 16-byte aligned tensors (no bulk copy otherwise)");
    p.drop_block = drop_block;
    p.wait_ns = 2ull * 1000 * 1000;  // 2 ms per wait: the CTA that owns the block gives up after ~4 ms
    return launch_decode(p, device, (cudaStream_t)stream);
}

namespace {
// Auxiliary buffer: decode table | seek points, high parts (uint32 per 32 groups, padded to 16
// bytes) | seek points, low parts (uint16 per group, 32 per chunk).
constexpr int64_t kMaxPreparedElements = 0xFFFFFFFFll - 32 * 32;  // group arithmetic is 32-bit
struct AuxLayout {
    int64_t n_chunks, hi_off, lo_off, total;
};
AuxLayout aux_layout(int64_t n_elements, int ept)
{
    AuxLayout a;
    const int64_t n_groups = (n_elements + ept - 1) / ept;
    a.n_chunks = (n_groups + 31) / 32;
    a.hi_off = kAuxTableBytes;
    a.lo_off = a.hi_off + (a.n_chunks * 4 + 15) / 16 * 16;
    a.total = a.lo_off + a.n_chunks * 64;
    return a;
}
}  // namespace

extern "C" int df11_seek_interval(int32_t elements)
{
    if (elements == 0) return elements_per_seek_point();
    if (elements != 16 && elements != 32)
        return df11_fail(DF11_ERR_BADARG, "a seek point every %d elements: 16 and 32 are supported", elements);
    g_ept.store(elements, std::memory_order_relaxed);
    return elements;
}

extern "C" int64_t df11_aux_bytes(int64_t n_bytes, int64_t n_elements)
{
    if (n_bytes < 0 || n_elements < 0) return df11_fail(DF11_ERR_BADARG, "negative size");
    return aux_layout(n_elements, elements_per_seek_point()).total;
}

extern "C" int df11_prepare(const void *luts, const void *codes, const void *output_positions,
                            const void *gaps, void *aux, int64_t aux_bytes, int32_t n_luts, int64_t n_bytes,
                            int64_t n_elements, void *status, int32_t device, void *stream)
{
    int rc = check_common(luts, codes, output_positions, gaps, n_luts, n_bytes, n_elements);
    if (rc != DF11_OK) return rc;
    if (!aux || ((uintptr_t)aux & 15)) return df11_fail(DF11_ERR_BADARG, "aux buffer is null or not 16-byte aligned");
    if (n_elements > kMaxPreparedElements)
        return df11_fail(DF11_ERR_BADARG, "the prepared form handles up to %lld elements per unit; use df11_decode",
                         (long long)kMaxPreparedElements);
    const int ept = elements_per_seek_point();
    const AuxLayout a = aux_layout(n_elements, ept);
    if (aux_bytes < a.total)
        return df11_fail(DF11_ERR_NOSPACE, "aux buffer holds %lld bytes, %lld needed", (long long)aux_bytes,
                         (long long)a.total);
    {
        DeviceGuard guard(device);
        if (!guard.ok) return df11_fail(DF11_ERR_CUDA, "cudaSetDevice(%d) failed", device);
        df11_table_kernel<<<1, 512, 0, (cudaStream_t)stream>>>((const uint8_t *)luts, n_luts, (Df11Entry *)aux);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return df11_fail(DF11_ERR_CUDA, "kernel launch failed: %s", cudaGetErrorString(e));
    }
    if (n_bytes == 0 || n_elements == 0) return DF11_OK;
    Params p = base_params(luts, codes, output_positions, gaps, n_luts, n_bytes, n_elements, status);
    p.sync_hi = (uint32_t *)((uint8_t *)aux + a.hi_off);
    p.sync_lo = (uint16_t *)((uint8_t *)aux + a.lo_off);
    p.n_chunks = a.n_chunks;
    p.ept = ept;
    const size_t smem = (4u << kTableBits) + small_tables_bytes(n_luts);
    return launch(df11_sync_kernel<kTableBits>, kThreads, 1, smem, p.n_blocks, p, device, (cudaStream_t)stream);
}

namespace {
// first_element / range_elements: which part of the unit to produce (range_elements < 0: all of
// it); `out_bf16` receives that part from its first element on.
int decode_prepared(const void *luts, const void *codes, const void *sign_mantissa, const void *output_positions,
                    const void *gaps, const void *aux, void *out_bf16, int32_t n_luts, int64_t n_bytes,
                    int64_t n_elements, void *status, int32_t device, void *stream, int max_ctas_per_sm,
                    int64_t first_element = 0, int64_t range_elements = -1)
{
    int rc = check_common(luts, codes, output_positions, gaps, n_luts, n_bytes, n_elements);
    if (rc != DF11_OK) return rc;
    if (n_bytes == 0 || n_elements == 0 || range_elements == 0) return DF11_OK;
    if (!sign_mantissa || !out_bf16 || !aux || ((uintptr_t)aux & 15))
        return df11_fail(DF11_ERR_BADARG, "null tensor pointer or misaligned aux buffer");
    if (n_elements > kMaxPreparedElements)
        return df11_fail(DF11_ERR_BADARG, "the prepared form handles up to %lld elements per unit; use df11_decode",
                         (long long)kMaxPreparedElements);
    const int ept = elements_per_seek_point();
    const AuxLayout a = aux_layout(n_elements, ept);
    Params p = base_params(luts, codes, output_positions, gaps, n_luts, n_bytes, n_elements, status);
    p.sm = (const uint8_t *)sign_mantissa;
    p.out = (uint16_t *)out_bf16;
    p.table_g = (const Df11Entry *)aux;
    p.sync_hi = (uint32_t *)((uint8_t *)aux + a.hi_off);
    p.sync_lo = (uint16_t *)((uint8_t *)aux + a.lo_off);
    p.n_chunks = a.n_chunks;
    p.ept = ept;
    p.sm_aligned = (((uintptr_t)sign_mantissa & 15) == 0 ? 1 : 0) | (((uintptr_t)sign_mantissa & 31) == 0 ? 2 : 0);
    p.out_aligned = (((uintptr_t)out_bf16 & 15) == 0 ? 1 : 0) | (((uintptr_t)out_bf16 & 31) == 0 ? 2 : 0);
    int64_t chunks = a.n_chunks;
    if (range_elements >= 0) {
        const int64_t chunk_elems = 32 * ept;
        const int64_t end = first_element + range_elements;
        if (first_element < 0 || end > n_elements || first_element % chunk_elems ||
            (end % chunk_elems && end != n_elements))
            return df11_fail(DF11_ERR_BADARG,
                             "range [%lld, %lld) of a unit of %lld elements: it must start on a multiple of %lld "
                             "elements and end on one or at the end of the unit",
                             (long long)first_element, (long long)end, (long long)n_elements, (long long)chunk_elems);
        p.chunk_first = (uint32_t)(first_element / chunk_elems);
        p.chunk_count = (uint32_t)((range_elements + chunk_elems - 1) / chunk_elems);
        chunks = p.chunk_count;
    }
    // work per CTA pass: one chunk (32 groups) per warp
    const int64_t cta_items = (chunks + kFastThreads / 32 - 1) / (kFastThreads / 32);
    const size_t smem = (8u << kFastTableBits) + (size_t)n_luts * 256;
    if (ept == 32)
        return launch(df11_fast_kernel<kFastTableBits, 32, false>, kFastThreads, 3, smem, cta_items, p, device,
                      (cudaStream_t)stream, max_ctas_per_sm);
    return launch(df11_fast_kernel<kFastTableBits, 16, false>, kFastThreads, 2, smem, cta_items, p, device,
                  (cudaStream_t)stream, max_ctas_per_sm);
}
}  // namespace

extern "C" int df11_decode_prepared(const void *luts, const void *codes, const void *sign_mantissa,
                                    const void *output_positions, const void *gaps, const void *aux,
                                    void *out_bf16, int32_t n_luts, int64_t n_bytes, int64_t n_elements,
                                    int32_t max_block_elems, void *status, int32_t device, void *stream)
{
    (void)max_block_elems;  // sizes the shared staging of df11_decode only
    return decode_prepared(luts, codes, sign_mantissa, output_positions, gaps, aux, out_bf16, n_luts, n_bytes,
                           n_elements, status, device, stream, 0);
}

extern "C" int df11_decode_prepared_shared(const void *luts, const void *codes, const void *sign_mantissa,
                                           const void *output_positions, const void *gaps, const void *aux,
                                           void *out_bf16, int32_t n_luts, int64_t n_bytes, int64_t n_elements,
                                           int32_t ctas_per_sm, void *status, int32_t device, void *stream)
{
    if (ctas_per_sm < 0) return df11_fail(DF11_ERR_BADARG, "ctas_per_sm = %d", ctas_per_sm);
    return decode_prepared(luts, codes, sign_mantissa, output_positions, gaps, aux, out_bf16, n_luts, n_bytes,
                           n_elements, status, device, stream, ctas_per_sm);
}

extern "C" int df11_decode_range_prepared(const void *luts, const void *codes, const void *sign_mantissa,
                                          const void *aux, int64_t first_element, int64_t range_elements,
                                          void *out_bf16, int32_t n_luts, int64_t n_bytes, int64_t n_elements,
                                          void *status, int32_t device, void *stream)
{
    if (range_elements < 0) return df11_fail(DF11_ERR_BADARG, "negative range length");
    // output_positions and gaps are not read by the fast decoder; any non-null pointer passes the check
    return decode_prepared(luts, codes, sign_mantissa, luts, luts, aux, out_bf16, n_luts, n_bytes, n_elements, status,
                           device, stream, 0, first_element, range_elements);
}

extern "C" int df11_decode_range_prepared_shared(const void *luts, const void *codes, const void *sign_mantissa,
                                                 const void *aux, int64_t first_element, int64_t range_elements,
                                                 void *out_bf16, int32_t n_luts, int64_t n_bytes, int64_t n_elements,
                                                 int32_t ctas_per_sm, void *status, int32_t device, void *stream)
{
    if (range_elements < 0) return df11_fail(DF11_ERR_BADARG, "negative range length");
    if (ctas_per_sm < 0) return df11_fail(DF11_ERR_BADARG, "ctas_per_sm = %d", ctas_per_sm);
    return decode_prepared(luts, codes, sign_mantissa, luts, luts, aux, out_bf16, n_luts, n_bytes, n_elements, status,
                           device, stream, ctas_per_sm, first_element, range_elements);
}

extern "C" int df11_decode_rows_prepared(const void *luts, const void *codes, const void *sign_mantissa,
                                         const void *aux, const void *rows, int64_t n_rows, int64_t row_elements,
                                         void *out_bf16, int32_t n_luts, int64_t n_bytes, int64_t n_elements,
                                         void *status, int32_t device, void *stream)
{
    // output_positions and gaps are not read by the fast decoder; any non-null pointer passes the check
    int rc = check_common(luts, codes, luts, luts, n_luts, n_bytes, n_elements);
    if (rc != DF11_OK) return rc;
    if (n_rows < 0 || row_elements <= 0) return df11_fail(DF11_ERR_BADARG, "bad row count or row length");
    if (n_rows == 0 || n_bytes == 0 || n_elements == 0) return DF11_OK;
    if (!sign_mantissa || !out_bf16 || !rows || !aux || ((uintptr_t)aux & 15))
        return df11_fail(DF11_ERR_BADARG, "null tensor pointer or misaligned aux buffer");
    if (n_elements > kMaxPreparedElements) return df11_fail(DF11_ERR_BADARG, "unit too large for the prepared form");
    const int ept = elements_per_seek_point();
    const int64_t chunk_elems = 32 * ept;
    if (row_elements % chunk_elems || n_elements % row_elements)
        return df11_fail(DF11_ERR_BADARG,
                         "row-wise decode needs rows of a multiple of %lld elements that tile the unit exactly "
                         "(row length %lld, unit %lld)",
                         (long long)chunk_elems, (long long)row_elements, (long long)n_elements);
    if (n_rows * (row_elements / chunk_elems) > 0x7FFFFFFFll || n_rows * row_elements > 0xFFFFFFFFll)
        return df11_fail(DF11_ERR_BADARG, "too many rows for one call");
    const AuxLayout a = aux_layout(n_elements, ept);
    Params p = base_params(luts, codes, luts, luts, n_luts, n_bytes, n_elements, status);
    p.sm = (const uint8_t *)sign_mantissa;
    p.out = (uint16_t *)out_bf16;
    p.table_g = (const Df11Entry *)aux;
    p.sync_hi = (uint32_t *)((uint8_t *)aux + a.hi_off);
    p.sync_lo = (uint16_t *)((uint8_t *)aux + a.lo_off);
    p.n_chunks = a.n_chunks;
    p.ept = ept;
    p.rows = (const int64_t *)rows;
    p.chunks_per_row = (uint32_t)(row_elements / chunk_elems);
    p.n_tasks = (uint32_t)(n_rows * p.chunks_per_row);
    p.n_rows_total = (uint32_t)(n_elements / row_elements);
    p.sm_aligned = (((uintptr_t)sign_mantissa & 15) == 0 ? 1 : 0) | (((uintptr_t)sign_mantissa & 31) == 0 ? 2 : 0);
    p.out_aligned = (((uintptr_t)out_bf16 & 15) == 0 ? 1 : 0) | (((uintptr_t)out_bf16 & 31) == 0 ? 2 : 0);
    const int64_t cta_items = ((int64_t)p.n_tasks + kFastThreads / 32 - 1) / (kFastThreads / 32);
    const size_t smem = (8u << kFastTableBits) + (size_t)n_luts * 256;
    if (ept == 32)
        return launch(df11_fast_kernel<kFastTableBits, 32, true>, kFastThreads, 5, smem, cta_items, p, device,
                      (cudaStream_t)stream);
    return launch(df11_fast_kernel<kFastTableBits, 16, true>, kFastThreads, 4, smem, cta_items, p, device,
                  (cudaStream_t)stream);
}

extern "C" int64_t df11_gemv_partials_bytes(int64_t n_rows, int64_t in_features, int32_t m)
{
    if (n_rows < 0 || in_features <= 0 || in_features % 512 || m < 1 || m > 4)
        return df11_fail(DF11_ERR_BADARG, "df11_gemv_partials_bytes(%lld, %lld, %d)", (long long)n_rows,
                         (long long)in_features, m);
    return (int64_t)m * n_rows * (in_features / 512) * 4;
}

namespace {
template <int EPT>
int launch_gemv_m(bool interior, int m, size_t smem, int64_t cta_items, const Params &p, const GemvArgs &g, int device,
                  cudaStream_t s)
{
    constexpr int base = EPT == 16 ? 6 : 14;  // kernel slots 6..13 and 14..21
    if (interior) {
        switch (m) {
        case 1: return launch_gemv(df11_gemv_kernel<kFastTableBits, EPT, 1, false>, base + 4, 1, smem, cta_items, p, g, device, s);
        case 2: return launch_gemv(df11_gemv_kernel<kFastTableBits, EPT, 2, false>, base + 5, 2, smem, cta_items, p, g, device, s);
        case 3: return launch_gemv(df11_gemv_kernel<kFastTableBits, EPT, 3, false>, base + 6, 3, smem, cta_items, p, g, device, s);
        default: return launch_gemv(df11_gemv_kernel<kFastTableBits, EPT, 4, false>, base + 7, 4, smem, cta_items, p, g, device, s);
        }
    }
    switch (m) {
    case 1: return launch_gemv(df11_gemv_kernel<kFastTableBits, EPT, 1, true>, base + 0, 1, smem, cta_items, p, g, device, s);
    case 2: return launch_gemv(df11_gemv_kernel<kFastTableBits, EPT, 2, true>, base + 1, 2, smem, cta_items, p, g, device, s);
    case 3: return launch_gemv(df11_gemv_kernel<kFastTableBits, EPT, 3, true>, base + 2, 3, smem, cta_items, p, g, device, s);
    default: return launch_gemv(df11_gemv_kernel<kFastTableBits, EPT, 4, true>, base + 3, 4, smem, cta_items, p, g, device, s);
    }
}
}  // namespace

extern "C" int df11_gemv_prepared(const void *luts, const void *codes, const void *sign_mantissa, const void *aux,
                                  const void *x_bf16, void *y_bf16, const void *bias_bf16, void *partials,
                                  int64_t first_element, int64_t n_rows, int64_t in_features,
                                  int32_t m, int32_t n_luts, int64_t n_bytes, int64_t n_elements, void *status,
                                  int32_t device, void *stream)
{
    if (!luts || !codes || !sign_mantissa || !aux || !x_bf16 || !y_bf16 || !partials)
        return df11_fail(DF11_ERR_BADARG, "null pointer");
    if (n_luts < 2 || n_luts > DF11_MAX_LUTS) return df11_fail(DF11_ERR_BADARG, "n_luts = %d", n_luts);
    if (n_bytes < 16 || n_elements <= 0 || n_elements > kMaxPreparedElements)
        return df11_fail(DF11_ERR_BADARG, "unit sizes out of range");
    if (m < 1 || m > 4) return df11_fail(DF11_ERR_BADARG, "m = %d: one to four activation vectors", m);
    const int ept = elements_per_seek_point();
    const int64_t chunk_elems = 32 * ept;
    if (in_features <= 0 || in_features % chunk_elems || first_element < 0 || first_element % chunk_elems ||
        n_rows < 0 || n_rows > 0x7FFFFFFF / (in_features / chunk_elems) ||
        first_element + n_rows * in_features > n_elements)
        return df11_fail(DF11_ERR_BADARG,
                         "matrix [%lld, %lld] at element %lld: rows must be multiples of %lld elements inside the unit",
                         (long long)n_rows, (long long)in_features, (long long)first_element, (long long)chunk_elems);
    if (((uintptr_t)codes & 3) || ((uintptr_t)sign_mantissa & 15) || ((uintptr_t)aux & 15) || ((uintptr_t)x_bf16 & 15) ||
        ((uintptr_t)partials & 3) || ((uintptr_t)y_bf16 & 1))
        return df11_fail(DF11_ERR_BADARG, "misaligned pointer (stream 4, sign_mantissa / aux / x 16 bytes)");
    if (n_rows == 0) return DF11_OK;
    const AuxLayout a = aux_layout(n_elements, ept);
    Params p = {};
    p.luts = (const uint8_t *)luts;
    p.codes = (const uint8_t *)codes;
    p.sm = (const uint8_t *)sign_mantissa;
    p.table_g = (const Df11Entry *)aux;
    p.sync_hi = (uint32_t *)((uint8_t *)aux + a.hi_off);
    p.sync_lo = (uint16_t *)((uint8_t *)aux + a.lo_off);
    p.status = (int *)status;
    p.n_bytes = n_bytes;
    p.n_elements = n_elements;
    p.n_chunks = a.n_chunks;
    p.n_luts = n_luts;
    p.ept = ept;
    p.sm_aligned = 1 | (((uintptr_t)sign_mantissa & 31) == 0 ? 2 : 0);
    GemvArgs g;
    g.x = (const uint16_t *)x_bf16;
    g.y = (uint16_t *)y_bf16;
    g.bias = (const uint16_t *)bias_bf16;
    g.partial = (float *)partials;
    g.first_chunk = (uint32_t)(first_element / chunk_elems);
    g.chunks_per_row = (uint32_t)(in_features / chunk_elems);
    g.n_rows = (uint32_t)n_rows;
    const size_t smem = (8u << kFastTableBits) + (size_t)n_luts * 256;
    const int64_t cta_items = (n_rows * g.chunks_per_row + kGemvThreads / 32 - 1) / (kGemvThreads / 32);
    // A matrix that stays clear of the unit's last two chunks needs no bounds checks on its
    // stream loads (see lean_tasks); the last matrix of a unit keeps them.
    const bool interior = (int64_t)g.first_chunk + n_rows * g.chunks_per_row + 2 <= a.n_chunks && (n_bytes >> 2) >= 4;
    if (ept == 32) return launch_gemv_m<32>(interior, m, smem, cta_items, p, g, device, (cudaStream_t)stream);
    return launch_gemv_m<16>(interior, m, smem, cta_items, p, g, device, (cudaStream_t)stream);
}


// ---------------------------------------------------------------------------------------
// Decode without any allocation by anybody: the auxiliary buffer of the prepared form lives
// in a fixed array inside the library image.
// ---------------------------------------------------------------------------------------
namespace {
// Decode table, then the seek points of a unit of at most DF11_STATIC_MAX_ELEMENTS elements
// (68 bytes per 512 elements).  About 4.3 MiB, held by every GPU that loads the library
// until the process exits.
constexpr int64_t kStaticAuxBytes =
    kAuxTableBytes + 68 * ((int64_t)DF11_STATIC_MAX_ELEMENTS / 512 + 1) + 64;
static __device__ __align__(256) uint8_t g_static_aux[kStaticAuxBytes];

// Device address of g_static_aux on each device.  In host code the array's name is only a
// handle for the runtime; the address a kernel can use comes from cudaGetSymbolAddress,
// asked once per device with that device current.
void *g_static_ptr[64] = {};

int static_aux_address(int device, void **out)
{
    if (device < 0 || device >= 64) return df11_fail(DF11_ERR_BADARG, "device index %d out of range", device);
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_static_ptr[device] == nullptr) {
        DeviceGuard guard(device);
        if (!guard.ok) return df11_fail(DF11_ERR_CUDA, "cudaSetDevice(%d) failed", device);
        void *ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_aux);
        if (e != cudaSuccess || ptr == nullptr)
            return df11_fail(DF11_ERR_CUDA, "cudaGetSymbolAddress failed on device %d: %s", device,
                             cudaGetErrorString(e));
        g_static_ptr[device] = ptr;
    }
    *out = g_static_ptr[device];
    return DF11_OK;
}
}  // namespace

extern "C" int df11_decode_static(const void *luts, const void *codes, const void *sign_mantissa,
                                  const void *output_positions, const void *gaps, void *out_bf16, int32_t n_luts,
                                  int64_t n_bytes, int64_t n_elements, void *status, int32_t device, void *stream)
{
    int rc = check_common(luts, codes, output_positions, gaps, n_luts, n_bytes, n_elements);
    if (rc != DF11_OK) return rc;  // argument errors come first: they must not cost the set-up below
    if (n_elements > (int64_t)DF11_STATIC_MAX_ELEMENTS)
        return df11_fail(DF11_ERR_NOSPACE,
                         "df11_decode_static handles units of up to %lld elements, this one has %lld; "
                         "use df11_prepare + df11_decode_prepared with a buffer of your own, or df11_decode",
                         (long long)DF11_STATIC_MAX_ELEMENTS, (long long)n_elements);
    if (df11_aux_bytes(n_bytes, n_elements) > kStaticAuxBytes)
        return df11_fail(DF11_ERR_NOSPACE, "the built-in buffer (%lld bytes) is too small for this unit",
                         (long long)kStaticAuxBytes);
    void *aux = nullptr;
    rc = static_aux_address(device, &aux);
    if (rc != DF11_OK) return rc;
    // Both steps go to the caller's stream, so the decode sees the seek points of THIS unit;
    // every entry it reads is written by the step before it, nothing needs to start at zero.
    rc = df11_prepare(luts, codes, output_positions, gaps, aux, kStaticAuxBytes, n_luts, n_bytes, n_elements, status,
                      device, stream);
    if (rc != DF11_OK) return rc;
    return df11_decode_prepared(luts, codes, sign_mantissa, output_positions, gaps, aux, out_bf16, n_luts, n_bytes,
                                n_elements, 0, status, device, stream);
}
