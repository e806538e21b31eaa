/*
 * libdf11 -- C ABI of the DFloat11 on-the-fly weight decompression path for
 * NVIDIA B200 (sm_100a).
 *
 * The reference project has no C interface: its Python package loads a PTX file
 * with cupy (`cp.RawModule(path=ptx_path).get_function('decode')`,
 * dfloat11/dfloat11.py:38-40) and launches it from two places
 * (dfloat11/dfloat11.py:142-151 in the forward pre-hook and :576-585 in the
 * compressor's self-check).  The entry points below are what a binding for that
 * path needs instead; each comment names the reference code it replaces.
 *
 * Conventions
 *   - Plain pointers and sizes only.  Pointers documented "device" must be valid
 *     on CUDA device `device`; "host" pointers are ordinary memory.
 *   - Nothing here allocates or frees device memory, synchronises the device or
 *     the stream, or keeps a pointer after returning.  Launches go to the given
 *     stream of the given device (the reference launches on cupy's current
 *     stream, dfloat11.py:142).  One exception, df11_decode_static: it works in a
 *     fixed array that is part of the library image, remembers that array's device
 *     address per device, and its calls on one device must not overlap (see there).
 *   - Every function returns DF11_OK (0) or a negative DF11_ERR_* code;
 *     df11_last_error() gives the message for the calling thread's last failure.
 *   - Functions are re-entrant and may be called from several threads.
 */
#ifndef DF11_H
#define DF11_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DF11_OK 0
#define DF11_ERR_BADARG (-1)  /* null pointer, negative size, unsupported table count ... */
#define DF11_ERR_CUDA (-2)    /* a CUDA runtime call failed (message has the CUDA error)   */
#define DF11_ERR_CORRUPT (-3) /* the DF11 tensors are inconsistent                         */
#define DF11_ERR_NOSPACE (-4) /* an output buffer given by the caller is too small         */

/* Bits a decode kernel ORs into the optional device status word. */
#define DF11_STATUS_BAD_TABLE 1    /* pointer outside `luts`, or a code length of 0 or > 32 */
#define DF11_STATUS_BAD_POSITIONS 2 /* output_positions not monotone / beyond n_elements    */
#define DF11_STATUS_TRUNCATED 4    /* a format block holds more elements than max_block_elems */
#define DF11_STATUS_TIMEOUT 8      /* a bounded wait for an asynchronous copy ran out        */

/* Library version, major*10000 + minor*100 + patch.  (The reference keeps a format
 * version string, dfloat11.py:44; this number versions the ABI below.) */
int df11_version(void);

/* Message of the last error on the calling thread ("" if none). */
const char *df11_last_error(void);

/*
 * Decompress one DF11 unit to BF16.  Replaces the reference's kernel launch
 *   _decode(grid, block, shared_mem, args=[luts, encoded_exponent, sign_mantissa,
 *           output_positions, gaps, out, n_luts, n_bytes, n_elements])
 * (dfloat11/dfloat11.py:142-151, kernel signature dfloat11/decode.cu:25-34).
 *
 *   luts              device, uint8  [n_luts * 256]
 *   codes             device, uint8  [n_bytes]           ("encoded_exponent")
 *   sign_mantissa     device, uint8  [n_elements]
 *   output_positions  device, uint32 [ceil(n_bytes/4096) + 1]
 *   gaps              device, uint8  [ceil(n_bytes/4096) * 320]
 *   out_bf16          device, uint16 [n_elements]        receives the BF16 bit patterns
 *   max_block_elems   largest output_positions[b+1] - output_positions[b]; it sizes the
 *                     kernel's shared-memory staging the way the reference's
 *                     `shared_mem_size` does (dfloat11.py:299-306).  <= 0: assume the
 *                     format's worst case (32768).
 *   status            device, int32, optional (may be NULL): DF11_STATUS_* bits are
 *                     ORed in when the kernel meets inconsistent tensors.  The kernel
 *                     never traps, reads out of bounds or loops without bound on bad
 *                     input; it only produces unspecified element values.
 *   stream            a cudaStream_t (NULL = the legacy default stream)
 *
 * 64-bit sizes: units above 2^31 elements are fine (the reference's `int`
 * arguments, decode.cu:33, overflow there).  The fast paths (TMA bulk copies, 16-byte
 * stores) need `codes`, `gaps`, `sign_mantissa` and `out_bf16` 16-byte aligned (any torch
 * allocation is); other alignments work but decode slower.
 */
int df11_decode(const void *luts, const void *codes, const void *sign_mantissa,
                const void *output_positions, const void *gaps, void *out_bf16,
                int32_t n_luts, int64_t n_bytes, int64_t n_elements,
                int32_t max_block_elems, void *status, int32_t device, void *stream);

/*
 * Self-test of the bounded waits in df11_decode's kernel.  Same arguments and launch as
 * df11_decode, except that the bulk copy of format block `drop_block`'s stream bytes is
 * announced to its barrier but never issued, and every wait is cut to 2 ms.  Nothing is in
 * flight, nothing faults: the CTA that owns that block finds its wait running out, ORs
 * DF11_STATUS_TIMEOUT into `status`, stops decoding and returns; the other CTAs finish their
 * blocks.  The call returns DF11_OK (the launch itself succeeded); the elements of the blocks
 * that CTA did not reach are unspecified.  For tests and for checking an installation; the
 * reference's kernel has no waits to bound (it loads synchronously, decode.cu:35-78).
 */
int df11_selftest_wait_timeout(const void *luts, const void *codes, const void *sign_mantissa,
                               const void *output_positions, const void *gaps, void *out_bf16,
                               int32_t n_luts, int64_t n_bytes, int64_t n_elements,
                               int32_t max_block_elems, int64_t drop_block, void *status,
                               int32_t device, void *stream);

/*
 * Optional two-step form for units that are decoded many times (every forward
 * pass, dfloat11.py:119-151).  df11_prepare() runs once per unit and device: it
 * fills a caller-owned auxiliary device buffer with (a) the multi-symbol decode
 * table derived from `luts` and (b) a seek point -- the stream bit position -- for
 * every group of 16 consecutive output elements, found by the counting pass and
 * block scan that the reference kernel redoes on every launch (decode.cu:104-178).
 * df11_decode_prepared() then lets every thread decode one group straight into its
 * final place.  The DF11 tensors on disk are unchanged; the auxiliary buffer is
 * derived data and can be rebuilt at any time.
 *
 * df11_aux_bytes(n_bytes, n_elements) is the size of that buffer (about
 * n_elements/8 + 32 KiB with a seek point every 16 elements, half of that with one
 * every 32, see df11_seek_interval).  The buffer must be 16-byte aligned.
 * `max_block_elems` is accepted for symmetry with df11_decode and ignored.  This
 * form has no counterpart in the reference.
 */
int64_t df11_aux_bytes(int64_t n_bytes, int64_t n_elements);

/*
 * How many consecutive output elements share one seek point of the prepared form: 16 or 32,
 * one setting for the whole process.  32 halves the auxiliary buffer (n_elements/16 bytes)
 * and makes the independently decodable chunk 1024 elements instead of 512.  elements = 0
 * only asks; 16 or 32 sets it; the return value is the setting in force (or a negative
 * error).  The initial value comes from DF11_EPT in the environment when it is 16 or 32.
 * A buffer filled by df11_prepare is only valid for calls made under the setting it was
 * filled under: change it before the first unit is prepared, not in between.
 * No counterpart in the reference.
 */
int df11_seek_interval(int32_t elements);

int df11_prepare(const void *luts, const void *codes, const void *output_positions,
                 const void *gaps, void *aux, int64_t aux_bytes, int32_t n_luts,
                 int64_t n_bytes, int64_t n_elements, void *status, int32_t device,
                 void *stream);

int df11_decode_prepared(const void *luts, const void *codes, const void *sign_mantissa,
                         const void *output_positions, const void *gaps, const void *aux,
                         void *out_bf16, int32_t n_luts, int64_t n_bytes, int64_t n_elements,
                         int32_t max_block_elems, void *status, int32_t device, void *stream);

/*
 * Row-wise decode for lookup tables (nn.Embedding): decompress only the rows that are
 * looked up instead of the whole unit, which the reference decodes on every forward
 * (dfloat11/dfloat11.py:158-161).  The seek points of the prepared form make any 512-element
 * chunk of a unit decodable on its own.
 *
 *   aux           the buffer filled by df11_prepare for this unit
 *   rows          device, int64 [n_rows]     row indices, in the order wanted; repeats allowed
 *   row_elements  elements per row: a multiple of 512 that divides n_elements
 *   out_bf16      device, uint16 [n_rows * row_elements]
 * An index outside the table sets DF11_STATUS_BAD_POSITIONS and yields row 0.
 * No counterpart in the reference.
 */
int df11_decode_rows_prepared(const void *luts, const void *codes, const void *sign_mantissa,
                              const void *aux, const void *rows, int64_t n_rows,
                              int64_t row_elements, void *out_bf16, int32_t n_luts, int64_t n_bytes,
                              int64_t n_elements, void *status, int32_t device, void *stream);

/*
 * Decode a contiguous part of a prepared unit: elements [first_element, first_element +
 * range_elements) go to out_bf16[0 .. range_elements).  The reference always decompresses a
 * whole unit into its buffer (dfloat11/dfloat11.py:139-151); decoding one matrix of a unit, or
 * a slab of its rows, right before the product that reads it lets the BF16 copy stay in the
 * L2 cache instead of travelling to HBM and back.  first_element must be a multiple of the
 * chunk (32 seek intervals: 512 or 1024 elements), and the range must end on such a multiple
 * or at the end of the unit.  Same bits as the matching part of df11_decode_prepared's output.
 * No counterpart in the reference.
 */
int df11_decode_range_prepared(const void *luts, const void *codes, const void *sign_mantissa,
                               const void *aux, int64_t first_element, int64_t range_elements,
                               void *out_bf16, int32_t n_luts, int64_t n_bytes, int64_t n_elements,
                               void *status, int32_t device, void *stream);

/*
 * df11_decode_range_prepared with the cap on CTAs per SM of df11_decode_prepared_shared: for a
 * part of a unit that is decompressed on a second stream beside the forward pass.
 */
int df11_decode_range_prepared_shared(const void *luts, const void *codes, const void *sign_mantissa,
                                      const void *aux, int64_t first_element, int64_t range_elements,
                                      void *out_bf16, int32_t n_luts, int64_t n_bytes, int64_t n_elements,
                                      int32_t ctas_per_sm, void *status, int32_t device, void *stream);

/*
 * Decode fused with a matrix-vector product: y[j][r] = sum_c W[r][c] * x[j][c] + bias[r] for
 * one [n_rows, in_features] matrix W that lies inside a prepared unit (its first weight is
 * element `first_element` of the unit) and m = 1..4 activation vectors, without writing W
 * anywhere.  It replaces, for batch-1 generation, the pair "decode the block, then
 * F.linear on the injected weight views" (dfloat11.py:139-166 plus torch's GEMV), which
 * writes 2 bytes per weight and reads them again.  x is [m][in_features] bf16, y is
 * [m][n_rows] bf16, bias is [n_rows] bf16 or NULL; products are exact and accumulated in
 * fp32 in a fixed order (bit-reproducible run to run; not the order of a library GEMV, so
 * not bit-identical to one).  in_features and first_element must be multiples of the chunk
 * (32 seek intervals: 512 or 1024 elements, see df11_seek_interval), `codes` 4-byte and
 * sign_mantissa / aux / x 16-byte aligned.  The kernel is launched with programmatic stream
 * serialization and reads the unit's tensors and `aux` BEFORE it waits for the kernel ahead
 * of it in the stream; that is safe behind any kernel of this library (none of those that
 * write such data signals its dependents early) and behind work that finished earlier, but
 * not behind a foreign kernel that writes these buffers and triggers dependent launches
 * before it is done.  x, y, bias and `partials` are only touched after the wait.
 * `partials` is caller-owned device scratch
 * of df11_gemv_partials_bytes() bytes whose contents do not matter; launches that share it
 * must not overlap.  Two kernels are queued: the products, then a small one that adds each
 * row's partial sums.  No counterpart in the reference.
 */
int64_t df11_gemv_partials_bytes(int64_t n_rows, int64_t in_features, int32_t m);

int df11_gemv_prepared(const void *luts, const void *codes, const void *sign_mantissa, const void *aux,
                       const void *x_bf16, void *y_bf16, const void *bias_bf16, void *partials,
                       int64_t first_element, int64_t n_rows, int64_t in_features,
                       int32_t m, int32_t n_luts, int64_t n_bytes, int64_t n_elements, void *status,
                       int32_t device, void *stream);

/*
 * df11_decode_prepared for a launch that is meant to run BESIDE other kernels: the decode
 * of the next transformer block on a second stream while the current block computes.  The
 * fast decoder is a persistent kernel that otherwise fills every SM (2 CTAs of 512 threads),
 * so kernels of other streams would wait for it to end; `ctas_per_sm` (1, or 0 = all) caps
 * the CTAs it places per SM and leaves the rest of each SM to them.  Same arguments, result
 * and bits as df11_decode_prepared.  No counterpart in the reference, which decodes in the
 * stream of the forward pass and overwrites one buffer (dfloat11.py:119-151).
 */
int df11_decode_prepared_shared(const void *luts, const void *codes, const void *sign_mantissa,
                                const void *output_positions, const void *gaps, const void *aux,
                                void *out_bf16, int32_t n_luts, int64_t n_bytes, int64_t n_elements,
                                int32_t ctas_per_sm, void *status, int32_t device, void *stream);

/*
 * Decode for callers that cannot allocate device memory at all and have nobody to do it
 * for them: code running inside a CUDA-graph capture or a stream callback, a plug-in
 * called from a serving loop whose memory pool is already carved up, a host runtime
 * that forbids cudaMalloc after start-up.  df11_decode needs no extra memory but is the
 * slower kernel; the fast kernel behind df11_decode_prepared needs an auxiliary buffer.
 * Here that buffer is a fixed array inside the library (about 4.3 MiB of every GPU that
 * loads libdf11, held until the process exits), so the call allocates nothing, and
 * neither does anything it calls.  Same tensors and meaning as df11_decode; the
 * auxiliary data is rebuilt on every call (two extra short launches on `stream`).
 *
 *   - Units of more than DF11_STATIC_MAX_ELEMENTS elements are refused with
 *     DF11_ERR_NOSPACE (the message says what to use instead).
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress); where the CUDA runtime loads modules lazily that lookup
 *     can make the driver load the library's image, array included, which is a
 *     driver-side allocation.  So "allocates nothing" holds from the second call on a
 *     device: make one warm-up call per device at start-up, outside any stream
 *     capture, before relying on it.  Argument errors are reported before that set-up.
 *   - All calls on one device share the array: two calls whose kernels may overlap on
 *     the GPU (different streams) corrupt each other.  Calls ordered on one stream are fine.
 * This entry point has no counterpart in the reference.
 */
#define DF11_STATIC_MAX_ELEMENTS (1 << 25)
int df11_decode_static(const void *luts, const void *codes, const void *sign_mantissa,
                       const void *output_positions, const void *gaps, void *out_bf16,
                       int32_t n_luts, int64_t n_bytes, int64_t n_elements, void *status,
                       int32_t device, void *stream);

/*
 * All-reduce (sum) of a small BF16 tensor across the ranks of the partitioned mode, in one
 * kernel over NVLink peer memory: plain peer loads and stores, no collective library, no
 * multicast.  For the [batch, hidden] activations that are summed after every row-parallel
 * layer (32 KB at batch 1 for hidden 16384), where a library collective is all latency.
 * Every rank calls it with the same n_elements, in the same order, on its own GPU.
 *
 *   peer_data    HOST array [world] of device addresses: rank r's buffer of 2 * slot_bytes
 *                bytes in memory that every rank can address (symmetric memory, or IPC
 *                mappings), as seen from THIS process; entry `rank` is this rank's own
 *   peer_flags   HOST array [world]: rank r's flag area of df11_allreduce_flag_bytes() bytes
 *                (about 2 MiB: the flags, and the cells of the pushed form below), in the
 *                same kind of memory, zeroed once before the first call on any rank
 *   counters     device, this rank only: df11_allreduce_counter_bytes() bytes (256), zeroed once;
 *                the kernels keep their call numbers there
 *   in_bf16 / out_bf16   device, n_elements BF16 each (a multiple of 8; in == out is fine),
 *                16-byte aligned; n_elements * 2 <= slot_bytes
 *   wait_ms      how long a rank waits for its peers' data before it gives up and sets
 *                DF11_STATUS_TIMEOUT in `status`; `out` is then undefined (<= 0: 2 s).  While
 *                that bit is set in `status`, later calls do not wait at all (they still keep
 *                the ranks' call numbers in step): clear it after dealing with the failure
 * Two forms, chosen by size alone (so every rank chooses alike).  Up to 64 KB on 1, 2, 4 or 8
 * ranks: every rank pushes its slice into every rank's flag area as 8-byte {data, call tag}
 * pairs and sums what has arrived with this call's tag -- one NVLink crossing, no fence, flag
 * or barrier.  Anything else: slices into the own data buffer, one flag per rank and CTA,
 * peer loads.
 * The sum is taken in rank order in fp32 and rounded once: identical bits on every rank.
 * The call numbers are kept in `counters`, so a launch captured in a CUDA graph replays.
 * No counterpart in the reference (its only multi-GPU form places whole layers on
 * different devices, dfloat11/dfloat11.py:455-460).
 */
int64_t df11_allreduce_flag_bytes(void);
int64_t df11_allreduce_counter_bytes(void);

int df11_allreduce_bf16(const uint64_t *peer_data, const uint64_t *peer_flags, void *counters,
                        int32_t rank, int32_t world, const void *in_bf16, void *out_bf16,
                        int64_t n_elements, int64_t slot_bytes, int64_t wait_ms, void *status,
                        int32_t device, void *stream);

/*
 * Self-test of df11_allreduce_bf16's kernels on ONE GPU: a single cooperative launch plays all
 * `world` ranks (2, 4 or 8: the specialised kernels; 3: the general one) -- row r of the grid runs rank r's code on rank r's buffers -- so
 * the exchange between ranks, the call tags and the alternating buffer halves are exercised
 * where only one GPU is at hand.  (Separate launches that wait for one another must never share
 * a GPU; one cooperative launch may.)
 *   data      device, world buffers of 2 * slot_bytes bytes one after another
 *   flags     device, world flag areas of df11_allreduce_flag_bytes() bytes, zeroed once
 *   counters  device, world blocks of df11_allreduce_counter_bytes() bytes, zeroed once
 *   in_bf16 / out_bf16   device, [world][n_elements] BF16: rank r's input and result
 * Size limits, forms, summation order and time-out as for df11_allreduce_bf16 (wait_ms <= 0:
 * 200 ms).  No counterpart in the reference.
 */
int df11_selftest_allreduce_one_gpu(int32_t world, void *data, void *flags, void *counters,
                                    const void *in_bf16, void *out_bf16, int64_t n_elements,
                                    int64_t slot_bytes, int64_t wait_ms, void *status, int32_t device,
                                    void *stream);

/*
 * Host-side check of one unit before its first launch (all pointers HOST memory).
 * The reference performs no validation: a zero entry in the length row makes its
 * kernel spin forever (decode.cu:116-118).  Checks: table count, pointers stay
 * inside `luts`, every symbol reachable from the root has a length in 1..32,
 * output_positions is monotone and ends at n_elements, tensor sizes agree.
 * On success *max_block_elems (optional) receives the value df11_decode wants.
 */
int df11_validate_host(const void *luts, int32_t n_luts, int64_t n_bytes, int64_t n_elements,
                       const void *output_positions, int64_t n_positions, int64_t n_gap_bytes,
                       int32_t *max_block_elems);

/*
 * Host-side bit packer for one unit; byte-identical to the reference's `encode`
 * (dfloat11/dfloat11_utils.py:118-170) for the same code table, but linear-time
 * native code instead of a per-symbol Python loop.  All pointers HOST memory.
 *
 *   exponents   uint8 [n_elements]        (W >> 7) & 0xFF of every BF16 weight
 *   code_len    uint8 [256], code_val uint32 [256]   code of each exponent value
 *               (length 0 = value does not occur)
 *   pad_len / pad_val   code whose leading bits complete the last byte when the
 *               stream does not end on a byte boundary (the reference uses its
 *               end-of-stream code, dfloat11_utils.py:153-160); pad_len 0 = zero bits
 * df11_encode_size() returns the stream length in bytes (or a negative error).
 * df11_encode_host() fills
 *   codes  [n_bytes], gaps [ceil(n_bytes/4096)*320], output_positions [ceil(n_bytes/4096)+1]
 * using up to n_threads host threads.
 */
int64_t df11_encode_size(const void *exponents, int64_t n_elements, const void *code_len);

int df11_encode_host(const void *exponents, int64_t n_elements, const void *code_len,
                     const void *code_val, int32_t pad_len, uint32_t pad_val, void *codes,
                     int64_t n_bytes, void *gaps, int64_t n_gap_bytes, void *output_positions,
                     int64_t n_positions, int32_t n_threads);

/*
 * The same bit packer on the GPU, for exponent bytes that are already in device memory
 * (a freshly loaded BF16 model): same outputs, byte for byte, as df11_encode_host.
 * Two steps, because the size of the stream is only known after a first pass:
 *   df11_encode_device_count()  queues the size pass and copies the total number of stream
 *                               BITS to *total_bits_host (8 bytes, host memory); synchronise
 *                               the stream before reading it;
 *   df11_encode_device_pack()   fills codes (4-byte aligned, room for n_bytes rounded up to a
 *                               multiple of 4), gaps and output_positions (4-byte aligned),
 *                               all caller-owned DEVICE buffers sized from that total.
 * `exponents` is device memory; `code_len` / `code_val` are HOST arrays of 256 entries, as for
 * df11_encode_host; `workspace` is caller-owned device memory of
 * df11_encode_device_workspace_bytes() bytes, 8-byte aligned, kept untouched between the two
 * steps.  A value that occurs but has no code sets DF11_STATUS_BAD_TABLE in `status`.
 * No counterpart in the reference, which packs on the CPU in Python.
 */
int64_t df11_encode_device_workspace_bytes(int64_t n_elements);

int df11_encode_device_count(const void *exponents, int64_t n_elements, const void *code_len,
                             const void *code_val, void *workspace, int64_t workspace_bytes,
                             void *total_bits_host, void *status, int32_t device, void *stream);

int df11_encode_device_pack(const void *exponents, int64_t n_elements, const void *code_len,
                            const void *code_val, int32_t pad_len, uint32_t pad_val, void *workspace,
                            void *codes, int64_t n_bytes, void *gaps, int64_t n_gap_bytes,
                            void *positions, int64_t n_positions, int32_t device, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* DF11_H */
