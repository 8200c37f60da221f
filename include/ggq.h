/*
 * ggq.h -- C ABI of the B200 (sm_100a) dequantize-and-multiply library, libggq_b200.so.
 *
 * Every entry point is plain C: pointers, sizes and integer codes only.  All device
 * pointers are caller-owned; the library never allocates or frees the caller's buffers,
 * never synchronises a stream and never reads results back, so every launcher can be
 * enqueued from a framework's custom-call handler (XLA FFI, torch, raw CUDA).
 *
 * qtype codes are the GGMLQuantizationType values of gguf-py / llama.cpp
 * (gguf/constants.py), e.g. Q4_K = 12, Q6_K = 14, IQ4_XS = 23.
 *
 * Every function that returns int32_t returns a ggq_status; 0 is success.  On failure a
 * thread-local message is available from ggq_last_error().  Nothing throws or exits.
 * All entry points may be called from several host threads at once; the library's own state
 * is per device and created once under std::call_once.
 *
 * Each declaration names the interface of the reference project (nshepperd/gguf-jax) it
 * stands in for, as path:line inside that project.
 */
#ifndef GGQ_H_
#define GGQ_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum ggq_status {
  GGQ_OK = 0,
  GGQ_BAD_QTYPE = 1,      /* qtype is not one of the 26 decodable types            */
  GGQ_BAD_SHAPE = 2,      /* K not a multiple of the block, N/M out of range, ...  */
  GGQ_MISALIGNED = 3,     /* a base pointer is not aligned as the kernel needs     */
  GGQ_UNSUPPORTED = 4,    /* no fused kernel for this qtype / batch                */
  GGQ_LAUNCH_FAILED = 5,  /* the CUDA runtime refused the launch                   */
  GGQ_TIMEOUT = 6,        /* a bounded device-side wait ran out (see ggq_read_status) */
  GGQ_NO_TABLES = 7,      /* a codebook qtype was used before ggq_set_tables       */
  GGQ_BAD_WORKSPACE = 8,  /* workspace missing or too small                        */
  GGQ_BAD_DTYPE = 9       /* output dtype code not one of ggq_dtype                */
} ggq_status;

typedef enum ggq_dtype { GGQ_F32 = 0, GGQ_BF16 = 1, GGQ_F16 = 2 } ggq_dtype;

/* Library ABI version (major * 100 + minor). No reference counterpart. */
int32_t ggq_version(void);

/* Message for the last non-zero status returned on this host thread. */
const char* ggq_last_error(void);

/* Block geometry of a qtype: elements per block and bytes per block.
 * Replaces the GGML_QUANT_SIZES lookups at src/gguf_jax/quants.py:720 and
 * src/gguf_jax/array.py:101. */
int32_t ggq_type_info(int32_t qtype, int32_t* block_elems, int32_t* block_bytes);

/* Byte size and layout of the codebook blob ggq_set_tables expects.  The blob is the
 * concatenation, in this order, of: IQ2_XXS grid u8[256*8], IQ2_XS grid u8[512*8],
 * IQ2_S grid u8[1024*8], IQ3_XXS grid u8[256*4], IQ3_S grid u8[512*4],
 * IQ1_S/IQ1_M grid i8[2048*8], IQ4_NL/IQ4_XS values i8[16], MXFP4/NVFP4 values i8[16].
 * The host side fills it from gguf.quants at import time, exactly where the reference
 * reads the same tables (src/gguf_jax/quants.py:476-483, cute/lowbit.py:401-420). */
size_t ggq_tables_bytes(void);

/* Upload the codebook blob (host memory) to `device` once.  The library keeps this one
 * immutable allocation per device until the process exits.  Idempotent. */
int32_t ggq_set_tables(int32_t device, const void* host_blob, size_t bytes);

/* Optional per-device set-up: allocates the 4-byte device status word that bounded device-side
 * waits raise (see ggq_read_status) and caches the multiprocessor count.  The launchers that can
 * wait (ggq_gemv_sharded, ggq_gemv_sharded_tagged, ggq_gemm) do the same on their first call on
 * a device; that first call allocates device memory, so make it -- or this call -- outside any
 * stream capture.  ggq_gemv never allocates: its kernels' waits for their own TMA copies (bounded like the others;
 * they run out only if the copy engine fails) are reported once the word exists, i.e. after this call or one of
 * those.  Thread-safe, idempotent.  No reference counterpart. */
int32_t ggq_init(int32_t device);

/* Decode n_blocks blocks of `qtype` (device bytes, n_blocks * block_bytes) into
 * n_blocks * block_elems values of out_dtype on `stream`.  The float32 result is
 * bit-identical to gguf.quants.dequantize; bf16/f16 are that result rounded once.
 * Replaces dequantize_blocks / the 26 registered decoders
 * (src/gguf_jax/quants.py:125-730) and the CuTe Q4_K kernel launch
 * (src/gguf_jax/cute/q4_k.py:78-101). */
int32_t ggq_dequant(int32_t qtype, const void* blocks, int64_t n_blocks, void* out,
                    int32_t out_dtype, void* stream);

/* 1 if a fused multiply kernel exists for qtype, else 0.
 * Replaces the key set of _fused() (src/gguf_jax/_matmul.py:52-75). */
int32_t ggq_has_fused(int32_t qtype);

/* Largest flattened batch M for which the fused route (ggq_gemv up to ggq_gemv_max_batch(), ggq_gemm above) is
 * the faster one for an (N, K) weight of qtype -- 16, or 256 / 512 for Q4_K / Q5_K / Q6_K weights of tens of MB; 0 when
 * there is no fused kernel.  Replaces the per-kernel caps
 * (src/gguf_jax/_matmul.py:60-75, cute/q4_k.py:117-118, cute/lowbit.py:97). */
int32_t ggq_fused_batch_limit(int32_t qtype, int64_t N, int64_t K);

/* Largest M served by the small-batch (GEMV) kernel; above it ggq_gemm is used. */
int32_t ggq_gemv_max_batch(void);

/* Scratch the fused kernels need for an (N, K) weight at batch M: the largest need of any kernel
 * ggq_gemv / ggq_gemm may pick for that shape (split-K partials, per-row-tile step counters,
 * per-unit partial slots).  The caller allocates at least this many bytes, 256-byte aligned,
 * ZERO-FILLED ONCE; the kernels leave it zeroed again, so one buffer serves any number of calls
 * that do not overlap on the GPU.  With less scratch than this the launchers fall back to the
 * kernels that need none where there is one, and return GGQ_INVALID_VALUE otherwise. */
size_t ggq_workspace_bytes(int32_t qtype, int64_t N, int64_t K, int32_t M);

/* y[M, N] = x[M, K] @ W[N, K]^T with W quantized (row-major blocks, N rows of
 * K / block_elems * block_bytes bytes), x bf16, y of y_dtype, 1 <= M <= ggq_gemv_max_batch().
 * Weights are applied at full float32 precision (exact integer codes times float32
 * scales), accumulation is float32, the only rounding to a narrow type is the output.
 * Replaces matmul_q4_k / matmul_q5_k / matmul_q6_k / matmul_iq4_xs / matmul_lowbit
 * (src/gguf_jax/cute/q4_k.py:282-329, q5_k.py:150-179, q6_k.py:115-144,
 * iq4_xs.py:146-175, lowbit.py:675-712).
 * Which kernel runs (all give the same product to float32 rounding; none is a CPU path):
 *   Q4_K / Q5_K / Q6_K at M = 1 and M = 5..16: the per-format kernels (integer codes fed to
 *     mma.sync as exact bf16 values, scales applied to the float32 accumulators);
 *   Q4_K / Q5_K / Q6_K at M = 2..4, and Q2_K, IQ4_XS, IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS, IQ3_S,
 *     IQ1_S, IQ1_M at every M: the tiled kernel (same arithmetic; warps own contiguous ranges of
 *     16-row x K-chunk steps; needs K % 256 == 0, rows of a multiple of 16 bytes and the workspace; serves M in slices of 8);
 *   everything else (the 32-element formats, float formats, shapes the above do not take): the
 *     streaming kernels that decode a block in registers and multiply it at once.
 * Launches are programmatic dependents: a kernel may begin to read `w` (only `w`) while the
 * previous launch of this library on the same stream is still finishing.  So `w` must not be an
 * output of that previous launch; x, y and the workspace carry no such restriction.  The weight
 * buffer must extend to the next 16-byte boundary (true of any device allocation). */
int32_t ggq_gemv(int32_t qtype, const void* w, int64_t N, int64_t K, const void* x_bf16,
                 int32_t M, void* y, int32_t y_dtype, void* workspace,
                 size_t workspace_bytes, void* stream);

/* The same product for larger M.  Replaces gemm_q4_k (src/gguf_jax/cute/q4_k_gemm.py:369-391).  Kernels:
 *   Q4_K / Q5_K / Q6_K, K % 256 == 0, rows of a multiple of 16 bytes, with the workspace:
 *     M <= 32: the batch-major mma.sync kernel of ggq_gemv (exact integer codes, nothing rounded);
 *     M  > 32: tcgen05 / tensor memory with the weights decoded exactly and rounded once to bf16 -- the
 *              reference's contract for its GEMM and its fallback (relative error of the result about 2e-3);
 *   any other block qtype (K % 256 == 0), or the above without workspace: tcgen05 with blocks decoded to float32 and
 *     multiplied as tf32 (weights rounded to 11 significant bits; relative error about 3e-4).
 * GGQ_GEMM_KERNEL = wide | bf16w | codes | tf32 in the environment pins one kernel (codes: integer-code tcgen05
 * operands with one accumulator per scale group, exact but slower).  With few row tiles a launch cuts K into ranges
 * (partials in the workspace, the last arriver adds them in a fixed order: results do not depend on timing).
 * ggq_fused_batch_limit says up to which M this entry beats decoding the weight and calling a library GEMM. */
int32_t ggq_gemm(int32_t qtype, const void* w, int64_t N, int64_t K, const void* x_bf16,
                 int32_t M, void* y, int32_t y_dtype, void* workspace,
                 size_t workspace_bytes, void* stream);

/* Row-sharded multiply with the exchange fused into the kernel.  No counterpart in the reference
 * (it runs on one device only); it stands where a sharded caller would otherwise follow ggq_gemv
 * with an all-gather.  `w` holds this rank's N_local rows of an (world * N_local, K) weight;
 * y_peers[p] is the address, valid on THIS device, of rank p's full (M, n_total) output buffer
 * (peer-mapped over NVLink for p != rank), flag_peers[p] likewise of rank p's flag array of
 * world + 2 uint32, zero-filled once.  The kernel stores its rows into every rank's buffer with
 * plain stores and, when its grid has finished, raises its flag on every rank.  With
 * wait_previous != 0 it first waits (bounded; GGQ_TIMEOUT through ggq_read_status) until every
 * rank has published the previous exchange, i.e. until x -- if it is the result of that exchange
 * -- is complete.  All ranks must issue the same sequence of calls.  Host arrays y_peers /
 * flag_peers are read during the call only.  Returns GGQ_UNSUPPORTED for qtype / batch
 * combinations without a publishing kernel (today: everything but Q4_K, Q5_K and Q6_K at
 * batch 1). */
int32_t ggq_gemv_sharded(int32_t qtype, const void* w, int64_t N_local, int64_t K, const void* x_bf16,
                         int32_t M, void* const* y_peers, uint32_t* const* flag_peers, int32_t world,
                         int32_t rank, int64_t n_total, int32_t y_dtype, int32_t wait_previous,
                         void* workspace, size_t workspace_bytes, void* stream);

/* Activations and results in page-locked host memory (no counterpart in the reference, whose arrays are
 * device-resident; what jax.device_put / device_get do around its calls).  In front of a 30 us product a
 * copy-engine transfer costs about 12 us of latency each way; these two uses avoid it:
 *  - ggq_stage_host copies `bytes` (a multiple of 16, both addresses 16-byte aligned, at most 64 MB) from a
 *    page-locked, device-visible host buffer (cudaHostAlloc / cudaHostRegister under unified addressing) to device
 *    memory with a small kernel that reads the host buffer over the bus; the product enqueued behind it is its
 *    programmatic dependent and prefetches weight tiles meanwhile.  The host buffer must stay unchanged until the
 *    stream has passed the call.
 *  - `y` of ggq_gemv may itself be such a host buffer: the kernels only ever store to y, the stores are
 *    visible to the host once the stream has been synchronised. */
int32_t ggq_stage_host(const void* host_src, void* device_dst, size_t bytes, void* stream);

/* Row-sharded batch-1 multiply with a tagged exchange: no flags and no fences.  No counterpart in
 * the reference.  Every output element is stored into every rank's buffer as one 32-bit word
 * (bf16 value in the low half, a 16-bit tag of the exchange in the high half), so each word
 * validates itself and the exchange costs one store flight.  y_peers[p] is the address, valid on
 * THIS device, of rank p's uint32[n_total] buffer.  The activations are either plain bf16
 * (x_bf16) or the tagged words a previous call of this function left in this rank's own buffer
 * (x_tagged, with x_back = how many sharded launches ago that call was, 1 = the previous one);
 * the kernel then polls each word until its tag is the expected one (bounded: GGQ_TIMEOUT via
 * ggq_read_status).  `state` is this rank's array of (world + 2) uint32, zero-filled once, that
 * only this function touches: it counts the exchanges, from which both tags are derived on the
 * device, so a captured CUDA graph can be replayed.  after_tagged (optional, may be NULL) names
 * after_words tagged words of the exchange after_back launches ago in this rank's own buffer:
 * the kernel does not read its activations before all of them have arrived, which orders it
 * after that exchange the way ggq_gemv_sharded's flags would.  All ranks must issue the same
 * sequence of calls.  A CTA polls only the part of the activations that its share of the weight touches, so
 * a rank may store exchange e while a peer still reads exchange e - 2 * x_back_max: a buffer may be reused for a
 * new exchange once 2 * x_back_max + 1 exchanges have passed (every call ordered with after_tagged behind the
 * exchange before it: x_back_max + 2). */
int32_t ggq_gemv_sharded_tagged(int32_t qtype, const void* w, int64_t N_local, int64_t K,
                                const void* x_bf16, const uint32_t* x_tagged, int32_t x_back,
                                const uint32_t* after_tagged, int64_t after_words,
                                int32_t after_back, uint32_t* const* y_peers, uint32_t* state, int32_t world,
                                int32_t rank, int64_t n_total, void* workspace,
                                size_t workspace_bytes, void* stream);

/* ggq_gemv_sharded for batches: M >= 1 rows of x, `ldx` elements apart (ldx >= K: x may be the leading K columns of a
 * wider buffer, e.g. of an earlier exchange's output), Q4_K / Q5_K / Q6_K shards with K % 256 == 0 and 16-byte aligned
 * rows.  y_peers[p] is rank p's (M, n_total) output; this rank's kernel stores its N_local columns of every batch row
 * into all of them and raises its flag once per launch.  Batches above 32 rows run as slices of 32, one exchange each;
 * a consumer that waits for the previous exchange (wait_previous of the next call) has all slices.  M == 1 is
 * ggq_gemv_sharded.  Needs ggq_workspace_bytes(qtype, N_local, K, M).  No reference counterpart. */
int32_t ggq_gemm_sharded(int32_t qtype, const void* w, int64_t N_local, int64_t K, const void* x_bf16, int64_t ldx,
                         int32_t M, void* const* y_peers, uint32_t* const* flag_peers, int32_t world, int32_t rank,
                         int64_t n_total, int32_t y_dtype, int32_t wait_previous, void* workspace,
                         size_t workspace_bytes, void* stream);

/* Batch-1 Q4_K multiply that needs no scratch from the caller and allocates nothing.
 * No counterpart in the reference.  It exists for hosts that cannot allocate device memory
 * around a call: a custom-call handler whose framework owns every buffer, a serving loop
 * with a fixed memory plan.  The scratch of ggq_gemv lives in a 192 KB device array
 * built into the library (held by every GPU that loads it until the process exits), which
 * bounds the weight to N <= 524288 rows; K as for the Q4_K path of ggq_gemv (multiple of 256,
 * activations resident in shared memory), w and x 16-byte aligned, M = 1.  Larger N or an
 * unsupported K returns GGQ_BAD_SHAPE with the limit in ggq_last_error().
 * The first call on a device looks up the array's device address (a synchronous runtime
 * query).  All calls on one device share the array: calls whose kernels
 * could overlap on the GPU (unordered streams) must be serialised by the caller.  The result
 * is identical to ggq_gemv on the same inputs. */
int32_t ggq_gemv_q4k_static(const void* w, int64_t N, int64_t K, const void* x_bf16, void* y,
                            int32_t y_dtype, void* stream);

/* Reads and clears the device-side status word of `device` (0 = no bounded wait ran
 * out since the last read; otherwise the call returns GGQ_TIMEOUT).  Synchronises the device.
 * The word exists from the first ggq_init / sharded / ggq_gemm call on the device, whether or
 * not ggq_set_tables was ever called; before that the function reports 0.  No reference
 * counterpart: the reference has no device-side waits. */
int32_t ggq_read_status(int32_t device, int32_t* status_word);

#ifdef __cplusplus
}
#endif
#endif /* GGQ_H_ */
