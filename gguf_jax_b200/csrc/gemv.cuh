// Internal interface between the multiply kernels and the ggq_gemv / ggq_gemm entry points.
#pragma once

#include "ggq_common.cuh"

#include <cuda.h>

#include <atomic>
#include <cstdlib>

namespace ggq {

// Single rounding of a float32 result to the caller's output dtype.
__device__ __forceinline__ void store_out(void* y, int y_dtype, int64_t idx, float v) {
  if (y_dtype == GGQ_F32) reinterpret_cast<float*>(y)[idx] = v;
  else if (y_dtype == GGQ_BF16) reinterpret_cast<__nv_bfloat16*>(y)[idx] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half*>(y)[idx] = __float2half_rn(v);
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against the driver library); null if the
// driver does not offer it.  Used for the TMA copy paths; every user keeps a cp.async path for that case.
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline EncodeTiledFn tensor_map_encoder() {
  static std::atomic<void*> cached{nullptr};
  static std::atomic<bool> tried{false};
  if (!tried.load(std::memory_order_acquire)) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      fn = nullptr;
    (void)cudaGetLastError();
    cached.store(fn, std::memory_order_release);
    tried.store(true, std::memory_order_release);
  }
  return reinterpret_cast<EncodeTiledFn>(cached.load(std::memory_order_acquire));
}
// A weight of `row_bytes` bytes per row (a multiple of 16) as a tensor map of 32-bit words [N rows, row_bytes / 4], box
// = box_words x 16 rows, no swizzle, zeros outside the tensor.  False if there is no encoder or it refuses.
inline bool make_weight_map(CUtensorMap* map, const uint8_t* w, int64_t N, int64_t row_bytes, int box_words) {
  EncodeTiledFn fn = tensor_map_encoder();
  if (!fn || row_bytes % 16 || (uintptr_t)w % 16) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)(row_bytes / 4), (cuuint64_t)N};
  const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)box_words, 16};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint8_t*>(w), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;   // the promotion size made no measurable difference
}
#ifdef __CUDACC__
// One lane: expect `bytes` on the mbarrier at shared address `bar`, then copy the box at word column x, row y of `map`
// to shared address `dst` (128-byte aligned).  x * 4 must be a multiple of 16.
__device__ __forceinline__ void tma_box_load(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar, uint32_t bytes) {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // the slot's last reads precede the copy
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
// All lanes: bounded wait for the phase `parity` of the mbarrier at `bar`; raises the status word when it runs out.
__device__ __forceinline__ void tma_box_wait(uint32_t bar, uint32_t parity, int* status, int lane) {
  uint32_t ok = 0;
  for (uint32_t spin = 0; spin < (1u << 20) && !ok; spin++)
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  if (!ok && status && lane == 0) atomicOr(status, STATUS_WAIT_EXPIRED);
}
__device__ __forceinline__ void tma_bars_init(uint32_t bars, int n, int lane) {
  if (lane == 0) {
    for (int d = 0; d < n; d++) asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bars + 8 * d), "r"(1u) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
}
#endif

// Coverage kernel: any block qtype, any M <= 16 (gemv_generic.cu).
cudaError_t gemv_generic(const TypeInfo* ti, const uint8_t* w, int64_t N, int64_t K, const void* x, int M,
                         void* y, int y_dtype, const uint8_t* tab, cudaStream_t st);

// Batch 1, any block qtype, K a multiple of 256, 16-byte aligned weight: warp per row with the raw
// blocks streamed through shared memory (gemv_stream.cu).
bool gemv_stream_applicable(const TypeInfo* ti, int64_t N, int64_t K, int M, const void* w, const void* x);
cudaError_t gemv_stream(const TypeInfo* ti, const uint8_t* w, int64_t N, int64_t K, const void* x, void* y,
                        int y_dtype, const uint8_t* tab, cudaStream_t st);

// Row-sharded output over several GPUs of one node (one process per GPU).  Instead of writing
// y into a local buffer and all-gathering it, a kernel can store its slice of the output rows
// straight into every peer's copy of y (peer-mapped pointers over NVLink) and, when the whole
// grid has finished, raise a per-rank sequence flag in every peer's flag array.  The consumer
// side is the same structure seen from the other end: before a kernel reads activations that a
// previous exchange produced, it waits (bounded) until every rank's flag has reached the
// sequence number of that exchange.  Plain stores and loads only; no multicast of any kind.
constexpr int kMaxPeers = 8;
struct PeerPublish {
  void* y[kMaxPeers];             // every rank's full (M, n_total) output buffer, index = rank
  uint32_t* flags[kMaxPeers];     // every rank's flag array (uint32[world]), index = rank
  int world;                      // 0: not sharded (write y locally, no flags)
  int rank;
  int64_t n_total;                // row stride of the full output
  int64_t row_offset;             // first output row of this rank's slice
  int wait_previous;              // 1: the activations come from the previous exchange, wait for it first
  // Tagged mode (no flags, no fences): every output element travels as one 32-bit word, bf16 value
  // in the low half and the exchange's 16-bit tag in the high half, so a word validates itself and
  // the only cost of the exchange is the flight time of the stores.  y[] are then uint32 buffers;
  // a consumer kernel given x_tagged polls each word until its tag is the expected one (bounded).
  int tagged;                     // 1: emit tagged words, do not raise flags
  const uint32_t* x_tagged;       // activations as tagged words of an earlier exchange (nullptr: plain bf16 x)
  int x_back;                     // that exchange was the x_back-th most recent one (1 = the previous launch)
  // Optional: do not start before an earlier exchange has landed completely in this rank's buffer
  // (the ordering the flag protocol gives, without its fences): every CTA polls these words.
  const uint32_t* after_tagged;   // nullptr: no such wait
  int64_t after_words;
  int after_back;
  // Each flag array has world + 2 words: [0, world) are raised by the peers; word `world` is this
  // rank's epoch (number of exchanges it has published), word world + 1 counts finished CTAs of
  // the running launch.  All ranks issue the same sequence of sharded launches, so "the previous
  // exchange" is the one whose number equals this rank's own epoch: no host-side sequence
  // numbers, and a captured CUDA graph can be replayed.  Tags are derived from the same epoch.
};

// Tag of exchange number e (1-based): 1..65535, never 0 (a zero-filled buffer is invalid).
__host__ __device__ inline uint32_t peer_tag_of(uint32_t e) { return e % 65535u + 1u; }

#ifdef __CUDACC__
// Programmatic dependent launch.  The batch-1 kernels are launched with the stream-serialization
// attribute: the next kernel of the stream may start while this one drains, stream its first
// weight tiles (which no kernel writes) into shared memory, and block in pdl_wait() until the
// previous kernel has completed and its memory is visible -- before it touches activations,
// scratch or outputs.  pdl_trigger() at the top of a kernel lets its own successor do the same.
// Both are no-ops when the launch did not carry the attribute.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), int grid, int block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3((unsigned)block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Consumer side, threads tid < world of one CTA (every CTA does it): the activations were produced
// by the previous exchange, whose number is this rank's own epoch; wait until every rank has
// raised its flag here to that number.  Bounded (about 50 ms of wall time); when it runs out the
// status word is raised and the launch carries on (its result is then meaningless, the host sees
// GGQ_TIMEOUT).
__device__ __forceinline__ void peer_wait_previous(const PeerPublish& pp, int tid, int* status) {
  if (pp.world > 0 && pp.wait_previous && tid < pp.world) {
    const uint32_t* mine = pp.flags[pp.rank];
    const uint32_t target = mine[pp.world];
    bool ok = false;
    uint64_t t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (uint32_t i = 0; i < (1u << 26) && !ok; i++) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine + tid) : "memory");
      ok = (int32_t)(v - target) >= 0;
      if (!ok && (i & 63) == 63) {
        uint64_t t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (t1 - t0 > 50000000ull) break;
      }
    }
    if (!ok && status) atomicOr(status, STATUS_WAIT_EXPIRED);
  }
}
// Eight consecutive activations (as raw bf16 pairs, the layout of a plain uint4 load) from a tagged
// vector: two 16-byte loads of tagged words, repeated until all eight tags match (bounded: about
// 50 ms, then the status word is raised and whatever is there is used).
__device__ __forceinline__ uint4 peer_load8_tagged(const uint32_t* xt, int idx8, uint32_t tag_hi, int* status) {
  const uint32_t* p = xt + 8 * (int64_t)idx8;
  uint4 a, b;
  uint64_t t0 = 0;
  for (uint32_t i = 0;; i++) {
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(p) : "memory");
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(p + 4) : "memory");
    const uint32_t bad = ((a.x ^ tag_hi) | (a.y ^ tag_hi) | (a.z ^ tag_hi) | (a.w ^ tag_hi) |
                          (b.x ^ tag_hi) | (b.y ^ tag_hi) | (b.z ^ tag_hi) | (b.w ^ tag_hi)) >> 16;
    if (!bad) break;
    if ((i & 63) == 0) {
      uint64_t t1;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
      if (i == 0) t0 = t1;
      else if (t1 - t0 > 50000000ull) { if (status) atomicOr(status, STATUS_WAIT_EXPIRED); break; }
    }
  }
  // word pairs (lo16 of even element | lo16 of odd element << 16)
  return make_uint4(__byte_perm(a.x, a.y, 0x5410), __byte_perm(a.z, a.w, 0x5410),
                    __byte_perm(b.x, b.y, 0x5410), __byte_perm(b.z, b.w, 0x5410));
}

// Wait (bounded, like peer_load8_tagged) until all `words` tagged words at `v` carry tag_hi.
// `words` is a multiple of 4 and `v` 16-byte aligned.
__device__ __forceinline__ void peer_wait_tagged(const uint32_t* v, int64_t words, uint32_t tag_hi, int tid, int n_threads,
                                                 int* status) {
  for (int64_t i = 4 * (int64_t)tid; i < words; i += 4 * (int64_t)n_threads) {
    uint64_t t0 = 0;
    for (uint32_t it = 0;; it++) {
      uint4 a;
      asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(v + i) : "memory");
      if (!(((a.x ^ tag_hi) | (a.y ^ tag_hi) | (a.z ^ tag_hi) | (a.w ^ tag_hi)) >> 16)) break;
      if ((it & 63) == 0) {
        uint64_t t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (it == 0) t0 = t1;
        else if (t1 - t0 > 50000000ull) { if (status) atomicOr(status, STATUS_WAIT_EXPIRED); break; }
      }
    }
  }
}

// One output value: locally, or into every rank's copy of the full output when row-sharded.
// out_tag: the running exchange's tag, already shifted into the high half (tagged mode only).
__device__ __forceinline__ void peer_emit(const PeerPublish& pp, void* y, int y_dtype, int64_t row, float v,
                                          uint32_t out_tag = 0) {
  if (pp.world == 0) {
    store_out(y, y_dtype, row, v);
  } else if (pp.tagged) {
    const uint32_t word = out_tag | (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v));
    for (int p = 0; p < pp.world; p++)
      asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(reinterpret_cast<uint32_t*>(pp.y[p]) + pp.row_offset + row),
                   "r"(word) : "memory");
  } else {
    for (int p = 0; p < pp.world; p++) store_out(pp.y[p], y_dtype, pp.row_offset + row, v);
  }
}
// Producer side, called by every thread of every CTA at the end of the kernel: once every CTA of
// the launch has pushed its rows to the peers, raise this rank's flag everywhere.
// Ordering: a CTA's peer stores -> bar.sync -> fence (GPU scope) -> counter; the last CTA reads the
// counter, fences at system scope and releases the flags.  Causality is transitive across the two
// scopes, so a peer that acquires the flag sees every CTA's stores; only one thread of the grid
// pays for a system-scope fence (148 of them at the tail of a 30 us kernel were measurable).
__device__ __forceinline__ void peer_publish(const PeerPublish& pp, int tid, int n_ctas) {
  if (pp.world > 0 && pp.tagged) {
    // tagged mode: nothing to tell the peers; the last CTA advances this rank's own epoch
    __syncthreads();
    if (tid == 0) {
      uint32_t* mine = pp.flags[pp.rank];
      const uint32_t done = atomicAdd(mine + pp.world + 1, 1u);
      if (done == (uint32_t)n_ctas - 1) {
        mine[pp.world + 1] = 0;
        mine[pp.world] = mine[pp.world] + 1;
      }
    }
  } else if (pp.world > 0) {
    __syncthreads();
    if (tid == 0) {
      uint32_t* mine = pp.flags[pp.rank];
      __threadfence();
      const uint32_t done = atomicAdd(mine + pp.world + 1, 1u);
      if (done == (uint32_t)n_ctas - 1) {
        __threadfence_system();
        mine[pp.world + 1] = 0;
        const uint32_t epoch = mine[pp.world] + 1;
        mine[pp.world] = epoch;
        for (int p = 0; p < pp.world; p++)
          asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(pp.flags[p] + pp.rank), "r"(epoch) : "memory");
      }
    }
  }
}
#endif

// Q4_K, batch 1: cp.async-staged tensor-core kernel (gemv_q4k.cu).
bool gemv_q4k_applicable(int64_t N, int64_t K, int M, const void* w, const void* x);
size_t gemv_q4k_workspace_bytes(int64_t N, int sm_count);
cudaError_t gemv_q4k(const uint8_t* w, int64_t N, int64_t K, const void* x, void* y, int y_dtype, void* ws,
                     size_t ws_bytes, int sm_count, int* status, cudaStream_t st,
                     const PeerPublish* peers = nullptr);

// Q6_K, batch 1: the same design on 210-byte superblocks (gemv_q6k.cu).  Scratch as for Q4_K.
bool gemv_q6k_applicable(int64_t N, int64_t K, int M, const void* w, const void* x);
cudaError_t gemv_q6k(const uint8_t* w, int64_t N, int64_t K, const void* x, void* y, int y_dtype, void* ws,
                     size_t ws_bytes, int sm_count, int* status, cudaStream_t st, const PeerPublish* peers = nullptr);

// Q5_K, batch 1: the Q4_K design plus a fifth-bit plane (gemv_q5k.cu).  Scratch as for Q4_K.
bool gemv_q5k_applicable(int64_t N, int64_t K, int M, const void* w, const void* x);
cudaError_t gemv_q5k(const uint8_t* w, int64_t N, int64_t K, const void* x, void* y, int y_dtype, void* ws,
                     size_t ws_bytes, int sm_count, int* status, cudaStream_t st, const PeerPublish* peers = nullptr);

// Tiled kernel for 1 <= M <= 8 (gemv_tile.cu): Q4_K, Q2_K, IQ4_XS and the IQ1/IQ2/IQ3 grid formats.
bool gemv_tile_applicable(int qtype, int64_t N, int64_t K, int M, const void* w, const void* x);
size_t gemv_tile_workspace_bytes(int qtype, int64_t N, int64_t K, int M);
cudaError_t gemv_tile(int qtype, const uint8_t* w, int64_t N, int64_t K, const void* x, int M, void* y, int y_dtype,
                      void* ws, size_t ws_bytes, int sm_count, int* status, const uint8_t* tab, cudaStream_t st,
                      const PeerPublish* peers = nullptr);
int gemv_tile_max_batch(int qtype);     // batch rows per launch (8, Q6_K: 4; 0 if qtype has no tile format)

// Same kernel with the scratch in a file-scope device array (no caller buffer); returns a ggq_status.
int32_t gemv_q4k_static(const void* w, int64_t N, int64_t K, const void* x, void* y, int32_t y_dtype,
                        int sm_count, cudaStream_t st);

// Any block qtype, M <= 16, K a multiple of 32: tensor-core kernel with exact three-way bf16 split
// of the decoded weights (gemv_mma.cu).
bool gemv_mma_applicable(const TypeInfo* ti, int64_t N, int64_t K, int M);
cudaError_t gemv_mma(const TypeInfo* ti, const uint8_t* w, int64_t N, int64_t K, const void* x, int M, void* y,
                     int y_dtype, const uint8_t* tab, cudaStream_t st);

// Larger batches: tcgen05 / TMEM tensor-core kernel with tf32 operands (gemm_tcgen05.cu).
bool gemm_applicable(const TypeInfo* ti, int64_t N, int64_t K, int M);
int gemm_splits(int64_t N, int64_t K, int M, int sm_count);
size_t gemm_workspace_bytes(int64_t N, int64_t K, int M, int sm_count);
cudaError_t gemm_tf32(const TypeInfo* ti, const uint8_t* w, int64_t N, int64_t K, const void* x, int M, void* y,
                      int y_dtype, const uint8_t* tab, int* status, void* ws, size_t ws_bytes, int sm_count,
                      cudaStream_t st);

// tcgen05 GEMM with the weights decoded to float32 exactly and rounded once to bf16 (the reference's own contract
// for its tensor-core GEMM), activations used as they are; Q4_K / Q5_K / Q6_K, any M (gemm_bf16w.cu).
bool gemm_bf16w_applicable(int qtype, int64_t N, int64_t K, int M);
size_t gemm_bf16w_workspace_bytes(int qtype, int64_t N, int64_t K, int M, int sm_count);
cudaError_t gemm_bf16w(int qtype, const uint8_t* w, int64_t N, int64_t K, const void* x, int M, void* y, int y_dtype,
                       int* status, void* ws, size_t ws_bytes, int sm_count, cudaStream_t st);

// Batches of 2 .. 32 rows per launch for Q4_K / Q5_K / Q6_K: all eight MMA columns are batch rows, one MMA
// (pair) per scale group, float32 scales on the accumulators (gemv_wide.cu).  Needs the workspace.
int gemv_wide_max_batch();
bool gemv_wide_applicable(int qtype, int64_t N, int64_t K, int M, const void* w, const void* x);
size_t gemv_wide_workspace_bytes(int qtype, int64_t N, int64_t K, int M, int sm_count);
// ldx: elements between batch rows of x (0: K); peers: row-sharded output with the flag protocol (then y is ignored).
cudaError_t gemv_wide(int qtype, const uint8_t* w, int64_t N, int64_t K, const void* x, int M, void* y, int y_dtype,
                      void* ws, size_t ws_bytes, int sm_count, cudaStream_t st, int64_t ldx = 0,
                      const PeerPublish* peers = nullptr, int* status = nullptr);

// Medium batches of Q4_K / Q5_K / Q6_K: tcgen05 kernel with exact integer codes as bf16 operands and one
// TMEM slot per scale group (gemm_codes.cu).
bool gemm_codes_applicable(int qtype, int64_t N, int64_t K, int M);
size_t gemm_codes_workspace_bytes(int qtype, int64_t N, int64_t K, int M, int sm_count);
cudaError_t gemm_codes(int qtype, const uint8_t* w, int64_t N, int64_t K, const void* x, int M, void* y, int y_dtype,
                       int* status, void* ws, size_t ws_bytes, int sm_count, cudaStream_t st);

// Fixed offsets inside the caller's scratch: GEMV partial slots first, then the arrival counters
// of every kernel (each launch leaves them at zero), then the float32 partial tiles of the GEMM.
constexpr size_t kWsCounterOffset = (size_t)256 * 2 * 64 * sizeof(float);   // 128 KB
constexpr size_t kWsGemmPartialOffset = (size_t)4 << 20;

// Upper bound on the SM count used when sizing scratch (the kernels use the real count).
constexpr int kMaxSmCount = 256;

}  // namespace ggq
