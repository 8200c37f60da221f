// Fused decode + GEMM for larger batches on the 5th-generation tensor cores (tcgen05 / TMEM).
//
//   y[M, N] = x[M, K] @ W[N, K]^T,   W quantized (any block qtype), x bf16, y bf16 / f16 / f32
//
// The weights are the 128-row operand of the MMA (D = W_tile . x^T, so D has one TMEM lane
// per weight row and one TMEM column per batch row); the batch is the N dimension of the
// instruction (16..256 columns).  A CTA owns one tile of 128 weight rows x up to 256 batch
// rows and walks K in blocks of 32 elements:
//
//   producer warps (16) first bring the raw block bytes of 128 rows x 256 weights into a ring in
//                       shared memory with 16-byte cp.async copies (two chunks ahead; rows of a
//                       GGUF tensor are only 2-byte aligned in general, so a copy takes the
//                       16-byte aligned window around the row's bytes and the decoder reads at
//                       the row's offset in it), then decode them from there -- shared-memory
//                       latency instead of a cache miss per block -- with the same per-qtype
//                       routines as the decode kernel (bit-exact values, rounded to tf32), widen
//                       the 32 x M activations from bf16 (prefetched one K block ahead), and
//                       store both into shared memory in the
//                       canonical K-major 128-byte-swizzled layout the MMA reads;
//   MMA warp (1 thread) issues four tcgen05.mma.kind::tf32 (K = 8 each) per K block,
//                       accumulating in TMEM, and tcgen05.commit hands the stage back;
//   epilogue            the producer warps read the accumulator with tcgen05.ld, round once to
//                       the output type and store y (32 consecutive n per warp and batch row).
//
// tf32 rather than bf16 operands: the contract is relative L2 <= 2e-3 against the float32
// product *including* the output rounding to bf16 (about 1.6e-3 by itself); bf16 weights
// would add another 1.6e-3 and miss it, tf32 weights (11 significant bits, rounded to
// nearest here) add 3e-4.  bf16 activations are exact in tf32.
//
// Small N leaves most SMs without a tile, so K is cut into `splits` ranges (grid.z): every CTA
// accumulates its range in TMEM, writes a float32 partial tile to the caller's scratch, and the
// last CTA of a tile to arrive adds the partials in range order (deterministic) and rounds once.
// The arrival counters return to zero, the partial area needs no initialisation.
//
// Every wait on an mbarrier is bounded; a wait that runs out raises the device status word
// (GGQ_TIMEOUT through ggq_read_status), lets the CTA fall through to the common exit, and
// the TMEM allocation is always released.
#define GGQ_DECODE_GENERIC_LOADS   // the decoders read staged blocks from shared memory
#include <algorithm>

#include "ggq_decode.cuh"
#include "gemv.cuh"

namespace ggq {
namespace gemm {

constexpr int kTileN = 128;        // weight rows per CTA (MMA M)
constexpr int kMaxTileM = 256;     // batch rows per CTA (MMA N)
constexpr int kBlockK = 32;        // elements per K block: 32 tf32 = one 128-byte swizzle row
constexpr int kMaxStages = 4;       // MMA operand stages (fewer when the batch tile is large)
constexpr int kProducerWarps = 16;
constexpr int kProducers = kProducerWarps * 32;
constexpr int kChunkK = 256;        // weights per row in one raw chunk
constexpr int kKbPerChunk = kChunkK / kBlockK;
constexpr int kRawStages = 3;       // raw chunks in shared memory: one being decoded, two in flight
constexpr int kMaxSplits = 8;
constexpr int kSmemLimit = 232448;
constexpr int kThreads = (kProducerWarps + 1) * 32;
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait; returns false (and raises the flags) when it gives up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status) {
  if (*abort_flag) return false;
  for (uint32_t i = 0; i < kSpinLimit; i++) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255) == 255 && *abort_flag) return false;
  }
  *abort_flag = 1;
  if (status) atomicOr(status, STATUS_WAIT_EXPIRED);
  return false;
}

// Shared-memory matrix descriptor, K-major, 128-byte swizzle: start address / 16 in bits 0-13,
// leading byte offset (unused for swizzled K-major, set to 1) in 16-29, stride byte offset
// (1024 B between 8-row groups) / 16 in 32-45, descriptor version 1 in 46-47, layout type 2
// (SWIZZLE_128B) in 61-63.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFF) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor for kind::tf32, float32 accumulate, both operands K-major:
// c_format F32 (bits 4-5 = 1), a/b format TF32 (bits 7-9, 10-12 = 2), N >> 3 in 17-22, M >> 4 in 24-28.
__device__ __forceinline__ uint32_t umma_idesc(int mma_m, int mma_n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(mma_n >> 3) << 17) | ((uint32_t)(mma_m >> 4) << 24);
}
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Byte offset of 16-byte chunk c (0..7) of row r in a K-major SWIZZLE_128B tile.
__device__ __forceinline__ uint32_t swz(int r, int c) {
  return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4));
}
// float32 -> tf32 container, round to nearest (ties away): the MMA ignores the low 13 bits.
__device__ __forceinline__ float to_tf32(float v) { return __uint_as_float(__float_as_uint(v) + 0x1000u); }

// Raw bytes of one row in one chunk, and the pitch of its 16-byte aligned window.
template <int QT> constexpr int raw_row_bytes() { return kChunkK / block_elems_of(QT) * block_bytes_of(QT); }
template <int QT> constexpr int raw_pitch() { return (raw_row_bytes<QT>() + 15 + 15) / 16 * 16; }

struct Layout {
  int a_bytes, b_bytes, stage_bytes, stages, raw_bytes;
  __host__ __device__ Layout(int tile_m, int pitch)
      : a_bytes(kTileN * 128), b_bytes(tile_m * 128), stage_bytes(kTileN * 128 + tile_m * 128),
        raw_bytes(kRawStages * kTileN * pitch) {
    stages = (kSmemLimit - raw_bytes - 256 - 1024) / stage_bytes;
    if (stages > kMaxStages) stages = kMaxStages;
  }
  __host__ __device__ int raw() const { return stages * stage_bytes; }
  __host__ __device__ int bars() const { return raw() + raw_bytes; }
  __host__ __device__ int total() const { return bars() + 256 + 1024; }   // + barriers/flags + alignment slack
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const uint8_t* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

// BIG: the batch tile has more than 128 rows, i.e. two 16-byte activation pieces per producer
// thread and K block instead of one.
template <int QT, bool BIG>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tf32_kernel(const uint8_t* __restrict__ w, int N, int K, const __nv_bfloat16* __restrict__ x, int M,
                 void* __restrict__ y, int y_dtype, const uint8_t* __restrict__ tab, int* __restrict__ status,
                 float* __restrict__ partials, int* __restrict__ counters) {
  constexpr int BS = block_elems_of(QT), TS = block_bytes_of(QT);
  extern __shared__ uint8_t smem_raw[];
  // the swizzle is a function of the address bits, so the tiles must start 1024-byte aligned
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * kTileN;
  const int m0 = blockIdx.y * kMaxTileM;
  const int m_here = min(kMaxTileM, M - m0);
  const int tile_m = max(16, (m_here + 15) & ~15);           // MMA N: multiple of 16
  int tmem_cols = 32;
  while (tmem_cols < tile_m) tmem_cols <<= 1;
  constexpr int RB = raw_row_bytes<QT>(), PITCH = raw_pitch<QT>();
  const Layout L(tile_m, PITCH);
  const int kStages = L.stages;
  const int splits = gridDim.z, split = blockIdx.z;
  // K ranges are whole chunks of 256 weights
  const int chunk_begin = (int)((int64_t)split * (K / kChunkK) / splits);
  const int n_chunks = (int)((int64_t)(split + 1) * (K / kChunkK) / splits) - chunk_begin;   // >= 1 (host guarantees)
  const int n_kb = n_chunks * kKbPerChunk;
  const int64_t row_bytes = (int64_t)(K / BS) * TS;

  const uint32_t bars = smem_u32(smem + L.bars());
  auto full_bar = [&](int s) { return bars + 8 * s; };
  auto empty_bar = [&](int s) { return bars + 8 * (kStages + s); };
  const uint32_t done_bar = bars + 8 * (2 * kStages);
  static_assert(8 * (2 * kMaxStages + 1) <= 96, "barriers overlap the flags behind them");
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L.bars() + 96);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L.bars() + 100);
  volatile int* last_flag = reinterpret_cast<volatile int*>(smem + L.bars() + 104);

  if (tid == 0) {
    for (int s = 0; s < kStages; s++) {
      mbar_init(full_bar(s), kProducerWarps);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(done_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kProducerWarps) {   // the MMA warp owns the TMEM allocation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == kProducerWarps) {
    // ------------------------------- MMA issue -------------------------------
    const uint32_t idesc = umma_idesc(kTileN, tile_m);
    for (int kb = 0; kb < n_kb; kb++) {
      const int s = kb % kStages, it = kb / kStages;
      if (!mbar_wait(full_bar(s), it & 1, abort_flag, status)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (lane == 0) {
        const uint32_t a_addr = smem_u32(smem + s * L.stage_bytes);
        const uint32_t b_addr = a_addr + L.a_bytes;
#pragma unroll
        for (int k8 = 0; k8 < kBlockK / 8; k8++)
          umma_tf32(tmem_base, umma_desc(a_addr + 32 * k8), umma_desc(b_addr + 32 * k8), idesc,
                    (kb > 0 || k8 > 0) ? 1u : 0u);
        umma_commit(empty_bar(s));          // the stage is free once these MMAs have read it
        if (kb == n_kb - 1) umma_commit(done_bar);
      }
      __syncwarp();
    }
  } else {
    // ------------------------------- producers -------------------------------
    // Thread (r, h): weight row r of the tile, eighth h of a 32-weight K block; it also copies
    // pieces h, h + 4, ... of row r's raw window.
    const int r = tid >> 2, h = tid & 3;
    const int row = min(n0 + r, N - 1);                       // rows past the end repeat the last one (never stored)
    const uint8_t* wsrc = w + (int64_t)row * row_bytes + (int64_t)chunk_begin * RB;
    // reads stop at the 16-byte boundary at or after the end of the tensor (any device allocation
    // extends that far)
    const uint8_t* const w_stop = w + (((int64_t)N * row_bytes + 15) & ~(int64_t)15);
    uint8_t* const raw_ring = smem + L.raw();
    auto issue_chunk = [&](int c) {
      if (c < n_chunks) {
        const uint8_t* p = wsrc + (int64_t)c * RB;
        const int skew = (int)((uintptr_t)p & 15);
        const uint8_t* p16 = p - skew;
        const int pieces = (skew + RB + 15) >> 4;
        const uint32_t dst = smem_u32(raw_ring + ((c % kRawStages) * kTileN + r) * PITCH);
        for (int q = h; q < pieces; q += 4)
          if (p16 + 16 * q + 16 <= w_stop) cp_async16(dst + 16 * q, p16 + 16 * q);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    issue_chunk(0);
    issue_chunk(1);
    // activations, fetched XD K blocks ahead into a small register ring (the loads come from L2
    // and a K block is only a few hundred cycles of work)
    constexpr int XP = BIG ? 2 : 1, XD = BIG ? 2 : 4;
    const int k_first = chunk_begin * kChunkK;
    uint4 xr[XD][XP];
    auto fetch_x = [&](int kb, uint4 (&dst)[XP]) {
#pragma unroll
      for (int u = 0; u < XP; u++) {
        const int q = tid + u * kProducers;
        const int mr = q >> 2, part = q & 3;
        dst[u] = make_uint4(0, 0, 0, 0);
        if (q < tile_m * 4 && mr < m_here && kb < n_kb)
          dst[u] = __ldg(reinterpret_cast<const uint4*>(x + (int64_t)(m0 + mr) * K + k_first + kb * kBlockK) + part);
      }
    };
#pragma unroll
    for (int d = 0; d < XD; d++) fetch_x(d, xr[d]);
    bool alive = true;
    int kb = 0;
    for (int c = 0; c < n_chunks; c++) {
      // every producer thread passes every one of these barriers, also after a wait has given up
      asm volatile("cp.async.wait_group 1;" ::: "memory");    // my copies of chunk c have landed
      asm volatile("bar.sync 2, %0;" ::"n"(kProducers) : "memory");   // everybody's have; chunk c-1 is decoded
      issue_chunk(c + 2);                                      // into the slot chunk c-1 occupied
      if (!alive) continue;
      const uint8_t* rawrow = raw_ring + ((c % kRawStages) * kTileN + r) * PITCH +
                              ((uintptr_t)(wsrc + (int64_t)c * RB) & 15);
#pragma unroll
      for (int k8 = 0; k8 < kKbPerChunk; k8++, kb++) {
        const int s = kb % kStages, it = kb / kStages;
        if (it > 0 && !mbar_wait(empty_bar(s), (it - 1) & 1, abort_flag, status)) { alive = false; break; }
        uint8_t* a_tile = smem + s * L.stage_bytes;
        uint8_t* b_tile = a_tile + L.a_bytes;
        // A: eight weights of row r
        {
          const int e = k8 * kBlockK + 8 * h;                  // element within the chunk
          float v[8];
          Dec<QT>::run(rawrow + (e / BS) * TS, (e % BS) >> 3, tab, v);
          *reinterpret_cast<float4*>(a_tile + swz(r, 2 * h)) =
              make_float4(to_tf32(v[0]), to_tf32(v[1]), to_tf32(v[2]), to_tf32(v[3]));
          *reinterpret_cast<float4*>(a_tile + swz(r, 2 * h + 1)) =
              make_float4(to_tf32(v[4]), to_tf32(v[5]), to_tf32(v[6]), to_tf32(v[7]));
        }
        // B: widen the activations; piece q = 8 consecutive k of one batch row
#pragma unroll
        for (int d = 0; d < XD; d++) {
          if ((k8 % XD) == d) {                              // k8 is a compile-time constant after unrolling
#pragma unroll
            for (int u = 0; u < XP; u++) {
              const int q = tid + u * kProducers;
              if (q < tile_m * 4) {
                const int mr = q >> 2, part = q & 3;
                const uint4 xv = xr[d][u];
                *reinterpret_cast<float4*>(b_tile + swz(mr, 2 * part)) =
                    make_float4(__uint_as_float(xv.x << 16), __uint_as_float(xv.x & 0xFFFF0000u),
                                __uint_as_float(xv.y << 16), __uint_as_float(xv.y & 0xFFFF0000u));
                *reinterpret_cast<float4*>(b_tile + swz(mr, 2 * part + 1)) =
                    make_float4(__uint_as_float(xv.z << 16), __uint_as_float(xv.z & 0xFFFF0000u),
                                __uint_as_float(xv.w << 16), __uint_as_float(xv.w & 0xFFFF0000u));
              }
            }
            fetch_x(kb + XD, xr[d]);
          }
        }
        // make the generic-proxy stores visible to the tensor core, then one arrival per warp
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(full_bar(s));
      }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    // ------------------------------- epilogue -------------------------------
    // A warp may read TMEM lanes 32 (warp % 4) .. + 31; the four warp groups deal the batch
    // columns among themselves in chunks of 8.
    const int quarter = warp & 3, cgroup = warp >> 2;
    const int out_row = n0 + 32 * quarter + lane;
    const bool ok = alive && mbar_wait(done_bar, 0, abort_flag, status);
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      for (int c = 8 * cgroup; c < tile_m; c += 32) {
        uint32_t v[8];
        const uint32_t taddr = tmem_base + ((uint32_t)(32 * quarter) << 16) + (uint32_t)c;
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                     : "r"(taddr));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const int m = m0 + c + i;
          if (c + i < m_here && out_row < N) {
            if (splits == 1) store_out(y, y_dtype, (int64_t)m * N + out_row, __uint_as_float(v[i]));
            else partials[((int64_t)split * M + m) * N + out_row] = __uint_as_float(v[i]);
          }
        }
      }
    }
    if (splits > 1) {
      // every producer thread takes part in both barriers, whatever happened above
      __threadfence();
      asm volatile("bar.sync 1, %0;" ::"n"(kProducers) : "memory");
      if (tid == 0) {
        int* counter = counters + blockIdx.y * gridDim.x + blockIdx.x;
        const int old = atomicAdd(counter, 1);
        *last_flag = old == splits - 1;
        if (old == splits - 1) *counter = 0;             // nobody else touches it until the next launch
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kProducers) : "memory");
      if (*last_flag) {
        __threadfence();
        for (int c = 8 * cgroup; c < tile_m; c += 32) {
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const int m = m0 + c + i;
            if (c + i < m_here && out_row < N) {
              float sum = 0.f;
              for (int z = 0; z < splits; z++) sum += __ldcg(partials + ((int64_t)z * M + m) * N + out_row);
              store_out(y, y_dtype, (int64_t)m * N + out_row, sum);
            }
          }
        }
      }
    }
  }
  // common exit: everybody is done with TMEM before it is released
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == kProducerWarps) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)tmem_cols) : "memory");
  }
}

template <int QT>
static cudaError_t launch(const uint8_t* w, int64_t N, int64_t K, const void* x, int M, void* y, int y_dtype,
                          const uint8_t* tab, int* status, int splits, float* partials, int* counters,
                          cudaStream_t st) {
  const int tile_m_max = M >= kMaxTileM ? kMaxTileM : ((M + 15) & ~15) < 16 ? 16 : ((M + 15) & ~15);
  const Layout lay(tile_m_max, raw_pitch<QT>());
  if (lay.stages < 2) return cudaErrorInvalidValue;
  // Every CTA lays its shared memory out for its own batch tile: the last tile of a batch that is not a multiple of
  // kMaxTileM is narrower, fits more stages, and can need more bytes than the full tiles do.
  int smem = lay.total();
  if (M > kMaxTileM && M % kMaxTileM) {
    const int last = std::max(16, (M % kMaxTileM + 15) & ~15);
    smem = std::max(smem, Layout(last, raw_pitch<QT>()).total());
  }
  static std::atomic<bool> attr_done[64];   // setting the attribute twice is harmless, so a flag per device suffices
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tf32_kernel<QT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gemm_tf32_kernel<QT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e != cudaSuccess) return e;
    attr_done[dev].store(true, std::memory_order_release);
  }
  dim3 grid((unsigned)((N + kTileN - 1) / kTileN), (unsigned)((M + kMaxTileM - 1) / kMaxTileM), (unsigned)splits);
  if (tile_m_max > 128)
    gemm_tf32_kernel<QT, true><<<grid, kThreads, smem, st>>>(w, (int)N, (int)K, (const __nv_bfloat16*)x, M, y, y_dtype,
                                                             tab, status, partials, counters);
  else
    gemm_tf32_kernel<QT, false><<<grid, kThreads, smem, st>>>(w, (int)N, (int)K, (const __nv_bfloat16*)x, M, y, y_dtype,
                                                              tab, status, partials, counters);
  return cudaPeekAtLastError();
}

}  // namespace gemm

bool gemm_applicable(const TypeInfo* ti, int64_t N, int64_t K, int M) {
  return ti && ti->block_elems >= 32 && K % gemm::kChunkK == 0 && N >= 1 && N < (1ll << 31) - 256 &&
         K < (1ll << 31) && M >= 1 && (int64_t)M * N < (1ll << 40);
}

// How many K ranges a launch uses: the count that minimises (waves of CTAs) / (ranges), with a
// small charge per range for the extra partial traffic.  One CTA is resident per SM.
int gemm_splits(int64_t N, int64_t K, int M, int sm_count) {
  if (sm_count <= 0) sm_count = 148;
  const int64_t tiles = ((N + gemm::kTileN - 1) / gemm::kTileN) * ((M + gemm::kMaxTileM - 1) / gemm::kMaxTileM);
  const int64_t n_chunks = K / gemm::kChunkK;
  int best = 1;
  double best_cost = 1e30;
  for (int s = 1; s <= gemm::kMaxSplits && s * 2 <= n_chunks; s++) {
    const double waves = (double)((tiles * s + sm_count - 1) / sm_count);
    const double cost = waves / s + 0.04 * s;
    if (cost < best_cost - 1e-9) { best_cost = cost; best = s; }
  }
  return best;
}

// Scratch of the K-split: [Q4_K GEMV partial slots, 128 KB][arrival counters up to 4 MB]
// [float32 partial tiles: splits x M x N].  The counter area is shared with the GEMV kernels
// (all of them leave their counters at zero); the partial tiles start at a fixed offset so that
// no launch ever writes floats where another shape keeps counters.
size_t gemm_workspace_bytes(int64_t N, int64_t K, int M, int sm_count) {
  const int s = gemm_splits(N, K, M, sm_count);
  if (s <= 1) return 0;
  return kWsGemmPartialOffset + (size_t)s * (size_t)M * (size_t)N * sizeof(float);
}

cudaError_t gemm_tf32(const TypeInfo* ti, const uint8_t* w, int64_t N, int64_t K, const void* x, int M, void* y,
                      int y_dtype, const uint8_t* tab, int* status, void* ws, size_t ws_bytes, int sm_count,
                      cudaStream_t st) {
  int splits = gemm_splits(N, K, M, sm_count);
  const int64_t tiles = ((N + gemm::kTileN - 1) / gemm::kTileN) * ((M + gemm::kMaxTileM - 1) / gemm::kMaxTileM);
  if (splits > 1 && (!ws || (uintptr_t)ws % 256 || ws_bytes < gemm_workspace_bytes(N, K, M, sm_count) ||
                     kWsCounterOffset + (size_t)tiles * sizeof(int) > kWsGemmPartialOffset))
    splits = 1;                                           // no usable scratch: one range per tile
  float* partials = splits > 1 ? reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ws) + kWsGemmPartialOffset) : nullptr;
  int* counters = splits > 1 ? reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(ws) + kWsCounterOffset) : nullptr;
  cudaError_t err = cudaErrorInvalidValue;
  dispatch_block_qtype(ti->qtype, [&]<int QT>() {
    err = gemm::launch<QT>(w, N, K, x, M, y, y_dtype, tab, status, splits, partials, counters, st);
  });
  return err;
}

}  // namespace ggq
