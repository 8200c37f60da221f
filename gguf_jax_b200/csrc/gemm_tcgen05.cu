// Fused decode + GEMM for larger batches on the 5th-generation tensor cores (tcgen05 / TMEM).
//
//   y[M, N] = x[M, K] @ W[N, K]^T,   W quantized (any block qtype), x bf16, y bf16 / f16 / f32
//
// The weights are the 128-row operand of the MMA (D = W_tile . x^T, so D has one TMEM lane
// per weight row and one TMEM column per batch row); the batch is the N dimension of the
// instruction (16..256 columns).  A CTA owns one tile of 128 weight rows x up to 256 batch
// rows and walks K in blocks of 32 elements:
//
//   producer warps (16) in four groups, one per pipeline stage: a group decodes 128 x 32 weights
//                       to float32 with the same per-qtype routines as
//                       the decode kernel (bit-exact values, rounded to tf32), widen the
//                       32 x M activations from bf16, and store both into shared memory in the
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
#include "ggq_decode.cuh"
#include "gemv.cuh"

namespace ggq {
namespace gemm {

constexpr int kTileN = 128;        // weight rows per CTA (MMA M)
constexpr int kMaxTileM = 256;     // batch rows per CTA (MMA N)
constexpr int kBlockK = 32;        // elements per K block: 32 tf32 = one 128-byte swizzle row
constexpr int kStages = 4;
constexpr int kProducerWarps = 16;
constexpr int kProducers = kProducerWarps * 32;
constexpr int kGroups = kProducerWarps / 4;   // one group of 128 threads per pipeline stage
static_assert(kGroups == kStages, "stage j belongs to producer group j");
constexpr int kPrefetchBytes = 1024;
constexpr int kMaxSplits = 8;
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

struct Layout {
  int a_bytes, b_bytes, stage_bytes;
  __host__ __device__ explicit Layout(int tile_m)
      : a_bytes(kTileN * 128), b_bytes(tile_m * 128), stage_bytes(kTileN * 128 + tile_m * 128) {}
  __host__ __device__ int bars() const { return kStages * stage_bytes; }
  __host__ __device__ int total() const { return bars() + 128 + 1024; }   // + barriers/flags + alignment slack
};

template <int QT>
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
  const Layout L(tile_m);
  const int splits = gridDim.z, split = blockIdx.z;
  const int kb_begin = (int)((int64_t)split * (K / kBlockK) / splits);
  const int n_kb = (int)((int64_t)(split + 1) * (K / kBlockK) / splits) - kb_begin;   // >= 1 (host guarantees)
  const int64_t row_bytes = (int64_t)(K / BS) * TS;

  const uint32_t bars = smem_u32(smem + L.bars());
  auto full_bar = [&](int s) { return bars + 8 * s; };
  auto empty_bar = [&](int s) { return bars + 8 * (kStages + s); };
  const uint32_t done_bar = bars + 8 * (2 * kStages);
  static_assert(8 * (2 * kStages + 1) <= 96, "barriers overlap the flags behind them");
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L.bars() + 96);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L.bars() + 100);
  volatile int* last_flag = reinterpret_cast<volatile int*>(smem + L.bars() + 104);

  if (tid == 0) {
    for (int s = 0; s < kStages; s++) {
      mbar_init(full_bar(s), 4);
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
    // Four groups of four warps; group j fills stage j with K blocks j, j + 4, ...  The 128 x 32
    // weights of a block are 512 decode8 jobs: job = 4 * row + eighth, dealt so that four
    // neighbouring lanes decode the four eighths of one row (their loads share cache lines) and a
    // thread's four jobs are four different rows (independent loads in flight together).
    const int r = tid & 127, group = tid >> 7;
    const int s = group;
    uint8_t* a_tile = smem + s * L.stage_bytes;
    uint8_t* b_tile = a_tile + L.a_bytes;
    const int h = r & 3;
    const uint8_t* wrow[4];
    bool row_ok[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int row = n0 + (r >> 2) + 32 * i;
      wrow[i] = w + (int64_t)min(row, N - 1) * row_bytes;
      row_ok[i] = row < N;
    }
    bool alive = true;
    for (int kb = group, it = 0; kb < n_kb; kb += kGroups, it++) {
      if (it > 0 && !mbar_wait(empty_bar(s), (it - 1) & 1, abort_flag, status)) { alive = false; break; }
      const int k0 = (kb_begin + kb) * kBlockK;
      const int64_t boff = (int64_t)(k0 / BS) * TS;
      // pull the rows' bytes of later K blocks towards L2 while this block is decoded
      if (boff + kPrefetchBytes < row_bytes)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(wrow[h] + boff + kPrefetchBytes));
      float v[4][8];
#pragma unroll
      for (int i = 0; i < 4; i++) {
        if (row_ok[i]) {
          Dec<QT>::run(wrow[i] + boff, ((k0 % BS) >> 3) + h, tab, v[i]);
        } else {
#pragma unroll
          for (int e = 0; e < 8; e++) v[i][e] = 0.f;
        }
      }
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const int rr = (r >> 2) + 32 * i;
        *reinterpret_cast<float4*>(a_tile + swz(rr, 2 * h)) =
            make_float4(to_tf32(v[i][0]), to_tf32(v[i][1]), to_tf32(v[i][2]), to_tf32(v[i][3]));
        *reinterpret_cast<float4*>(a_tile + swz(rr, 2 * h + 1)) =
            make_float4(to_tf32(v[i][4]), to_tf32(v[i][5]), to_tf32(v[i][6]), to_tf32(v[i][7]));
      }
      // B: widen the activations; chunk q = 8 consecutive k of one batch row
      for (int q = r; q < tile_m * 4; q += 128) {
        const int mr = q >> 2, part = q & 3;
        uint4 u = make_uint4(0, 0, 0, 0);
        if (mr < m_here) u = __ldg(reinterpret_cast<const uint4*>(x + (int64_t)(m0 + mr) * K + k0) + part);
        *reinterpret_cast<float4*>(b_tile + swz(mr, 2 * part)) =
            make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xFFFF0000u),
                        __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xFFFF0000u));
        *reinterpret_cast<float4*>(b_tile + swz(mr, 2 * part + 1)) =
            make_float4(__uint_as_float(u.z << 16), __uint_as_float(u.z & 0xFFFF0000u),
                        __uint_as_float(u.w << 16), __uint_as_float(u.w & 0xFFFF0000u));
      }
      // make the generic-proxy stores visible to the tensor core, then one arrival per warp
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(full_bar(s));
    }
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
  const int smem = Layout(tile_m_max).total();
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tf32_kernel<QT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Layout(kMaxTileM).total());
    if (e != cudaSuccess) return e;
    attr_done[dev] = true;
  }
  dim3 grid((unsigned)((N + kTileN - 1) / kTileN), (unsigned)((M + kMaxTileM - 1) / kMaxTileM), (unsigned)splits);
  gemm_tf32_kernel<QT><<<grid, kThreads, smem, st>>>(w, (int)N, (int)K, (const __nv_bfloat16*)x, M, y, y_dtype, tab,
                                                     status, partials, counters);
  return cudaPeekAtLastError();
}

}  // namespace gemm

bool gemm_applicable(const TypeInfo* ti, int64_t N, int64_t K, int M) {
  return ti && ti->block_elems >= 32 && K % 32 == 0 && K % ti->block_elems == 0 && N >= 1 && N < (1ll << 31) - 256 &&
         K < (1ll << 31) && M >= 1 && (int64_t)M * N < (1ll << 40);
}

// How many K ranges a launch uses: the count that minimises (waves of CTAs) / (ranges), with a
// small charge per range for the extra partial traffic.  One CTA is resident per SM.
int gemm_splits(int64_t N, int64_t K, int M, int sm_count) {
  if (sm_count <= 0) sm_count = 148;
  const int64_t tiles = ((N + gemm::kTileN - 1) / gemm::kTileN) * ((M + gemm::kMaxTileM - 1) / gemm::kMaxTileM);
  const int64_t n_kb = K / gemm::kBlockK;
  int best = 1;
  double best_cost = 1e30;
  for (int s = 1; s <= gemm::kMaxSplits && s * 8 <= n_kb; s++) {
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
