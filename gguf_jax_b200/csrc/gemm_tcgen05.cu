// Fused decode + GEMM for larger batches on the 5th-generation tensor cores (tcgen05 / TMEM).
//
//   y[M, N] = x[M, K] @ W[N, K]^T,   W quantized (any block qtype), x bf16, y bf16 / f16 / f32
//
// The weights are the 128-row operand of the MMA (D = W_tile . x^T, so D has one TMEM lane
// per weight row and one TMEM column per batch row); the batch is the N dimension of the
// instruction (16..256 columns).  A CTA owns one tile of 128 weight rows x up to 256 batch
// rows and walks K in blocks of 32 elements:
//
//   producer warps (8)  decode 128 x 32 weights to float32 with the same per-qtype routines as
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
constexpr int kStages = 3;
constexpr int kProducerWarps = 8;
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
                 void* __restrict__ y, int y_dtype, const uint8_t* __restrict__ tab, int* __restrict__ status) {
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
  const int n_kb = K / kBlockK;
  const int64_t row_bytes = (int64_t)(K / BS) * TS;

  const uint32_t bars = smem_u32(smem + L.bars());
  auto full_bar = [&](int s) { return bars + 8 * s; };
  auto empty_bar = [&](int s) { return bars + 8 * (kStages + s); };
  const uint32_t done_bar = bars + 8 * (2 * kStages);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L.bars() + 64);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L.bars() + 72);

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
    const int r = tid & 127, half = tid >> 7;          // weight row in the tile, which 16 of the 32 elements
    const int row = n0 + r;
    const uint8_t* wrow = w + (int64_t)min(row, N - 1) * row_bytes;
    const bool row_ok = row < N;
    bool alive = true;
    for (int kb = 0; kb < n_kb && alive; kb++) {
      const int s = kb % kStages, it = kb / kStages;
      if (it > 0 && !mbar_wait(empty_bar(s), (it - 1) & 1, abort_flag, status)) { alive = false; break; }
      uint8_t* a_tile = smem + s * L.stage_bytes;
      uint8_t* b_tile = a_tile + L.a_bytes;
      // A: decode 16 weights of this thread's row
      const int e0 = kb * kBlockK + 16 * half;
#pragma unroll
      for (int h = 0; h < 2; h++) {
        const int e = e0 + 8 * h;
        float v[8];
        if (row_ok) {
          Dec<QT>::run(wrow + (int64_t)(e / BS) * TS, (e % BS) >> 3, tab, v);
        } else {
#pragma unroll
          for (int i = 0; i < 8; i++) v[i] = 0.f;
        }
        const int c = 4 * half + 2 * h;
        *reinterpret_cast<float4*>(a_tile + swz(r, c)) = make_float4(to_tf32(v[0]), to_tf32(v[1]), to_tf32(v[2]), to_tf32(v[3]));
        *reinterpret_cast<float4*>(a_tile + swz(r, c + 1)) = make_float4(to_tf32(v[4]), to_tf32(v[5]), to_tf32(v[6]), to_tf32(v[7]));
      }
      // B: widen the activations; chunk q = 8 consecutive k of one batch row
      for (int q = tid; q < tile_m * 4; q += kProducerWarps * 32) {
        const int mr = q >> 2, part = q & 3;
        uint4 u = make_uint4(0, 0, 0, 0);
        if (mr < m_here) u = __ldg(reinterpret_cast<const uint4*>(x + (int64_t)(m0 + mr) * K + kb * kBlockK) + part);
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
    if (alive && mbar_wait(done_bar, 0, abort_flag, status)) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int quarter = warp & 3;                     // a warp may read TMEM lanes 32 (warp % 4) .. + 31
      const int col_half = warp >> 2;                   // the two warp groups split the batch columns
      const int out_row = n0 + 32 * quarter + lane;
      const int c_begin = col_half * (tile_m / 2), c_end = c_begin + tile_m / 2;
      for (int c = c_begin; c < c_end; c += 8) {
        uint32_t v[8];
        const uint32_t taddr = tmem_base + ((uint32_t)(32 * quarter) << 16) + (uint32_t)c;
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                     : "r"(taddr));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const int m = m0 + c + i;
          if (c + i < m_here && out_row < N) store_out(y, y_dtype, (int64_t)m * N + out_row, __uint_as_float(v[i]));
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
                          const uint8_t* tab, int* status, cudaStream_t st) {
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
  dim3 grid((unsigned)((N + kTileN - 1) / kTileN), (unsigned)((M + kMaxTileM - 1) / kMaxTileM));
  gemm_tf32_kernel<QT><<<grid, kThreads, smem, st>>>(w, (int)N, (int)K, (const __nv_bfloat16*)x, M, y, y_dtype, tab, status);
  return cudaPeekAtLastError();
}

}  // namespace gemm

bool gemm_applicable(const TypeInfo* ti, int64_t N, int64_t K, int M) {
  return ti && ti->block_elems >= 32 && K % 32 == 0 && K % ti->block_elems == 0 && N >= 1 && N < (1ll << 31) - 256 &&
         K < (1ll << 31) && M >= 1 && (int64_t)M * N < (1ll << 40);
}

cudaError_t gemm_tf32(const TypeInfo* ti, const uint8_t* w, int64_t N, int64_t K, const void* x, int M, void* y,
                      int y_dtype, const uint8_t* tab, int* status, cudaStream_t st) {
  cudaError_t err = cudaErrorInvalidValue;
  dispatch_block_qtype(ti->qtype, [&]<int QT>() { err = gemm::launch<QT>(w, N, K, x, M, y, y_dtype, tab, status, st); });
  return err;
}

}  // namespace ggq
