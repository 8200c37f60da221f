// Fused decode + GEMM for medium batches (17 .. a few hundred rows) on the 5th-generation tensor
// cores (tcgen05 / TMEM) with *exact integer codes* as the bf16 A operand -- Q4_K, Q5_K, Q6_K.
//
//   y[M, N] = x[M, K] @ W[N, K]^T
//
// Idea.  A quantized weight is  scale(row, group) * code  (+ offset(row, group)), with small integer
// codes.  A bf16 whose upper byte is 0x00 / 0x80 is linear in its lower byte (0x00vv = v * 2^-133), so
// a masked word of quant bytes *is* a pair of bf16 codes (tile_formats.cuh) and a weight tile costs the
// producers about one instruction per weight -- no float decode, no rounding, half the shared-memory
// bytes of a tf32 tile.  The scales cannot go into the operands, so they go onto the accumulators:
// every scale group along K (32 or 64 codes) is multiplied into its *own* TMEM slot,
//     D_g[128 rows x MT batch columns] = codes_g . x_g ,
// and eight epilogue warps read the slots back (tcgen05.ld), multiply each by its row's float32 group
// scale, add the offset terms (min * sum(x), -32 * sum(x)) and keep the running y in registers.
// The tensor cores do the 2 M N K multiply-adds; the CUDA cores do M N K / 32 scale multiply-adds.
//
// A CTA owns 128 weight rows x MT = 64 batch columns and walks K in phases of 128 codes:
//   producers (8 warps)   raw block bytes of 128 rows arrive through a ring of whole superblocks (cp.async,
//                         two blocks ahead); per phase a thread turns (row, run) into 16-byte groups of eight
//                         codes and stores them into the K-major 128-byte-swizzled A tile; the matching
//                         activations come from a copy prepared by a small kernel (pre-scaled by a power of
//                         two, permuted to the code order, with the per-group sums) and go into the B tile;
//   MMA warp (1 thread)   per phase: one tcgen05.mma.kind::f16 (bf16 x bf16 -> f32) per 16 codes of every
//                         group into the group's TMEM slot (no accumulation across groups), then
//                         tcgen05.commit to the barriers;
//   epilogue (8 warps)    per phase: slots -> registers -> y += a(row, g) * D_g + b(row, g) * sum_g(x).
// Two shared-memory stages and two TMEM buffers (4 slots x 64 columns each) keep the three roles
// overlapped.  With few row tiles K is cut into ranges (grid.z); partial tiles go to scratch and the last
// CTA of a tile adds them in range order (deterministic).
//
// Every mbarrier wait is bounded; a wait that runs out raises the device status word (GGQ_TIMEOUT
// through ggq_read_status), lets the CTA fall through to the common exit, and TMEM is always released.
#include "gemv.cuh"
#include "tile_formats.cuh"

#include <algorithm>

namespace ggq {
namespace gemmc {

constexpr int kTileN = 128;          // weight rows per CTA (MMA M)
constexpr int kMT = 64;              // batch columns per CTA (MMA N)
constexpr int kPhaseK = 128;         // codes per phase = two 128-byte swizzle atoms of bf16
constexpr int kStages = 2;
constexpr int kRawStages = 3;
constexpr int kProducerWarps = 8, kEpilogueWarps = 8;
constexpr int kProducers = kProducerWarps * 32;
constexpr int kThreads = (kProducerWarps + kEpilogueWarps + 1) * 32;
constexpr int kSlots = 4;            // TMEM slots (scale groups) per buffer
constexpr int kTmemCols = 2 * kSlots * kMT;     // 512
constexpr int kMaxSplits = 8;
constexpr int kSmemLimit = 232448;
constexpr uint32_t kSpinLimit = 1u << 18;        // tries of up to 2 us each

constexpr int kABytes = kTileN * kPhaseK * 2;    // 32 KB: two atoms of 128 rows x 128 B
constexpr int kBBytes = kMT * kPhaseK * 2;       // 16 KB: two atoms of 64 rows x 128 B
constexpr int kScBytes = kSlots * kTileN * 8;    // float2 (a, b) per group and row
constexpr int kXsBytes = kSlots * kMT * 4;       // sum(x) per group and batch column
constexpr int kStageBytes = kABytes + kBBytes + kScBytes + kXsBytes;

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
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"      // may sleep up to %3 ns: a waiting warp
      "selp.u32 %0, 1, 0, p;\n\t}"                                          // must not take issue slots from the others
      : "=r"(ok) : "r"(bar), "r"(parity), "r"(2000u) : "memory");
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
// Shared-memory matrix descriptor, K-major, 128-byte swizzle: start address / 16 in bits 0-13, leading
// byte offset (unused for swizzled K-major, 1) in 16-29, stride byte offset (1024 B between 8-row groups)
// / 16 in 32-45, descriptor version 1 in 46-47, layout type 2 (SWIZZLE_128B) in 61-63.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFF) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor for kind::f16 with bf16 operands and float32 accumulation, both operands K-major:
// c_format F32 (bits 4-5 = 1), a / b format BF16 (bits 7-9, 10-12 = 1), N >> 3 in 17-22, M >> 4 in 24-28.
__device__ __forceinline__ uint32_t umma_idesc(int mma_m, int mma_n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(mma_n >> 3) << 17) | ((uint32_t)(mma_m >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// Byte offset of 16-byte chunk c (0..7) of row r in a K-major SWIZZLE_128B atom.
__device__ __forceinline__ uint32_t swz(int r, int c) {
  return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const uint8_t* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void sts_v4(uint32_t a, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ float bf16lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16hi(uint32_t u) { return __uint_as_float(u & 0xFFFF0000u); }
__device__ __forceinline__ float pow2f(int e) { return __uint_as_float((uint32_t)(127 + e) << 23); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}

// Packed float32 pairs (Blackwell executes fma.rn.f32x2 as one instruction).
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  return (uint64_t)__float_as_uint(lo) | ((uint64_t)__float_as_uint(hi) << 32);
}
__device__ __forceinline__ uint64_t pack2u(uint32_t lo, uint32_t hi) { return (uint64_t)lo | ((uint64_t)hi << 32); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}

// The fold of a format as two coefficients: contribution = a * acc + b * sum(x).
template <class F>
__device__ __forceinline__ float2 fold_coeffs(const typename F::Group& g) {
  if constexpr (F::kQt == QT_Q6_K) return make_float2(g.dl, -32.0f * g.dl);
  else return make_float2(g.dl, g.ndm);
}

// ---------------------------------------------------------------------------------------------
// Activation copy: xp[m][block][run][octet][8] bf16 in the code order of format F, scaled by
// 2^(S[m] + x_exp); xs[m][block][run][group] = sum(x) * 2^(S[m] - 133); S[m] puts the row's largest
// magnitude near 2^24..2^120 (96 for any sane tensor).  One CTA per batch row.
template <class F>
__global__ void __launch_bounds__(256)
prepare_x_kernel(const __nv_bfloat16* __restrict__ x, int K, uint4* __restrict__ xp, float* __restrict__ xs, int* __restrict__ S_out) {
  __shared__ int s_max;
  const int m = blockIdx.x, tid = threadIdx.x;
  const int n_oct = (K / 256) * 4 * F::kOct;
  const __nv_bfloat16* xr = x + (int64_t)m * K;
  if (tid == 0) s_max = 0;
  __syncthreads();
  float amax = 0.f;
  for (int i = tid; i < K / 8; i += 256) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(xr) + i);
    const float s = (fabsf(bf16lo(v.x)) + fabsf(bf16hi(v.x))) + (fabsf(bf16lo(v.y)) + fabsf(bf16hi(v.y))) +
                    (fabsf(bf16lo(v.z)) + fabsf(bf16hi(v.z))) + (fabsf(bf16lo(v.w)) + fabsf(bf16hi(v.w)));
    amax = fmaxf(amax, s);
  }
  atomicMax(&s_max, (int)__float_as_uint(amax));
  __syncthreads();
  const int emax = min((s_max >> 23) & 0xFF, 254);
  const int S = (emax > 156 || (emax < 97 && emax > 0)) ? max(8, min(120, 247 - emax)) : 96;
  if (tid == 0) S_out[m] = S;
  const float sum_scale = pow2f(S - 133);
  uint4* dst = xp + (int64_t)m * n_oct;
  float* sums = xs + (int64_t)m * (n_oct / F::kGroupOct);
  for (int o = tid; o < n_oct; o += 256) {
    const int blk = o / (4 * F::kOct), tt = (o / F::kOct) & 3, oo = o % F::kOct;
    int qa, qb;
    F::src_quads(tt, oo, qa, qb);
    const uint2 va = __ldg(reinterpret_cast<const uint2*>(xr + blk * 256 + qa));
    const uint2 vb = __ldg(reinterpret_cast<const uint2*>(xr + blk * 256 + qb));
    const float a0 = bf16lo(va.x), a1 = bf16hi(va.x), a2 = bf16lo(va.y), a3 = bf16hi(va.y);
    const float b0 = bf16lo(vb.x), b1 = bf16hi(vb.x), b2 = bf16lo(vb.y), b3 = bf16hi(vb.y);
    const float up = pow2f(S + F::x_exp(tt, oo));
    dst[o] = make_uint4(pack_bf16(a0 * up, a2 * up), pack_bf16(a1 * up, a3 * up), pack_bf16(b0 * up, b2 * up), pack_bf16(b1 * up, b3 * up));
    float sum = ((a0 + a1) + (a2 + a3)) + ((b0 + b1) + (b2 + b3));
    if ((oo & (F::kGroupOct - 1)) >= F::kSumOct) sum = 0.f;
    if (F::kGroupOct >= 2) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
    if (F::kGroupOct >= 4) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
    if (F::kGroupOct >= 8) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 4);
    if ((oo & (F::kGroupOct - 1)) == 0) sums[o / F::kGroupOct] = sum * sum_scale;
  }
}

// ---------------------------------------------------------------------------------------------
template <class F>
struct Shape {
  static constexpr int kRunK = F::kOct * 8;                        // codes per run: 64 or 128
  static constexpr int kRunsPerPhase = kPhaseK / kRunK;            // 2 or 1
  static constexpr int kPhasesPerBlock = 4 / kRunsPerPhase;        // 2 or 4
  static constexpr int kGroupK = F::kGroupOct * 8;                 // codes per scale group: 32 or 64
  static constexpr int kGroupsPerRun = F::kOct / F::kGroupOct;
  static constexpr int kGroupsPerPhase = kGroupsPerRun * kRunsPerPhase;     // 4 (Q4_K, Q6_K) or 2 (Q5_K)
  static constexpr int kSplit = kProducers / (kTileN * kRunsPerPhase);      // threads per (row, run): 1 or 2
  static constexpr int kOctPerTask = F::kOct / kSplit;
  static constexpr int kRawPitch = (F::kTs + 15 + 15) / 16 * 16 + ((((F::kTs + 15 + 15) / 16) % 2) ? 0 : 16);
  static_assert(kGroupsPerPhase <= kSlots, "a phase's scale groups must fit one TMEM buffer");
  static_assert(kPhaseK % kRunK == 0 && kProducers % (kTileN * kRunsPerPhase) == 0, "phase geometry");
};

template <class F>
__global__ void __launch_bounds__(kThreads, 1)
gemm_codes_kernel(const uint8_t* __restrict__ w, int N, int K, const uint4* __restrict__ xp, const float* __restrict__ xs,
                  const int* __restrict__ S_in, int M, void* __restrict__ y, int y_dtype, int* __restrict__ status,
                  float* __restrict__ partials, int* __restrict__ counters) {
  using Sh = Shape<F>;
  extern __shared__ uint8_t smem_raw[];
  // the swizzle is a function of the address bits: tiles start 1024-byte aligned
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * kTileN, m0 = blockIdx.y * kMT;
  const int splits = gridDim.z, split = blockIdx.z;
  const int SB = K / 256;
  const int blk_begin = (int)((int64_t)split * SB / splits);
  const int n_blocks = (int)((int64_t)(split + 1) * SB / splits) - blk_begin;      // >= 1 (host guarantees)
  const int n_phases = n_blocks * Sh::kPhasesPerBlock;
  const int64_t row_bytes = (int64_t)SB * F::kTs;
  const int n_oct_row = SB * 4 * F::kOct;                                            // 16-byte groups of xp per batch row

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t raw_base = smem_base + kStages * kStageBytes;
  constexpr int kRawBytes = kTileN * Sh::kRawPitch;
  const uint32_t bars = raw_base + kRawStages * kRawBytes;
  auto full_bar = [&](int s) { return bars + 8 * s; };
  auto empty_bar = [&](int s) { return bars + 8 * (kStages + s); };
  auto tfull_bar = [&](int s) { return bars + 8 * (2 * kStages + s); };
  uint8_t* flags = smem + kStages * kStageBytes + kRawStages * kRawBytes + 64;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(flags);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(flags + 4);
  volatile int* last_flag = reinterpret_cast<volatile int*>(flags + 8);

  if (tid == 0) {
    for (int s = 0; s < kStages; s++) {
      mbar_init(full_bar(s), kProducerWarps);
      mbar_init(empty_bar(s), 1 + kEpilogueWarps);     // the MMAs have read the tiles, the epilogue the scales
      mbar_init(tfull_bar(s), 1);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  const int mma_warp = kProducerWarps + kEpilogueWarps;
  if (warp == mma_warp) {   // the MMA warp owns the TMEM allocation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == mma_warp) {
    // ------------------------------- MMA issue -------------------------------
    const uint32_t idesc = umma_idesc(kTileN, kMT);
    for (int ph = 0; ph < n_phases; ph++) {
      const int s = ph & 1, it = ph >> 1;
      // the stage's tiles are written, and (same barrier as the stage's reuse) the epilogue has drained
      // the TMEM buffer this phase overwrites: buffer s was last filled in phase ph - 2, whose epilogue
      // arrival the producers waited for before they refilled stage s
      if (!mbar_wait(full_bar(s), it & 1, abort_flag, status)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (lane == 0) {
        const uint32_t a_addr = smem_base + s * kStageBytes;
        const uint32_t b_addr = a_addr + kABytes;
#pragma unroll
        for (int g = 0; g < Sh::kGroupsPerPhase; g++) {
#pragma unroll
          for (int i = 0; i < Sh::kGroupK / 16; i++) {
            const int kk = g * (Sh::kGroupK / 16) + i;             // 16-code step within the phase
            const uint32_t ao = (kk >> 2) * (kTileN * 128) + (kk & 3) * 32;
            const uint32_t bo = (kk >> 2) * (kMT * 128) + (kk & 3) * 32;
            umma_bf16(tmem_base + (uint32_t)((s * kSlots + g) * kMT), umma_desc(a_addr + ao), umma_desc(b_addr + bo), idesc,
                      i > 0 ? 1u : 0u);
          }
        }
        umma_commit(tfull_bar(s));         // the epilogue may read the slots
        umma_commit(empty_bar(s));         // and the producers may (once the epilogue is done too) refill the stage
      }
      __syncwarp();
    }
  } else if (warp < kProducerWarps) {
    // ------------------------------- producers -------------------------------
    const int ptid = tid;                                            // 0..255
    // raw copies: thread (row = ptid >> 1, half = ptid & 1) copies every second 16-byte piece of its row's block window
    const int crow = ptid >> 1, chalf = ptid & 1;
    const uint8_t* wrow = w + (int64_t)min(n0 + crow, N - 1) * row_bytes;   // rows past the end repeat the last one (never stored)
    auto issue_raw = [&](int b) {
      if (b < n_blocks) {
        const int64_t off = (int64_t)(blk_begin + b) * F::kTs;
        const int skew = (int)(off & 15);
        const uint8_t* p16 = wrow + (off - skew);
        const int pieces = (skew + F::kTs + 15) >> 4;
        const uint32_t dst = raw_base + (b % kRawStages) * kRawBytes + crow * Sh::kRawPitch;
        for (int q = chalf; q < pieces; q += 2) cp_async16(dst + 16 * q, p16 + 16 * q);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    issue_raw(0);
    issue_raw(1);
    // tasks of a phase: (row, run of the phase, part of the run's octets)
    const int t_row = ptid % kTileN, t_rest = ptid / kTileN;
    const int t_run = t_rest / Sh::kSplit, t_part = t_rest % Sh::kSplit;
    tf::Tables tb{};
    bool alive = true;
    int ph = 0;
    constexpr int kBx = kMT * (kPhaseK / 8) / kProducers;             // 16-byte groups of the B tile per thread: 4
    uint4 bx[kBx];
    float xsum = 0.f;
    auto fetch_b = [&](int blk, int pb) {
#pragma unroll
      for (int u = 0; u < kBx; u++) {
        const int q = ptid + u * kProducers;
        const int mr = q >> 4, ch = q & 15;                         // batch row of the tile, 16-byte chunk of the phase
        bx[u] = make_uint4(0, 0, 0, 0);
        if (m0 + mr < M)
          bx[u] = __ldg(xp + (int64_t)(m0 + mr) * n_oct_row + (int64_t)blk * (4 * F::kOct) + pb * (kPhaseK / 8) + ch);
      }
      const int g = ptid / kMT, mr = ptid % kMT;                   // 4 x 64 sums per phase
      xsum = 0.f;
      if (g < Sh::kGroupsPerPhase && m0 + mr < M)
        xsum = __ldg(xs + ((int64_t)(m0 + mr) * SB + blk) * (4 * Sh::kGroupsPerRun) + pb * Sh::kGroupsPerPhase + g);
    };
    for (int b = 0; b < n_blocks; b++) {
      // every producer thread passes every one of these barriers, also after a wait has given up
      asm volatile("cp.async.wait_group 1;" ::: "memory");             // my pieces of block b have landed
      asm volatile("bar.sync 2, %0;" ::"n"(kProducers) : "memory");    // everybody's have; block b - 1 is consumed
      issue_raw(b + 2);                                                // into the slot block b - 1 occupied
      if (!alive) continue;
      const int blk = blk_begin + b;
      const uint32_t braw = raw_base + (b % kRawStages) * kRawBytes + t_row * Sh::kRawPitch + (uint32_t)(((int64_t)blk * F::kTs) & 15);
      const tf::BlockLd ld{braw};
      for (int pb = 0; pb < Sh::kPhasesPerBlock; pb++, ph++) {
        const int s = ph & 1, it = ph >> 1;
        if (it > 0 && !mbar_wait(empty_bar(s), (it - 1) & 1, abort_flag, status)) { alive = false; break; }
        const uint32_t stage = smem_base + s * kStageBytes;
        // ---- B tile (64 batch rows x 16 groups of eight activations) and the groups' sums: fetched one phase
        // ahead (the L2 round trip overlaps the wait above and the code extraction below)
        if (ph == 0) fetch_b(blk, pb);
        // ---- A tile: this thread's octets of (row, run)
        const int run = pb * Sh::kRunsPerPhase + t_run;
        const typename F::Run rr = F::load_run(ld, run);
#pragma unroll
        for (int gi = 0; gi < Sh::kGroupsPerRun; gi++) {
          const typename F::Group gg = F::load_group(ld, rr, run, gi);
          if (t_part == 0) {
            const float2 ab = fold_coeffs<F>(gg);
            *reinterpret_cast<float2*>(smem + s * kStageBytes + kABytes + kBBytes + ((t_run * Sh::kGroupsPerRun + gi) * kTileN + t_row) * 8) = ab;
          }
#pragma unroll
          for (int q = 0; q < F::kGroupOct; q++) {
            const int oo = gi * F::kGroupOct + q;
            if (oo / Sh::kOctPerTask != t_part) continue;
            uint32_t p[4];
            F::octet(gg, q, tb, p);
            const int kpos = t_run * Sh::kRunK + oo * 8;            // code position within the phase
            sts_v4(stage + (kpos >> 6) * (kTileN * 128) + swz(t_row, (kpos >> 3) & 7), p[0], p[1], p[2], p[3]);
          }
        }
#pragma unroll
        for (int u = 0; u < kBx; u++) {
          const int q = ptid + u * kProducers;
          const int mr = q >> 4, ch = q & 15;
          sts_v4(stage + kABytes + (ch >> 3) * (kMT * 128) + swz(mr, ch & 7), bx[u].x, bx[u].y, bx[u].z, bx[u].w);
        }
        *reinterpret_cast<float*>(smem + s * kStageBytes + kABytes + kBBytes + kScBytes + ptid * 4) = xsum;
        // make the generic-proxy stores visible to the tensor core, then one arrival per warp
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(full_bar(s));
        // the next phase's activations (of this block, or of the first phase of the next one)
        if (pb + 1 < Sh::kPhasesPerBlock) fetch_b(blk, pb + 1);
        else if (b + 1 < n_blocks) fetch_b(blk + 1, 0);
      }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  } else {
    // ------------------------------- epilogue -------------------------------
    // warp e: TMEM lanes (rows) 32 (e & 3) .. + 31, batch columns 32 (e >> 2) .. + 31 of every slot
    const int e = warp - kProducerWarps;
    const int quarter = e & 3, chalf = e >> 2;
    const int row = 32 * quarter + lane;
    uint64_t out2[16];             // 32 running outputs as 16 float pairs
#pragma unroll
    for (int i = 0; i < 16; i++) out2[i] = 0ull;
    bool ok = true;
    for (int ph = 0; ph < n_phases && ok; ph++) {
      const int s = ph & 1, it = ph >> 1;
      ok = mbar_wait(tfull_bar(s), it & 1, abort_flag, status);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint8_t* stage = smem + s * kStageBytes;
#pragma unroll
      for (int g = 0; g < Sh::kGroupsPerPhase; g++) {
        uint32_t v[32];
        const uint32_t taddr = tmem_base + ((uint32_t)(32 * quarter) << 16) + (uint32_t)((s * kSlots + g) * kMT + 32 * chalf);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
            "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
              "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
              "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
              "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
            : "r"(taddr));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const float2 ab = *reinterpret_cast<const float2*>(stage + kABytes + kBBytes + (g * kTileN + row) * 8);
        const float4* sx = reinterpret_cast<const float4*>(stage + kABytes + kBBytes + kScBytes + (g * kMT + 32 * chalf) * 4);
        // two batch columns per instruction (fma.rn.f32x2): out = a * D + (b * sum(x) + out)
        const uint64_t a2 = pack2(ab.x, ab.x), b2 = pack2(ab.y, ab.y);
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const float4 s4 = sx[i];
          out2[2 * i] = fma2(a2, pack2u(v[4 * i], v[4 * i + 1]), fma2(b2, pack2(s4.x, s4.y), out2[2 * i]));
          out2[2 * i + 1] = fma2(a2, pack2u(v[4 * i + 2], v[4 * i + 3]), fma2(b2, pack2(s4.z, s4.w), out2[2 * i + 1]));
        }
      }
      // the slots and the stage's scales are consumed
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar(s));
    }
    // ---- store: undo the activations' power-of-two scale, round once
    const int out_row = n0 + row;
    if (ok && out_row < N) {
#pragma unroll
      for (int i = 0; i < 32; i++) {
        const int m = m0 + 32 * chalf + i;
        if (m < M) {
          const float val = __uint_as_float((uint32_t)(out2[i >> 1] >> (32 * (i & 1)))) * pow2f(133 - __ldg(S_in + m));
          if (splits == 1) store_out(y, y_dtype, (int64_t)m * N + out_row, val);
          else partials[((int64_t)split * M + m) * N + out_row] = val;
        }
      }
    }
    if (splits > 1) {
      // every epilogue thread takes part in both barriers, whatever happened above
      __threadfence();
      asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueWarps * 32) : "memory");
      if (e == 0 && lane == 0) {
        int* counter = counters + blockIdx.y * gridDim.x + blockIdx.x;
        const int old = atomicAdd(counter, 1);
        *last_flag = old == splits - 1;
        if (old == splits - 1) *counter = 0;             // nobody else touches it until the next launch
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueWarps * 32) : "memory");
      if (*last_flag && out_row < N) {
        __threadfence();
        for (int i = 0; i < 32; i++) {
          const int m = m0 + 32 * chalf + i;
          if (m < M) {
            float sum = 0.f;
            for (int z = 0; z < splits; z++) sum += __ldcg(partials + ((int64_t)z * M + m) * N + out_row);
            store_out(y, y_dtype, (int64_t)m * N + out_row, sum);
          }
        }
      }
    }
  }
  // common exit: everybody is done with TMEM before it is released
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == mma_warp) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols) : "memory");
  }
}

template <class F>
constexpr int smem_bytes() {
  return kStages * kStageBytes + kRawStages * kTileN * Shape<F>::kRawPitch + 64 + 64 + 1024;
}

static int oct_of(int qtype) { return qtype == QT_Q4_K ? 8 : 16; }
static int group_oct_of(int qtype) { return qtype == QT_Q4_K ? 4 : qtype == QT_Q5_K ? 8 : 4; }

template <class F>
static cudaError_t launch(const uint8_t* w, int64_t N, int64_t K, const void* x, int M, void* y, int y_dtype, int* status,
                          int splits, uint8_t* ws, cudaStream_t st) {
  static_assert(smem_bytes<F>() <= kSmemLimit, "shared memory");
  static std::atomic<bool> attr_done[64];   // setting the attribute twice is harmless, so a flag per device suffices
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(gemm_codes_kernel<F>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<F>());
    if (e != cudaSuccess) return e;
    attr_done[dev].store(true, std::memory_order_release);
  }
  const int64_t n_oct_row = K / 256 * 4 * F::kOct;
  uint8_t* p = ws + kWsGemmPartialOffset;
  uint4* xp = reinterpret_cast<uint4*>(p);
  p += (size_t)M * n_oct_row * 16;
  float* xs = reinterpret_cast<float*>(p);
  p += ((size_t)M * (n_oct_row / F::kGroupOct) * 4 + 255) / 256 * 256;
  int* S = reinterpret_cast<int*>(p);
  p += ((size_t)M * 4 + 255) / 256 * 256;
  float* partials = reinterpret_cast<float*>(p);
  int* counters = reinterpret_cast<int*>(ws + kWsCounterOffset);
  prepare_x_kernel<F><<<M, 256, 0, st>>>((const __nv_bfloat16*)x, (int)K, xp, xs, S);
  dim3 grid((unsigned)((N + kTileN - 1) / kTileN), (unsigned)((M + kMT - 1) / kMT), (unsigned)splits);
  gemm_codes_kernel<F><<<grid, kThreads, smem_bytes<F>(), st>>>(w, (int)N, (int)K, xp, xs, S, M, y, y_dtype, status, partials, counters);
  return cudaPeekAtLastError();
}

}  // namespace gemmc

bool gemm_codes_applicable(int qtype, int64_t N, int64_t K, int M) {
  if (qtype != QT_Q4_K && qtype != QT_Q5_K && qtype != QT_Q6_K) return false;
  const int ts = qtype == QT_Q4_K ? 144 : qtype == QT_Q5_K ? 176 : 210;
  return K > 0 && K % 256 == 0 && (K / 256 * ts) % 16 == 0 && N >= 1 && N < (1ll << 31) - 256 && M >= 1 && M <= 4096 &&
         (int64_t)M * N < (1ll << 40);
}

// How many K ranges a launch uses: the count that minimises (waves of CTAs) / (ranges), with a small
// charge per range for the extra partial traffic.  One CTA is resident per SM.
int gemm_codes_splits(int64_t N, int64_t K, int M, int sm_count) {
  if (sm_count <= 0) sm_count = 148;
  const int64_t tiles = ((N + gemmc::kTileN - 1) / gemmc::kTileN) * ((M + gemmc::kMT - 1) / gemmc::kMT);
  const int64_t SB = K / 256;
  int best = 1;
  double best_cost = 1e30;
  for (int s = 1; s <= gemmc::kMaxSplits && s * 2 <= SB; s++) {
    const double waves = (double)((tiles * s + sm_count - 1) / sm_count);
    const double cost = waves / s + 0.04 * s;
    if (cost < best_cost - 1e-9) { best_cost = cost; best = s; }
  }
  return best;
}

// Scratch: [partial slots 128 KB][arrival counters up to 4 MB][activation copy, its sums and scales][partial tiles]
size_t gemm_codes_workspace_bytes(int qtype, int64_t N, int64_t K, int M, int sm_count) {
  const int64_t n_oct_row = K / 256 * 4 * gemmc::oct_of(qtype);
  const int s = gemm_codes_splits(N, K, M, sm_count);
  size_t need = kWsGemmPartialOffset + (size_t)M * n_oct_row * 16;
  need += ((size_t)M * (n_oct_row / gemmc::group_oct_of(qtype)) * 4 + 255) / 256 * 256;
  need += ((size_t)M * 4 + 255) / 256 * 256;
  if (s > 1) need += (size_t)s * M * N * sizeof(float);
  return (need + 255) / 256 * 256;
}

cudaError_t gemm_codes(int qtype, const uint8_t* w, int64_t N, int64_t K, const void* x, int M, void* y, int y_dtype,
                       int* status, void* ws, size_t ws_bytes, int sm_count, cudaStream_t st) {
  if (!ws || (uintptr_t)ws % 256 || ws_bytes < gemm_codes_workspace_bytes(qtype, N, K, M, sm_count)) return cudaErrorInvalidValue;
  const int splits = gemm_codes_splits(N, K, M, sm_count);
  const int64_t tiles = ((N + gemmc::kTileN - 1) / gemmc::kTileN) * ((M + gemmc::kMT - 1) / gemmc::kMT);
  if (kWsCounterOffset + (size_t)tiles * sizeof(int) > kWsGemmPartialOffset) return cudaErrorInvalidValue;
  uint8_t* base = reinterpret_cast<uint8_t*>(ws);
  switch (qtype) {
    case QT_Q4_K: return gemmc::launch<tf::Q4K>(w, N, K, x, M, y, y_dtype, status, splits, base, st);
    case QT_Q5_K: return gemmc::launch<tf::Q5K>(w, N, K, x, M, y, y_dtype, status, splits, base, st);
    case QT_Q6_K: return gemmc::launch<tf::Q6K>(w, N, K, x, M, y, y_dtype, status, splits, base, st);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace ggq
