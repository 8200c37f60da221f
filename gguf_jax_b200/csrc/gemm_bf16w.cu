// Fused decode + GEMM for batches from a few dozen to thousands of rows on the 5th-generation tensor cores
// (tcgen05 / TMEM): Q4_K, Q5_K and Q6_K weights are decoded to float32 (Q6_K exactly as the decode kernel does;
// Q4_K / Q5_K to within 2^-20 of a weight, see decode4), rounded once to bf16 and written straight into the K-major, 128-byte-swizzled A tile in shared memory;
// the activations are used as they are (bf16, K-major: the B tile is a copy of 64 consecutive elements per
// batch row); tcgen05.mma.kind::f16 accumulates the whole K range of the CTA in TMEM in float32.
//
//   y[M, N] = x[M, K] @ bf16(W)[N, K]^T
//
// Precision.  This is the reference's own contract for its tensor-core GEMM and for its fallback (weights
// rounded to the activation dtype before the product): relative error of a weight 2^-9, of the result about
// 2e-3 on random data.  The small-batch kernels of this library (exact integer codes, float32 scales) do
// not round the weights at all; this kernel trades that for tensor-core throughput.
//
// A CTA owns 128 weight rows x MT batch columns (MT = 32 .. 256 = the MMA N, or 512 as two MMAs of 256 columns into
// the two halves of the 512-column tensor memory) and a range of K:
//   producers (16 warps)  raw block bytes of the 128 rows arrive through a ring of whole superblocks
//                         (cp.async, two superblocks ahead); per superblock a thread unpacks the float32 scale and
//                         offset of its groups once; per stage of 64 weights it decodes 16 weights of one row (one
//                         byte permute and one FMA per weight, packed conversion to bf16) and stores two 16-byte
//                         chunks of the A tile; with an even number of stages two stages are filled per round;
//   loaders (4 warps)     copy the stage's 64 activations of every batch row of the tile straight from x into the
//                         swizzled B tile (cp.async, 16 bytes), two stages ahead of announcing them;
//   MMA warp (1 thread)   per stage four tcgen05.mma (K = 16 each) into the same TMEM accumulator,
//                         tcgen05.commit frees the stage;
//   epilogue              the producer warps, once their last stage is written: tcgen05.ld -> y, or, when K
//                         is split over several CTAs (few row tiles), -> partial tiles in the scratch that the
//                         last CTA of a tile adds in range order (deterministic).
// Every mbarrier wait is bounded; a wait that runs out raises the device status word (GGQ_TIMEOUT through
// ggq_read_status), the CTA falls through to the common exit and TMEM is always released.
#include "gemv.cuh"

#include <cuda.h>

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>

namespace ggq {
namespace gemmb {

constexpr int kTileN = 128;                  // weight rows per CTA (MMA M)
constexpr int kStageK = 64;                  // weights per stage: one 128-byte swizzle atom of bf16 per row
constexpr int kProducerWarps = 16;
constexpr int kProducers = kProducerWarps * 32;
constexpr int kLoaderWarps = 4;              // copy the activations' B tiles
constexpr int kThreads = kProducers + 32 + 32 * kLoaderWarps;    // + the MMA warp + the loaders
constexpr int kABytes = kTileN * 128;        // 16 KB
constexpr int kMaxSplits = 16;
constexpr int kSmemLimit = 232448;
constexpr uint32_t kSpinLimit = 1u << 22;    // tries (each returns after a short hardware-defined wait)

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
// Bounded wait; returns false (and raises the flags) when it gives up.  (Pausing between tries with nanosleep was
// measured: the sleeps overshoot and stall the pipeline, up to 2 x slower.)
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*abort_flag) return false;
  for (uint32_t i = 0; i < kSpinLimit; i++) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255) == 255 && *abort_flag) return false;
  }
  *abort_flag = 1;
  if (status) atomicOr(status, STATUS_WAIT_EXPIRED);
  return false;
}
// Shared-memory matrix descriptor, K-major, 128-byte swizzle: start address / 16 in bits 0-13, leading byte
// offset (unused for swizzled K-major, 1) in 16-29, stride byte offset (1024 B between 8-row groups) / 16 in
// 32-45, descriptor version 1 in 46-47, layout type 2 (SWIZZLE_128B) in 61-63.
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
// Byte offset of 16-byte chunk c (0..7) of row r in a K-major SWIZZLE_128B tile of 128-byte rows.
__device__ __forceinline__ uint32_t swz(int r, int c) {
  return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const uint8_t* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void sts_v4(uint32_t a, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t a) { uint32_t v; asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a)); return v; }
__device__ __forceinline__ uint32_t lds_u16(uint32_t a) { uint32_t v; asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(a)); return v; }
__device__ __forceinline__ uint32_t lds_u8(uint32_t a) { uint32_t v; asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a)); return v; }
// four consecutive bytes at a 2-byte aligned shared address
__device__ __forceinline__ uint32_t ldw2(uint32_t a) {
  if (a & 2) return __byte_perm(lds_u32(a - 2), lds_u32(a + 2), 0x5432);
  return lds_u32(a);
}
__device__ __forceinline__ float h2f(uint32_t bits) { return __half2float(__ushort_as_half((unsigned short)bits)); }
// byte SEL of v as a float, exact: the bits 0x4B0000vv are 2^23 + v
template <int SEL>
__device__ __forceinline__ float byte_to_float(uint32_t v) {
  return __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7440 + SEL)) - 8388608.0f;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}
// byte SEL of v plus 128 as a float, exact, in one instruction: the bits 0x43vv0000 are 128 + v for v < 128
template <int SEL>
__device__ __forceinline__ float byte_plus_128(uint32_t v) {
  return __uint_as_float(__byte_perm(v, 0x43000000u, 0x7044 + (SEL << 8)));
}
// four code bytes (each < 128) -> four weights a * code + b -> two words of bf16 pairs.  One permute and one FMA per
// weight: a * (128 + code) + c with c = b - 128 a.  The FMA rounds once; c is exact for Q6_K (b = -32 a) and carries
// one float32 rounding of about |a| 2^-17 for Q4_K / Q5_K, i.e. 2^-20 of a typical weight, before the bf16 rounding.
__device__ __forceinline__ void decode4(uint32_t codes, float a, float c, uint32_t& lo, uint32_t& hi) {
  lo = pack_bf16(fmaf(a, byte_plus_128<0>(codes), c), fmaf(a, byte_plus_128<1>(codes), c));
  hi = pack_bf16(fmaf(a, byte_plus_128<2>(codes), c), fmaf(a, byte_plus_128<3>(codes), c));
}

// ---------------------------------------------------------------------------------------------
// Formats.  A thread owns quarter qd (16 weights) of every 64-weight stage of one row.  prep() reads the
// superblock's header once and leaves the float32 scale / offset pairs of the thread's groups; decode16()
// turns the 16 weights [64 s + 16 qd, + 16) into eight words of bf16 pairs.  blk = shared address of the
// superblock's bytes (2-byte aligned for Q6_K, 16-byte aligned otherwise).

__device__ __forceinline__ uint4 lds_v4(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
template <int SEL>
__device__ __forceinline__ float byte_of(uint32_t lo, uint32_t hi, int which) {       // byte SEL of lo (which = 0) or hi
  return byte_to_float<SEL>(which ? hi : lo);
}

struct FQ4K {
  static constexpr int kQt = QT_Q4_K, kTs = 144, kRawPitch = 176;
  static constexpr bool kSplitChunks = false;
  struct Prep { float a[4], b[4]; };          // group 2 s + h of stage s, h = qd / 2: weight = a * (128 + code) + b
  __device__ static Prep prep(uint32_t blk, int qd) {
    const uint4 hd = lds_v4(blk);              // d | dmin, scales[0..3], scales[4..7], scales[8..11]
    const int h = qd >> 1;
    // groups j = h, 2 + h (plain 6-bit fields) and 4 + h, 6 + h (split fields)
    const uint32_t sc_lo = hd.y & 0x3F3F3F3Fu, mn_lo = hd.z & 0x3F3F3F3Fu;
    const uint32_t sc_hi = (hd.w & 0x0F0F0F0Fu) | ((hd.y >> 2) & 0x30303030u);
    const uint32_t mn_hi = ((hd.w >> 4) & 0x0F0F0F0Fu) | ((hd.z >> 2) & 0x30303030u);
    const float d = h2f(hd.x & 0xFFFF), nd = -h2f(hd.x >> 16);
    Prep p;
    p.a[0] = __fmul_rn(d, h ? byte_to_float<1>(sc_lo) : byte_to_float<0>(sc_lo));
    p.a[1] = __fmul_rn(d, h ? byte_to_float<3>(sc_lo) : byte_to_float<2>(sc_lo));
    p.a[2] = __fmul_rn(d, h ? byte_to_float<1>(sc_hi) : byte_to_float<0>(sc_hi));
    p.a[3] = __fmul_rn(d, h ? byte_to_float<3>(sc_hi) : byte_to_float<2>(sc_hi));
    p.b[0] = __fmul_rn(nd, h ? byte_to_float<1>(mn_lo) : byte_to_float<0>(mn_lo));
    p.b[1] = __fmul_rn(nd, h ? byte_to_float<3>(mn_lo) : byte_to_float<2>(mn_lo));
    p.b[2] = __fmul_rn(nd, h ? byte_to_float<1>(mn_hi) : byte_to_float<0>(mn_hi));
    p.b[3] = __fmul_rn(nd, h ? byte_to_float<3>(mn_hi) : byte_to_float<2>(mn_hi));
#pragma unroll
    for (int i = 0; i < 4; i++) p.b[i] = fmaf(-128.0f, p.a[i], p.b[i]);     // the offset decode4 wants
    return p;
  }
  template <int S>
  __device__ static void decode16(uint32_t blk, const Prep& p, int qd, uint32_t (&o)[8]) {
    const uint4 q = lds_v4(blk + 16 + 32 * S + 16 * (qd & 1));
    const int sh = 4 * (qd >> 1);                                 // low or high nibbles of qs[32 S ..]
    const float a = p.a[S], b = p.b[S];
    decode4((q.x >> sh) & 0x0F0F0F0Fu, a, b, o[0], o[1]);
    decode4((q.y >> sh) & 0x0F0F0F0Fu, a, b, o[2], o[3]);
    decode4((q.z >> sh) & 0x0F0F0F0Fu, a, b, o[4], o[5]);
    decode4((q.w >> sh) & 0x0F0F0F0Fu, a, b, o[6], o[7]);
  }
};
struct FQ5K {
  static constexpr int kQt = QT_Q5_K, kTs = 176, kRawPitch = 208;
  static constexpr bool kSplitChunks = false;
  struct Prep { float a[4], b[4]; uint4 qh; };
  __device__ static Prep prep(uint32_t blk, int qd) {
    const FQ4K::Prep q = FQ4K::prep(blk, qd);                     // same header layout
    Prep p;
#pragma unroll
    for (int i = 0; i < 4; i++) { p.a[i] = q.a[i]; p.b[i] = q.b[i]; }
    p.qh = lds_v4(blk + 16 + 16 * (qd & 1));                      // bit j of byte i: fifth bit of weight i of group j
    return p;
  }
  template <int S>
  __device__ static void decode16(uint32_t blk, const Prep& p, int qd, uint32_t (&o)[8]) {
    const uint4 q = lds_v4(blk + 48 + 32 * S + 16 * (qd & 1));
    const int h = qd >> 1, sh = 4 * h, j = 2 * S + h;
    const float a = p.a[S], b = p.b[S];
    auto code = [&](uint32_t w, uint32_t hb) { return ((w >> sh) & 0x0F0F0F0Fu) | (((hb >> j) & 0x01010101u) << 4); };
    decode4(code(q.x, p.qh.x), a, b, o[0], o[1]);
    decode4(code(q.y, p.qh.y), a, b, o[2], o[3]);
    decode4(code(q.z, p.qh.z), a, b, o[4], o[5]);
    decode4(code(q.w, p.qh.w), a, b, o[6], o[7]);
  }
};
struct FQ6K {
  static constexpr int kQt = QT_Q6_K, kTs = 210, kRawPitch = 240;
  static constexpr bool kSplitChunks = true;   // a thread's two chunks are qd and 4 + qd (not 2 qd, 2 qd + 1)
  // Stage s = half n = s / 2, quarters c0 = 2 (s & 1) and c0 + 1 (32 weights each).  A thread takes the eight
  // weights l = 8 qd .. + 7 of both quarters: ql[64 n + l] and ql[64 n + 32 + l] (nibble s & 1), qh[32 n + l]
  // (bits 4 (s & 1) .. + 3), scales 8 n + 2 c + qd / 2.  All shifts are compile-time.
  struct Prep { float a[8]; };                 // a[2 s + i]: quarter c0 + i of stage s
  // 2 * cnt bytes starting at a 2-byte aligned address, as cnt / 2 .. words (cnt words loaded + 1 when misaligned)
  template <int NW>
  __device__ static void load_words(uint32_t a, uint32_t (&w)[NW]) {
    if (a & 2) {
      uint32_t t[NW + 1];
#pragma unroll
      for (int i = 0; i <= NW; i++) t[i] = lds_u32(a - 2 + 4 * i);
#pragma unroll
      for (int i = 0; i < NW; i++) w[i] = __byte_perm(t[i], t[i + 1], 0x5432);
    } else {
#pragma unroll
      for (int i = 0; i < NW; i++) w[i] = lds_u32(a + 4 * i);
    }
  }
  __device__ static Prep prep(uint32_t blk, int qd) {
    const float d = h2f(lds_u16(blk + 208));
    uint32_t sc[4];
    load_words<4>(blk + 192, sc);
    const int hh = qd >> 1;                    // which 16-weight group of a quarter
    Prep p;
#pragma unroll
    for (int i = 0; i < 8; i++) {              // scale index 2 i + hh: byte (2 i + hh) & 3 of word i / 2
      const uint32_t x = sc[i >> 1] ^ 0x80808080u;                  // int8 + 128
      const float f = (i & 1) ? (hh ? byte_to_float<3>(x) : byte_to_float<2>(x)) : (hh ? byte_to_float<1>(x) : byte_to_float<0>(x));
      p.a[i] = __fmul_rn(d, f - 128.0f);
    }
    return p;
  }
  template <int S>
  __device__ static void decode16(uint32_t blk, const Prep& p, int qd, uint32_t (&o)[8]) {
    constexpr int n = S >> 1, nib = 4 * (S & 1), hs = 4 * (S & 1);
    uint32_t q0[2], q1[2], qh[2];
    load_words<2>(blk + 64 * n + 8 * qd, q0);
    load_words<2>(blk + 64 * n + 32 + 8 * qd, q1);
    load_words<2>(blk + 128 + 32 * n + 8 * qd, qh);
    const float a0 = p.a[2 * S], a1 = p.a[2 * S + 1];
    const float b0 = -160.0f * a0, b1 = -160.0f * a1;           // a * (128 + q) - 160 a = a * (q - 32), rounded once
#pragma unroll
    for (int i = 0; i < 2; i++) {
      const uint32_t c0 = ((q0[i] >> nib) & 0x0F0F0F0Fu) | (((qh[i] >> hs) & 0x03030303u) << 4);
      const uint32_t c1 = ((q1[i] >> nib) & 0x0F0F0F0Fu) | (((qh[i] >> (hs + 2)) & 0x03030303u) << 4);
      decode4(c0, a0, b0, o[2 * i], o[2 * i + 1]);          // chunk qd
      decode4(c1, a1, b1, o[4 + 2 * i], o[4 + 2 * i + 1]);  // chunk 4 + qd
    }
  }
};

template <int MT> constexpr int stages_of() { return MT >= 512 ? 2 : MT >= 256 ? 3 : 4; }
template <class F, int MT> constexpr int raw_stages_of() {
  return (stages_of<MT>() * (kABytes + MT * 128) + 3 * kTileN * F::kRawPitch + 2304 <= kSmemLimit) ? 3 : 2;
}
template <class F, int MT> constexpr int smem_bytes() {
  return stages_of<MT>() * (kABytes + MT * 128) + raw_stages_of<F, MT>() * kTileN * F::kRawPitch + 256 + 1024;
}

template <class F, int MT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16w_kernel(const uint8_t* __restrict__ w, int N, int K, const __nv_bfloat16* __restrict__ x, int M,
                  void* __restrict__ y, int y_dtype, int* __restrict__ status, float* __restrict__ partials,
                  int* __restrict__ counters, const __grid_constant__ CUtensorMap x_map, const int use_tma) {
  constexpr int kStages = stages_of<MT>(), kRawStages = raw_stages_of<F, MT>();
  constexpr int kBBytes = MT * 128, kStageBytes = kABytes + kBBytes, kRawBytes = kTileN * F::kRawPitch;
  extern __shared__ uint8_t smem_raw[];
  // the swizzle is a function of the address bits: tiles start 1024-byte aligned
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * kTileN, m0 = blockIdx.y * MT;
  const int splits = gridDim.z, split = blockIdx.z;
  const int SB = K / 256;
  const int blk_begin = (int)((int64_t)split * SB / splits);
  const int n_blocks = (int)((int64_t)(split + 1) * SB / splits) - blk_begin;      // >= 1 (host guarantees)
  const int n_stages = n_blocks * 4;
  const int64_t row_bytes = (int64_t)SB * F::kTs;

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t raw_base = smem_base + kStages * kStageBytes;
  const uint32_t bars = raw_base + kRawStages * kRawBytes;
  auto full_bar = [&](int s) { return bars + 8 * s; };
  auto empty_bar = [&](int s) { return bars + 8 * (kStages + s); };
  const uint32_t acc_bar = bars + 8 * (2 * kStages);
  uint8_t* flags = smem + kStages * kStageBytes + kRawStages * kRawBytes + 128;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(flags);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(flags + 4);
  volatile int* last_flag = reinterpret_cast<volatile int*>(flags + 8);

  if (tid == 0) {
    for (int s = 0; s < kStages; s++) {
      mbar_init(full_bar(s), kProducerWarps + (use_tma ? 1 : kLoaderWarps));   // + the B tile's announcement(s)
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (!use_tma && m0 + MT > M) {
    // batch rows past the end are never copied: their B rows stay zero (the tensor-map copy fills them itself)
    for (int i = tid; i < kStages * (kBBytes / 16); i += kThreads) {
      const int st = i / (kBBytes / 16), q = i % (kBBytes / 16);
      sts_v4(smem_base + st * kStageBytes + kABytes + 16 * q, 0u, 0u, 0u, 0u);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  const int mma_warp = kProducerWarps;
  constexpr uint32_t kTmemCols = MT < 32 ? 32 : MT;      // 32 .. 512: a power of two
  if (warp == mma_warp) {   // the MMA warp owns the TMEM allocation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == mma_warp) {
    // ------------------------------- MMA issue -------------------------------
    constexpr int kMmaN = MT > 256 ? 256 : MT;       // 512 columns are two MMAs per step into the two halves of the accumulator
    const uint32_t idesc = umma_idesc(kTileN, kMmaN);
    bool ok = true;
    for (int st = 0; st < n_stages && ok; st++) {
      const int s = st % kStages, it = st / kStages;
      ok = mbar_wait(full_bar(s), it & 1, abort_flag, status);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (lane == 0) {
        const uint32_t a_addr = smem_base + s * kStageBytes, b_addr = a_addr + kABytes;
#pragma unroll
        for (int kk = 0; kk < kStageK / 16; kk++) {
#pragma unroll
          for (int half = 0; half < MT / kMmaN; half++)
            umma_bf16(tmem_base + half * kMmaN, umma_desc(a_addr + kk * 32), umma_desc(b_addr + half * (kMmaN * 128) + kk * 32), idesc,
                      (st > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(empty_bar(s));                  // the stage may be refilled once these MMAs have read it
        if (st == n_stages - 1) umma_commit(acc_bar);   // and the accumulator is complete
      }
      __syncwarp();
    }
  } else if (warp > mma_warp) {
    // ------------------------------- B-tile loaders -------------------------------
    // Copy the stage's 64 activations of every batch row of the tile (cp.async, 16 bytes) into the swizzled B tile; the
    // arrival for a stage follows one stage later, after its copies have landed and a proxy fence (cp.async writes through
    // the generic proxy, the tensor core reads through the async proxy).
    const int ltid = (warp - mma_warp - 1) * 32 + lane;
    if (use_tma) {
      // One thread, one instruction per stage: a 64-element x MT-row box of x (bf16, row-major [M, K]) lands in the
      // 128-byte-swizzled B tile; rows past M are zero-filled by the copy; completion is counted in bytes on the
      // stage's "full" barrier.  The other loader lanes have nothing to do.
      if (ltid == 0) {
        bool ok = true;
        for (int st = 0; st < n_stages && ok; st++) {
          const int s = st % kStages, it = st / kStages;
          if (it > 0) ok = mbar_wait(empty_bar(s), (it - 1) & 1, abort_flag, status);
          if (!ok) break;
          const uint32_t bt = smem_base + s * kStageBytes + kABytes, bar = full_bar(s);
          const int k0 = (blk_begin * 4 + st) * kStageK;
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)kBBytes) : "memory");
          constexpr int kBoxRows = MT > 256 ? 256 : MT;      // a box has at most 256 rows
#pragma unroll
          for (int half = 0; half < MT / kBoxRows; half++)
            asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                         ::"r"(bt + half * (kBoxRows * 128)), "l"(&x_map), "r"(k0), "r"(m0 + half * kBoxRows), "r"(bar) : "memory");
        }
      }
    } else {
    constexpr int kL = 32 * kLoaderWarps, kPer = (MT * 8 + kL - 1) / kL;      // chunks per loader thread and stage
    // chunk q = ltid + i * kL: batch row q / 8, 16-byte piece q % 8; consecutive i are kL / 8 rows apart, i.e. a whole
    // number of 8-row swizzle groups, so both addresses advance by constants
    const int mr0 = ltid >> 3, ch = ltid & 7;
    const uint32_t dst0 = kABytes + swz(mr0, ch);
    const uint8_t* src0 = reinterpret_cast<const uint8_t*>(x + (int64_t)(m0 + mr0) * K + (int64_t)blk_begin * 256) + 16 * ch;
    const int64_t src_step = (int64_t)(kL / 8) * K * 2;
    constexpr uint32_t dst_step = (kL / 8 / 8) * 1024;
    constexpr int kAhead = 2;                       // a stage is announced after two more have been issued
    bool ok = true;
    for (int st = 0; st < n_stages + kAhead; st++) {
      // first announce the stage whose copies were issued kAhead iterations ago (so that the MMAs never wait for this
      // warp's next wait), then take the next free stage
      if (st >= kAhead) {
        asm volatile("cp.async.wait_group %0;" ::"n"(kAhead - 1) : "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0 && ok) mbar_arrive(full_bar((st - kAhead) % kStages));
      }
      if (st < n_stages) {
        const int s = st % kStages, it = st / kStages;
        if (ok && it > 0) ok = mbar_wait(empty_bar(s), (it - 1) & 1, abort_flag, status);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (ok) {
          const uint32_t bt = smem_base + s * kStageBytes + dst0;
          const uint8_t* src = src0 + (int64_t)st * (kStageK * 2);
#pragma unroll
          for (int i = 0; i < kPer; i++) {
            const int mr = mr0 + i * (kL / 8);
            if (mr < MT && m0 + mr < M) cp_async16(bt + i * dst_step, src + i * src_step);
          }
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
    }
  } else {
    // ------------------------------- producers -------------------------------
    const int ptid = tid;                                            // 0..511
    // raw copies: four threads per row, every fourth 16-byte piece of the row's block window each
    const int crow = ptid >> 2, cq = ptid & 3;
    const uint8_t* wrow = w + (int64_t)min(n0 + crow, N - 1) * row_bytes;   // rows past the end repeat the last one (never stored)
    auto issue_raw = [&](int b) {
      if (b < n_blocks) {
        const int64_t off = (int64_t)(blk_begin + b) * F::kTs;
        const int skew = (int)(off & 15);
        const uint8_t* p16 = wrow + (off - skew);
        const int pieces = (skew + F::kTs + 15) >> 4;
        const uint32_t dst = raw_base + (b % kRawStages) * kRawBytes + crow * F::kRawPitch;
        for (int q = cq; q < pieces; q += 4) cp_async16(dst + 16 * q, p16 + 16 * q);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    for (int b = 0; b < kRawStages - 1; b++) issue_raw(b);
    // decode task: row = ptid >> 2, quarter qd = ptid & 3 of the stage's 64 weights
    const int t_row = ptid >> 2, qd = ptid & 3;
    bool alive = true;
    const uint32_t a_dst0 = swz(t_row, F::kSplitChunks ? qd : 2 * qd), a_dst1 = swz(t_row, F::kSplitChunks ? 4 + qd : 2 * qd + 1);
    int s = 0;                      // stage slot of the next stage
    uint32_t round = 0;             // how many times the ring has wrapped
    for (int b = 0; b < n_blocks; b++) {
      // every producer thread passes every one of these barriers, also after a wait has given up
      if (kRawStages == 3) asm volatile("cp.async.wait_group 1;" ::: "memory");      // my pieces of block b have landed
      else asm volatile("cp.async.wait_group 0;" ::: "memory");
      asm volatile("bar.sync 2, %0;" ::"n"(kProducers) : "memory");    // everybody's have; block b - 1 is consumed
      issue_raw(b + kRawStages - 1);                                   // into the slot block b - 1 occupied
      if (!alive) continue;
      const int blk = blk_begin + b;
      const uint32_t braw = raw_base + (b % kRawStages) * kRawBytes + t_row * F::kRawPitch + (uint32_t)(((int64_t)blk * F::kTs) & 15);
      const typename F::Prep pr = F::prep(braw, qd);
      if constexpr (kStages % 2 == 0 && kStages >= 4) {
        // two stages per round: two independent decode chains per thread, half as many fences, waits and arrivals
        // (a superblock starts at an even stage slot: the ring has an even number of slots and a superblock four stages)
#pragma unroll
        for (int sq = 0; sq < 4; sq += 2) {
          if (round > 0 && !(mbar_wait(empty_bar(s), (round - 1) & 1, abort_flag, status) &&
                             mbar_wait(empty_bar(s + 1), (round - 1) & 1, abort_flag, status))) { alive = false; break; }
          const uint32_t stage = smem_base + s * kStageBytes;
          uint32_t o[8], o2[8];
          if (sq == 0) { F::template decode16<0>(braw, pr, qd, o); F::template decode16<1>(braw, pr, qd, o2); }
          else { F::template decode16<2>(braw, pr, qd, o); F::template decode16<3>(braw, pr, qd, o2); }
          sts_v4(stage + a_dst0, o[0], o[1], o[2], o[3]);
          sts_v4(stage + a_dst1, o[4], o[5], o[6], o[7]);
          sts_v4(stage + kStageBytes + a_dst0, o2[0], o2[1], o2[2], o2[3]);
          sts_v4(stage + kStageBytes + a_dst1, o2[4], o2[5], o2[6], o2[7]);
          // make the generic-proxy stores visible to the tensor core, then one arrival per warp and stage
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) { mbar_arrive(full_bar(s)); mbar_arrive(full_bar(s + 1)); }
          s += 2;
          if (s == kStages) { s = 0; ++round; }
        }
      } else {
#pragma unroll
        for (int sq = 0; sq < 4; sq++) {
          if (round > 0 && !mbar_wait(empty_bar(s), (round - 1) & 1, abort_flag, status)) { alive = false; break; }
          const uint32_t stage = smem_base + s * kStageBytes;
          uint32_t o[8];
          if (sq == 0) F::template decode16<0>(braw, pr, qd, o);
          else if (sq == 1) F::template decode16<1>(braw, pr, qd, o);
          else if (sq == 2) F::template decode16<2>(braw, pr, qd, o);
          else F::template decode16<3>(braw, pr, qd, o);
          sts_v4(stage + a_dst0, o[0], o[1], o[2], o[3]);
          sts_v4(stage + a_dst1, o[4], o[5], o[6], o[7]);
          // make the generic-proxy stores visible to the tensor core, then one arrival per warp
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(full_bar(s));
          if (++s == kStages) { s = 0; ++round; }
        }
      }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    // ------------------------------- epilogue -------------------------------
    // warp e: TMEM lanes (rows) 32 (e & 3) .. + 31; the column range is split over the four warps of a quarter
    const int quarter = warp & 3, cpart = warp >> 2;                 // cpart 0..3
    constexpr int kColsPerWarp = MT / 4 >= 8 ? MT / 4 : 8;           // 8 (MT = 32), 16, 32, 64
    const int row = 32 * quarter + lane, out_row = n0 + row;
    bool ok = alive && mbar_wait(acc_bar, 0, abort_flag, status);
    ok = __all_sync(0xFFFFFFFFu, ok);                               // tcgen05.ld needs the whole warp
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
    for (int c0 = 0; c0 < kColsPerWarp; c0 += 8) {
      const int col = cpart * kColsPerWarp + c0;
      uint32_t v[8];
      if (ok) {       // warp-uniform
        const uint32_t taddr = tmem_base + ((uint32_t)(32 * quarter) << 16) + (uint32_t)col;
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                     : "r"(taddr));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (out_row < N) {
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const int m = m0 + col + i;
            if (m < M) {
              if (splits == 1) store_out(y, y_dtype, (int64_t)m * N + out_row, __uint_as_float(v[i]));
              else partials[((int64_t)split * M + m) * N + out_row] = __uint_as_float(v[i]);
            }
          }
        }
      }
    }
    if (splits > 1) {
      // every producer thread takes part in both barriers, whatever happened above
      __threadfence();
      asm volatile("bar.sync 1, %0;" ::"n"(kProducers) : "memory");
      if (ptid == 0) {
        int* counter = counters + blockIdx.y * gridDim.x + blockIdx.x;
        const int old = atomicAdd(counter, 1);
        *last_flag = old == splits - 1;
        if (old == splits - 1) *counter = 0;             // nobody else touches it until the next launch
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kProducers) : "memory");
      if (*last_flag && out_row < N) {
        __threadfence();
        const int64_t zs = (int64_t)M * N;                          // stride between the ranges' partial tiles
        // four batch columns at a time, the ranges in order: 4 independent chains keep 4 loads in flight per thread
        for (int c = 0; c < kColsPerWarp; c += 4) {
          const int mb = m0 + cpart * kColsPerWarp + c;
          const float* p = partials + (int64_t)mb * N + out_row;
          float sum[4] = {0.f, 0.f, 0.f, 0.f};
          // columns past M read column mb again (never stored): no branches around the loads
          const int64_t o1 = mb + 1 < M ? N : 0, o2 = mb + 2 < M ? 2 * (int64_t)N : 0, o3 = mb + 3 < M ? 3 * (int64_t)N : 0;
          if (mb < M) {
#pragma unroll 4
            for (int z = 0; z < splits; z++) {
              const float* q = p + z * zs;
              const float v0 = __ldcg(q), v1 = __ldcg(q + o1), v2 = __ldcg(q + o2), v3 = __ldcg(q + o3);
              sum[0] += v0; sum[1] += v1; sum[2] += v2; sum[3] += v3;
            }
          }
#pragma unroll
          for (int i = 0; i < 4; i++)
            if (mb + i < M) store_out(y, y_dtype, (int64_t)(mb + i) * N + out_row, sum[i]);
        }
      }
    }
  }
  // common exit: everybody is done with TMEM before it is released
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == mma_warp) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

static int tile_m_of(int M) { return M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : M <= 256 ? 256 : 512; }

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against the driver library).
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
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
// Tensor map of x as bf16 [M rows, K columns], box = 64 columns x box_rows rows, 128-byte swizzle, zero fill outside.
static bool make_x_map(CUtensorMap* map, const void* x, int64_t M, int64_t K, int box_rows) {
  static const bool off = [] { const char* e = getenv("GGQ_GEMM_NO_TMA"); return e && e[0] == '1'; }();
  EncodeTiledFn fn = off ? nullptr : encode_tiled_fn();
  if (!fn || (uintptr_t)x % 16 || (K * 2) % 16) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kStageK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <class F, int MT>
static cudaError_t launch_mt(const uint8_t* w, int64_t N, int64_t K, const void* x, int M, void* y, int y_dtype, int* status,
                             int splits, uint8_t* ws, cudaStream_t st) {
  static_assert(smem_bytes<F, MT>() <= kSmemLimit, "shared memory");
  static std::atomic<bool> attr_done[64];   // setting the attribute twice is harmless, so a flag per device suffices
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16w_kernel<F, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<F, MT>());
    if (e != cudaSuccess) return e;
    attr_done[dev].store(true, std::memory_order_release);
  }
  float* partials = reinterpret_cast<float*>(ws + kWsGemmPartialOffset);
  int* counters = reinterpret_cast<int*>(ws + kWsCounterOffset);
  // the B tile comes by TMA when the driver offers the tensor-map encoder (it does from CUDA 12.0 on); otherwise the
  // loader warps copy it with cp.async
  alignas(64) CUtensorMap x_map;
  memset(&x_map, 0, sizeof(x_map));
  const int use_tma = make_x_map(&x_map, x, M, K, MT > 256 ? 256 : MT) ? 1 : 0;
  dim3 grid((unsigned)((N + kTileN - 1) / kTileN), (unsigned)((M + MT - 1) / MT), (unsigned)splits);
  gemm_bf16w_kernel<F, MT><<<grid, kThreads, smem_bytes<F, MT>(), st>>>(w, (int)N, (int)K, (const __nv_bfloat16*)x, M, y, y_dtype,
                                                                        status, partials, counters, x_map, use_tma);
  return cudaPeekAtLastError();
}

template <class F>
static cudaError_t launch(const uint8_t* w, int64_t N, int64_t K, const void* x, int M, void* y, int y_dtype, int* status,
                          int mt, int splits, uint8_t* ws, cudaStream_t st) {
  switch (mt) {
    case 32: return launch_mt<F, 32>(w, N, K, x, M, y, y_dtype, status, splits, ws, st);
    case 64: return launch_mt<F, 64>(w, N, K, x, M, y, y_dtype, status, splits, ws, st);
    case 128: return launch_mt<F, 128>(w, N, K, x, M, y, y_dtype, status, splits, ws, st);
    case 256: return launch_mt<F, 256>(w, N, K, x, M, y, y_dtype, status, splits, ws, st);
    default: return launch_mt<F, 512>(w, N, K, x, M, y, y_dtype, status, splits, ws, st);
  }
}

}  // namespace gemmb

bool gemm_bf16w_applicable(int qtype, int64_t N, int64_t K, int M) {
  if (qtype != QT_Q4_K && qtype != QT_Q5_K && qtype != QT_Q6_K) return false;
  const int ts = qtype == QT_Q4_K ? 144 : qtype == QT_Q5_K ? 176 : 210;
  return K > 0 && K % 256 == 0 && (K / 256 * ts) % 16 == 0 && N >= 1 && N < (1ll << 31) - 256 && M >= 1 && M <= 65536 &&
         (int64_t)M * N < (1ll << 40);
}

// Batch tile and number of K ranges of a launch: the pair that minimises
//   waves of CTAs x (superblocks of a CTA x time per superblock + 4 us to start and drain a CTA) + the partial tiles' round trip,
// with the time per superblock (2.3 us + 3.5 ns per batch column) and the other constants fitted to B200 timings.
// One CTA is resident per SM.  Above 256 rows the choice is between one 512-column tile (the weights are decoded once,
// fewer CTAs) and 256-column tiles (twice the decoding, twice the CTAs: better for few row tiles).
static void choose_tiling(int64_t N, int64_t K, int M, int sm_count, int* mt_out, int* splits_out) {
  if (sm_count <= 0) sm_count = 148;
  const int64_t SB = K / 256;
  const int mt_lo = gemmb::tile_m_of(M > 256 ? 256 : M), mt_hi = gemmb::tile_m_of(M);
  double best_cost = 1e30;
  for (int mt = mt_lo; mt <= mt_hi; mt *= 2) {
    const int64_t tiles = ((N + gemmb::kTileN - 1) / gemmb::kTileN) * ((M + mt - 1) / mt);
    const double t_sb = 2.3 + 0.0035 * mt;
    // a 512-column tile is cut into at most two K ranges: its partial tiles are 256 KB each, and four or more of them
    // per row tile were measured far slower than the model says (4096 x 14336 at 512 rows: 205 us against 120 us)
    for (int s = 1; s <= (mt > 256 ? 2 : gemmb::kMaxSplits) && s <= SB; s++) {
      const double waves = (double)((tiles * s + sm_count - 1) / sm_count);
      const double cost = waves * ((double)((SB + s - 1) / s) * t_sb + 4.0) + (s > 1 ? 2.0 + 0.02 * s * mt : 0.0);
      if (cost < best_cost - 1e-9) { best_cost = cost; *mt_out = mt; *splits_out = s; }
    }
  }
}
int gemm_bf16w_splits(int64_t N, int64_t K, int M, int sm_count) {
  int mt = 32, s = 1;
  choose_tiling(N, K, M, sm_count, &mt, &s);
  return s;
}

// Scratch: arrival counters in the counter area every kernel shares; partial tiles (splits x M x N float32) when K is split.
size_t gemm_bf16w_workspace_bytes(int qtype, int64_t N, int64_t K, int M, int sm_count) {
  (void)qtype;
  const int s = gemm_bf16w_splits(N, K, M, sm_count);
  size_t need = kWsGemmPartialOffset;
  if (s > 1) need += (size_t)s * M * N * sizeof(float);
  return (need + 255) / 256 * 256;
}

cudaError_t gemm_bf16w(int qtype, const uint8_t* w, int64_t N, int64_t K, const void* x, int M, void* y, int y_dtype,
                       int* status, void* ws, size_t ws_bytes, int sm_count, cudaStream_t st) {
  if (!ws || (uintptr_t)ws % 256 || ws_bytes < gemm_bf16w_workspace_bytes(qtype, N, K, M, sm_count)) return cudaErrorInvalidValue;
  int mt = 32, splits = 1;
  choose_tiling(N, K, M, sm_count, &mt, &splits);
  const int64_t tiles = ((N + gemmb::kTileN - 1) / gemmb::kTileN) * ((M + mt - 1) / mt);
  if (kWsCounterOffset + (size_t)tiles * sizeof(int) > kWsGemmPartialOffset) return cudaErrorInvalidValue;
  uint8_t* base = reinterpret_cast<uint8_t*>(ws);
  switch (qtype) {
    case QT_Q4_K: return gemmb::launch<gemmb::FQ4K>(w, N, K, x, M, y, y_dtype, status, mt, splits, base, st);
    case QT_Q5_K: return gemmb::launch<gemmb::FQ5K>(w, N, K, x, M, y, y_dtype, status, mt, splits, base, st);
    case QT_Q6_K: return gemmb::launch<gemmb::FQ6K>(w, N, K, x, M, y, y_dtype, status, mt, splits, base, st);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace ggq
