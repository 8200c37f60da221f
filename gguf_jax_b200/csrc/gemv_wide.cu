// Fused decode + multiply for batches of 5 to 32 rows per launch (larger batches in slices) on B200:
// Q4_K, Q5_K and Q6_K weights, y[M, N] = x[M, K] W[N, K]^T with W as GGUF blocks.
//
// Where the small-batch kernels (gemv_tile.cu) spend the eight columns of an MMA on four lane-run
// channels x two batch rows, this one gives all eight columns to batch rows and keeps the scale
// groups apart in time instead: every mma.sync.m16n8k16 (or pair of them) covers exactly one scale
// group of 16 weight rows, its accumulator tile is multiplied by the group's float32 scale and
// added to the running sums, and the next group starts from zero.  A lane therefore holds a
// quarter of every group (not a private run of 64 weights), and the decoded A registers of a group
// serve all batch-column tiles (1, 2 or 4 tiles of 8 columns).  The arithmetic is the exact-code
// scheme of the other kernels: quants become bf16 values with a zero upper byte (v * 2^-133),
// activations are pre-scaled by a power of two, float32 scales meet float32 accumulators.  Offsets
// (Q4_K / Q5_K: -dmin * m_j * sum(x_j); Q6_K: -32 * d * sc_j * sum(x_j)) are one more MMA per
// superblock: A = the per-group integers (exact codes), B = the per-group sums of x split into three
// bf16 terms (exact to 24 bits).
//
// Work split.  A CTA (8 warps, two CTAs per SM so that one's barriers and dependent chains overlap the other's
// work) takes row blocks of 128 rows -- warp w the rows 16 w .. 16 w + 15 -- and walks along K one superblock
// per step; all steps of the launch (row block major) are dealt to the CTAs as equal contiguous ranges.  A row block cut by a range boundary is finished by the last
// CTA to arrive: each contributor leaves its 128 x M partial sums in one of its two scratch slots,
// bumps the row block's counter, and the last one adds the slots in CTA order (deterministic).
// The activations of a step are the same for all warps: a separate launch (prepare kernel) writes
// them once, already in B-fragment order, and the CTAs copy one superblock's worth per step into a
// ring in shared memory next to each warp's private ring of raw weight bytes (one TMA box of 16 rows per warp and step on a
// per-warp mbarrier; per-lane 16-byte cp.async where no tensor-map encoder is to be had).
#include "gemv.cuh"

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace ggq {
namespace wide {

constexpr int kWarps = 8;
constexpr int kCtasPerSm = 2;
constexpr int kThreads = kWarps * 32;
constexpr int kBlockRows = 16 * kWarps;          // rows of a row block
constexpr int kSmemLimit = 232448;
constexpr int kMaxBatch = 32;                    // four column tiles

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_pending(int n) {
  switch (n) {
    case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
  }
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// the same with a zero C operand: starts a fresh accumulator tile without clearing registers first
__device__ __forceinline__ void mma16816_first(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t a) { uint32_t v; asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a)); return v; }
__device__ __forceinline__ uint2 lds_v2(uint32_t a) { uint2 v; asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a)); return v; }
__device__ __forceinline__ uint4 lds_v4(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ float bf16lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16hi(uint32_t u) { return __uint_as_float(u & 0xFFFF0000u); }
__device__ __forceinline__ float pow2f(int e) { return __uint_as_float((uint32_t)(127 + e) << 23); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}
// o0 += s * a0, o1 += s * a1 as one packed instruction
__device__ __forceinline__ void fma_pair(float& o0, float& o1, float s, float a0, float a1) {
  asm("{ .reg .b64 o, a, ss;\n mov.b64 o, {%0, %1};\n mov.b64 a, {%3, %4};\n mov.b64 ss, {%2, %2};\n fma.rn.f32x2 o, ss, a, o;\n mov.b64 {%0, %1}, o; }"
      : "+f"(o0), "+f"(o1) : "f"(s), "f"(a0), "f"(a1));
}
// byte SEL of x as a float, exact: the bits 0x4B0000vv are 2^23 + v
template <int SEL>
__device__ __forceinline__ float byte_to_float(uint32_t x) {
  return __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7440 + SEL)) - 8388608.0f;
}
// a float32 as three bf16 terms whose sum is the float (each residual is exact)
__device__ __forceinline__ void split3(float s, uint32_t& hi, uint32_t& mid, uint32_t& lo) {
  const __nv_bfloat16 h = __float2bfloat16_rn(s);
  const float r1 = s - __bfloat162float(h);
  const __nv_bfloat16 m = __float2bfloat16_rn(r1);
  const float r2 = r1 - __bfloat162float(m);
  const __nv_bfloat16 l = __float2bfloat16_rn(r2);
  hi = __bfloat16_as_ushort(h); mid = __bfloat16_as_ushort(m); lo = __bfloat16_as_ushort(l);
}

// ---------------------------------------------------------------------------------------------
// Formats.  A superblock's activations are staged per batch column as 512 bytes in "piece" order:
// the piece of (MMA group q, lane group t) holds the activations of the weights lane t feeds to
// group q's MMAs, in the k-slot order of its A registers.  kPiece = bytes of a piece (16: two MMAs
// per group, 8: one), kOffBytes = bytes per column of the offset operand.

struct FQ4K {
  static constexpr int kQt = QT_Q4_K, kTs = 144, kPitch = 160, kPiece = 16, kGroups = 8, kOffBytes = 64;
  // weight index and power-of-two exponent of element e (0..7) of piece (q, t)
  __host__ __device__ static int src(int q, int t, int e) { return 32 * q + 8 * t + e; }
  __host__ __device__ static int x_exp(int q) { return (q & 1) ? -4 : 0; }       // high nibbles stay in place: codes * 16
  static constexpr int kSumGroups = 8, kSumLen = 32;
};
struct FQ5K {
  static constexpr int kQt = QT_Q5_K, kTs = 176, kPitch = 224, kPiece = 16, kGroups = 8, kOffBytes = 64;
  __host__ __device__ static int src(int q, int t, int e) { return 32 * q + 8 * t + e; }
  __host__ __device__ static int x_exp(int) { return 0; }
  static constexpr int kSumGroups = 8, kSumLen = 32;
};
struct FQ6K {
  static constexpr int kQt = QT_Q6_K, kTs = 210, kPitch = 240, kPiece = 8, kGroups = 16, kOffBytes = 128;
  // group q = 8 n + 2 quarter + half: the 16 weights 128 n + 32 quarter + 16 half + (0..15)
  __host__ __device__ static int src(int q, int t, int e) { return 16 * q + 4 * t + e; }
  __host__ __device__ static int x_exp(int) { return 0; }
  static constexpr int kSumGroups = 16, kSumLen = 16;
};

// Launch geometry (host-computed).
struct Geo {
  int SB, RB;                 // superblocks per row, row blocks
  int64_t S;                  // steps = RB * SB
  int depth;                  // ring depth (steps)
  int wslot_bytes;            // 16 * pitch
  int xstage_bytes;           // XR * (512 + kOffBytes)
  int off_x, total;
  int tma;                    // weight slots arrive as TMA boxes (one per warp and step) instead of cp.async copies
  int vec_store;              // 2-byte outputs whose 8-row runs are 16-byte aligned: stored as 16-byte vectors
};

// ---------------------------------------------------------------------------------------------
// Prepare kernel: one CTA per staged batch column (columns >= M are zero-filled).
//   xp[sb][q][col][t]   kPiece bytes: activations * 2^(S + x_exp), permuted (0,2,1,3[,4,6,5,7]) to the A registers' pairing
//   xo[sb][col][...]    kOffBytes: the group sums of x (times 2^S), three bf16 terms each, in offset-MMA order
//   S_col[col]          the column's power-of-two exponent
template <class F, int XR>
__global__ void __launch_bounds__(256)
prepare_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, int K, int M, uint8_t* __restrict__ xp, uint8_t* __restrict__ xo,
               int* __restrict__ S_col, const PeerPublish pp, int* __restrict__ status) {
  __shared__ int s_max;
  pdl_wait();            // x may be the previous kernel's output, and the previous launch may still read the staged copy
  pdl_trigger();         // the multiply kernel may start fetching weights
  const int col = blockIdx.x, tid = threadIdx.x;
  // row-sharded: x is what the peers stored during the previous exchange; wait (bounded) for all of their flags
  peer_wait_previous(pp, tid, status);
  if (pp.world > 0 && pp.wait_previous) __syncthreads();
  const int SB = K / 256;
  const bool real = col < M;
  const __nv_bfloat16* xr = x + (int64_t)(real ? col : 0) * ldx;
  if (tid == 0) s_max = 0;
  __syncthreads();
  float amax = 0.f;
  if (real)
    for (int i = tid; i < K / 8; i += 256) {
      const uint4 v = __ldcg(reinterpret_cast<const uint4*>(xr) + i);
      const float s = (fabsf(bf16lo(v.x)) + fabsf(bf16hi(v.x))) + (fabsf(bf16lo(v.y)) + fabsf(bf16hi(v.y))) +
                      (fabsf(bf16lo(v.z)) + fabsf(bf16hi(v.z))) + (fabsf(bf16lo(v.w)) + fabsf(bf16hi(v.w)));
      amax = fmaxf(amax, s);
    }
  atomicMax(&s_max, (int)__float_as_uint(amax));
  __syncthreads();
  // 2^96 suits any octet sum of |x| in about [2^-30, 2^30); otherwise put the largest near 2^120
  const int emax = min((s_max >> 23) & 0xFF, 254);
  const int S = (emax > 156 || (emax < 97 && emax > 0)) ? max(8, min(120, 247 - emax)) : 96;
  if (tid == 0) S_col[col] = S;
  constexpr int kE = F::kPiece / 2;                       // elements per piece: 8 or 4
  constexpr int kPiecesPerSum = F::kSumLen / kE;          // pieces (consecutive t) that make one scale group: 4
  static_assert(kPiecesPerSum == 4, "a scale group is the four lane groups of one MMA group");
  const int n_pieces = SB * F::kGroups * 4;
  for (int o = tid; o < (n_pieces + 255) / 256 * 256; o += 256) {
    const bool in = o < n_pieces;
    const int sb = o / (F::kGroups * 4), q = (o / 4) % F::kGroups, t = o & 3;
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (in && real) {
      const __nv_bfloat16* p = xr + (int64_t)sb * 256 + F::src(q, t, 0);
      if (kE == 8) {
        const uint4 u = __ldcg(reinterpret_cast<const uint4*>(p));
        v[0] = bf16lo(u.x); v[1] = bf16hi(u.x); v[2] = bf16lo(u.y); v[3] = bf16hi(u.y);
        v[4] = bf16lo(u.z); v[5] = bf16hi(u.z); v[6] = bf16lo(u.w); v[7] = bf16hi(u.w);
      } else {
        const uint2 u = __ldcg(reinterpret_cast<const uint2*>(p));
        v[0] = bf16lo(u.x); v[1] = bf16hi(u.x); v[2] = bf16lo(u.y); v[3] = bf16hi(u.y);
      }
    }
    const float up = pow2f(S + F::x_exp(q));
    if (in) {
      uint8_t* dst = xp + (((int64_t)sb * F::kGroups + q) * XR + col) * (4 * F::kPiece) + t * F::kPiece;
      const uint2 lo2 = make_uint2(pack_bf16(v[0] * up, v[2] * up), pack_bf16(v[1] * up, v[3] * up));
      if (kE == 8) *reinterpret_cast<uint4*>(dst) = make_uint4(lo2.x, lo2.y, pack_bf16(v[4] * up, v[6] * up), pack_bf16(v[5] * up, v[7] * up));
      else *reinterpret_cast<uint2*>(dst) = lo2;
    }
    float sum = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
    if (in && t == 0) {
      uint32_t hi, mid, lo;
      split3(sum * pow2f(S), hi, mid, lo);
      uint8_t* ob = xo + ((int64_t)sb * XR + col) * F::kOffBytes;
      if (F::kGroups == 8) {
        // offset MMAs 1 and 2, lane group t' = q / 2: slots (hi, mid) of groups 2t', 2t'+1, then (lo, 0) of both
        uint32_t* piece = reinterpret_cast<uint32_t*>(ob + (q >> 1) * 16);
        piece[q & 1] = hi | (mid << 16);
        piece[2 + (q & 1)] = lo;
      } else {
        // sixteen groups: lane group t' = q / 4 holds groups 4t' .. 4t'+3; three MMAs (hi, mid, lo), 8 bytes each:
        // k-slots (2t', 2t'+1) = groups 4t', 4t'+1 and (2t'+8, 2t'+9) = groups 4t'+2, 4t'+3
        uint16_t* piece = reinterpret_cast<uint16_t*>(ob + (q >> 2) * 32);
        piece[0 + (q & 3)] = (uint16_t)hi;
        piece[4 + (q & 3)] = (uint16_t)mid;
        piece[8 + (q & 3)] = (uint16_t)lo;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// One superblock of 16 rows against NT column tiles.  blk0 / blk1: shared addresses of the block in rows
// g and g + 8; xs: shared address of the step's staged activations; out[nt] = {row g: cols 2t, 2t+1; row g+8: same}.

template <int NT>
__device__ __forceinline__ void group_mma2(float (&acc)[NT][4], uint32_t a00, uint32_t a01, uint32_t a10, uint32_t a11,
                                           uint32_t a20, uint32_t a21, uint32_t a30, uint32_t a31, uint32_t xq) {
  // a{r}{row}: register r (0..3) of the lane's octet for row g (0) / g + 8 (1); xq: this lane's piece of column tile 0
  // all first halves, then all second halves: the two MMAs of a column tile depend on each other, the tiles do not
  uint4 xv[NT];
#pragma unroll
  for (int nt = 0; nt < NT; nt++) xv[nt] = lds_v4(xq + nt * (8 * 64));
#pragma unroll
  for (int nt = 0; nt < NT; nt++) mma16816_first(acc[nt], a00, a01, a10, a11, xv[nt].x, xv[nt].y);
#pragma unroll
  for (int nt = 0; nt < NT; nt++) mma16816(acc[nt], a20, a21, a30, a31, xv[nt].z, xv[nt].w);
}

template <int NT>
__device__ __forceinline__ void block_q4k(uint32_t blk0, uint32_t blk1, int g, int t, uint32_t xs, float (&out)[NT][4]) {
  constexpr int XR = 8 * NT;
  const uint4 h0 = lds_v4(blk0), h1 = lds_v4(blk1);
  // 6-bit scales and mins of the eight groups, one byte each
  const uint32_t sc0[2] = {h0.y & 0x3F3F3F3Fu, (h0.w & 0x0F0F0F0Fu) | ((h0.y >> 2) & 0x30303030u)};
  const uint32_t mn0[2] = {h0.z & 0x3F3F3F3Fu, ((h0.w >> 4) & 0x0F0F0F0Fu) | ((h0.z >> 2) & 0x30303030u)};
  const uint32_t sc1[2] = {h1.y & 0x3F3F3F3Fu, (h1.w & 0x0F0F0F0Fu) | ((h1.y >> 2) & 0x30303030u)};
  const uint32_t mn1[2] = {h1.z & 0x3F3F3F3Fu, ((h1.w >> 4) & 0x0F0F0F0Fu) | ((h1.z >> 2) & 0x30303030u)};
  const __half2 dd0 = *reinterpret_cast<const __half2*>(&h0.x), dd1 = *reinterpret_cast<const __half2*>(&h1.x);
  const float d0 = __low2float(dd0), nm0 = -__high2float(dd0), d1 = __low2float(dd1), nm1 = -__high2float(dd1);
  const uint32_t xl = xs + (g * 4 + t) * 16;
#pragma unroll
  for (int p = 0; p < 4; p++) {
    const uint2 q0 = lds_v2(blk0 + 16 + 32 * p + 8 * t), q1 = lds_v2(blk1 + 16 + 32 * p + 8 * t);
    const uint32_t q0xs = q0.x >> 8, q0ys = q0.y >> 8, q1xs = q1.x >> 8, q1ys = q1.y >> 8;
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const uint32_t mk = h ? 0x00F000F0u : 0x000F000Fu;
      float acc[NT][4];
      group_mma2<NT>(acc, q0.x & mk, q1.x & mk, q0xs & mk, q1xs & mk, q0.y & mk, q1.y & mk, q0ys & mk, q1ys & mk,
                     xl + (2 * p + h) * (XR * 64));
      const int j = 2 * p + h;
      const float s0 = (j & 3) == 0 ? byte_to_float<0>(sc0[j >> 2]) : (j & 3) == 1 ? byte_to_float<1>(sc0[j >> 2]) :
                       (j & 3) == 2 ? byte_to_float<2>(sc0[j >> 2]) : byte_to_float<3>(sc0[j >> 2]);
      const float s1 = (j & 3) == 0 ? byte_to_float<0>(sc1[j >> 2]) : (j & 3) == 1 ? byte_to_float<1>(sc1[j >> 2]) :
                       (j & 3) == 2 ? byte_to_float<2>(sc1[j >> 2]) : byte_to_float<3>(sc1[j >> 2]);
      const float ds0 = __fmul_rn(d0, s0), ds1 = __fmul_rn(d1, s1);      // exact: 11 x 6 bits
#pragma unroll
      for (int nt = 0; nt < NT; nt++) {
        fma_pair(out[nt][0], out[nt][1], ds0, acc[nt][0], acc[nt][1]);
        fma_pair(out[nt][2], out[nt][3], ds1, acc[nt][2], acc[nt][3]);
      }
    }
  }
  // offsets: A = (m_2t, m_2t | m_2t+1, m_2t+1) as exact codes, B = three-term sums of x
  const uint32_t mw0 = t < 2 ? mn0[0] : mn0[1], mw1 = t < 2 ? mn1[0] : mn1[1];
  const uint32_t bsel = (2 * t) & 3;
  const uint32_t sel_a = bsel | (4u << 4) | (bsel << 8) | (4u << 12), sel_b = sel_a + 0x0101u;
  const uint32_t ma0 = __byte_perm(mw0, 0u, sel_a), mb0 = __byte_perm(mw0, 0u, sel_b);
  const uint32_t ma1 = __byte_perm(mw1, 0u, sel_a), mb1 = __byte_perm(mw1, 0u, sel_b);
  const uint32_t xo = xs + XR * 512 + (g * 4 + t) * 16;
#pragma unroll
  for (int nt = 0; nt < NT; nt++) {
    const uint4 ov = lds_v4(xo + nt * (8 * 64));
    float a2[4];
    mma16816_first(a2, ma0, ma1, mb0, mb1, ov.x, ov.y);
    mma16816(a2, ma0, ma1, mb0, mb1, ov.z, ov.w);
    out[nt][0] = fmaf(nm0, a2[0], out[nt][0]); out[nt][1] = fmaf(nm0, a2[1], out[nt][1]);
    out[nt][2] = fmaf(nm1, a2[2], out[nt][2]); out[nt][3] = fmaf(nm1, a2[3], out[nt][3]);
  }
}

// Q5_K: Q4_K plus a fifth bit per weight (qh byte i, bit j = weight i of group j); codes 0..31 assembled per byte.
template <int NT>
__device__ __forceinline__ void block_q5k(uint32_t blk0, uint32_t blk1, int g, int t, uint32_t xs, float (&out)[NT][4]) {
  constexpr int XR = 8 * NT;
  const uint4 h0 = lds_v4(blk0), h1 = lds_v4(blk1);
  const uint32_t sc0[2] = {h0.y & 0x3F3F3F3Fu, (h0.w & 0x0F0F0F0Fu) | ((h0.y >> 2) & 0x30303030u)};
  const uint32_t mn0[2] = {h0.z & 0x3F3F3F3Fu, ((h0.w >> 4) & 0x0F0F0F0Fu) | ((h0.z >> 2) & 0x30303030u)};
  const uint32_t sc1[2] = {h1.y & 0x3F3F3F3Fu, (h1.w & 0x0F0F0F0Fu) | ((h1.y >> 2) & 0x30303030u)};
  const uint32_t mn1[2] = {h1.z & 0x3F3F3F3Fu, ((h1.w >> 4) & 0x0F0F0F0Fu) | ((h1.z >> 2) & 0x30303030u)};
  const uint2 qh0 = lds_v2(blk0 + 16 + 8 * t), qh1 = lds_v2(blk1 + 16 + 8 * t);
  const __half2 dd0 = *reinterpret_cast<const __half2*>(&h0.x), dd1 = *reinterpret_cast<const __half2*>(&h1.x);
  const float d0 = __low2float(dd0), nm0 = -__high2float(dd0), d1 = __low2float(dd1), nm1 = -__high2float(dd1);
  const uint32_t xl = xs + (g * 4 + t) * 16;
#pragma unroll
  for (int p = 0; p < 4; p++) {
    const uint2 q0 = lds_v2(blk0 + 48 + 32 * p + 8 * t), q1 = lds_v2(blk1 + 48 + 32 * p + 8 * t);
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const int j = 2 * p + h;
      auto code = [&](uint32_t q, uint32_t qh) -> uint32_t {
        const uint32_t hb = (j < 4 ? (qh << (4 - j)) : (qh >> (j - 4))) & 0x10101010u;
        return ((h ? (q >> 4) : q) & 0x0F0F0F0Fu) | hb;
      };
      const uint32_t v0x = code(q0.x, qh0.x), v0y = code(q0.y, qh0.y), v1x = code(q1.x, qh1.x), v1y = code(q1.y, qh1.y);
      float acc[NT][4];
      group_mma2<NT>(acc, v0x & 0x00FF00FFu, v1x & 0x00FF00FFu, (v0x >> 8) & 0x00FF00FFu, (v1x >> 8) & 0x00FF00FFu,
                     v0y & 0x00FF00FFu, v1y & 0x00FF00FFu, (v0y >> 8) & 0x00FF00FFu, (v1y >> 8) & 0x00FF00FFu,
                     xl + j * (XR * 64));
      const float s0 = (j & 3) == 0 ? byte_to_float<0>(sc0[j >> 2]) : (j & 3) == 1 ? byte_to_float<1>(sc0[j >> 2]) :
                       (j & 3) == 2 ? byte_to_float<2>(sc0[j >> 2]) : byte_to_float<3>(sc0[j >> 2]);
      const float s1 = (j & 3) == 0 ? byte_to_float<0>(sc1[j >> 2]) : (j & 3) == 1 ? byte_to_float<1>(sc1[j >> 2]) :
                       (j & 3) == 2 ? byte_to_float<2>(sc1[j >> 2]) : byte_to_float<3>(sc1[j >> 2]);
      const float ds0 = __fmul_rn(d0, s0), ds1 = __fmul_rn(d1, s1);      // exact: 11 x 6 bits
#pragma unroll
      for (int nt = 0; nt < NT; nt++) {
        fma_pair(out[nt][0], out[nt][1], ds0, acc[nt][0], acc[nt][1]);
        fma_pair(out[nt][2], out[nt][3], ds1, acc[nt][2], acc[nt][3]);
      }
    }
  }
  const uint32_t mw0 = t < 2 ? mn0[0] : mn0[1], mw1 = t < 2 ? mn1[0] : mn1[1];
  const uint32_t bsel = (2 * t) & 3;
  const uint32_t sel_a = bsel | (4u << 4) | (bsel << 8) | (4u << 12), sel_b = sel_a + 0x0101u;
  const uint32_t ma0 = __byte_perm(mw0, 0u, sel_a), mb0 = __byte_perm(mw0, 0u, sel_b);
  const uint32_t ma1 = __byte_perm(mw1, 0u, sel_a), mb1 = __byte_perm(mw1, 0u, sel_b);
  const uint32_t xo = xs + XR * 512 + (g * 4 + t) * 16;
#pragma unroll
  for (int nt = 0; nt < NT; nt++) {
    const uint4 ov = lds_v4(xo + nt * (8 * 64));
    float a2[4];
    mma16816_first(a2, ma0, ma1, mb0, mb1, ov.x, ov.y);
    mma16816(a2, ma0, ma1, mb0, mb1, ov.z, ov.w);
    out[nt][0] = fmaf(nm0, a2[0], out[nt][0]); out[nt][1] = fmaf(nm0, a2[1], out[nt][1]);
    out[nt][2] = fmaf(nm1, a2[2], out[nt][2]); out[nt][3] = fmaf(nm1, a2[3], out[nt][3]);
  }
}

// Q6_K: sixteen groups of 16 weights, one MMA each; codes 0..63 = nibble | two bits of qh << 4, the -32 rides on the
// offset MMAs (A = the int8 scales as sign-magnitude codes, B = three-term sums of x).  A 210-byte block is only
// 2-byte aligned: MIS = 1 when the block sits at 2 (mod 4), then a word is two aligned loads and a byte permute.
template <int MIS>
__device__ __forceinline__ uint32_t ldw(uint32_t a) {
  if (MIS) return __byte_perm(lds_u32(a - 2), lds_u32(a + 2), 0x5432);
  return lds_u32(a);
}
__device__ __forceinline__ float sbyte_to_float(uint32_t x_xor80, int sel) {   // x_xor80 = int8 bytes ^ 0x80
  const uint32_t u = sel == 0 ? __byte_perm(x_xor80, 0x4B000000u, 0x7440) : sel == 1 ? __byte_perm(x_xor80, 0x4B000000u, 0x7441) :
                     sel == 2 ? __byte_perm(x_xor80, 0x4B000000u, 0x7442) : __byte_perm(x_xor80, 0x4B000000u, 0x7443);
  return __uint_as_float(u) - 8388736.0f;          // 2^23 + 128
}
template <int NT, int MIS>
__device__ __forceinline__ void block_q6k(uint32_t blk0, uint32_t blk1, int g, int t, uint32_t xs, float (&out)[NT][4]) {
  constexpr int XR = 8 * NT;
  uint32_t s0w[4], s1w[4];
#pragma unroll
  for (int i = 0; i < 4; i++) { s0w[i] = ldw<MIS>(blk0 + 192 + 4 * i); s1w[i] = ldw<MIS>(blk1 + 192 + 4 * i); }
  float ts[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; nt++) ts[nt][0] = ts[nt][1] = ts[nt][2] = ts[nt][3] = 0.f;
  const uint32_t xl = xs + (g * 4 + t) * 8;
#pragma unroll
  for (int n = 0; n < 2; n++) {
#pragma unroll
    for (int hh = 0; hh < 2; hh++) {
      const uint32_t o = 64 * n + 16 * hh + 4 * t;
      const uint32_t A0 = ldw<MIS>(blk0 + o), B0 = ldw<MIS>(blk0 + o + 32), H0 = ldw<MIS>(blk0 + 128 + 32 * n + 16 * hh + 4 * t);
      const uint32_t A1 = ldw<MIS>(blk1 + o), B1 = ldw<MIS>(blk1 + o + 32), H1 = ldw<MIS>(blk1 + 128 + 32 * n + 16 * hh + 4 * t);
#pragma unroll
      for (int c = 0; c < 4; c++) {
        const int q = 8 * n + 2 * c + hh;
        auto code = [&](uint32_t A, uint32_t B, uint32_t H) -> uint32_t {
          const uint32_t nib = (c == 0 ? A : c == 1 ? B : c == 2 ? (A >> 4) : (B >> 4)) & 0x0F0F0F0Fu;
          const uint32_t hi = (c == 0 ? (H << 4) : c == 1 ? (H << 2) : c == 2 ? H : (H >> 2)) & 0x30303030u;
          return nib | hi;
        };
        const uint32_t v0 = code(A0, B0, H0), v1 = code(A1, B1, H1);
        const uint32_t a0 = v0 & 0x00FF00FFu, a1 = v1 & 0x00FF00FFu, a2 = (v0 >> 8) & 0x00FF00FFu, a3 = (v1 >> 8) & 0x00FF00FFu;
        const float f0 = sbyte_to_float(s0w[q >> 2] ^ 0x80808080u, q & 3), f1 = sbyte_to_float(s1w[q >> 2] ^ 0x80808080u, q & 3);
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
          const uint2 xv = lds_v2(xl + q * (XR * 32) + nt * (8 * 32));
          float acc[4];
          mma16816_first(acc, a0, a1, a2, a3, xv.x, xv.y);
          fma_pair(ts[nt][0], ts[nt][1], f0, acc[0], acc[1]);
          fma_pair(ts[nt][2], ts[nt][3], f1, acc[2], acc[3]);
        }
      }
    }
  }
  // offsets: lane group t holds the scales of groups 4t .. 4t+3 (one word) as sign-magnitude codes
  const uint32_t w0 = t == 0 ? s0w[0] : t == 1 ? s0w[1] : t == 2 ? s0w[2] : s0w[3];
  const uint32_t w1 = t == 0 ? s1w[0] : t == 1 ? s1w[1] : t == 2 ? s1w[2] : s1w[3];
  const uint32_t m0 = (w0 >> 7) & 0x01010101u, m1 = (w1 >> 7) & 0x01010101u;
  const uint32_t ab0 = (w0 ^ (m0 * 0xFFu)) + m0, ab1 = (w1 ^ (m1 * 0xFFu)) + m1;
  const uint32_t ca0 = __byte_perm(ab0, 0u, 0x4140) | (__byte_perm(m0, 0u, 0x4140) << 15);
  const uint32_t cb0 = __byte_perm(ab0, 0u, 0x4342) | (__byte_perm(m0, 0u, 0x4342) << 15);
  const uint32_t ca1 = __byte_perm(ab1, 0u, 0x4140) | (__byte_perm(m1, 0u, 0x4140) << 15);
  const uint32_t cb1 = __byte_perm(ab1, 0u, 0x4342) | (__byte_perm(m1, 0u, 0x4342) << 15);
  uint32_t dh0, dh1;
  asm volatile("ld.shared.u16 %0, [%1];" : "=r"(dh0) : "r"(blk0 + 208));
  asm volatile("ld.shared.u16 %0, [%1];" : "=r"(dh1) : "r"(blk1 + 208));
  const float d0 = __half2float(__ushort_as_half((unsigned short)dh0)), d1 = __half2float(__ushort_as_half((unsigned short)dh1));
  const uint32_t xo = xs + XR * 512 + (g * 4 + t) * 32;
#pragma unroll
  for (int nt = 0; nt < NT; nt++) {
    const uint4 ov = lds_v4(xo + nt * (8 * 128));
    const uint2 ol = lds_v2(xo + nt * (8 * 128) + 16);
    float a2[4];
    mma16816_first(a2, ca0, ca1, cb0, cb1, ov.x, ov.y);
    mma16816(a2, ca0, ca1, cb0, cb1, ov.z, ov.w);
    mma16816(a2, ca0, ca1, cb0, cb1, ol.x, ol.y);
    out[nt][0] = fmaf(d0, fmaf(-32.f, a2[0], ts[nt][0]), out[nt][0]);
    out[nt][1] = fmaf(d0, fmaf(-32.f, a2[1], ts[nt][1]), out[nt][1]);
    out[nt][2] = fmaf(d1, fmaf(-32.f, a2[2], ts[nt][2]), out[nt][2]);
    out[nt][3] = fmaf(d1, fmaf(-32.f, a2[3], ts[nt][3]), out[nt][3]);
  }
}

template <class F, int NT>
__device__ __forceinline__ void block_mul(uint32_t blk0, uint32_t blk1, int g, int t, uint32_t xs, float (&out)[NT][4]) {
  if constexpr (F::kQt == QT_Q4_K) block_q4k<NT>(blk0, blk1, g, t, xs, out);
  else if constexpr (F::kQt == QT_Q5_K) block_q5k<NT>(blk0, blk1, g, t, xs, out);
  else {
    if (blk0 & 2) block_q6k<NT, 1>(blk0, blk1, g, t, xs, out);
    else block_q6k<NT, 0>(blk0, blk1, g, t, xs, out);
  }
}

// the CTA whose range holds step s (ranges are [S b / G, S (b + 1) / G))
__device__ __forceinline__ int cta_of_step(int64_t s, int64_t S, int G) {
  int b = (int)((s * G) / S);
  while (b + 1 < G && S * (b + 1) / G <= s) ++b;
  while (b > 0 && S * b / G > s) --b;
  return b;
}

template <class F, int NT>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
gemv_wide_kernel(const uint8_t* __restrict__ w, int N, int K, const uint8_t* __restrict__ xp, const uint8_t* __restrict__ xo,
                 const int* __restrict__ S_col, int M, void* __restrict__ y, int y_dtype, int* __restrict__ counters,
                 float* __restrict__ slots, const Geo geo, const PeerPublish pp, int* __restrict__ status,
                 const __grid_constant__ CUtensorMap w_map) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int s_last;
  __shared__ __align__(8) uint64_t w_bars[kWarps][4];     // one mbarrier per warp and ring slot (depth <= 4)
  constexpr int XR = 8 * NT;
  constexpr int kStageX = XR * 512, kStageO = XR * F::kOffBytes;
  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xFFFFFFFFu, tid >> 5, 0);
  const int g = lane >> 2, t = lane & 3;
  const int SB = geo.SB, depth = geo.depth;
  const int64_t row_bytes = (int64_t)SB * F::kTs;
  const int b = blockIdx.x, G = gridDim.x;
  const int64_t s_begin = geo.S * b / G, s_end = geo.S * (b + 1) / G;
  const int n_steps = (int)(s_end - s_begin);
  const int rb_first = (int)(s_begin / SB);

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t my_ring = smem_base + warp * (depth * geo.wslot_bytes);
  const uint32_t x_ring = smem_base + geo.off_x;
  const int hl = lane >> 4, kl = lane & 15;
  const bool tma = geo.tma != 0;
  const uint32_t my_bars = smem_u32(&w_bars[warp][0]);
  if (tma) tma_bars_init(my_bars, depth, lane);
  // weights and activations are issued by separate cursors: the first weight copies go out before this kernel
  // waits for its predecessor (the weights are immutable), the activations only after it
  int w_issued = 0, w_slot = 0, w_rb = rb_first, w_k = (int)(s_begin - (int64_t)rb_first * SB);
  auto issue_w = [&]() {
    if (w_issued < n_steps) {
      // this warp's 16 rows of superblock w_k: a half-warp copies one row (the 16-byte aligned window around the block)
      const int row0 = w_rb * kBlockRows + warp * 16;
      if (tma) {
        // one box: the slot's pitch in words x 16 rows from the 16-byte aligned window around the block; words past the
        // row's end and rows past N arrive as zeros (a box wholly outside still completes its bytes)
        if (lane == 0)
          tma_box_load(my_ring + w_slot * geo.wslot_bytes, &w_map, ((w_k * F::kTs) & ~15) >> 2, row0, my_bars + 8 * w_slot,
                       (uint32_t)geo.wslot_bytes);
      } else if (row0 < N) {
        const int boff = w_k * F::kTs;
        const int pieces = ((boff & 15) + F::kTs + 15) >> 4;
        const uint32_t dst0 = my_ring + w_slot * geo.wslot_bytes + hl * F::kPitch + 16 * kl;
        if (kl < pieces) {
          if (row0 + 16 <= N) {
            const uint8_t* src = w + (int64_t)(row0 + hl) * row_bytes + ((boff & ~15) + 16 * kl);
#pragma unroll
            for (int i = 0; i < 8; i++) { cp_async16(dst0 + i * (2 * F::kPitch), src); src += 2 * row_bytes; }
          } else {        // ragged last rows: rows past the end repeat row N - 1 (multiplied, never stored)
            const uint8_t* src0 = w + ((boff & ~15) + 16 * kl);
#pragma unroll
            for (int i = 0; i < 8; i++) cp_async16(dst0 + i * (2 * F::kPitch), src0 + (int64_t)min(row0 + 2 * i + hl, N - 1) * row_bytes);
          }
        }
      }
      ++w_issued;
      if (++w_slot == depth) w_slot = 0;
      if (++w_k == SB) { w_k = 0; ++w_rb; }
    }
  };
  int x_issued = 0, x_slot = 0, x_k = w_k;
  auto issue_x = [&]() {
    if (x_issued < n_steps) {
      // the step's activations, the same for every warp
      const uint32_t xdst = x_ring + x_slot * geo.xstage_bytes;
      const uint8_t* xsrc = xp + (int64_t)x_k * kStageX;
      for (int q = tid; q < kStageX / 16; q += kThreads) cp_async16(xdst + q * 16, xsrc + q * 16);
      const uint8_t* osrc = xo + (int64_t)x_k * kStageO;
      for (int q = tid; q < kStageO / 16; q += kThreads) cp_async16(xdst + kStageX + q * 16, osrc + q * 16);
      ++x_issued;
      if (++x_slot == depth) x_slot = 0;
      if (++x_k == SB) x_k = 0;
    }
  };
  for (int d = 0; d < depth - 1; d++) issue_w();
  pdl_wait();            // the prepare kernel's output (and the previous launch's use of the scratch) is behind us
  pdl_trigger();
  for (int d = 0; d < depth - 1; d++) { issue_x(); cp_async_commit(); }
  auto issue_next = [&]() { issue_w(); issue_x(); cp_async_commit(); };

  float out[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; nt++) out[nt][0] = out[nt][1] = out[nt][2] = out[nt][3] = 0.f;

  // scale of the staged columns this lane owns: 2^(133 - S)
  float unscale[NT][2];
#pragma unroll
  for (int nt = 0; nt < NT; nt++) {
    unscale[nt][0] = pow2f(133 - S_col[nt * 8 + 2 * t]);
    unscale[nt][1] = pow2f(133 - S_col[nt * 8 + 2 * t + 1]);
  }
  auto store_rows = [&](int rb, const float (&v)[NT][4]) {
    const int row_base = rb * kBlockRows + warp * 16;
    if (geo.vec_store && row_base + 16 <= N) {
      // Turn the fragment layout (a lane holds 2 rows x 2 columns per column tile) into runs of 8 rows of one column
      // with shuffles, so that every store is 16 bytes: a quarter of the store instructions and, row-sharded, NVLink
      // packets of 16 and 32 bytes instead of 2-byte ones (the store phase is what grows with the ranks).
      // Lanes 0..15 end up with (column c = lane / 2, row half h = lane & 1) of the column tile.
      const int c = (lane >> 1) & 7, h = lane & 1;
#pragma unroll
      for (int nt = 0; nt < NT; nt++) {
        const float a0 = v[nt][0] * unscale[nt][0], a1 = v[nt][1] * unscale[nt][1];
        const float a2 = v[nt][2] * unscale[nt][0], a3 = v[nt][3] * unscale[nt][1];
        uint32_t p0, p1;       // (column 2t, column 2t + 1) of row g and of row g + 8
        if (y_dtype == GGQ_BF16) {
          const __nv_bfloat162 q0 = __floats2bfloat162_rn(a0, a1), q1 = __floats2bfloat162_rn(a2, a3);
          p0 = *reinterpret_cast<const uint32_t*>(&q0); p1 = *reinterpret_cast<const uint32_t*>(&q1);
        } else {
          const __half2 q0 = __floats2half2_rn(a0, a1), q1 = __floats2half2_rn(a2, a3);
          p0 = *reinterpret_cast<const uint32_t*>(&q0); p1 = *reinterpret_cast<const uint32_t*>(&q1);
        }
        uint32_t e[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
          const int src = j * 4 + (c >> 1);            // the lane with g = j, t = c / 2
          const uint32_t u0 = __shfl_sync(0xFFFFFFFFu, p0, src), u1 = __shfl_sync(0xFFFFFFFFu, p1, src);
          const uint32_t u = h ? u1 : u0;
          e[j] = (c & 1) ? (u >> 16) : (u & 0xFFFFu);
        }
        const uint4 run = make_uint4(e[0] | (e[1] << 16), e[2] | (e[3] << 16), e[4] | (e[5] << 16), e[6] | (e[7] << 16));
        const int col = nt * 8 + c;
        if (lane < 16 && col < M) {
          if (pp.world == 0) {
            *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(y) + (int64_t)col * N + row_base + 8 * h) = run;
          } else {
#pragma unroll 1
            for (int p = 0; p < pp.world; p++)
              *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(pp.y[p]) + (int64_t)col * pp.n_total + pp.row_offset + row_base + 8 * h) = run;
          }
        }
      }
      return;
    }
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const int row = rb * kBlockRows + warp * 16 + g + 8 * (i >> 1), col = nt * 8 + 2 * t + (i & 1);
        if (row < N && col < M) {
          const float val = v[nt][i] * unscale[nt][i & 1];
          if (pp.world == 0) store_out(y, y_dtype, (int64_t)col * N + row, val);
          else {            // row-sharded: this rank's rows of every rank's (M, n_total) output
#pragma unroll 1
            for (int p = 0; p < pp.world; p++) store_out(pp.y[p], y_dtype, (int64_t)col * pp.n_total + pp.row_offset + row, val);
          }
        }
      }
    }
  };

  int rb = rb_first, k = (int)(s_begin - (int64_t)rb_first * SB), slot = 0, seg_k = k;
  uint32_t ring_round = 0;              // how often the ring has wrapped: the parity a slot's barrier shows
  for (int i = 0; i < n_steps; i++) {
    cp_async_wait_pending(depth - 2);
    __syncthreads();                    // everybody's copies of step i have landed; everybody is done with step i - 1
    issue_next();
    if (tma) { tma_box_wait(my_bars + 8 * slot, ring_round & 1, status, lane); __syncwarp(); }
    const int row0 = rb * kBlockRows + warp * 16;
    if (row0 < N) {
      const uint32_t blk0 = my_ring + slot * geo.wslot_bytes + g * F::kPitch + ((k * F::kTs) & 15);
      block_mul<F, NT>(blk0, blk0 + 8 * F::kPitch, g, t, x_ring + slot * geo.xstage_bytes, out);
    }
    if (++slot == depth) { slot = 0; ++ring_round; }

    if (k == SB - 1 || i == n_steps - 1) {
      // ---- the CTA's segment of row block rb ends here
      const bool whole = seg_k == 0 && k == SB - 1;
      if (whole) {
        store_rows(rb, out);
      } else {
        const int part = rb == rb_first ? 0 : 1;
        float* sl = slots + (((int64_t)b * 2 + part) * kBlockRows + warp * 16) * XR;
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
          __stcg(reinterpret_cast<float2*>(sl + g * XR + nt * 8 + 2 * t), make_float2(out[nt][0], out[nt][1]));
          __stcg(reinterpret_cast<float2*>(sl + (g + 8) * XR + nt * 8 + 2 * t), make_float2(out[nt][2], out[nt][3]));
        }
        const int64_t rb_s0 = (int64_t)rb * SB;
        const int c_first = cta_of_step(rb_s0, geo.S, G), c_last = cta_of_step(rb_s0 + SB - 1, geo.S, G);
        __threadfence();
        __syncthreads();
        if (tid == 0) {
          const int old = atomicAdd(counters + rb, 1);
          s_last = old + 1 == c_last - c_first + 1;
        }
        __syncthreads();
        if (s_last) {
          __threadfence();
          float sum[NT][4];
#pragma unroll
          for (int nt = 0; nt < NT; nt++) sum[nt][0] = sum[nt][1] = sum[nt][2] = sum[nt][3] = 0.f;
          for (int c = c_first; c <= c_last; c++) {
            const int cpart = (int)((geo.S * c / G) / SB) == rb ? 0 : 1;
            const float* cs = slots + (((int64_t)c * 2 + cpart) * kBlockRows + warp * 16) * XR;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
              const float2 lo = __ldcg(reinterpret_cast<const float2*>(cs + g * XR + nt * 8 + 2 * t));
              const float2 hi = __ldcg(reinterpret_cast<const float2*>(cs + (g + 8) * XR + nt * 8 + 2 * t));
              sum[nt][0] += lo.x; sum[nt][1] += lo.y; sum[nt][2] += hi.x; sum[nt][3] += hi.y;
            }
          }
          store_rows(rb, sum);
          if (tid == 0) counters[rb] = 0;
        }
      }
#pragma unroll
      for (int nt = 0; nt < NT; nt++) out[nt][0] = out[nt][1] = out[nt][2] = out[nt][3] = 0.f;
      seg_k = 0;
    }
    if (++k == SB) { k = 0; ++rb; }
  }
  cp_async_wait_pending(0);
  peer_publish(pp, tid, gridDim.x);        // row-sharded: raise this rank's flag on every rank once the whole grid has stored
}

// ---------------------------------------------------------------------------------------------
// host side

struct FormatInfo { int qt, ts, pitch, off_bytes; };
static bool format_of(int qtype, FormatInfo* fi) {
  switch (qtype) {
    case QT_Q4_K: *fi = {FQ4K::kQt, FQ4K::kTs, FQ4K::kPitch, FQ4K::kOffBytes}; return true;
    case QT_Q5_K: *fi = {FQ5K::kQt, FQ5K::kTs, FQ5K::kPitch, FQ5K::kOffBytes}; return true;
    case QT_Q6_K: *fi = {FQ6K::kQt, FQ6K::kTs, FQ6K::kPitch, FQ6K::kOffBytes}; return true;
    default: return false;
  }
}
static int tiles_of(int M) { return M <= 8 ? 1 : M <= 16 ? 2 : 4; }

static bool plan(const FormatInfo& fi, int64_t N, int64_t K, int M, Geo* geo) {
  const int XR = 8 * tiles_of(M);
  Geo g{};
  g.SB = (int)(K / 256);
  g.RB = (int)((N + kBlockRows - 1) / kBlockRows);
  g.S = (int64_t)g.RB * g.SB;
  g.wslot_bytes = 16 * fi.pitch;
  g.xstage_bytes = XR * (512 + fi.off_bytes);
  const int per_depth = kWarps * g.wslot_bytes + g.xstage_bytes;
  g.depth = std::min(4, (kSmemLimit / kCtasPerSm - 1024) / per_depth);
  if (g.depth < 2) return false;
  g.off_x = kWarps * g.depth * g.wslot_bytes;
  g.total = g.off_x + g.depth * g.xstage_bytes;
  *geo = g;
  return true;
}

struct WsLayout { size_t xp, xo, scol, slots, total; };
static WsLayout ws_layout(const FormatInfo& fi, int64_t K, int M, int sm_count) {
  const int XR = 8 * tiles_of(M);
  const int64_t SB = K / 256;
  WsLayout l{};
  size_t p = kWsGemmPartialOffset;
  l.xp = p; p += (size_t)SB * XR * 512;
  l.xo = p; p += (size_t)SB * XR * fi.off_bytes;
  l.scol = p; p += 256;
  l.slots = p; p += (size_t)sm_count * kCtasPerSm * 2 * kBlockRows * XR * sizeof(float);
  l.total = (p + 255) / 256 * 256;
  return l;
}

template <class F, int NT>
static cudaError_t launch(const Geo& geo, int grid, cudaStream_t st, const uint8_t* w, int N, int K, const void* x, int64_t ldx, int M,
                          void* y, int y_dtype, uint8_t* ws, const WsLayout& l, const PeerPublish& pp, int* status,
                          const CUtensorMap& w_map) {
  static std::atomic<bool> attr_done[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(gemv_wide_kernel<F, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit / kCtasPerSm - 1024);
    if (e != cudaSuccess) return e;
    attr_done[dev].store(true, std::memory_order_release);
  }
  constexpr int XR = 8 * NT;
  cudaError_t err = launch_pdl(prepare_kernel<F, XR>, XR, 256, 0, st, (const __nv_bfloat16*)x, ldx, K, M, ws + l.xp, ws + l.xo,
                               reinterpret_cast<int*>(ws + l.scol), pp, status);
  if (err != cudaSuccess) return err;
  err = launch_pdl(gemv_wide_kernel<F, NT>, grid, kThreads, (size_t)geo.total, st, w, N, K, (const uint8_t*)(ws + l.xp),
                   (const uint8_t*)(ws + l.xo), reinterpret_cast<const int*>(ws + l.scol), M, y, y_dtype,
                   reinterpret_cast<int*>(ws + kWsCounterOffset), reinterpret_cast<float*>(ws + l.slots), geo, pp, status, w_map);
  return err != cudaSuccess ? err : cudaPeekAtLastError();
}

template <class F>
static cudaError_t launch_tiles(int NT, const Geo& geo, int grid, cudaStream_t st, const uint8_t* w, int N, int K, const void* x,
                                int64_t ldx, int M, void* y, int y_dtype, uint8_t* ws, const WsLayout& l, const PeerPublish& pp,
                                int* status, const CUtensorMap& w_map) {
  switch (NT) {
    case 1: return launch<F, 1>(geo, grid, st, w, N, K, x, ldx, M, y, y_dtype, ws, l, pp, status, w_map);
    case 2: return launch<F, 2>(geo, grid, st, w, N, K, x, ldx, M, y, y_dtype, ws, l, pp, status, w_map);
    default: return launch<F, 4>(geo, grid, st, w, N, K, x, ldx, M, y, y_dtype, ws, l, pp, status, w_map);
  }
}

}  // namespace wide

int gemv_wide_max_batch() { return wide::kMaxBatch; }

bool gemv_wide_applicable(int qtype, int64_t N, int64_t K, int M, const void* w, const void* x) {
  wide::FormatInfo fi;
  if (!wide::format_of(qtype, &fi)) return false;
  if (M < 1 || M > wide::kMaxBatch || K <= 0 || K % 256 || N < 1 || N > (1ll << 24)) return false;
  if ((K / 256 * fi.ts) % 16 || (uintptr_t)w % 16 || (uintptr_t)x % 16) return false;
  if (N * (K / 256 * fi.ts) >= (1ll << 40)) return false;
  wide::Geo geo;
  return wide::plan(fi, N, K, M, &geo);
}

// Scratch: arrival counters (one per row block) in the counter area every kernel shares; in the float area the
// staged activations, their offset operand, the column exponents, and two partial slots per CTA.
size_t gemv_wide_workspace_bytes(int qtype, int64_t N, int64_t K, int M, int sm_count) {
  wide::FormatInfo fi;
  if (!wide::format_of(qtype, &fi) || M < 1) return 0;
  if (sm_count <= 0) sm_count = 148;
  return wide::ws_layout(fi, K, std::min(M, wide::kMaxBatch), sm_count).total;
}

cudaError_t gemv_wide(int qtype, const uint8_t* w, int64_t N, int64_t K, const void* x, int M, void* y, int y_dtype,
                      void* ws, size_t ws_bytes, int sm_count, cudaStream_t st, int64_t ldx, const PeerPublish* peers, int* status) {
  using namespace wide;
  FormatInfo fi;
  if (!format_of(qtype, &fi)) return cudaErrorInvalidValue;
  if (sm_count <= 0) sm_count = 148;
  Geo geo;
  if (!plan(fi, N, K, M, &geo)) return cudaErrorInvalidValue;
  const WsLayout l = ws_layout(fi, K, M, sm_count);
  if (!ws || ws_bytes < l.total || (uintptr_t)ws % 256) return cudaErrorInvalidValue;
  if (kWsCounterOffset + (size_t)geo.RB * sizeof(int) > kWsGemmPartialOffset) return cudaErrorInvalidValue;
  const int grid = (int)std::min<int64_t>((int64_t)sm_count * kCtasPerSm, geo.S);
  const int NT = tiles_of(M);
  uint8_t* base = reinterpret_cast<uint8_t*>(ws);
  PeerPublish pp = {};
  if (peers) pp = *peers;
  if (ldx <= 0) ldx = K;
  if (ldx < K || (ldx * 2) % 16) return cudaErrorInvalidValue;
  // Copy path: the weight as a tensor map of 32-bit words [N rows, row bytes / 4], box = slot pitch x 16 rows (measured on
  // B200, 8192 x 28672 at 8 / 32 batch rows: Q4_K 60.3 / 92.8 against 63.5 / 99.8 us, Q6_K 80.7 / 117.1 against 89.1 / 126.7);
  // per-lane cp.async copies where the driver offers no encoder and under GGQ_WIDE_TMA=0.
  const char* tma_env = getenv("GGQ_WIDE_TMA");        // read per call, so that one process can take both paths
  const bool want_tma = !(tma_env && tma_env[0] == '0');
  CUtensorMap w_map;
  memset(&w_map, 0, sizeof(w_map));
  geo.tma = want_tma && make_weight_map(&w_map, w, N, K / 256 * fi.ts, fi.pitch / 4) ? 1 : 0;
  // 16-byte output stores: 2-byte outputs, and every run of 8 rows of a column starts on a 16-byte boundary
  bool vec = y_dtype == GGQ_BF16 || y_dtype == GGQ_F16;
  if (pp.world == 0) {
    vec = vec && N % 8 == 0 && (uintptr_t)y % 16 == 0;
  } else {
    vec = vec && pp.n_total % 8 == 0 && pp.row_offset % 8 == 0;
    for (int p = 0; p < pp.world; p++) vec = vec && (uintptr_t)pp.y[p] % 16 == 0;
  }
  const char* vec_env = getenv("GGQ_WIDE_VEC_STORE");       // "0": element-wise stores (read per call; the tests take both)
  geo.vec_store = vec && !(vec_env && vec_env[0] == '0') ? 1 : 0;
  switch (qtype) {
    case QT_Q4_K: return launch_tiles<FQ4K>(NT, geo, grid, st, w, (int)N, (int)K, x, ldx, M, y, y_dtype, base, l, pp, status, w_map);
    case QT_Q5_K: return launch_tiles<FQ5K>(NT, geo, grid, st, w, (int)N, (int)K, x, ldx, M, y, y_dtype, base, l, pp, status, w_map);
    case QT_Q6_K: return launch_tiles<FQ6K>(NT, geo, grid, st, w, (int)N, (int)K, x, ldx, M, y, y_dtype, base, l, pp, status, w_map);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace ggq
