// Fused decode + multiply for small batches (1 <= M <= 16), every block qtype, on the tensor cores.
//
// The per-element FMA kernel (gemv_generic.cu) spends 2.5 instructions per weight *per batch
// row*; this kernel pays a fixed price per weight whatever the batch:
//   * each lane decodes eight consecutive weights of two rows with the shared decode8 routines
//     (bit-exact float32 values),
//   * splits every float32 weight into three bf16 terms  w = b0 + b1 + b2  (8 significant bits
//     each, so the split is exact),
//   * and feeds them to mma.sync.m16n8k16 (16 weight rows x 16 k  times  16 k x 8 batch rows)
//     with float32 accumulation.  The products b_i * x are exact and the three terms re-assemble
//     the float32 weight in the accumulator, so the result carries the weight at full precision
//     (a one-hot x returns bf16(float32 weight) exactly) and the cost does not grow with M.
// k-slots of the MMA are assigned so that the four lanes of a quad hold 32 consecutive weights
// of their row (eight each); the activations are read in exactly that order, 16 bytes per lane.
//
// A CTA owns 16 output rows; its eight warps split K in steps of 32 weights and their partial
// tiles are added through shared memory (fixed order, deterministic).  HBM-bound in principle;
// in practice bound by the decode + split instruction count (about 10 per weight).
#include "ggq_decode.cuh"
#include "gemv.cuh"

namespace ggq {
namespace mmav {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// bf16 pair (lo = high half of a's bits, hi = high half of b's bits): truncation, exact for values
// that already have at most 8 significant bits.
__device__ __forceinline__ uint32_t pack_hi(float a, float b) {
  return __byte_perm(__float_as_uint(a), __float_as_uint(b), 0x7632);
}
__device__ __forceinline__ float trunc_bf16(float v) { return __uint_as_float(__float_as_uint(v) & 0xFFFF0000u); }

// Split eight float32 weights into three exact bf16 layers, packed as the MMA wants them:
// layer[l][j] = bf16 pair (elements 2j, 2j+1) of layer l.
__device__ __forceinline__ void split3(const float* v, uint32_t (&layer)[3][4]) {
  float r1[8], r2[8];
#pragma unroll
  for (int i = 0; i < 8; i++) {
    r1[i] = __fsub_rn(v[i], trunc_bf16(v[i]));          // exact: removes the top 8 significant bits
    r2[i] = __fsub_rn(r1[i], trunc_bf16(r1[i]));        // exact: what is left has at most 8 bits
  }
#pragma unroll
  for (int j = 0; j < 4; j++) {
    layer[0][j] = pack_hi(v[2 * j], v[2 * j + 1]);
    layer[1][j] = pack_hi(r1[2 * j], r1[2 * j + 1]);
    layer[2][j] = pack_hi(r2[2 * j], r2[2 * j + 1]);
  }
}

template <int QT, int NCG>   // NCG column groups of 8 batch rows
__global__ void __launch_bounds__(kThreads)
gemv_mma_kernel(const uint8_t* __restrict__ w, int N, int K, const __nv_bfloat16* __restrict__ x, int M,
                void* __restrict__ y, int y_dtype, const uint8_t* __restrict__ tab) {
  constexpr int BS = block_elems_of(QT), TS = block_bytes_of(QT);
  __shared__ float red[kWarps][NCG][4][32];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * 16;
  const int64_t row_bytes = (int64_t)(K / BS) * TS;
  const uint8_t* w0 = w + (int64_t)min(n0 + g, N - 1) * row_bytes;
  const uint8_t* w1 = w + (int64_t)min(n0 + g + 8, N - 1) * row_bytes;
  const int n_steps = K / 32;

  float acc[NCG][4];
#pragma unroll
  for (int c = 0; c < NCG; c++)
#pragma unroll
    for (int i = 0; i < 4; i++) acc[c][i] = 0.f;

  for (int s = warp; s < n_steps; s += kWarps) {
    const int e = 32 * s + 8 * t;                       // this lane's eight weights of the step
    const int64_t boff = (int64_t)(e / BS) * TS;
    const int grp = (e % BS) >> 3;
    float v0[8], v1[8];
    Dec<QT>::run(w0 + boff, grp, tab, v0);
    Dec<QT>::run(w1 + boff, grp, tab, v1);
    uint32_t l0[3][4], l1[3][4];
    split3(v0, l0);
    split3(v1, l1);
#pragma unroll
    for (int c = 0; c < NCG; c++) {
      const int m = 8 * c + g;                          // the batch row this lane feeds as B column g
      uint4 xq = make_uint4(0, 0, 0, 0);
      if (m < M) xq = __ldg(reinterpret_cast<const uint4*>(x + (int64_t)m * K + e));
#pragma unroll
      for (int l = 0; l < 3; l++) {
        // k-slots (2t, 2t+1) <- weights 0,1 ; (2t+8, 2t+9) <- weights 2,3 ; second MMA: weights 4..7
        mma16816(acc[c], l0[l][0], l1[l][0], l0[l][1], l1[l][1], xq.x, xq.y);
        mma16816(acc[c], l0[l][2], l1[l][2], l0[l][3], l1[l][3], xq.z, xq.w);
      }
    }
  }
#pragma unroll
  for (int c = 0; c < NCG; c++)
#pragma unroll
    for (int i = 0; i < 4; i++) red[warp][c][i][lane] = acc[c][i];
  __syncthreads();
  // fold the eight warps (fixed order) and store: fragment element i of lane (g, t) is
  // row g + 8 (i >> 1), batch column 2t + (i & 1) of its group
  for (int idx = tid; idx < NCG * 4 * 32; idx += kThreads) {
    const int c = idx / 128, i = (idx >> 5) & 3, ln = idx & 31;
    float sum = 0.f;
#pragma unroll
    for (int ww = 0; ww < kWarps; ww++) sum += red[ww][c][i][ln];
    const int row = n0 + (ln >> 2) + 8 * (i >> 1);
    const int m = 8 * c + 2 * (ln & 3) + (i & 1);
    if (row < N && m < M) store_out(y, y_dtype, (int64_t)m * N + row, sum);
  }
}

// ---------------------------------------------------------------------------------------------
// Q4_K and Q5_K, 2 <= M <= 16, without the float32 detour: the 4-bit codes go to the tensor cores as exact
// bf16 integers (0x000v = v * 2^-133; the high nibbles as 16 v), one MMA layer instead of three,
// and the float32 scales are applied to the 32-weight partial sums:
//     y[m] += (d * sc) * sum(q * x[m]) - (dmin * mn) * sum(x[m])      per sub-block,
// with sum(x[m]) from a second MMA against an all-ones A operand.  Activations are multiplied by
// 2^64 on the way in so that the products are normal float32 numbers (valid for activation
// magnitudes from about 2^-50 to 2^62).  Warp j of a CTA takes sub-block j of every superblock.
// Q5: the block is Q5_K (176 bytes: the same header, then 32 bytes of fifth bits, then the nibbles)
// and the code is nibble | bit << 4, assembled per byte before it is spread into bf16 pairs.
template <int NCG, bool Q5>
__global__ void __launch_bounds__(kThreads)
gemv_mma_q45k_kernel(const uint8_t* __restrict__ w, int N, int K, const __nv_bfloat16* __restrict__ x, int M,
                    void* __restrict__ y, int y_dtype) {
  __shared__ float red[kWarps][NCG][4][32];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * 16;
  const int n_sb = K / 256;
  constexpr int TS = Q5 ? 176 : 144, QS = Q5 ? 48 : 16;
  const int64_t row_bytes = (int64_t)n_sb * TS;
  const uint8_t* w0 = w + (int64_t)min(n0 + g, N - 1) * row_bytes;
  const uint8_t* w1 = w + (int64_t)min(n0 + g + 8, N - 1) * row_bytes;
  const int sbk = warp, pair = sbk >> 1;
  const bool high = sbk & 1;
  const uint32_t mask = high ? 0x00F000F0u : 0x000F000Fu;
  const float up_codes = (high && !Q5) ? 0x1p65f : 0x1p69f;   // 2^(133 - 64); Q4_K keeps high nibbles as 16 q
  const __nv_bfloat162 x_up = __floats2bfloat162_rn(0x1p64f, 0x1p64f);
  const uint32_t ones = 0x3F803F80u;                    // bf16 (1.0, 1.0)

  float acc[NCG][4];
#pragma unroll
  for (int c = 0; c < NCG; c++)
#pragma unroll
    for (int i = 0; i < 4; i++) acc[c][i] = 0.f;

  // the loads of superblock b + 1 are issued before superblock b is multiplied (a deeper register
  // pipeline measured slower: the registers it takes cost more occupancy than the latency it hides)
  struct Raw { uint4 h0, h1; uint2 q0, q1, e0, e1; uint4 xq[NCG]; };
  auto load = [&](int b) {
    Raw r;
    const uint8_t* blk0 = w0 + (int64_t)b * TS;
    const uint8_t* blk1 = w1 + (int64_t)b * TS;
    r.h0 = __ldg(reinterpret_cast<const uint4*>(blk0));
    r.h1 = __ldg(reinterpret_cast<const uint4*>(blk1));
    r.q0 = __ldg(reinterpret_cast<const uint2*>(blk0 + QS + 32 * pair + 8 * t));
    r.q1 = __ldg(reinterpret_cast<const uint2*>(blk1 + QS + 32 * pair + 8 * t));
    r.e0 = r.e1 = make_uint2(0, 0);
    if constexpr (Q5) {
      r.e0 = __ldg(reinterpret_cast<const uint2*>(blk0 + 16 + 8 * t));
      r.e1 = __ldg(reinterpret_cast<const uint2*>(blk1 + 16 + 8 * t));
    }
#pragma unroll
    for (int c = 0; c < NCG; c++) {
      const int m = 8 * c + g;                          // the batch row this lane feeds as B column g
      r.xq[c] = make_uint4(0, 0, 0, 0);
      if (m < M) r.xq[c] = __ldg(reinterpret_cast<const uint4*>(x + (int64_t)m * K + (int64_t)b * 256 + 32 * sbk + 8 * t));
    }
    return r;
  };
  Raw cur = load(0);
  for (int b = 0; b < n_sb; b++) {
    Raw nxt = cur;
    if (b + 1 < n_sb) nxt = load(b + 1);
    const uint4 h0 = cur.h0, h1 = cur.h1;
    const uint2 q0 = cur.q0, q1 = cur.q1;
    // 6-bit scale and min of sub-block sbk from the 12 packed bytes (header words y, z, w)
    float dl[2], ndm[2];
#pragma unroll
    for (int rr = 0; rr < 2; rr++) {
      const uint4& h = rr ? h1 : h0;
      const __half2 dd = *reinterpret_cast<const __half2*>(&h.x);
      uint32_t sc, mn;
      if (sbk < 4) {
        sc = (h.y >> (8 * sbk)) & 63;
        mn = (h.z >> (8 * sbk)) & 63;
      } else {
        const uint32_t md = (h.w >> (8 * (sbk - 4))) & 0xFF;
        sc = (md & 15) | (((h.y >> (8 * (sbk - 4) + 6)) & 3) << 4);
        mn = (md >> 4) | (((h.z >> (8 * (sbk - 4) + 6)) & 3) << 4);
      }
      dl[rr] = __fmul_rn(__fmul_rn(__low2float(dd), (float)sc), up_codes);
      ndm[rr] = -__fmul_rn(__fmul_rn(__high2float(dd), (float)mn), 0x1p-64f);
    }
    // bytes (0,2) of a word fill k-slots 2t, 2t+1, bytes (1,3) fill k-slots 2t+8, 2t+9
    uint32_t a00, a01, a02, a03, a10, a11, a12, a13;
    if constexpr (Q5) {
      const int ns = high ? 4 : 0;
      auto code = [&](uint32_t q, uint32_t e) { return ((q >> ns) & 0x0F0F0F0Fu) | (((e >> sbk) & 0x01010101u) << 4); };
      const uint32_t c0x = code(q0.x, cur.e0.x), c1x = code(q1.x, cur.e1.x), c0y = code(q0.y, cur.e0.y), c1y = code(q1.y, cur.e1.y);
      a00 = c0x & 0x00FF00FFu; a01 = c1x & 0x00FF00FFu; a02 = (c0x >> 8) & 0x00FF00FFu; a03 = (c1x >> 8) & 0x00FF00FFu;
      a10 = c0y & 0x00FF00FFu; a11 = c1y & 0x00FF00FFu; a12 = (c0y >> 8) & 0x00FF00FFu; a13 = (c1y >> 8) & 0x00FF00FFu;
    } else {
      a00 = q0.x & mask; a01 = q1.x & mask; a02 = (q0.x >> 8) & mask; a03 = (q1.x >> 8) & mask;
      a10 = q0.y & mask; a11 = q1.y & mask; a12 = (q0.y >> 8) & mask; a13 = (q1.y >> 8) & mask;
    }
#pragma unroll
    for (int c = 0; c < NCG; c++) {
      const uint4 xq = cur.xq[c];
      // (e0,e2) / (e1,e3) pairs to match the byte order of the codes, scaled by 2^64
      uint32_t bf[4] = {__byte_perm(xq.x, xq.y, 0x5410), __byte_perm(xq.x, xq.y, 0x7632),
                        __byte_perm(xq.z, xq.w, 0x5410), __byte_perm(xq.z, xq.w, 0x7632)};
#pragma unroll
      for (int i = 0; i < 4; i++) {
        __nv_bfloat162 v = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&bf[i]), x_up);
        bf[i] = *reinterpret_cast<uint32_t*>(&v);
      }
      float u[4] = {0.f, 0.f, 0.f, 0.f}, sx[4] = {0.f, 0.f, 0.f, 0.f};
      mma16816(u, a00, a01, a02, a03, bf[0], bf[1]);
      mma16816(u, a10, a11, a12, a13, bf[2], bf[3]);
      mma16816(sx, ones, ones, ones, ones, bf[0], bf[1]);
      mma16816(sx, ones, ones, ones, ones, bf[2], bf[3]);
      acc[c][0] = fmaf(ndm[0], sx[0], fmaf(dl[0], u[0], acc[c][0]));
      acc[c][1] = fmaf(ndm[0], sx[1], fmaf(dl[0], u[1], acc[c][1]));
      acc[c][2] = fmaf(ndm[1], sx[2], fmaf(dl[1], u[2], acc[c][2]));
      acc[c][3] = fmaf(ndm[1], sx[3], fmaf(dl[1], u[3], acc[c][3]));
    }
    cur = nxt;
  }
#pragma unroll
  for (int c = 0; c < NCG; c++)
#pragma unroll
    for (int i = 0; i < 4; i++) red[warp][c][i][lane] = acc[c][i];
  __syncthreads();
  for (int idx = tid; idx < NCG * 4 * 32; idx += kThreads) {
    const int c = idx / 128, i = (idx >> 5) & 3, ln = idx & 31;
    float sum = 0.f;
#pragma unroll
    for (int ww = 0; ww < kWarps; ww++) sum += red[ww][c][i][ln];
    const int row = n0 + (ln >> 2) + 8 * (i >> 1);
    const int m = 8 * c + 2 * (ln & 3) + (i & 1);
    if (row < N && m < M) store_out(y, y_dtype, (int64_t)m * N + row, sum);
  }
}

// Q6_K, 2 <= M <= 16, the same idea: the 6-bit code (low nibble | high bits << 4) is one exact bf16
// integer, an MMA of 16 k-slots is exactly one 16-weight scale group, and
//     y[m] += (d * sc) * (sum(q * x[m]) - 32 * sum(x[m]))      per group.
// Warp j takes quarter j of every superblock (32 weights: half j >> 2, quarter j & 3 of that
// half); a lane holds bytes 4t..4t+3 of the quarter's first group and of its second group.
// Blocks are 2-byte aligned, so words are assembled from 16-bit loads.
__device__ __forceinline__ uint32_t ldg_u32_a2(const uint8_t* p) {
  const unsigned short* q = reinterpret_cast<const unsigned short*>(p);
  return (uint32_t)__ldg(q) | ((uint32_t)__ldg(q + 1) << 16);
}

template <int NCG>
__global__ void __launch_bounds__(kThreads)
gemv_mma_q6k_kernel(const uint8_t* __restrict__ w, int N, int K, const __nv_bfloat16* __restrict__ x, int M,
                    void* __restrict__ y, int y_dtype) {
  __shared__ float red[kWarps][NCG][4][32];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * 16;
  const int n_sb = K / 256;
  const int64_t row_bytes = (int64_t)n_sb * 210;
  const uint8_t* w0 = w + (int64_t)min(n0 + g, N - 1) * row_bytes;
  const uint8_t* w1 = w + (int64_t)min(n0 + g + 8, N - 1) * row_bytes;
  const int h = warp >> 2, c = warp & 3;                // half and quarter
  const int ql_off = 64 * h + 32 * (c & 1) + 4 * t, qh_off = 128 + 32 * h + 4 * t, sc_off = 192 + 8 * h + 2 * c;
  const int nib_shift = 4 * (c >> 1), hi_shift = 2 * c;
  const __nv_bfloat162 x_up = __floats2bfloat162_rn(0x1p64f, 0x1p64f);
  const uint32_t ones = 0x3F803F80u;

  float acc[NCG][4];
#pragma unroll
  for (int cg = 0; cg < NCG; cg++)
#pragma unroll
    for (int i = 0; i < 4; i++) acc[cg][i] = 0.f;

  // the loads of superblock b + 1 are issued before superblock b is multiplied (a deeper register
  // pipeline measured slower: the registers it takes cost more occupancy than the latency it hides)
  struct Raw { uint32_t d[2], sc[2], ql[2][2], qh[2][2]; uint2 xa[NCG], xb[NCG]; };
  auto load = [&](int b) {
    Raw r;
#pragma unroll
    for (int rr = 0; rr < 2; rr++) {
      const uint8_t* blk = (rr ? w1 : w0) + (int64_t)b * 210;
      r.d[rr] = __ldg(reinterpret_cast<const unsigned short*>(blk + 208));
      r.sc[rr] = __ldg(reinterpret_cast<const unsigned short*>(blk + sc_off));
#pragma unroll
      for (int grp = 0; grp < 2; grp++) {
        r.ql[rr][grp] = ldg_u32_a2(blk + ql_off + 16 * grp);
        r.qh[rr][grp] = ldg_u32_a2(blk + qh_off + 16 * grp);
      }
    }
#pragma unroll
    for (int cg = 0; cg < NCG; cg++) {
      const int m = 8 * cg + g;
      r.xa[cg] = make_uint2(0, 0);
      r.xb[cg] = make_uint2(0, 0);
      if (m < M) {
        const __nv_bfloat16* xp = x + (int64_t)m * K + (int64_t)b * 256 + 32 * warp + 4 * t;
        r.xa[cg] = __ldg(reinterpret_cast<const uint2*>(xp));
        r.xb[cg] = __ldg(reinterpret_cast<const uint2*>(xp + 16));
      }
    }
    return r;
  };
  Raw cur = load(0);
  for (int b = 0; b < n_sb; b++) {
    Raw nxt = cur;
    if (b + 1 < n_sb) nxt = load(b + 1);
    uint32_t a[2][4];        // [group][a0..a3]
    float ds[2][2];          // [row][group]: d * sc * 2^69
#pragma unroll
    for (int rr = 0; rr < 2; rr++) {
      const float d = __half2float(__ushort_as_half((unsigned short)cur.d[rr]));
      const uint32_t scw = cur.sc[rr];
      ds[rr][0] = __fmul_rn(__fmul_rn(d, (float)(int)(int8_t)(scw & 0xFF)), 0x1p69f);
      ds[rr][1] = __fmul_rn(__fmul_rn(d, (float)(int)(int8_t)(scw >> 8)), 0x1p69f);
#pragma unroll
      for (int grp = 0; grp < 2; grp++) {
        const uint32_t qlw = cur.ql[rr][grp], qhw = cur.qh[rr][grp];
        const uint32_t cw = ((qlw >> nib_shift) & 0x0F0F0F0Fu) | (((qhw >> hi_shift) & 0x03030303u) << 4);
        a[grp][rr] = cw & 0x00FF00FFu;                   // bytes (0,2): k-slots 2t, 2t+1
        a[grp][2 + rr] = (cw >> 8) & 0x00FF00FFu;        // bytes (1,3): k-slots 2t+8, 2t+9
      }
    }
#pragma unroll
    for (int cg = 0; cg < NCG; cg++) {
      const uint2 xa = cur.xa[cg], xb = cur.xb[cg];
      uint32_t bf[4] = {__byte_perm(xa.x, xa.y, 0x5410), __byte_perm(xa.x, xa.y, 0x7632),
                        __byte_perm(xb.x, xb.y, 0x5410), __byte_perm(xb.x, xb.y, 0x7632)};
#pragma unroll
      for (int i = 0; i < 4; i++) {
        __nv_bfloat162 v = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&bf[i]), x_up);
        bf[i] = *reinterpret_cast<uint32_t*>(&v);
      }
#pragma unroll
      for (int grp = 0; grp < 2; grp++) {
        float u[4] = {0.f, 0.f, 0.f, 0.f}, sx[4] = {0.f, 0.f, 0.f, 0.f};
        mma16816(u, a[grp][0], a[grp][1], a[grp][2], a[grp][3], bf[2 * grp], bf[2 * grp + 1]);
        mma16816(sx, ones, ones, ones, ones, bf[2 * grp], bf[2 * grp + 1]);
        // sum(x) carries 2^64 where sum(q x) carries 2^-69: 32 * 2^-133
        acc[cg][0] = fmaf(ds[0][grp], fmaf(-0x1p-128f, sx[0], u[0]), acc[cg][0]);
        acc[cg][1] = fmaf(ds[0][grp], fmaf(-0x1p-128f, sx[1], u[1]), acc[cg][1]);
        acc[cg][2] = fmaf(ds[1][grp], fmaf(-0x1p-128f, sx[2], u[2]), acc[cg][2]);
        acc[cg][3] = fmaf(ds[1][grp], fmaf(-0x1p-128f, sx[3], u[3]), acc[cg][3]);
      }
    }
    cur = nxt;
  }
#pragma unroll
  for (int cg = 0; cg < NCG; cg++)
#pragma unroll
    for (int i = 0; i < 4; i++) red[warp][cg][i][lane] = acc[cg][i];
  __syncthreads();
  for (int idx = tid; idx < NCG * 4 * 32; idx += kThreads) {
    const int cg = idx / 128, i = (idx >> 5) & 3, ln = idx & 31;
    float sum = 0.f;
#pragma unroll
    for (int ww = 0; ww < kWarps; ww++) sum += red[ww][cg][i][ln];
    const int row = n0 + (ln >> 2) + 8 * (i >> 1);
    const int m = 8 * cg + 2 * (ln & 3) + (i & 1);
    if (row < N && m < M) store_out(y, y_dtype, (int64_t)m * N + row, sum);
  }
}

template <int QT>
static cudaError_t launch(const uint8_t* w, int64_t N, int64_t K, const void* x, int M, void* y, int y_dtype,
                          const uint8_t* tab, cudaStream_t st) {
  const unsigned grid = (unsigned)((N + 15) / 16);
  const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
  if (M <= 8) gemv_mma_kernel<QT, 1><<<grid, kThreads, 0, st>>>(w, (int)N, (int)K, xb, M, y, y_dtype, tab);
  else gemv_mma_kernel<QT, 2><<<grid, kThreads, 0, st>>>(w, (int)N, (int)K, xb, M, y, y_dtype, tab);
  return cudaPeekAtLastError();
}

}  // namespace mmav

bool gemv_mma_applicable(const TypeInfo* ti, int64_t N, int64_t K, int M) {
  return ti && ti->block_elems >= 32 && K % 32 == 0 && K % ti->block_elems == 0 && M >= 1 && M <= 16 && N >= 1 &&
         N < (1ll << 31) - 64 && K < (1ll << 31);
}

cudaError_t gemv_mma(const TypeInfo* ti, const uint8_t* w, int64_t N, int64_t K, const void* x, int M, void* y,
                     int y_dtype, const uint8_t* tab, cudaStream_t st) {
  if ((ti->qtype == QT_Q4_K || ti->qtype == QT_Q5_K) && K % 256 == 0 && (uintptr_t)w % 16 == 0) {
    const unsigned grid = (unsigned)((N + 15) / 16);
    const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
    const bool q5 = ti->qtype == QT_Q5_K;
    if (M <= 8 && !q5) mmav::gemv_mma_q45k_kernel<1, false><<<grid, mmav::kThreads, 0, st>>>(w, (int)N, (int)K, xb, M, y, y_dtype);
    else if (!q5) mmav::gemv_mma_q45k_kernel<2, false><<<grid, mmav::kThreads, 0, st>>>(w, (int)N, (int)K, xb, M, y, y_dtype);
    else if (M <= 8) mmav::gemv_mma_q45k_kernel<1, true><<<grid, mmav::kThreads, 0, st>>>(w, (int)N, (int)K, xb, M, y, y_dtype);
    else mmav::gemv_mma_q45k_kernel<2, true><<<grid, mmav::kThreads, 0, st>>>(w, (int)N, (int)K, xb, M, y, y_dtype);
    return cudaPeekAtLastError();
  }
  if (ti->qtype == QT_Q6_K && K % 256 == 0 && (uintptr_t)w % 2 == 0) {
    const unsigned grid = (unsigned)((N + 15) / 16);
    const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
    if (M <= 8) mmav::gemv_mma_q6k_kernel<1><<<grid, mmav::kThreads, 0, st>>>(w, (int)N, (int)K, xb, M, y, y_dtype);
    else mmav::gemv_mma_q6k_kernel<2><<<grid, mmav::kThreads, 0, st>>>(w, (int)N, (int)K, xb, M, y, y_dtype);
    return cudaPeekAtLastError();
  }
  cudaError_t err = cudaErrorInvalidValue;
  dispatch_block_qtype(ti->qtype, [&]<int QT>() { err = mmav::launch<QT>(w, N, K, x, M, y, y_dtype, tab, st); });
  return err;
}

}  // namespace ggq
