// Q5_K fused decode + multiply for batch 1 on B200: the Q4_K batch-1 design (gemv_q4k.cu) with a
// fifth-bit plane.
//
// Block layout (src/gguf_jax/quants.py, Q5_K decoder; gguf/quants.py Q5_K): d, dmin (float16),
// twelve bytes of packed 6-bit scales and mins, qh[32], qs[128].  Element e = 64 t + 32 u + p
// (pair t, nibble u, p in 0..31) has code = nibble u of qs[32 t + p] + 16 * bit (2t + u) of qh[p]
// and weight = d * sc[2t + u] * code - dmin * mn[2t + u].
//
// As for Q4_K the codes go to the tensor cores as exact bf16 integers (0x00vv = v * 2^-133): the
// nibbles as (w & 0x000F000F) / (w & 0x00F000F0), the fifth bits as (qh & (0x00010001 << 2t)) and
// (qh & (0x00020002 << 2t)) -- single bits, so the masked word is a valid bf16 pair whatever the
// bit position -- accumulated in tiles of their own and folded with a per-lane power of two:
//     u = nib + f * bit,      y += (d * sc) * u - (dmin * mn) * sum(x).
// Everything else (persistent CTA per SM, per-warp rings filled by one TMA box per step -- 52 words x 16 rows --
// or by cp.async where no tensor-map encoder is to be had, activations staged once as
// scaled pair-permuted bf16, the eight B columns as eight sub-block channels, contiguous unit
// ranges with a last-arriver reduction) is the Q4_K design; a step is one superblock (176 B per
// row, pitch 208 = 80 mod 128 so the 128-bit reads of a quarter-warp hit distinct banks).
#include "gemv.cuh"

#include <cstdlib>
#include <cstring>

namespace ggq {
namespace q5k {

constexpr int kBlockBytes = 176;
constexpr int kRowTiles = 2;                   // 16-row tiles per unit
constexpr int kWarps = 8 * kRowTiles;
constexpr int kThreads = (kWarps + 1) * 32;    // sixteen tile warps and one reducer warp
constexpr int kBarFull = 1, kBarFree = 3;      // named barriers (two each, alternating) of the flush hand-off
constexpr int kRowsPerUnit = 16 * kRowTiles;
constexpr int kSbPerUnit = 8;                  // one superblock per warp and step
constexpr int kPieces = 11;                    // 16-byte pieces per row and step
constexpr int kSlotPitch = 208;
constexpr int kSlotBytes = 16 * kSlotPitch;
constexpr int kSmemLimit = 232448;

struct Smem {
  int x;                                                                         // bf16[K], scaled + permuted
  __host__ __device__ explicit Smem(int depth) : x(kWarps * depth * kSlotBytes) {}
  __host__ __device__ int xs(int K) const { return x + 2 * K; }                  // float[K/32] sub-block sums
  __host__ __device__ int zero(int K) const { return xs(K) + (K / 32) * 4; }     // 64 zero bytes
  __host__ __device__ int red(int K) const { return zero(K) + 64; }              // float[2][kWarps][16]
  __host__ __device__ int misc(int K) const { return red(K) + 2 * kWarps * 16 * 4; }
  __host__ __device__ int bars(int K) const { return misc(K) + 16; }   // uint64[kWarps][4]: per-warp slot barriers (tensor-map copies)
  __host__ __device__ int total(int K) const { return bars(K) + kWarps * 4 * 8; }
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint4 lds128(uint32_t a) { return *reinterpret_cast<const uint4*>(__cvta_shared_to_generic(a)); }
__device__ __forceinline__ float2 lds64f(uint32_t a) { return *reinterpret_cast<const float2*>(__cvta_shared_to_generic(a)); }
__device__ __forceinline__ uint32_t lds32(uint32_t a) { return *reinterpret_cast<const uint32_t*>(__cvta_shared_to_generic(a)); }
__device__ __forceinline__ uint32_t lds16(uint32_t a) { return *reinterpret_cast<const uint16_t*>(__cvta_shared_to_generic(a)); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const uint8_t* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void bar_sync(int id, int count) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory"); }
__device__ __forceinline__ void bar_arrive(int id, int count) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory"); }
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float bf16lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16hi(uint32_t u) { return __uint_as_float(u & 0xFFFF0000u); }
// byte `SEL` (0..3) of x as a float, exact: bits 0x4B0000vv are 2^23 + v.
template <int SEL>
__device__ __forceinline__ float byte_to_float(uint32_t x) {
  return __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7440 + SEL)) - 8388608.0f;
}
// Which CTA owns unit u when U units are dealt to G CTAs as ranges [U*b/G, U*(b+1)/G).
__device__ __forceinline__ int owner_of(int64_t u, int64_t U, int G) { return (int)(((u + 1) * G - 1) / U); }

// Per-lane constants of the 6-bit scale unpack: lanes t < 2 own sub-blocks 0..3 (plain 6-bit
// fields), lanes t >= 2 own sub-blocks 4..7 (4 low bits in bytes 8..11, 2 high bits on top of
// bytes 0..7).  Written with selects and masks so the unpack is branch-free.
struct LaneScale {
  bool low;          // t < 2
  int sh, sh2, shm;  // 16 (t & 1), sh + 2, sh + (low ? 0 : 4)
  uint32_t ma, mb;   // 0x3F3F / 0 for low lanes, 0x0F0F / 0x3030 otherwise
  __device__ explicit LaneScale(int t)
      : low(t < 2), sh(16 * (t & 1)), sh2(16 * (t & 1) + 2), shm(16 * (t & 1) + (t < 2 ? 0 : 4)),
        ma(t < 2 ? 0x3F3Fu : 0x0F0Fu), mb(t < 2 ? 0u : 0x3030u) {}
};

// Scales of the sub-block pair (2t, 2t+1) from a block header (d|dmin, s0-3, s4-7, s8-11):
// dl = d * sc, ndm = -(dmin * mn), the products exact in float32 (src/gguf_jax/quants.py:275-305).
__device__ __forceinline__ void pair_scales(const uint4& h, const LaneScale& c, float& dl_a, float& ndm_a,
                                            float& dl_b, float& ndm_b) {
  const __half2 dd = *reinterpret_cast<const __half2*>(&h.x);
  const float d = __low2float(dd), ndmin = -__high2float(dd);
  const uint32_t a_sc = c.low ? h.y : h.w, a_mn = c.low ? h.z : h.w;
  const uint32_t scp = ((a_sc >> c.sh) & c.ma) | ((h.y >> c.sh2) & c.mb);
  const uint32_t mnp = ((a_mn >> c.shm) & c.ma) | ((h.z >> c.sh2) & c.mb);
  dl_a = __fmul_rn(d, byte_to_float<0>(scp));
  dl_b = __fmul_rn(d, byte_to_float<1>(scp));
  ndm_a = __fmul_rn(ndmin, byte_to_float<0>(mnp));
  ndm_b = __fmul_rn(ndmin, byte_to_float<1>(mnp));
}

// Multiply one tile (16 rows x one superblock) by its activations (at xa, sub-block sums at xsa)
// and add this lane's share of the row sums to out0 (row g) / out1 (row g + 8).
__device__ __forceinline__ void compute_tile(uint32_t tile, int g, int t, const LaneScale& lc, uint32_t m1,
                                             float f_lo, float f_hi, uint32_t xa, uint32_t x_step, uint32_t xsa,
                                             float& out0, float& out1) {
  const uint32_t base0 = tile + g * kSlotPitch, base1 = base0 + 8 * kSlotPitch;
  const uint4 h0 = lds128(base0), h1 = lds128(base1);
  const uint4 ea0 = lds128(base0 + 16), eb0 = lds128(base0 + 32);                       // qh, all 32 bytes
  const uint4 ea1 = lds128(base1 + 16), eb1 = lds128(base1 + 32);
  const uint4 qa0 = lds128(base0 + 48 + 32 * t), qb0 = lds128(base0 + 64 + 32 * t);     // qs of pair t
  const uint4 qa1 = lds128(base1 + 48 + 32 * t), qb1 = lds128(base1 + 64 + 32 * t);
  // A lane feeds column g of the B operand; that column is live only in the k-slots of lane
  // group g/2, so every other lane reads the zero page (base = zero page, strides = 0).
  const uint4 x0 = lds128(xa), x1 = lds128(xa + x_step), x2 = lds128(xa + 2 * x_step), x3 = lds128(xa + 3 * x_step);
  const float2 sx = lds64f(xsa);                                                         // X[2t], X[2t+1], scaled

  // Four accumulator tiles: nibbles and fifth bits of the low-nibble sub-block (column 2t is kept)
  // and of the high-nibble sub-block (column 2t+1 is kept).
  float lo[4] = {0.f, 0.f, 0.f, 0.f}, hi[4] = {0.f, 0.f, 0.f, 0.f};
  float lob[4] = {0.f, 0.f, 0.f, 0.f}, hib[4] = {0.f, 0.f, 0.f, 0.f};
  const uint32_t m2 = m1 << 1;
  const uint32_t w0[8] = {qa0.x, qa0.y, qa0.z, qa0.w, qb0.x, qb0.y, qb0.z, qb0.w};
  const uint32_t w1[8] = {qa1.x, qa1.y, qa1.z, qa1.w, qb1.x, qb1.y, qb1.z, qb1.w};
  const uint32_t e0[8] = {ea0.x, ea0.y, ea0.z, ea0.w, eb0.x, eb0.y, eb0.z, eb0.w};
  const uint32_t e1[8] = {ea1.x, ea1.y, ea1.z, ea1.w, eb1.x, eb1.y, eb1.z, eb1.w};
  const uint32_t xr[16] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w,
                           x2.x, x2.y, x2.z, x2.w, x3.x, x3.y, x3.z, x3.w};
#pragma unroll
  for (int i = 0; i < 8; i++) {
    // word i = bytes p = 4i..4i+3 of the pair's run and of qh; bytes (0,2) fill k-slots 2t,2t+1,
    // bytes (1,3) fill k-slots 2t+8,2t+9, matching the pair-permuted activations
    const uint32_t a = w0[i], b = w1[i], as = a >> 8, bs = b >> 8;
    const uint32_t c = e0[i], d = e1[i], cs = c >> 8, ds = d >> 8;
    mma16816(lo, a & 0x000F000Fu, b & 0x000F000Fu, as & 0x000F000Fu, bs & 0x000F000Fu, xr[2 * i], xr[2 * i + 1]);
    mma16816(hi, a & 0x00F000F0u, b & 0x00F000F0u, as & 0x00F000F0u, bs & 0x00F000F0u, xr[2 * i], xr[2 * i + 1]);
    mma16816(lob, c & m1, d & m1, cs & m1, ds & m1, xr[2 * i], xr[2 * i + 1]);
    mma16816(hib, c & m2, d & m2, cs & m2, ds & m2, xr[2 * i], xr[2 * i + 1]);
  }
  float dla, dma, dlb, dmb;
  pair_scales(h0, lc, dla, dma, dlb, dmb);
  out0 = fmaf(dla, fmaf(f_lo, lob[0], lo[0]), out0); out0 = fmaf(dma, sx.x, out0);
  out0 = fmaf(dlb, fmaf(f_hi, hib[1], hi[1]), out0); out0 = fmaf(dmb, sx.y, out0);
  pair_scales(h1, lc, dla, dma, dlb, dmb);
  out1 = fmaf(dla, fmaf(f_lo, lob[2], lo[2]), out1); out1 = fmaf(dma, sx.x, out1);
  out1 = fmaf(dlb, fmaf(f_hi, hib[3], hi[3]), out1); out1 = fmaf(dmb, sx.y, out1);
}

// TMA: a step's 16 rows x 208 bytes (the block and the 32 bytes behind it, which keep the slot's row pitch) arrive as one
// two-dimensional tensor-map box issued by one lane, as in gemv_q4k.cu.
template <int DEPTH, bool TMA>
__global__ void __launch_bounds__(kThreads, 1)
gemv_q5k_m1_kernel(const uint8_t* __restrict__ w, int N, int K, const __nv_bfloat16* __restrict__ x,
                   void* __restrict__ y, int y_dtype, int* __restrict__ counters, float* __restrict__ partials,
                   const PeerPublish pp, int* __restrict__ status, const __grid_constant__ CUtensorMap w_map) {
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_trigger();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int SB = K / 256;                        // superblocks per row
  const int row_bytes = SB * kBlockBytes;
  const int C = (SB + kSbPerUnit - 1) / kSbPerUnit;   // chunks per row group
  const int RG = (N + kRowsPerUnit - 1) / kRowsPerUnit;
  const int64_t U = (int64_t)RG * C;
  const int G = gridDim.x, b = blockIdx.x;
  const int64_t u_begin = U * b / G, u_end = U * (b + 1) / G;
  const int n_units = (int)(u_end - u_begin);
  const int rg_begin = (int)(u_begin / C), c_begin = (int)(u_begin - (int64_t)rg_begin * C);

  const int g = lane >> 2, t = lane & 3;
  const int rt = warp >> 3, j = warp & 7;        // row tile (16 rows) and superblock slot of this warp

  const Smem L(DEPTH);
  const uint32_t my_ring = smem_u32(smem) + warp * (DEPTH * kSlotBytes);
  const uint32_t my_bars = smem_u32(smem) + L.bars(K) + warp * 32;        // DEPTH (<= 4) barriers of 8 bytes
  if (TMA && warp < kWarps) tma_bars_init(my_bars, DEPTH, lane);

  // ---- copy side: 8 instructions per step, each copying the 11 pieces of two rows ----
  const int hl = lane >> 4, kl = lane & 15;
  const bool copier = kl < kPieces;
  const int32_t src_a = hl * row_bytes + 16 * kl;
  const uint32_t dst_a = hl * kSlotPitch + 16 * kl;
  const uint8_t* src = w;
  int rg_i = rg_begin, c_i = c_begin, issued = 0, slot_i = 0;
  auto seek_row_group = [&]() {
    src = w + (int64_t)(rg_i * kRowsPerUnit + 16 * rt) * row_bytes + (int64_t)(c_i * kSbPerUnit + j) * kBlockBytes;
  };
  seek_row_group();
  auto issue_next = [&]() {
    if (TMA) {
      if (issued < n_units) {
        // words and rows outside the tensor (a chunk past the end of a ragged row, rows past N) arrive as zeros
        if (lane == 0)
          tma_box_load(my_ring + slot_i * kSlotBytes, &w_map, (c_i * kSbPerUnit + j) * (kBlockBytes / 4),
                       rg_i * kRowsPerUnit + 16 * rt, my_bars + 8 * slot_i, (uint32_t)kSlotBytes);
        ++issued;
        if (++slot_i == DEPTH) slot_i = 0;
        if (++c_i == C) { c_i = 0; ++rg_i; }
      }
      return;
    }
    if (issued < n_units) {
      const uint32_t dst = my_ring + slot_i * kSlotBytes;
      const int row0 = rg_i * kRowsPerUnit + 16 * rt;
      if (c_i * kSbPerUnit + j < SB) {           // a chunk past the end of a ragged row is never multiplied
        if (row0 + 16 <= N) {
          if (copier) {
            const uint8_t* pa = src + src_a;
#pragma unroll
            for (int i = 0; i < 8; i++) cp_async16(dst + dst_a + i * (2 * kSlotPitch), pa + (int64_t)i * (2 * row_bytes));
          }
        } else {
          for (int p = lane; p < 16 * kPieces; p += 32) {
            const int row = p / kPieces, k = p - row * kPieces;
            cp_async16(dst + row * kSlotPitch + 16 * k,
                       src + (int64_t)(min(row0 + row, N - 1) - row0) * row_bytes + 16 * k);
          }
        }
      }
      ++issued;
      if (++slot_i == DEPTH) slot_i = 0;
      src += kSbPerUnit * kBlockBytes;
      if (++c_i == C) { c_i = 0; ++rg_i; seek_row_group(); }
    }
    cp_async_commit();
  };
  const bool tile_warp = warp < kWarps;           // the last warp only reduces and publishes row sums
  if (tile_warp) {
#pragma unroll
    for (int d = 0; d < DEPTH - 1; d++) issue_next();
  }

  float* xs = reinterpret_cast<float*>(smem + L.xs(K));
  int* xmax = reinterpret_cast<int*>(smem + L.misc(K));
  uint32_t out_tag = 0, x_tag = 0;   // tagged exchange: this launch's tag and the tag its activations carry
  int S;  // activations are held as x * 2^S (even sub-blocks) / x * 2^(S-4) (odd sub-blocks)
  {
    if (tid < 16) reinterpret_cast<uint32_t*>(smem + L.zero(K))[tid] = 0;
    if (tid == 0) *xmax = 0;
    pdl_wait();   // everything below reads or writes memory that the previous kernel may still be using
    peer_wait_previous(pp, tid, status);
    if (pp.world > 0 && pp.tagged) {
      const uint32_t e = pp.flags[pp.rank][pp.world];        // exchanges this rank has completed
      out_tag = peer_tag_of(e + 1) << 16;
      x_tag = peer_tag_of(e + 1 - (uint32_t)pp.x_back) << 16;
      if (pp.after_tagged)
        peer_wait_tagged(pp.after_tagged, pp.after_words, peer_tag_of(e + 1 - (uint32_t)pp.after_back) << 16, tid,
                         kThreads, status);
    }
    __syncthreads();
    const uint4* xg = reinterpret_cast<const uint4*>(x);
    uint4* xv = reinterpret_cast<uint4*>(smem + L.x);
    // One pass over x: sub-block sums, largest magnitude, and the scaled pair-permuted copy:
    // word 2i = (x[4i], x[4i+2]), word 2i+1 = (x[4i+1], x[4i+3]).
    auto stage_x = [&](int S_) -> float {
      const float up_even = __uint_as_float((uint32_t)(127 + S_) << 23);
      const float up_odd = __uint_as_float((uint32_t)(127 + S_ - 4) << 23);
      const float xs_scale = __uint_as_float((uint32_t)(127 + S_ - 133) << 23);
      float amax = 0.f;
      const int n_sub = K / 32;
      const int rot = (int)(((int64_t)b * n_sub) / G) & ~1;      // even: keeps sub-block parity
      // two sub-blocks per thread and round, both loads issued before either is converted
      auto fetch = [&](int sblk, uint4 (&v)[4]) {
#pragma unroll
        for (int q = 0; q < 4; q++)
          v[q] = pp.x_tagged ? peer_load8_tagged(pp.x_tagged, sblk * 4 + q, x_tag, status) : __ldcg(xg + sblk * 4 + q);   // L2-coherent: x may have been stored by peers or by the previous launch while this kernel was already resident
      };
      auto convert = [&](int sblk, const uint4 (&v)[4]) {
        const float up = (sblk & 1) ? up_odd : up_even;
        float sum = 0.f, asum = 0.f;
#pragma unroll
        for (int q = 0; q < 4; q++) {
          const float e0 = bf16lo(v[q].x), e1 = bf16hi(v[q].x), e2 = bf16lo(v[q].y), e3 = bf16hi(v[q].y);
          const float e4 = bf16lo(v[q].z), e5 = bf16hi(v[q].z), e6 = bf16lo(v[q].w), e7 = bf16hi(v[q].w);
          sum += (e0 + e1) + (e2 + e3) + ((e4 + e5) + (e6 + e7));
          asum += (fabsf(e0) + fabsf(e1)) + (fabsf(e2) + fabsf(e3)) + ((fabsf(e4) + fabsf(e5)) + (fabsf(e6) + fabsf(e7)));
          __nv_bfloat162 p0 = __floats2bfloat162_rn(e0 * up, e2 * up);
          __nv_bfloat162 p1 = __floats2bfloat162_rn(e1 * up, e3 * up);
          __nv_bfloat162 p2 = __floats2bfloat162_rn(e4 * up, e6 * up);
          __nv_bfloat162 p3 = __floats2bfloat162_rn(e5 * up, e7 * up);
          xv[sblk * 4 + q] = make_uint4(*reinterpret_cast<uint32_t*>(&p0), *reinterpret_cast<uint32_t*>(&p1),
                                        *reinterpret_cast<uint32_t*>(&p2), *reinterpret_cast<uint32_t*>(&p3));
        }
        xs[sblk] = sum * xs_scale;
        amax = fmaxf(amax, asum);
      
      };
      // A CTA whose units cover fewer chunks than a row has (small shards, small weights) stages only those chunks:
      // `count` sub-blocks from the first chunk on, wrapping at the end of the padded row (C whole chunks); places
      // past the real end of a row are skipped.  Otherwise all of x, from the rotated start.
      const bool part = n_units < C;
      const int wrap = part ? C * (kSbPerUnit * 8) : n_sub;
      const int first = part ? c_begin * (kSbPerUnit * 8) : rot;
      const int count = part ? n_units * (kSbPerUnit * 8) : n_sub;
      auto rotated = [&](int i) { int sblk = i + first; return sblk >= wrap ? sblk - wrap : sblk; };
      for (int i = tid; i < count; i += 2 * kThreads) {
        const int s0 = rotated(i), i1 = i + kThreads;
        const int s1 = i1 < count ? rotated(i1) : n_sub;
        const bool one = s0 < n_sub, two = s1 < n_sub;
        uint4 v0[4], v1[4];
        if (one) fetch(s0, v0);
        if (two) fetch(s1, v1);
        if (one) convert(s0, v0);
        if (two) convert(s1, v1);
      }
      return amax;
    };
    // Optimistic scale 2^96, staged again with a fitted scale when the magnitudes are far from
    // unit scale (same rule as the Q4_K kernel).
    S = 96;
    atomicMax(xmax, (int)__float_as_uint(stage_x(S)));
    __syncthreads();
    const int emax = min((*xmax >> 23) & 0xFF, 254);
    if (emax > 156 || emax < 97) {
      S = max(8, min(120, 247 - emax));
      stage_x(S);
      __syncthreads();
    }
  }
  const float d_up = __uint_as_float((uint32_t)(127 + 133 - S) << 23);   // 2^(133-S)
  const bool live = (g >> 1) == t;
  const uint32_t x_lane_base = live ? smem_u32(smem + L.x) + g * 64 : smem_u32(smem + L.zero(K));
  const uint32_t x_sb_stride = live ? 512u : 0u, x_step = live ? 16u : 0u;
  const uint32_t xs_lane_base = smem_u32(xs) + 8 * t;
  const LaneScale lc(t);
  // fifth bits: bit 2t of qh (value 4^t in the accumulator, wanted 16) belongs to sub-block 2t,
  // bit 2t+1 (value 2 * 4^t against activations that carry 2^-4, wanted 16) to sub-block 2t+1
  const uint32_t m1 = 0x00010001u << (2 * t);
  const float f_lo = 16.f / (float)(1 << (2 * t)), f_hi = 128.f / (float)(1 << (2 * t));
  float* red = reinterpret_cast<float*>(smem + L.red(K));

  // The tile warps leave their row sums in shared memory at the end of a row group and go on; the
  // reducer warp folds them, settles split row groups with the other CTAs and stores the outputs
  // (hand-off through two pairs of named barriers, as in gemv_q4k.cu).
  if (tile_warp) {
    int rg = rg_begin, c = c_begin, done = 0, slot = 0, flush_i = 0;
    uint32_t ring_round = 0;                               // how often the ring has wrapped: the parity the slot's barrier shows
    while (done < n_units) {
      const int c_first = c;
      const int c_stop = min(C, c + (n_units - done));
      float out0 = 0.f, out1 = 0.f;
      int sbg = c * kSbPerUnit + j;
      uint32_t xa = x_lane_base + (uint32_t)sbg * x_sb_stride;
      uint32_t xsa = xs_lane_base + (uint32_t)sbg * 32u;
      for (; c < c_stop; ++c) {
        issue_next();
        if (TMA) tma_box_wait(my_bars + 8 * slot, ring_round & 1, status, lane);
        else cp_async_wait<DEPTH - 1>();
        __syncwarp();
        if (sbg < SB) compute_tile(my_ring + slot * kSlotBytes, g, t, lc, m1, f_lo, f_hi, xa, x_step, xsa, out0, out1);
        __syncwarp();
        if (++slot == DEPTH) { slot = 0; ++ring_round; }
        sbg += kSbPerUnit;
        xa += kSbPerUnit * x_sb_stride;
        xsa += kSbPerUnit * 32u;
      }
      done += c_stop - c_first;

      float v0 = out0, v1 = out1;
      v0 += __shfl_xor_sync(0xFFFFFFFFu, v0, 1); v0 += __shfl_xor_sync(0xFFFFFFFFu, v0, 2);
      v1 += __shfl_xor_sync(0xFFFFFFFFu, v1, 1); v1 += __shfl_xor_sync(0xFFFFFFFFu, v1, 2);
      const int p = flush_i & 1;
      if (flush_i >= 2) bar_sync(kBarFree + p, kThreads);  // the reducer has read this buffer's previous content
      float* redbuf = red + p * (kWarps * 16);
      if (t == 0) {
        redbuf[warp * 16 + g] = v0 * d_up;
        redbuf[warp * 16 + g + 8] = v1 * d_up;
      }
      __threadfence_block();
      bar_arrive(kBarFull + p, kThreads);
      ++flush_i;
      if (c == C) { c = 0; ++rg; }
    }
  } else {
    int rg = rg_begin, c = c_begin, done = 0, flush_i = 0;
    while (done < n_units) {
      const int c_first = c;
      const int c_stop = min(C, c + (n_units - done));
      done += c_stop - c_first;
      c = c_stop;
      const int p = flush_i & 1;
      bar_sync(kBarFull + p, kThreads);                    // all sixteen tile warps have written their sums
      const float* redbuf = red + p * (kWarps * 16);
      const bool complete = (c_first == 0) && (c_stop == C);
      const int64_t rg_first_unit = (int64_t)rg * C, rg_last_unit = rg_first_unit + C - 1;
      const int r = lane;                         // row within the unit
      float v = 0.f;
#pragma unroll
      for (int jj = 0; jj < 8; jj++) v += redbuf[((r >> 4) * 8 + jj) * 16 + (r & 15)];
      __syncwarp();
      bar_arrive(kBarFree + p, kThreads);                  // the buffer may be overwritten
      ++flush_i;
      const int row = rg * kRowsPerUnit + r;
      if (complete) {
        if (row < N) peer_emit(pp, y, y_dtype, row, v, out_tag);
      } else {
        const int slot_p = (rg == rg_begin) ? 0 : 1;
        float* mine = partials + ((int64_t)b * 2 + slot_p) * 64;
        __stcg(&mine[lane], v);
        __threadfence();
        __syncwarp();
        const int bf = owner_of(rg_first_unit, U, G), bl = owner_of(rg_last_unit, U, G);
        int old = 0;
        if (lane == 0) old = atomicAdd(&counters[rg], 1);
        old = __shfl_sync(0xFFFFFFFFu, old, 0);
        if (old == bl - bf) {
          __threadfence();
          float s0 = 0.f;
          for (int bb = bf; bb <= bl; bb++) {
            const int sl = (rg == (int)((U * bb / G) / C)) ? 0 : 1;
            s0 += __ldcg(partials + ((int64_t)bb * 2 + sl) * 64 + lane);
          }
          if (row < N) peer_emit(pp, y, y_dtype, row, s0, out_tag);
          if (lane == 0) counters[rg] = 0;
        }
      }
      if (c == C) { c = 0; ++rg; }
    }
  }
  if (!TMA) cp_async_wait<0>();
  peer_publish(pp, tid, G);
}

}  // namespace q5k

bool gemv_q5k_applicable(int64_t N, int64_t K, int M, const void* w, const void* x) {
  return M == 1 && K % 256 == 0 && q5k::Smem(2).total((int)K) <= q5k::kSmemLimit && N >= 1 && N <= (1ll << 24) &&
         N * (K / 256 * 176) < (1ll << 40) && (uintptr_t)w % 16 == 0 && (uintptr_t)x % 16 == 0;
}

cudaError_t gemv_q5k(const uint8_t* w, int64_t N, int64_t K, const void* x, void* y, int y_dtype, void* ws,
                     size_t ws_bytes, int sm_count, int* status, cudaStream_t st, const PeerPublish* peers) {
  using namespace q5k;
  PeerPublish pp = {};
  if (peers) pp = *peers;
  if (ws_bytes < gemv_q4k_workspace_bytes(N, sm_count) || !ws || sm_count > kMaxSmCount) return cudaErrorInvalidValue;
  const int64_t RG = (N + kRowsPerUnit - 1) / kRowsPerUnit;
  const int64_t U = RG * ((K / 256 + kSbPerUnit - 1) / kSbPerUnit);
  const int grid = (int)(U < sm_count ? U : sm_count);
  int depth = 4;
  while (depth > 2 && Smem(depth).total((int)K) > kSmemLimit) depth--;
  const int smem = Smem(depth).total((int)K);
  if (smem > kSmemLimit) return cudaErrorInvalidValue;
  static std::atomic<bool> attr_done[64];   // setting the attribute twice is harmless, so a flag per device suffices
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(gemv_q5k_m1_kernel<4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_q5k_m1_kernel<3, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_q5k_m1_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_q5k_m1_kernel<4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_q5k_m1_kernel<3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_q5k_m1_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e != cudaSuccess) return e;
    attr_done[dev].store(true, std::memory_order_release);
  }
  float* partials = reinterpret_cast<float*>(ws);
  int* counters = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(ws) + kWsCounterOffset);
  const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
  // copy path: tensor-map boxes where the driver offers the encoder (GGQ_Q5K_TMA=0 keeps cp.async, also the fallback)
  alignas(64) CUtensorMap w_map;
  memset(&w_map, 0, sizeof(w_map));
  static const bool want_tma = [] { const char* e = getenv("GGQ_Q5K_TMA"); return !(e && e[0] == '0'); }();
  const bool tma = want_tma && make_weight_map(&w_map, w, N, K / 256 * kBlockBytes, kSlotPitch / 4);
  cudaError_t err;
#define GGQ_Q5K_LAUNCH(D, T) launch_pdl(gemv_q5k_m1_kernel<D, T>, grid, kThreads, smem, st, w, (int)N, (int)K, xb, y, y_dtype, counters, partials, pp, status, w_map)
  if (tma) err = depth == 4 ? GGQ_Q5K_LAUNCH(4, true) : depth == 3 ? GGQ_Q5K_LAUNCH(3, true) : GGQ_Q5K_LAUNCH(2, true);
  else err = depth == 4 ? GGQ_Q5K_LAUNCH(4, false) : depth == 3 ? GGQ_Q5K_LAUNCH(3, false) : GGQ_Q5K_LAUNCH(2, false);
#undef GGQ_Q5K_LAUNCH
  return err != cudaSuccess ? err : cudaPeekAtLastError();
}

}  // namespace ggq
