// Q6_K fused decode + multiply for batch 1 on B200: the Q4_K batch-1 design (gemv_q4k.cu)
// carried over to the 210-byte Q6_K superblock.
//
// Block layout (src/gguf_jax/quants.py, Q6_K decoder; gguf/quants.py Q6_K): ql[128] low nibbles,
// qh[64] two high bits, sc[16] int8 scales of 16-element groups, d (float16).  Element
// e = 128 h + 32 c + p (half h, quarter c, p in 0..31) has
//     low nibble  = nibble (c >> 1) of ql[64 h + 32 (c & 1) + p]
//     high bits   = bits 2c, 2c+1 of qh[32 h + p]
//     weight      = d * sc[8 h + 2 c + (p >> 4)] * (low + 16 high - 32).
//
// Arithmetic.  Exact integer codes on the tensor cores, as for Q4_K: a bf16 whose upper byte is
// zero is linear in its lower byte (0x00vv = v * 2^-133), so (w & 0x000F000F) is a pair of bf16
// low nibbles and (qh & 0x00030003 << 2c) a pair of (scaled) high-bit fields.  The low nibbles
// and the high bits are multiplied as two separate planes into two accumulator tiles,
//     u = lo + f * hi - 32 * sum(x),      y += (d * sc) * u,
// with f a power of two that depends only on the lane.  Activations are staged once per CTA in
// shared memory, scaled by 2^S (2^(S-4) for quarters 2 and 3, which absorbs the 16 of a high
// nibble), pair-permuted for the MMA fragment layout, next to the 16-element sums of x.
//
// The eight columns of the MMA's B operand are the eight scale groups of a half: lane group t
// holds bytes p in [8t, 8t+8) of every quarter, which belong to group 2c + (t >> 1); column
// gamma carries activations only in the k-slots of the lanes that hold its elements (quarter
// gamma >> 1, lane groups with t >> 1 == gamma & 1) and zeros elsewhere, so one accumulator
// tile collects all eight group sums of 16 rows and lane (g, t) ends up with the sums of rows
// g, g+8 and groups 2t, 2t+1 -- whose two int8 scales are one 16-bit load.
//
// Data movement.  Persistent CTA per SM, sixteen tile warps (plus a reducer warp, as in
// gemv_q4k.cu), each streaming its own tiles (16 rows
// x one superblock) into a private ring of shared-memory slots: one two-dimensional TMA box per step (72 words x 16
// rows of a tensor map over the weight, issued by one lane, counted on a per-warp mbarrier; 45.7 against 49.2 us on
// 8192 x 28672), or 16-byte cp.async copies where the driver offers no tensor-map encoder.
// A 210-byte block is only 2-byte aligned, so a step copies the 16-byte aligned window of 224
// bytes that contains the block and the multiply reads its fields at the block's offset in that
// window (skew); warp j always works on superblocks j, j+8, ... whose skew 2j mod 16 is constant.
// Fields of an odd-skew block are 2 (mod 4) aligned: three aligned words and two funnel shifts
// replace two word loads.  Requires rows that start 16-byte aligned (K a multiple of 2048).
//
// Work split and reduction: as in gemv_q4k.cu (contiguous unit ranges per CTA, partial sums and
// a last-arriver reduction in CTA order for row groups cut by a range boundary).
#include "gemv.cuh"

#include <cstdlib>
#include <cstring>

namespace ggq {
namespace q6k {

constexpr int kBlockBytes = 210;
constexpr int kRowTiles = 2;                   // 16-row tiles per unit
constexpr int kWarps = 8 * kRowTiles;
constexpr int kThreads = (kWarps + 1) * 32;    // sixteen tile warps and one reducer warp
constexpr int kBarFull = 1, kBarFree = 3;      // named barriers (two each, alternating) of the flush hand-off
constexpr int kRowsPerUnit = 16 * kRowTiles;
constexpr int kSbPerUnit = 8;                  // one superblock per warp and step
constexpr int kPieces = 14;                    // 16-byte pieces of the aligned window (skew + 210 <= 224)
// Row pitch = 32 (mod 128): the 4-byte reads of the 32 lanes (8 rows x 4 lane groups, 8 bytes apart)
// fall into 32 different banks.
constexpr int kSlotPitch = 288;
constexpr int kSlotBytes = 16 * kSlotPitch;
constexpr int kSmemLimit = 232448;

struct Smem {
  int x;                                                                         // bf16[K], scaled + permuted
  __host__ __device__ explicit Smem(int depth) : x(kWarps * depth * kSlotBytes) {}
  __host__ __device__ int xs(int K) const { return x + 2 * K; }                  // float[K/16] group sums
  __host__ __device__ int zero(int K) const { return xs(K) + (K / 16) * 4; }     // 64 zero bytes
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
// int8 in byte SEL of v as a float, exact: flip the sign bit, read the byte as 2^23 + (s + 128).
template <int SEL>
__device__ __forceinline__ float int8_to_float(uint32_t v_flipped) {
  return __uint_as_float(__byte_perm(v_flipped, 0x4B000000u, 0x7440 + SEL)) - (8388608.0f + 128.0f);
}
__device__ __forceinline__ int owner_of(int64_t u, int64_t U, int G) { return (int)(((u + 1) * G - 1) / U); }

// Eight bytes of a block field at shared address a.  ALIGN: 8 (one 64-bit load, conflict free at
// this pitch), 4 (two words) or 2 (a = 2 mod 4: three aligned words and two funnel shifts).
template <int ALIGN>
__device__ __forceinline__ uint2 ld_field(uint32_t a) {
  if constexpr (ALIGN == 8) {
    return *reinterpret_cast<const uint2*>(__cvta_shared_to_generic(a));
  } else if constexpr (ALIGN == 4) {
    return make_uint2(lds32(a), lds32(a + 4));
  } else {
    const uint32_t w0 = lds32(a - 2), w1 = lds32(a + 2), w2 = lds32(a + 6);
    return make_uint2(__funnelshift_r(w0, w1, 16), __funnelshift_r(w1, w2, 16));
  }
}

// Per-lane addressing of the activations: pass c (quarter c of a half) reads the lane's eight
// activations if the lane feeds a live column in that pass, the zero page otherwise.
struct LaneX {
  uint32_t addr[4];     // running shared address per pass
  uint32_t stride[4];   // bytes per superblock (512 when live, 0 on the zero page)
};

// Multiply one tile (16 rows x one superblock at `blk`, the block's first byte in the slot of row 0)
// by its activations and add this lane's share of the row sums to out0 (row g) / out1 (row g + 8).
template <int ALIGN>
__device__ __forceinline__ void compute_tile(uint32_t blk, int g, int t, const LaneX& lx, uint32_t xsa, float f_hi,
                                             float& out0, float& out1) {
  const uint32_t b0 = blk + g * kSlotPitch, b1 = b0 + 8 * kSlotPitch;
  const float d0 = __half2float(__ushort_as_half((unsigned short)lds16(b0 + 208)));
  const float d1 = __half2float(__ushort_as_half((unsigned short)lds16(b1 + 208)));
#pragma unroll
  for (int h = 0; h < 2; h++) {
    const uint2 qa0 = ld_field<ALIGN>(b0 + 64 * h + 8 * t), qb0 = ld_field<ALIGN>(b0 + 64 * h + 32 + 8 * t);
    const uint2 qh0 = ld_field<ALIGN>(b0 + 128 + 32 * h + 8 * t);
    const uint2 qa1 = ld_field<ALIGN>(b1 + 64 * h + 8 * t), qb1 = ld_field<ALIGN>(b1 + 64 * h + 32 + 8 * t);
    const uint2 qh1 = ld_field<ALIGN>(b1 + 128 + 32 * h + 8 * t);
    uint4 xb[4];
#pragma unroll
    for (int c = 0; c < 4; c++) xb[c] = lds128(lx.addr[c] + h * (lx.stride[c] >> 1));
    const uint32_t s0 = lds16(b0 + 192 + 8 * h + 2 * t) ^ 0x8080u, s1 = lds16(b1 + 192 + 8 * h + 2 * t) ^ 0x8080u;
    const float2 X = lds64f(xsa + 32 * h);

    float lo[4] = {0.f, 0.f, 0.f, 0.f}, hi[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int m = 0; m < 2; m++) {
      const uint32_t a0 = m ? qa0.y : qa0.x, a1 = m ? qa1.y : qa1.x;
      const uint32_t c0 = m ? qb0.y : qb0.x, c1 = m ? qb1.y : qb1.x;
      const uint32_t e0 = m ? qh0.y : qh0.x, e1 = m ? qh1.y : qh1.x;
      const uint32_t a0s = a0 >> 8, a1s = a1 >> 8, c0s = c0 >> 8, c1s = c1 >> 8, e0s = e0 >> 8, e1s = e1 >> 8;
      const uint32_t x00 = m ? xb[0].z : xb[0].x, x01 = m ? xb[0].w : xb[0].y;
      const uint32_t x10 = m ? xb[1].z : xb[1].x, x11 = m ? xb[1].w : xb[1].y;
      const uint32_t x20 = m ? xb[2].z : xb[2].x, x21 = m ? xb[2].w : xb[2].y;
      const uint32_t x30 = m ? xb[3].z : xb[3].x, x31 = m ? xb[3].w : xb[3].y;
      // quarter 0: low nibbles of ql[0..31], bits 0-1 of qh
      mma16816(lo, a0 & 0x000F000Fu, a1 & 0x000F000Fu, a0s & 0x000F000Fu, a1s & 0x000F000Fu, x00, x01);
      mma16816(hi, e0 & 0x00030003u, e1 & 0x00030003u, e0s & 0x00030003u, e1s & 0x00030003u, x00, x01);
      // quarter 1: low nibbles of ql[32..63], bits 2-3
      mma16816(lo, c0 & 0x000F000Fu, c1 & 0x000F000Fu, c0s & 0x000F000Fu, c1s & 0x000F000Fu, x10, x11);
      mma16816(hi, e0 & 0x000C000Cu, e1 & 0x000C000Cu, e0s & 0x000C000Cu, e1s & 0x000C000Cu, x10, x11);
      // quarter 2: high nibbles of ql[0..31] (x carries 2^-4), bits 4-5
      mma16816(lo, a0 & 0x00F000F0u, a1 & 0x00F000F0u, a0s & 0x00F000F0u, a1s & 0x00F000F0u, x20, x21);
      mma16816(hi, e0 & 0x00300030u, e1 & 0x00300030u, e0s & 0x00300030u, e1s & 0x00300030u, x20, x21);
      // quarter 3: high nibbles of ql[32..63], bits 6-7
      mma16816(lo, c0 & 0x00F000F0u, c1 & 0x00F000F0u, c0s & 0x00F000F0u, c1s & 0x00F000F0u, x30, x31);
      mma16816(hi, e0 & 0x00C000C0u, e1 & 0x00C000C0u, e0s & 0x00C000C0u, e1s & 0x00C000C0u, x30, x31);
    }
    // groups 2t and 2t+1 of this half: u = lo + f hi - 32 X, y += (d sc) u
    float ua = fmaf(f_hi, hi[0], lo[0]), ub = fmaf(f_hi, hi[1], lo[1]);
    ua = fmaf(-32.f, X.x, ua);
    ub = fmaf(-32.f, X.y, ub);
    out0 = fmaf(__fmul_rn(d0, int8_to_float<0>(s0)), ua, out0);
    out0 = fmaf(__fmul_rn(d0, int8_to_float<1>(s0)), ub, out0);
    float va = fmaf(f_hi, hi[2], lo[2]), vb = fmaf(f_hi, hi[3], lo[3]);
    va = fmaf(-32.f, X.x, va);
    vb = fmaf(-32.f, X.y, vb);
    out1 = fmaf(__fmul_rn(d1, int8_to_float<0>(s1)), va, out1);
    out1 = fmaf(__fmul_rn(d1, int8_to_float<1>(s1)), vb, out1);
  }
}

// TMA: a step's 16 rows x 288 bytes (the 224-byte window and the 64 bytes behind it, which keep the slot's row pitch)
// arrive as one two-dimensional tensor-map box issued by one lane, as in gemv_q4k.cu.
template <int DEPTH, bool TMA>
__global__ void __launch_bounds__(kThreads, 1)
gemv_q6k_m1_kernel(const uint8_t* __restrict__ w, int N, int K, const __nv_bfloat16* __restrict__ x,
                   void* __restrict__ y, int y_dtype, int* __restrict__ counters, float* __restrict__ partials,
                   const PeerPublish pp, int* __restrict__ status, const __grid_constant__ CUtensorMap w_map) {
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_trigger();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int SB = K / 256;                        // superblocks per row (a multiple of 8)
  const int row_bytes = SB * kBlockBytes;        // a multiple of 16
  const int C = SB / kSbPerUnit;                 // chunks per row group
  const int RG = (N + kRowsPerUnit - 1) / kRowsPerUnit;
  const int64_t U = (int64_t)RG * C;
  const int G = gridDim.x, b = blockIdx.x;
  const int64_t u_begin = U * b / G, u_end = U * (b + 1) / G;
  const int n_units = (int)(u_end - u_begin);
  const int rg_begin = (int)(u_begin / C), c_begin = (int)(u_begin - (int64_t)rg_begin * C);

  const int g = lane >> 2, t = lane & 3;
  const int rt = warp >> 3, j = warp & 7;        // row tile (16 rows) and superblock slot of this warp
  // superblock 8c + j starts at byte 1680 c + 210 j of its row: 1680 = 0 (mod 16), so the offset
  // of the block inside its aligned window depends on j only
  const int skew = (kBlockBytes * j) & 15;
  const int win0 = kBlockBytes * j - skew;       // window start within the chunk, 16-byte aligned

  const Smem L(DEPTH);
  const uint32_t my_ring = smem_u32(smem) + warp * (DEPTH * kSlotBytes);
  const uint32_t my_bars = smem_u32(smem) + L.bars(K) + warp * 32;        // DEPTH (<= 4) barriers of 8 bytes
  if (TMA && warp < kWarps) tma_bars_init(my_bars, DEPTH, lane);
  const uint8_t* const w_end = w + (int64_t)N * row_bytes;

  // ---- copy side: 8 instructions per step, each copying the 14 window pieces of two rows ----
  const int hl = lane >> 4, kl = lane & 15;
  const bool copier = kl < kPieces;
  const int32_t src_a = hl * row_bytes + 16 * kl;
  const uint32_t dst_a = hl * kSlotPitch + 16 * kl;
  const uint8_t* src = w;
  int rg_i = rg_begin, c_i = c_begin, issued = 0, slot_i = 0;
  auto seek_row_group = [&]() {
    src = w + (int64_t)(rg_i * kRowsPerUnit + 16 * rt) * row_bytes + (int64_t)c_i * (kSbPerUnit * kBlockBytes) + win0;
  };
  seek_row_group();
  auto issue_next = [&]() {
    if (TMA) {
      if (issued < n_units) {
        // words and rows outside the tensor (the window of a row's last blocks, rows past N) arrive as zeros
        if (lane == 0)
          tma_box_load(my_ring + slot_i * kSlotBytes, &w_map, (c_i * (kSbPerUnit * kBlockBytes) + win0) / 4,
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
      // the window of the tensor's very last block may reach past the end of the tensor
      if (row0 + 16 <= N && src + (int64_t)15 * row_bytes + 16 * kPieces <= w_end) {
        if (copier) {
          const uint8_t* pa = src + src_a;
#pragma unroll
          for (int i = 0; i < 8; i++) cp_async16(dst + dst_a + i * (2 * kSlotPitch), pa + (int64_t)i * (2 * row_bytes));
        }
      } else {
        for (int p = lane; p < 16 * kPieces; p += 32) {
          const int row = p / kPieces, k = p - row * kPieces;
          const uint8_t* s = src + (int64_t)(min(row0 + row, N - 1) - row0) * row_bytes + 16 * k;
          if (s + 16 <= w_end) cp_async16(dst + row * kSlotPitch + 16 * k, s);
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
  int S;  // activations are held as x * 2^S (quarters 0, 1 of a half) / x * 2^(S-4) (quarters 2, 3)
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
    // One pass over x: group sums, largest magnitude, and the scaled pair-permuted copy:
    // word 2i = (x[4i], x[4i+2]), word 2i+1 = (x[4i+1], x[4i+3]).
    auto stage_x = [&](int S_) -> float {
      const float up_lo = __uint_as_float((uint32_t)(127 + S_) << 23);
      const float up_hi = __uint_as_float((uint32_t)(127 + S_ - 4) << 23);
      const float xs_scale = __uint_as_float((uint32_t)(127 + S_ - 133) << 23);
      float amax = 0.f;
      const int n_sub = K / 32;
      const int rot = (int)(((int64_t)b * n_sub) / G) & ~3;      // keeps the quarter index
      // two sub-blocks per thread and round, both loads issued before either is converted
      auto fetch = [&](int sblk, uint4 (&v)[4]) {
#pragma unroll
        for (int q = 0; q < 4; q++)
          v[q] = pp.x_tagged ? peer_load8_tagged(pp.x_tagged, sblk * 4 + q, x_tag, status) : __ldcg(xg + sblk * 4 + q);   // L2-coherent: x may have been stored by peers or by the previous launch while this kernel was already resident
      };
      auto convert = [&](int sblk, const uint4 (&v)[4]) {
        const float up = (sblk & 2) ? up_hi : up_lo;
        float sum[2] = {0.f, 0.f}, asum = 0.f;
#pragma unroll
        for (int q = 0; q < 4; q++) {
          const float e0 = bf16lo(v[q].x), e1 = bf16hi(v[q].x), e2 = bf16lo(v[q].y), e3 = bf16hi(v[q].y);
          const float e4 = bf16lo(v[q].z), e5 = bf16hi(v[q].z), e6 = bf16lo(v[q].w), e7 = bf16hi(v[q].w);
          sum[q >> 1] += (e0 + e1) + (e2 + e3) + ((e4 + e5) + (e6 + e7));
          asum += (fabsf(e0) + fabsf(e1)) + (fabsf(e2) + fabsf(e3)) + ((fabsf(e4) + fabsf(e5)) + (fabsf(e6) + fabsf(e7)));
          __nv_bfloat162 p0 = __floats2bfloat162_rn(e0 * up, e2 * up);
          __nv_bfloat162 p1 = __floats2bfloat162_rn(e1 * up, e3 * up);
          __nv_bfloat162 p2 = __floats2bfloat162_rn(e4 * up, e6 * up);
          __nv_bfloat162 p3 = __floats2bfloat162_rn(e5 * up, e7 * up);
          xv[sblk * 4 + q] = make_uint4(*reinterpret_cast<uint32_t*>(&p0), *reinterpret_cast<uint32_t*>(&p1),
                                        *reinterpret_cast<uint32_t*>(&p2), *reinterpret_cast<uint32_t*>(&p3));
        }
        xs[2 * sblk] = sum[0] * xs_scale;
        xs[2 * sblk + 1] = sum[1] * xs_scale;
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
  // Lane (g, t) feeds column g of B: group g of a half = quarter g >> 1, bytes p with (p >> 4) == (g & 1),
  // which lane groups t with (t >> 1) == (g & 1) hold.
  const bool feeds = (g & 1) == (t >> 1);
  LaneX lx;
#pragma unroll
  for (int c = 0; c < 4; c++) {
    const bool live = feeds && (g >> 1) == c;
    lx.addr[c] = live ? smem_u32(smem + L.x) + 64 * c + 16 * t : smem_u32(smem + L.zero(K));
    lx.stride[c] = live ? 512u : 0u;
  }
  // high-bit plane: field of quarter c sits at bits 2c (value * 4^c); quarters 2, 3 meet activations
  // that carry 2^-4.  The lane reads groups 2t, 2t+1, i.e. quarter t.
  const float f_hi = (t & 1) ? 4.f : 16.f;
  const uint32_t xs_lane_base = smem_u32(xs) + 8 * t;
  float* red = reinterpret_cast<float*>(smem + L.red(K));
  const bool odd = (skew & 2) != 0;

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
      LaneX cur = lx;
#pragma unroll
      for (int q = 0; q < 4; q++) cur.addr[q] += (uint32_t)sbg * lx.stride[q];
      uint32_t xsa = xs_lane_base + (uint32_t)sbg * 64u;
      for (; c < c_stop; ++c) {
        issue_next();
        if (TMA) tma_box_wait(my_bars + 8 * slot, ring_round & 1, status, lane);
        else cp_async_wait<DEPTH - 1>();
        __syncwarp();
        const uint32_t blk = my_ring + slot * kSlotBytes + skew;
        if (odd) compute_tile<2>(blk, g, t, cur, xsa, f_hi, out0, out1);
        else if (skew & 4) compute_tile<4>(blk, g, t, cur, xsa, f_hi, out0, out1);
        else compute_tile<8>(blk, g, t, cur, xsa, f_hi, out0, out1);
        __syncwarp();
        if (++slot == DEPTH) { slot = 0; ++ring_round; }
#pragma unroll
        for (int q = 0; q < 4; q++) cur.addr[q] += kSbPerUnit * lx.stride[q];
        xsa += kSbPerUnit * 64u;
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

}  // namespace q6k

bool gemv_q6k_applicable(int64_t N, int64_t K, int M, const void* w, const void* x) {
  return M == 1 && K % 2048 == 0 && q6k::Smem(2).total((int)K) <= q6k::kSmemLimit && N >= 1 && N <= (1ll << 24) &&
         N * (K / 256 * 210) < (1ll << 40) && (uintptr_t)w % 16 == 0 && (uintptr_t)x % 16 == 0;
}

cudaError_t gemv_q6k(const uint8_t* w, int64_t N, int64_t K, const void* x, void* y, int y_dtype, void* ws,
                     size_t ws_bytes, int sm_count, int* status, cudaStream_t st, const PeerPublish* peers) {
  using namespace q6k;
  PeerPublish pp = {};
  if (peers) pp = *peers;
  if (ws_bytes < gemv_q4k_workspace_bytes(N, sm_count) || !ws || sm_count > kMaxSmCount) return cudaErrorInvalidValue;
  const int64_t RG = (N + kRowsPerUnit - 1) / kRowsPerUnit;
  const int64_t U = RG * (K / 256 / kSbPerUnit);
  const int grid = (int)(U < sm_count ? U : sm_count);
  int depth = 4;
  while (depth > 2 && Smem(depth).total((int)K) > kSmemLimit) depth--;
  const int smem = Smem(depth).total((int)K);
  if (smem > kSmemLimit) return cudaErrorInvalidValue;
  static std::atomic<bool> attr_done[64];   // setting the attribute twice is harmless, so a flag per device suffices
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(gemv_q6k_m1_kernel<4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_q6k_m1_kernel<3, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_q6k_m1_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_q6k_m1_kernel<4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_q6k_m1_kernel<3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_q6k_m1_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e != cudaSuccess) return e;
    attr_done[dev].store(true, std::memory_order_release);
  }
  float* partials = reinterpret_cast<float*>(ws);
  int* counters = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(ws) + kWsCounterOffset);
  const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
  // copy path: tensor-map boxes where the driver offers the encoder (GGQ_Q6K_TMA=0 keeps cp.async, also the fallback)
  alignas(64) CUtensorMap w_map;
  memset(&w_map, 0, sizeof(w_map));
  static const bool want_tma = [] { const char* e = getenv("GGQ_Q6K_TMA"); return !(e && e[0] == '0'); }();
  const bool tma = want_tma && make_weight_map(&w_map, w, N, K / 256 * kBlockBytes, kSlotPitch / 4);
  cudaError_t err;
#define GGQ_Q6K_LAUNCH(D, T) launch_pdl(gemv_q6k_m1_kernel<D, T>, grid, kThreads, smem, st, w, (int)N, (int)K, xb, y, y_dtype, counters, partials, pp, status, w_map)
  if (tma) err = depth == 4 ? GGQ_Q6K_LAUNCH(4, true) : depth == 3 ? GGQ_Q6K_LAUNCH(3, true) : GGQ_Q6K_LAUNCH(2, true);
  else err = depth == 4 ? GGQ_Q6K_LAUNCH(4, false) : depth == 3 ? GGQ_Q6K_LAUNCH(3, false) : GGQ_Q6K_LAUNCH(2, false);
#undef GGQ_Q6K_LAUNCH
  return err != cudaSuccess ? err : cudaPeekAtLastError();
}

}  // namespace ggq
