// Tiled fused decode + multiply for small batches (1 <= M <= 8 per launch) on B200, one kernel template
// for every format of tile_formats.cuh (Q4_K, Q5_K, Q6_K, Q2_K, IQ4_XS, IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS,
// IQ3_S, IQ1_S, IQ1_M).
//
// Work split.  K is cut into chunks of spu * nb superblocks; a unit is one 16-row tile x one chunk and
// takes spu steps of nb superblocks.  All steps of the launch, numbered chunk-major (chunk, row tile,
// position in the chunk), are dealt to the warps of the grid as equal contiguous ranges -- a warp, not
// a CTA, is the unit of scheduling: no warp ever waits for another one.  The warps of a CTA sit in one
// or two adjacent chunks, so the CTA stages only those chunks' activations in shared memory (a few KB
// per batch row instead of all of x): a short prologue however the rows are sharded, and room for
// batch rows.  A warp keeps a unit's 16 x M sums in registers while it walks along K and stores them
// to a scratch slot when the unit (or its range) ends; a range boundary cuts a unit into at most two
// segments, which have a slot each.  A counter per row tile collects the steps done; the warp that
// completes a row tile adds its 2 C slots in a fixed order and stores the outputs.  No float atomics:
// a launch is deterministic.
//
// Data movement.  Sixteen warps per CTA, one persistent CTA per SM.  A warp streams its own steps
// (16 rows x nb superblocks) through a private ring of shared-memory slots with 16-byte cp.async
// copies, one to five steps ahead of the one it is multiplying; consecutive steps of a warp are
// consecutive bytes of the same 16 rows.  There is no block-wide barrier after the prologue.  Blocks
// of most formats are only 2-byte aligned, so a step copies the 16-byte aligned window around its
// bytes; rows must start 16-byte aligned (K / 256 * block bytes a multiple of 16).
//
// Arithmetic.  mma.sync.m16n8k16 with exact integer codes as bf16 operands (tile_formats.cuh).
// The eight B columns are four lane-run channels x two batch rows: column 2t carries batch row
// 2p and column 2t+1 batch row 2p+1 of pass p, and only in the k-slots of lane group t, so lane
// (g, t) collects the sums of its own run of rows g and g+8 for two batch rows per MMA, applies
// its own scales, and further passes reuse the decoded A registers for more batch rows.
// Activations are staged pre-scaled by a power of two (per batch row and chunk) so that products
// of sub-normal bf16 codes land in the normal float32 range; the inverse goes into the row sums.
// mma.sync rather than tcgen05: the operands are produced in registers, lane by lane, from bytes
// that were just decoded; tcgen05 wants both operands in shared memory.
#include "gemv.cuh"
#include "tile_formats.cuh"

#include <algorithm>
#include <cstdio>
#include <cstdlib>

namespace ggq {
namespace tile {

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr int kSmemLimit = 232448;              // 227 KB opt-in limit per CTA
constexpr int kMaxDepth = 6;
constexpr int kMaxBatch = 8;                    // four passes of two batch rows
constexpr int kMaxXBufs = 16;                   // K chunks whose activations a CTA can hold at once

// Launch geometry, computed on the host (plan()) and passed by value.
struct Geo {
  int nb;                // superblocks per step
  int spu;               // steps per unit (a unit = one 16-row tile x one K chunk)
  int chunk_sb;          // superblocks per chunk = spu * nb
  int C, RT;             // chunks per row, 16-row tiles
  int64_t S;             // warp steps in all = C * RT * spu
  int W;                 // warps that take part (each gets a contiguous range of at least one unit)
  int depth, pitch, slot_bytes;
  int xbufs;             // chunk buffers: the most adjacent chunks the warps of one CTA touch
  int x_rows;            // staged batch rows = 2 * passes (rows >= M are zero)
  int x_row_bytes;       // staged bytes per batch row and chunk, padded to 64 (mod 128)
  int xs_row_floats;     // sums per batch row and chunk
  int off_x, off_xs, off_zero, off_tab, off_misc, total;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const uint8_t* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_pending(int n) {
  switch (n) {
    case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
    case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
  }
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float bf16lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16hi(uint32_t u) { return __uint_as_float(u & 0xFFFF0000u); }
__device__ __forceinline__ float pow2f(int e) { return __uint_as_float((uint32_t)(127 + e) << 23); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}
__device__ __forceinline__ float lds_f32(uint32_t a) { float v; asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a)); return v; }

// ---- Q4_K at batch 1 and 2: one B register set serves the low- and the high-nibble MMA of a word.
// Lane g = 2t of a quad's column pair reads the activations of sub-block 2t, lane g = 2t + 1 those of
// sub-block 2t + 1 (staged times 2^-4); column 2t of the low-nibble accumulator and column 2t + 1 of the
// high-nibble accumulator are the two sub-block sums, the other two columns are not used.
// byte `SEL` (0..3) of x as a float, exact: bits 0x4B0000vv are 2^23 + v.
template <int SEL>
__device__ __forceinline__ float byte_to_float(uint32_t x) {
  return __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7440 + SEL)) - 8388608.0f;
}
struct Q4kLane {          // per-lane constants of the 6-bit scale unpack (t < 2: plain fields, else split fields)
  bool low;
  int sh, sh2, shm;
  uint32_t ma, mb;
  __device__ explicit Q4kLane(int t)
      : low(t < 2), sh(16 * (t & 1)), sh2(16 * (t & 1) + 2), shm(16 * (t & 1) + (t < 2 ? 0 : 4)),
        ma(t < 2 ? 0x3F3Fu : 0x0F0Fu), mb(t < 2 ? 0u : 0x3030u) {}
};
__device__ __forceinline__ void q4k_pair_scales(const uint4& h, const Q4kLane& c, float& dl_a, float& ndm_a, float& dl_b,
                                                float& ndm_b) {
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
// One superblock of 16 rows: blk0 / blk1 = shared addresses of the block in rows g / g + 8, xa = this
// lane's 64 bytes of activations (or the zero page, step 0), xsa = the two sub-block sums of x.
__device__ __forceinline__ void q4k_block_m1(uint32_t blk0, uint32_t blk1, int t, const Q4kLane& lc, uint32_t xa, uint32_t x_step,
                                             uint32_t xsa, float& out0, float& out1) {
  const uint4 h0 = tf::lds_v4(blk0), h1 = tf::lds_v4(blk1);
  const uint4 qa0 = tf::lds_v4(blk0 + 16 + 32 * t), qb0 = tf::lds_v4(blk0 + 32 + 32 * t);
  const uint4 qa1 = tf::lds_v4(blk1 + 16 + 32 * t), qb1 = tf::lds_v4(blk1 + 32 + 32 * t);
  const uint4 x0 = tf::lds_v4(xa), x1 = tf::lds_v4(xa + x_step), x2 = tf::lds_v4(xa + 2 * x_step), x3 = tf::lds_v4(xa + 3 * x_step);
  const uint2 sxu = tf::lds_v2(xsa);
  const float sx0 = __uint_as_float(sxu.x), sx1 = __uint_as_float(sxu.y);
  float lo[4] = {0.f, 0.f, 0.f, 0.f}, hi[4] = {0.f, 0.f, 0.f, 0.f};
  const uint32_t w0[8] = {qa0.x, qa0.y, qa0.z, qa0.w, qb0.x, qb0.y, qb0.z, qb0.w};
  const uint32_t w1[8] = {qa1.x, qa1.y, qa1.z, qa1.w, qb1.x, qb1.y, qb1.z, qb1.w};
  const uint32_t xr[16] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w, x2.x, x2.y, x2.z, x2.w, x3.x, x3.y, x3.z, x3.w};
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const uint32_t a = w0[i], b = w1[i];
    const uint32_t as = a >> 8, bs = b >> 8;
    mma16816(lo, a & 0x000F000Fu, b & 0x000F000Fu, as & 0x000F000Fu, bs & 0x000F000Fu, xr[2 * i], xr[2 * i + 1]);
    mma16816(hi, a & 0x00F000F0u, b & 0x00F000F0u, as & 0x00F000F0u, bs & 0x00F000F0u, xr[2 * i], xr[2 * i + 1]);
  }
  float dla, dma, dlb, dmb;
  q4k_pair_scales(h0, lc, dla, dma, dlb, dmb);
  out0 = fmaf(dla, lo[0], out0); out0 = fmaf(dma, sx0, out0);
  out0 = fmaf(dlb, hi[1], out0); out0 = fmaf(dmb, sx1, out0);
  q4k_pair_scales(h1, lc, dla, dma, dlb, dmb);
  out1 = fmaf(dla, lo[2], out1); out1 = fmaf(dma, sx0, out1);
  out1 = fmaf(dlb, hi[3], out1); out1 = fmaf(dmb, sx1, out1);
}

template <class F, int MP>
__global__ void __launch_bounds__(kThreads, 1)
gemv_tile_kernel(const uint8_t* __restrict__ w, int N, int K, const __nv_bfloat16* __restrict__ x, int M,
                 void* __restrict__ y, int y_dtype, int* __restrict__ counters, float* __restrict__ slots,
                 const Geo geo, const PeerPublish pp, int* __restrict__ status, const uint8_t* __restrict__ tab) {
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_trigger();
  const int tid = threadIdx.x, lane = tid & 31;
  // the shuffle tells the compiler that the warp index (and all the step bookkeeping derived from
  // it) is the same in every lane, so branches on it are uniform and the warp provably converged
  const int warp = __shfl_sync(0xFFFFFFFFu, tid >> 5, 0);
  const int g = lane >> 2, t = lane & 3;
  const int SB = K / 256;
  const int64_t row_bytes = (int64_t)SB * F::kTs;
  const int b = blockIdx.x;
  const int nb = geo.nb, spu = geo.spu, depth = geo.depth, pitch = geo.pitch, RT = geo.RT;
  constexpr int XR = 2 * MP;                      // staged batch rows

  // ---- this warp's range of steps and where it starts: step s = (chunk c, row tile rt, position k)
  const int gw = b * kWarps + warp;
  const bool active = gw < geo.W;
  const int64_t s_begin = active ? geo.S * gw / geo.W : 0, s_end = active ? geo.S * (gw + 1) / geo.W : 0;
  const int n_steps = (int)(s_end - s_begin);
  const int unit_steps = RT * spu;                // steps per chunk
  int c0 = (int)(s_begin / unit_steps);
  int rem0 = (int)(s_begin - (int64_t)c0 * unit_steps);
  const int rt0 = rem0 / spu, k0 = rem0 - rt0 * spu;
  // the chunks this CTA's warps touch (at most geo.xbufs, by construction of the plan)
  const int w_lo = b * kWarps, w_hi = min(w_lo + kWarps, geo.W);
  const int c_lo = (int)((geo.S * w_lo / geo.W) / unit_steps);
  const int c_hi = (int)((geo.S * w_hi / geo.W - 1) / unit_steps);

  // ---- copy side
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t my_ring = smem_base + warp * (depth * geo.slot_bytes);
  const int hl = lane >> 4, kl = lane & 15;
  int issued = 0, slot_i = 0;
  int c_i = c0, rt_i = rt0, k_i = k0;
  auto issue_next = [&]() {
    if (issued < n_steps) {
      const int sb0 = c_i * geo.chunk_sb + k_i * nb;
      const int nbh = min(nb, SB - sb0);
      if (nbh > 0) {
        const int boff = sb0 * F::kTs;
        const int pieces = ((boff & 15) + nbh * F::kTs + 15) >> 4;
        const int row0 = rt_i * 16;
        const uint8_t* src0 = w + (boff & ~15) + 16 * kl;
        const uint32_t dst0 = my_ring + slot_i * geo.slot_bytes + hl * pitch + 16 * kl;
        // a half-warp copies one row: lane kl takes pieces kl, kl + 16 (and kl + 32 where a step can be
        // wider than 512 bytes); predicated single instructions, no loops, so the warp stays converged
        const bool q0 = kl < pieces, q1 = kl + 16 < pieces, q2 = kl + 32 < pieces;
        constexpr bool kWide = 14 + 4 * F::kTs + 15 > 512;
        if (row0 + 16 <= N) {
          const uint8_t* src = src0 + (int64_t)(row0 + hl) * row_bytes;
#pragma unroll
          for (int i = 0; i < 8; i++) {
            if (q0) cp_async16(dst0 + i * (2 * pitch), src);
            if (q1) cp_async16(dst0 + i * (2 * pitch) + 256, src + 256);
            if (kWide && q2) cp_async16(dst0 + i * (2 * pitch) + 512, src + 512);
            src += 2 * row_bytes;
          }
        } else {            // last, ragged row tile: rows past the end repeat row N - 1 (multiplied, never stored)
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const uint8_t* src = src0 + (int64_t)min(row0 + 2 * i + hl, N - 1) * row_bytes;
            if (q0) cp_async16(dst0 + i * (2 * pitch), src);
            if (q1) cp_async16(dst0 + i * (2 * pitch) + 256, src + 256);
            if (kWide && q2) cp_async16(dst0 + i * (2 * pitch) + 512, src + 512);
          }
        }
      }
      ++issued;
      if (++slot_i == depth) slot_i = 0;
      if (++k_i == spu) { k_i = 0; if (++rt_i == RT) { rt_i = 0; ++c_i; } }
    }
    cp_async_commit();
  };
  for (int d = 0; d < depth - 1; d++) issue_next();

  // ---- shared-memory tables (immutable inputs: may be read before the previous kernel has finished)
  tf::Tables tb{};
  tb.grid = smem_base + geo.off_tab;
  if constexpr (F::kTableBytes > 0) {
    uint32_t* dst = reinterpret_cast<uint32_t*>(smem + geo.off_tab);
    if constexpr (F::kQt == QT_IQ1_S || F::kQt == QT_IQ1_M) {
      // int8 grid {-1, 0, 1} -> code bytes 8 * grid + 9
      const uint32_t* src = reinterpret_cast<const uint32_t*>(tab + TAB_IQ1);
      for (int i = tid; i < F::kTableBytes / 4; i += kThreads) {
        const uint32_t v = __ldg(src + i);
        const uint32_t neg = (v >> 7) & 0x01010101u, pos = v & ~(v >> 7) & 0x01010101u;    // per byte: 0xFF / 0x01
        dst[i] = 0x09090909u - 8u * neg + 8u * pos;
      }
    } else {
      constexpr int kOff = F::kQt == QT_IQ2_XXS ? TAB_IQ2_XXS : F::kQt == QT_IQ2_XS ? TAB_IQ2_XS :
                           F::kQt == QT_IQ2_S ? TAB_IQ2_S : F::kQt == QT_IQ3_XXS ? TAB_IQ3_XXS : TAB_IQ3_S;
      const uint32_t* src = reinterpret_cast<const uint32_t*>(tab + kOff);
      for (int i = tid; i < F::kTableBytes / 4; i += kThreads) dst[i] = __ldg(src + i);
    }
  }
  if constexpr (F::kQt == QT_IQ4_XS) {
    const uint32_t* src = reinterpret_cast<const uint32_t*>(tab + TAB_KV_IQ4);
#pragma unroll
    for (int i = 0; i < 4; i++) tb.kv[i] = __ldg(src + i) ^ 0x80808080u;     // int8 + 128, per byte
  }
  if (tid < 16) reinterpret_cast<uint32_t*>(smem + geo.off_zero)[tid] = 0;
  int* misc = reinterpret_cast<int*>(smem + geo.off_misc);     // [buf][0..7] S per batch row, [buf][8..15] largest octet sum of |x|
  if (tid < 16 * geo.xbufs) misc[tid] = (tid & 15) < 8 ? 96 : 0;

  // ---- everything below reads or writes memory the previous kernel may still be using
  pdl_wait();
  uint32_t out_tag = 0, x_tag = 0;
  peer_wait_previous(pp, tid, status);
  if (pp.world > 0 && pp.tagged) {
    const uint32_t e = pp.flags[pp.rank][pp.world];
    out_tag = peer_tag_of(e + 1) << 16;
    x_tag = peer_tag_of(e + 1 - (uint32_t)pp.x_back) << 16;
    // every thread polls its own few words: the wait is a chain of L2 round trips, so it is the number of
    // words per thread, not the number of threads, that costs time
    if (pp.after_tagged)
      peer_wait_tagged(pp.after_tagged, pp.after_words, peer_tag_of(e + 1 - (uint32_t)pp.after_back) << 16, tid, kThreads, status);
  }
  __syncthreads();

  // Stage the activations of chunk c into buffer cb: destination order [block][run t][octet][8 values],
  // 16 bytes per octet, so a lane's run of a block is 128 contiguous bytes.
  constexpr uint32_t kRunBytes = F::kOct * 16;          // staged activations of one lane run
  constexpr uint32_t kRunStride = kRunBytes + 16;
  auto stage_pass = [&](int cb, int c, int m, int S) -> float {
    const int n_oct = geo.chunk_sb * (4 * F::kOct);
    uint4* xv = reinterpret_cast<uint4*>(smem + geo.off_x + (cb * XR + m) * geo.x_row_bytes);
    float* xs = reinterpret_cast<float*>(smem + geo.off_xs) + (cb * XR + m) * geo.xs_row_floats;
    const float sum_scale = pow2f(S - 133);
    float amax = 0.f;
    for (int o = tid; o < n_oct; o += kThreads) {
      const int blk = o / (4 * F::kOct), tt = (o / F::kOct) & 3, oo = o % F::kOct;
      int qa, qb;
      F::src_quads(tt, oo, qa, qb);
      const int64_t kk = ((int64_t)c * geo.chunk_sb + blk) * 256;
      uint2 va = make_uint2(0, 0), vb = make_uint2(0, 0);
      if (m < M && kk < K) {
        if (F::kPairOrder == 0 && pp.x_tagged) {
          const uint4 v = peer_load8_tagged(pp.x_tagged, (int)((kk + qa) >> 3), x_tag, status);
          va = make_uint2(v.x, v.y); vb = make_uint2(v.z, v.w);
        } else {
          const __nv_bfloat16* xr = x + (int64_t)m * K + kk;
          va = __ldcg(reinterpret_cast<const uint2*>(xr + qa));
          vb = __ldcg(reinterpret_cast<const uint2*>(xr + qb));
        }
      }
      const float a0 = bf16lo(va.x), a1 = bf16hi(va.x), a2 = bf16lo(va.y), a3 = bf16hi(va.y);
      const float b0 = bf16lo(vb.x), b1 = bf16hi(vb.x), b2 = bf16lo(vb.y), b3 = bf16hi(vb.y);
      const float up = pow2f(S + F::x_exp(tt, oo));
      uint4 o4;
      if (F::kPairOrder == 0) o4 = make_uint4(pack_bf16(a0 * up, a2 * up), pack_bf16(a1 * up, a3 * up),
                                               pack_bf16(b0 * up, b2 * up), pack_bf16(b1 * up, b3 * up));
      else o4 = make_uint4(pack_bf16(a0 * up, a1 * up), pack_bf16(b0 * up, b1 * up),
                           pack_bf16(a2 * up, a3 * up), pack_bf16(b2 * up, b3 * up));
      // a run takes kRunBytes + 16 bytes and a batch row 64 (mod 128) bytes, so that the eight lanes that
      // read activations at once (four runs x two batch rows) hit eight different 16-byte bank groups
      *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(xv) + (blk * 4 + tt) * kRunStride + oo * 16) = o4;
      float sum = ((a0 + a1) + (a2 + a3)) + ((b0 + b1) + (b2 + b3));
      const float asum = ((fabsf(a0) + fabsf(a1)) + (fabsf(a2) + fabsf(a3))) + ((fabsf(b0) + fabsf(b1)) + (fabsf(b2) + fabsf(b3)));
      amax = fmaxf(amax, asum);
      if constexpr (F::kSums) {
        if ((oo & (F::kGroupOct - 1)) >= F::kSumOct) sum = 0.f;      // second plane of a two-plane format: same weights again
        if (F::kGroupOct >= 2) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
        if (F::kGroupOct >= 4) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
        if (F::kGroupOct >= 8) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 4);
        if ((oo & (F::kGroupOct - 1)) == 0) xs[o / F::kGroupOct] = sum * sum_scale;
      }
    }
    return amax;
  };
  // Optimistic scale 2^96: right whenever the largest |x| of a chunk lies in about [2^-30, 2^24); a row
  // outside that range is staged a second time with a scale that puts its largest magnitude near 2^120.
  for (int c = c_lo; c <= c_hi; c++)
    for (int m = 0; m < XR; m++) {
      const float amax = stage_pass(c - c_lo, c, m, 96);
      if (m < M) atomicMax(&misc[(c - c_lo) * 16 + 8 + m], (int)__float_as_uint(amax));   // non-negative floats order like integers
    }
  __syncthreads();
  for (int c = c_lo; c <= c_hi; c++)
    for (int m = 0; m < M; m++) {
      const int emax = min((misc[(c - c_lo) * 16 + 8 + m] >> 23) & 0xFF, 254);   // biased exponent of the largest octet sum of |x|
      if (emax > 156 || (emax < 97 && emax > 0)) {
        const int S = max(8, min(120, 247 - emax));
        stage_pass(c - c_lo, c, m, S);
        if (tid == 0) misc[(c - c_lo) * 16 + m] = S;
      }
    }
  __syncthreads();

  const bool live = (g >> 1) == t;
  const uint32_t zero_addr = smem_base + geo.off_zero;
  const uint32_t x_lane = live ? smem_base + geo.off_x + (g & 1) * geo.x_row_bytes + t * kRunStride : zero_addr;
  const uint32_t x_pass = live ? 2u * geo.x_row_bytes : 0u, x_oct = live ? 16u : 0u, x_blk = live ? 4u * kRunStride : 0u;
  const uint32_t x_buf = live ? (uint32_t)(XR * geo.x_row_bytes) : 0u;
  const uint32_t xs_base = smem_base + geo.off_xs;
  constexpr int kGroups = F::kOct / F::kGroupOct;
  const int total_steps = geo.C * spu;            // arrivals that complete a row tile

  auto emit = [&](int row, int m, float val) {
    if (pp.world == 0) store_out(y, y_dtype, (int64_t)m * N + row, val);
    else peer_emit(pp, y, y_dtype, row, val, out_tag);
  };
  // Completion of a row tile: whoever brings its step count to C * spu adds the 2 C slots in order.
  int pend_rt = -1, pend_steps = 0, pend_old = 0;
  auto settle = [&]() {
    const int old = __shfl_sync(0xFFFFFFFFu, pend_old, 0);
    if (old + pend_steps == total_steps) {
      constexpr int kPer = XR / 2;                 // floats per lane: 16 rows x XR values over 32 lanes
      float sum[kPer];
#pragma unroll
      for (int i = 0; i < kPer; i++) sum[i] = 0.f;
      for (int cc = 0; cc < geo.C; cc++) {
#pragma unroll
        for (int part = 0; part < 2; part++) {
          const float* sl = slots + ((((int64_t)cc * RT + pend_rt) * 2 + part) * 16 * XR) + lane * kPer;
#pragma unroll
          for (int i = 0; i < kPer; i++) sum[i] += __ldcg(sl + i);
        }
      }
      const int idx0 = lane * kPer;
#pragma unroll
      for (int i = 0; i < kPer; i++) {
        const int row = pend_rt * 16 + (idx0 + i) / XR, m = (idx0 + i) % XR;
        if (row < N && m < M) emit(row, m, sum[i]);
      }
      if (lane == 0) counters[pend_rt] = 0;
    }
    pend_rt = -1;
  };

  // Q4_K at batch 1: the dedicated inner loop (see q4k_block_m1); everything else takes the generic one
  constexpr bool kQ4kM1 = F::kQt == QT_Q4_K && MP == 1;
  const bool q4k_fast = kQ4kM1 && M == 1;
  const Q4kLane q4k_lane(t);
  const uint32_t q4k_x_lane = live ? smem_base + geo.off_x + t * kRunStride + (g & 1) * 64 : zero_addr;

  if (active) {
    int c = c0, rt = rt0, k = k0, slot = 0, seg_k = k0;
    float out[MP][4];
#pragma unroll
    for (int p = 0; p < MP; p++) out[p][0] = out[p][1] = out[p][2] = out[p][3] = 0.f;
    for (int i = 0; i < n_steps; i++) {
      issue_next();
      cp_async_wait_pending(depth - 1);
      __syncwarp();
      const int sb0 = c * geo.chunk_sb + k * nb;
      const int nbh = min(nb, SB - sb0);
      const int cb = c - c_lo;
      const uint32_t tile = my_ring + slot * geo.slot_bytes + g * pitch + ((sb0 * F::kTs) & 15);
      const uint32_t xr0 = x_lane + cb * x_buf + (k * nb) * x_blk;
      const uint32_t xs0 = xs_base + (uint32_t)(((cb * XR) * geo.xs_row_floats + (k * nb * 4 + t) * kGroups) * 4);
      if constexpr (kQ4kM1) {
        if (q4k_fast) {
          const uint32_t xa0 = q4k_x_lane + cb * x_buf + (k * nb) * x_blk;
          const uint32_t xsa0 = xs0;           // the run's two sub-block sums: xs[(blk * 4 + t) * 2 + {0, 1}]
          for (int blk = 0; blk < nbh; blk++)
            q4k_block_m1(tile + blk * F::kTs, tile + blk * F::kTs + 8 * pitch, t, q4k_lane, xa0 + blk * x_blk, x_oct,
                         xsa0 + blk * (4 * kGroups * 4), out[0][0], out[0][2]);
        }
      }
      for (int blk = 0; blk < (q4k_fast ? 0 : nbh); blk++) {
        const tf::BlockLd ld0{tile + blk * F::kTs}, ld1{tile + blk * F::kTs + 8 * pitch};
        const typename F::Run run0 = F::load_run(ld0, t), run1 = F::load_run(ld1, t);
        const uint32_t xr = xr0 + blk * x_blk;
        const uint32_t xsb = xs0 + blk * (4 * kGroups * 4);
        auto do_group = [&](int grp) {
          const typename F::Group g0 = F::load_group(ld0, run0, t, grp), g1 = F::load_group(ld1, run1, t, grp);
          const uint32_t xg = xr + grp * (F::kGroupOct * x_oct);
          float acc[MP][4], acc2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int p = 0; p < MP; p++) acc[p][0] = acc[p][1] = acc[p][2] = acc[p][3] = 0.f;
#pragma unroll
          for (int q = 0; q < F::kGroupOct; q++) {
            uint32_t p0[4], p1[4];
            F::octet(g0, q, tb, p0);
            F::octet(g1, q, tb, p1);
#pragma unroll
            for (int p = 0; p < MP; p++) {
              const uint4 xv = tf::lds_v4(xg + q * x_oct + p * x_pass);
              if (MP == 1 && (q & 1)) {      // a second accumulation chain when there is only one pass
                mma16816(acc2, p0[0], p1[0], p0[1], p1[1], xv.x, xv.y);
                mma16816(acc2, p0[2], p1[2], p0[3], p1[3], xv.z, xv.w);
              } else {
                mma16816(acc[p], p0[0], p1[0], p0[1], p1[1], xv.x, xv.y);
                mma16816(acc[p], p0[2], p1[2], p0[3], p1[3], xv.z, xv.w);
              }
            }
          }
#pragma unroll
          for (int p = 0; p < MP; p++) {
            float s0 = 0.f, s1 = 0.f;
            if constexpr (F::kSums) {
              s0 = lds_f32(xsb + ((2 * p) * geo.xs_row_floats + grp) * 4);
              s1 = lds_f32(xsb + ((2 * p + 1) * geo.xs_row_floats + grp) * 4);
            }
            if (MP == 1) { acc[0][0] += acc2[0]; acc[0][1] += acc2[1]; acc[0][2] += acc2[2]; acc[0][3] += acc2[3]; }
            out[p][0] = F::fold(g0, acc[p][0], s0, out[p][0]);
            out[p][1] = F::fold(g0, acc[p][1], s1, out[p][1]);
            out[p][2] = F::fold(g1, acc[p][2], s0, out[p][2]);
            out[p][3] = F::fold(g1, acc[p][3], s1, out[p][3]);
          }
        };
        if constexpr (F::kUnrollGroups) {
#pragma unroll
          for (int grp = 0; grp < kGroups; grp++) do_group(grp);
        } else {
#pragma unroll 1
          for (int grp = 0; grp < kGroups; grp++) do_group(grp);
        }
      }
      __syncwarp();          // every lane is done with the slot before a later copy overwrites it
      if (++slot == depth) slot = 0;

      // ---- end of a unit, or of this warp's range: the segment's 16 x XR sums go to scratch
      if (k == spu - 1 || i == n_steps - 1) {
        const bool whole = seg_k == 0 && k == spu - 1;
        const int part = seg_k == 0 ? 0 : 1;
        if (pend_rt >= 0) settle();
        float v[MP][4];
#pragma unroll
        for (int p = 0; p < MP; p++) {
#pragma unroll
          for (int q = 0; q < 4; q++) {
            float s = out[p][q];
            s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);
            s += __shfl_xor_sync(0xFFFFFFFFu, s, 2);
            v[p][q] = s * pow2f(133 - misc[cb * 16 + 2 * p + (q & 1)]);     // undo the activations' power-of-two scale
            out[p][q] = 0.f;
          }
        }
        if (geo.C == 1 && whole) {
          if (t == 0) {
#pragma unroll
            for (int p = 0; p < MP; p++) {
#pragma unroll
              for (int q = 0; q < 4; q++) {
                const int row = rt * 16 + g + 8 * (q >> 1), m = 2 * p + (q & 1);
                if (row < N && m < M) emit(row, m, v[p][q]);
              }
            }
          }
        } else {
          float* sl = slots + (((int64_t)c * RT + rt) * 2) * 16 * XR;
          if (t == 0) {
#pragma unroll
            for (int p = 0; p < MP; p++) {
              __stcg(reinterpret_cast<float2*>(sl + (part * 16 + g) * XR + 2 * p), make_float2(v[p][0], v[p][1]));
              __stcg(reinterpret_cast<float2*>(sl + (part * 16 + g + 8) * XR + 2 * p), make_float2(v[p][2], v[p][3]));
              if (whole) {
                __stcg(reinterpret_cast<float2*>(sl + (16 + g) * XR + 2 * p), make_float2(0.f, 0.f));
                __stcg(reinterpret_cast<float2*>(sl + (16 + g + 8) * XR + 2 * p), make_float2(0.f, 0.f));
              }
            }
          }
          __syncwarp();
          // release: this warp's slot stores are visible to whoever sees the increment; acquire: if this is
          // the last arrival, every other segment's slot is visible to this warp.  The old value is first
          // looked at when the next segment is flushed, so the round trip never holds the warp up.
          pend_steps = k - seg_k + 1;
          if (lane == 0)
            asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(pend_old) : "l"(counters + rt), "r"(pend_steps) : "memory");
          pend_rt = rt;
        }
        seg_k = 0;
      }
      if (++k == spu) { k = 0; if (++rt == RT) { rt = 0; ++c; } }
    }
    if (pend_rt >= 0) settle();
  }
  cp_async_wait_pending(0);
  peer_publish(pp, tid, gridDim.x);
}

// ---------------------------------------------------------------------------------------------
// host side

struct FormatInfo { int qt, ts, table_bytes, sum_groups, oct; bool sums; };

template <class F>
constexpr FormatInfo info_of() { return {F::kQt, F::kTs, F::kTableBytes, F::kOct / F::kGroupOct, F::kOct, F::kSums}; }

static bool format_of(int qtype, FormatInfo* fi) {
  switch (qtype) {
    case QT_Q4_K: *fi = info_of<tf::Q4K>(); return true;
    case QT_Q5_K: *fi = info_of<tf::Q5K>(); return true;
    case QT_Q6_K: *fi = info_of<tf::Q6K>(); return true;
    case QT_Q2_K: *fi = info_of<tf::Q2K>(); return true;
    case QT_IQ4_XS: *fi = info_of<tf::IQ4XS>(); return true;
    case QT_IQ2_XXS: *fi = info_of<tf::IQ2XXS>(); return true;
    case QT_IQ2_XS: *fi = info_of<tf::IQ2XS>(); return true;
    case QT_IQ2_S: *fi = info_of<tf::IQ2S>(); return true;
    case QT_IQ3_XXS: *fi = info_of<tf::IQ3XXS>(); return true;
    case QT_IQ3_S: *fi = info_of<tf::IQ3S>(); return true;
    case QT_IQ1_S: *fi = info_of<tf::IQ1S>(); return true;
    case QT_IQ1_M: *fi = info_of<tf::IQ1M>(); return true;
    default: return false;
  }
}

static int passes_of(int M) { return M <= 2 ? 1 : M <= 4 ? 2 : 4; }

// Smallest K chunk (in superblocks) the plan may use.  Eight for weights with enough (chunk, row tile)
// units to give every warp of the device at least one; smaller for small weights, so that they still
// spread over the whole device.  The scratch is sized by the same rule.
static int min_chunk_sb(int64_t N, int64_t K) {
  const int64_t RT = (N + 15) / 16, SB = K / 256;
  int chunk = 8;
  while (chunk > 1 && RT * ((SB + chunk - 1) / chunk) < 148 * kWarps) chunk /= 2;
  return chunk;
}

// Shared-memory layout and work split for one launch; false if nothing fits.
static bool plan(const FormatInfo& fi, int64_t N, int64_t K, int M, int sm_count, int nb_forced, int chunk_forced, Geo* out) {
  const int SB = (int)(K / 256);
  const int x_rows = 2 * passes_of(M);
  Geo best{};
  double best_cost = 1e30;
  for (int nb = 1; nb <= 4; nb *= 2) {
    if (nb_forced > 0 && nb != nb_forced) continue;
    for (int chunk = min_chunk_sb(N, K); ; chunk *= 2) {
      const bool whole_k = chunk >= SB;
      if (chunk % nb == 0 && (chunk_forced <= 0 || chunk == chunk_forced || whole_k)) {
        Geo g{};
        g.nb = nb;
        g.chunk_sb = whole_k ? (SB + nb - 1) / nb * nb : chunk;
        g.spu = g.chunk_sb / nb;
        g.C = (SB + g.chunk_sb - 1) / g.chunk_sb;
        g.RT = (int)((N + 15) / 16);
        g.S = (int64_t)g.C * g.RT * g.spu;
        const int64_t units = (int64_t)g.C * g.RT;
        g.W = (int)std::min<int64_t>((int64_t)sm_count * kWarps, units);
        g.x_rows = x_rows;
        g.x_row_bytes = g.chunk_sb * 4 * (16 * fi.oct + 16);
        g.x_row_bytes += (64 - g.x_row_bytes % 128 + 128) % 128;      // 64 (mod 128): see the staging
        g.xs_row_floats = fi.sums ? g.chunk_sb * 4 * fi.sum_groups : 0;
        const int pieces = (14 + nb * fi.ts + 15) / 16;
        g.pitch = 16 * pieces;
        if (g.pitch % 32 == 0) g.pitch += 16;          // odd multiple of 16: rows fall into different bank groups
        g.slot_bytes = 16 * g.pitch;
        // chunks a CTA's sixteen warps can touch: their steps span at most this many chunks
        const int64_t cta_steps = (g.S * kWarps + g.W - 1) / g.W + 1;
        const int64_t span = (cta_steps + (int64_t)g.RT * g.spu - 2) / ((int64_t)g.RT * g.spu) + 1;
        const int bufs = (int)std::min<int64_t>(span, g.C);
        const bool span_ok = bufs <= kMaxXBufs;
        g.xbufs = bufs;
        const int fixed = bufs * x_rows * (g.x_row_bytes + g.xs_row_floats * 4) + 64 + (fi.table_bytes + 15) / 16 * 16 + 64 * kMaxXBufs;
        const int room = kSmemLimit - fixed;
        if (span_ok && room >= 2 * kWarps * g.slot_bytes) {
          g.depth = std::min(kMaxDepth, room / (kWarps * g.slot_bytes));
          g.off_x = kWarps * g.depth * g.slot_bytes;
          g.off_xs = g.off_x + bufs * x_rows * g.x_row_bytes;
          g.off_zero = g.off_xs + bufs * x_rows * g.xs_row_floats * 4;
          g.off_tab = g.off_zero + 64;
          g.off_misc = g.off_tab + (fi.table_bytes + 15) / 16 * 16;
          g.total = g.off_misc + 64 * kMaxXBufs;
          // time ~ steps of the busiest warp x (blocks per step + a fixed cost per step) + staging + a flush per
          // unit, in units of one block's multiply; the constants are fitted to B200 timings (8192 x 28672:
          // nb = 2 with chunks of 16 superblocks is the fastest split for every format)
          const double steps = (double)((g.S + g.W - 1) / g.W);
          const double cost = steps * (nb + 0.6) * (g.depth >= 3 ? 1.0 : 1.03) + bufs * g.chunk_sb * x_rows * 0.02 + steps / g.spu * 0.6;
          if (cost < best_cost) { best_cost = cost; best = g; }
        }
      }
      if (whole_k) break;
    }
  }
  if (best_cost >= 1e30) return false;
  *out = best;
  return true;
}

static int env_int(const char* name) {
  const char* s = getenv(name);
  return s ? atoi(s) : 0;
}
static int forced_nb() { static const int v = env_int("GGQ_TILE_NB"); return v; }
static int forced_chunk() { static const int v = env_int("GGQ_TILE_CHUNK"); return v; }

template <class F, int MP>
static cudaError_t launch(const Geo& geo, int grid, cudaStream_t st, const uint8_t* w, int N, int K, const void* x, int M,
                          void* y, int y_dtype, int* counters, float* slots, const PeerPublish& pp, int* status,
                          const uint8_t* tab) {
  static std::atomic<bool> attr_done[64];   // setting the attribute twice is harmless, so a flag per device suffices
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(gemv_tile_kernel<F, MP>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e != cudaSuccess) return e;
    attr_done[dev].store(true, std::memory_order_release);
  }
  cudaError_t err = launch_pdl(gemv_tile_kernel<F, MP>, grid, kThreads, (size_t)geo.total, st, w, N, K,
                               (const __nv_bfloat16*)x, M, y, y_dtype, counters, slots, geo, pp, status, tab);
  return err != cudaSuccess ? err : cudaPeekAtLastError();
}

template <class F>
static cudaError_t launch_passes(int MP, const Geo& geo, int grid, cudaStream_t st, const uint8_t* w, int N, int K,
                                 const void* x, int M, void* y, int y_dtype, int* counters, float* slots,
                                 const PeerPublish& pp, int* status, const uint8_t* tab) {
  switch (MP) {
    case 1: return launch<F, 1>(geo, grid, st, w, N, K, x, M, y, y_dtype, counters, slots, pp, status, tab);
    case 2: return launch<F, 2>(geo, grid, st, w, N, K, x, M, y, y_dtype, counters, slots, pp, status, tab);
    default: return launch<F, 4>(geo, grid, st, w, N, K, x, M, y, y_dtype, counters, slots, pp, status, tab);
  }
}

}  // namespace tile

// Most batch rows one launch takes for qtype (0: not a tile format).  Four passes only pay where decoding
// dominates; Q6_K, with two planes and 32 MMAs per block and pass, is faster as two launches of two passes.
int gemv_tile_max_batch(int qtype) {
  tile::FormatInfo fi;
  if (!tile::format_of(qtype, &fi)) return 0;
  return qtype == QT_Q6_K ? 4 : tile::kMaxBatch;
}

bool gemv_tile_applicable(int qtype, int64_t N, int64_t K, int M, const void* w, const void* x) {
  tile::FormatInfo fi;
  if (!tile::format_of(qtype, &fi)) return false;
  if (M < 1 || M > gemv_tile_max_batch(qtype) || K <= 0 || K % 256 || N < 1 || N > (1ll << 24)) return false;
  if ((K / 256 * fi.ts) % 16 || (uintptr_t)w % 16 || (uintptr_t)x % 16 || (K * 2) % 16) return false;
  if (N * (K / 256 * fi.ts) >= (1ll << 31)) return false;      // block offsets are 32-bit inside a row; rows are 64-bit
  tile::Geo geo;
  return tile::plan(fi, N, K, M, 148, 0, 0, &geo);
}

// Scratch: one arrival counter per 16-row tile in the counter area every kernel shares, and two
// 16 x batch-row float slots per (chunk, row tile) in the float area; sized for the smallest chunk
// the plan may pick.
size_t gemv_tile_workspace_bytes(int qtype, int64_t N, int64_t K, int M) {
  tile::FormatInfo fi;
  if (!tile::format_of(qtype, &fi) || M < 1 || M > tile::kMaxBatch) return 0;
  const int64_t RT = (N + 15) / 16;
  const int chunk = tile::min_chunk_sb(N, K);
  const int64_t C = (K / 256 + chunk - 1) / chunk;
  const size_t slots = (size_t)(RT * C) * 2 * 16 * 2 * tile::passes_of(M) * sizeof(float);
  return kWsGemmPartialOffset + (slots + 255) / 256 * 256;
}

cudaError_t gemv_tile(int qtype, const uint8_t* w, int64_t N, int64_t K, const void* x, int M, void* y, int y_dtype,
                      void* ws, size_t ws_bytes, int sm_count, int* status, const uint8_t* tab, cudaStream_t st,
                      const PeerPublish* peers) {
  using namespace tile;
  FormatInfo fi;
  if (!format_of(qtype, &fi)) return cudaErrorInvalidValue;
  Geo geo;
  if (!plan(fi, N, K, M, sm_count, forced_nb(), forced_chunk(), &geo) && !plan(fi, N, K, M, sm_count, 0, 0, &geo))
    return cudaErrorInvalidValue;
  if (!ws || ws_bytes < gemv_tile_workspace_bytes(qtype, N, K, M) || (uintptr_t)ws % 256) return cudaErrorInvalidValue;
  if (kWsCounterOffset + (size_t)geo.RT * sizeof(int) > kWsGemmPartialOffset) return cudaErrorInvalidValue;
  static const bool debug = env_int("GGQ_TILE_DEBUG") != 0;     // prints the plan of every launch (a tuning aid)
  if (debug)
    fprintf(stderr, "gemv_tile qtype %d N=%lld K=%lld M=%d: nb=%d chunk=%d spu=%d C=%d RT=%d S=%lld W=%d depth=%d pitch=%d xbufs=%d smem=%d\n",
            qtype, (long long)N, (long long)K, M, geo.nb, geo.chunk_sb, geo.spu, geo.C, geo.RT, (long long)geo.S, geo.W, geo.depth,
            geo.pitch, geo.xbufs, geo.total);
  PeerPublish pp = {};
  if (peers) pp = *peers;
  int* counters = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(ws) + kWsCounterOffset);
  float* slots = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ws) + kWsGemmPartialOffset);
  const int grid = (geo.W + kWarps - 1) / kWarps;
  const int MP = passes_of(M);
#define GGQ_TILE_CASE(QT, F) \
  case QT: return launch_passes<tf::F>(MP, geo, grid, st, w, (int)N, (int)K, x, M, y, y_dtype, counters, slots, pp, status, tab);
  switch (qtype) {
    GGQ_TILE_CASE(QT_Q4_K, Q4K)
    GGQ_TILE_CASE(QT_Q5_K, Q5K)
    GGQ_TILE_CASE(QT_Q6_K, Q6K)
    GGQ_TILE_CASE(QT_Q2_K, Q2K)
    GGQ_TILE_CASE(QT_IQ4_XS, IQ4XS)
    GGQ_TILE_CASE(QT_IQ2_XS, IQ2XS)
    GGQ_TILE_CASE(QT_IQ2_S, IQ2S)
    GGQ_TILE_CASE(QT_IQ3_XXS, IQ3XXS)
    GGQ_TILE_CASE(QT_IQ3_S, IQ3S)
    GGQ_TILE_CASE(QT_IQ1_S, IQ1S)
    GGQ_TILE_CASE(QT_IQ1_M, IQ1M)
    GGQ_TILE_CASE(QT_IQ2_XXS, IQ2XXS)
    default: return cudaErrorInvalidValue;
  }
#undef GGQ_TILE_CASE
}

}  // namespace ggq
