// Tiled fused decode + multiply for small batches (1 <= M <= 16) on B200, one kernel template for
// every format of tile_formats.cuh (Q4_K, Q2_K, IQ4_XS, IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS, IQ3_S,
// IQ1_S, IQ1_M).
//
// Work split.  A unit is 32 output rows x one K chunk of 8 * nb superblocks (nb = 1, 2 or 4, picked
// per launch).  Units are numbered chunk-major (all row groups of chunk 0, then chunk 1, ...) and
// dealt to the persistent CTAs (one per SM) as equal contiguous ranges, so a CTA works inside one
// chunk, sometimes two: it stages only that chunk's activations in shared memory (a few KB per
// batch row instead of all of x), which keeps the prologue short however the rows are sharded and
// leaves room for batch rows.  Every unit leaves its 32 x M partial sums in scratch; the CTA that
// completes a row group (a counter per row group tells which one) adds the chunks' partials in
// chunk order and stores the outputs.  The order of every float32 addition therefore depends on K
// and nb only -- not on the grid or on how many rows a launch has.
//
// Data movement.  Sixteen tile warps (2 row tiles x 8 K positions) and one reducer warp per CTA.
// A tile warp streams its own steps (16 rows x nb superblocks) through a private ring of
// shared-memory slots with 16-byte cp.async copies, one to five steps ahead of the one it is
// multiplying; no block-wide barrier sits in the main loop.  Blocks of most formats are only
// 2-byte aligned, so a step copies the 16-byte aligned window around its bytes; rows must start
// 16-byte aligned (K / 256 * block bytes a multiple of 16).
//
// Arithmetic.  mma.sync.m16n8k16 with exact integer codes as bf16 operands (tile_formats.cuh).
// The eight B columns are four lane-run channels x two batch rows: column 2t carries batch row
// 2p and column 2t+1 batch row 2p+1 of pass p, and only in the k-slots of lane group t, so lane
// (g, t) collects the sums of its own run of rows g and g+8 for two batch rows per MMA, applies
// its own scales, and further passes reuse the decoded A registers for more batch rows.
// Activations are staged pre-scaled by a power of two (per batch row and chunk) so that products
// of sub-normal bf16 codes land in the normal float32 range; the inverse goes into the row sums.
#include "gemv.cuh"
#include "tile_formats.cuh"

#include <algorithm>
#include <cstdlib>

namespace ggq {
namespace tile {

constexpr int kWarps = 16;                      // tile warps: (row tile rt = warp >> 3, K position j = warp & 7)
constexpr int kThreads = (kWarps + 1) * 32;     // plus the reducer warp
constexpr int kRowsPerUnit = 32;
constexpr int kBarFull = 1, kBarFree = 3, kBarStage = 5;
constexpr int kSmemLimit = 232448;              // 227 KB opt-in limit per CTA
constexpr int kMaxDepth = 6;
constexpr int kMaxBatch = 8;                    // four passes of two batch rows

// Launch geometry, computed on the host (plan()) and passed by value.
struct Geo {
  int nb, depth, pitch, slot_bytes;
  int chunk_sb;          // superblocks per chunk = 8 * nb
  int C, RG;             // chunks per row, row groups
  int64_t U;             // units = C * RG
  int x_rows;            // staged batch rows = 2 * passes (rows >= M are zero)
  int x_row_bytes;       // chunk_sb * 512
  int xs_row_floats;     // sums per batch row and chunk
  int off_x, off_xs, off_zero, off_red, off_tab, off_misc, total;
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
__device__ __forceinline__ void bar_sync(int id, int count) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory"); }
__device__ __forceinline__ void bar_arrive(int id, int count) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory"); }
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

// 17 warps put five on one of the four sub-cores (16384 registers each): 96 registers per thread.
template <class F, int MP>
__global__ void __launch_bounds__(kThreads, 1)
gemv_tile_kernel(const uint8_t* __restrict__ w, int N, int K, const __nv_bfloat16* __restrict__ x, int M,
                 void* __restrict__ y, int y_dtype, int* __restrict__ counters, float* __restrict__ partials,
                 const Geo geo, const PeerPublish pp, int* __restrict__ status, const uint8_t* __restrict__ tab) {
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_trigger();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int rt = warp >> 3, j = warp & 7;
  const bool tile_warp = warp < kWarps;
  const int SB = K / 256;
  const int64_t row_bytes = (int64_t)SB * F::kTs;
  const int G = gridDim.x, b = blockIdx.x;
  const int64_t u_begin = geo.U * b / G, u_end = geo.U * (b + 1) / G;
  const int n_units = (int)(u_end - u_begin);
  const int nb = geo.nb, depth = geo.depth, pitch = geo.pitch, RG = geo.RG;

  // ---- copy side: step i of this warp covers unit u_begin + i
  const uint32_t my_ring = smem_u32(smem) + warp * (depth * geo.slot_bytes);
  const int a_off = (j * nb * F::kTs) & 15;           // where the warp's first block sits in its 16-byte window
  const int hl = lane >> 4, kl = lane & 15;
  int issued = 0, slot_i = 0;
  int c_i = (int)(u_begin / RG), rg_i = (int)(u_begin - (int64_t)c_i * RG);
  auto issue_next = [&]() {
    if (issued < n_units) {
      const int sb0 = c_i * geo.chunk_sb + j * nb;
      const int nbh = min(nb, SB - sb0);
      if (nbh > 0) {
        const int pieces = (a_off + nbh * F::kTs + 15) >> 4;
        const int row0 = rg_i * kRowsPerUnit + 16 * rt;
        const uint8_t* src0 = w + (((int64_t)sb0 * F::kTs) & ~(int64_t)15);
        const uint32_t dst0 = my_ring + slot_i * geo.slot_bytes;
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const int r = 2 * i + hl;
          const uint8_t* src = src0 + (int64_t)min(row0 + r, N - 1) * row_bytes;
          const uint32_t dst = dst0 + r * pitch;
          for (int k = kl; k < pieces; k += 16) cp_async16(dst + 16 * k, src + 16 * k);
        }
      }
      ++issued;
      if (++slot_i == depth) slot_i = 0;
      if (++rg_i == RG) { rg_i = 0; ++c_i; }
    }
    cp_async_commit();
  };
  if (tile_warp)
    for (int d = 0; d < depth - 1; d++) issue_next();

  // ---- shared-memory tables (immutable inputs: may be read before the previous kernel has finished)
  tf::Tables tb{};
  tb.grid = smem + geo.off_tab;
  if constexpr (F::kTableBytes > 0) {
    uint32_t* dst = reinterpret_cast<uint32_t*>(smem + geo.off_tab);
    if constexpr (F::kQt == QT_IQ1_S || F::kQt == QT_IQ1_M) {
      // int8 grid {-1, 0, 1} -> code bytes 8 * grid + 9
      const uint32_t* src = reinterpret_cast<const uint32_t*>(tab + TAB_IQ1);
      for (int i = tid; i < F::kTableBytes / 4; i += kThreads) {
        const uint32_t v = __ldg(src + i);
        // per byte: 0xFF -> 1, 0x00 -> 9, 0x01 -> 17
        const uint32_t neg = (v >> 7) & 0x01010101u, pos = v & ~(v >> 7) & 0x01010101u;
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
  int* misc = reinterpret_cast<int*>(smem + geo.off_misc);     // [0..15] S per batch row, [16..31] max exponent word
  float* xs_all = reinterpret_cast<float*>(smem + geo.off_xs);
  float* red = reinterpret_cast<float*>(smem + geo.off_red);

  // ---- everything below reads or writes memory the previous kernel may still be using
  pdl_wait();
  uint32_t out_tag = 0, x_tag = 0;
  peer_wait_previous(pp, tid, status);
  if (pp.world > 0 && pp.tagged) {
    const uint32_t e = pp.flags[pp.rank][pp.world];
    out_tag = peer_tag_of(e + 1) << 16;
    x_tag = peer_tag_of(e + 1 - (uint32_t)pp.x_back) << 16;
    if (pp.after_tagged && warp == kWarps)
      peer_wait_tagged(pp.after_tagged, pp.after_words, peer_tag_of(e + 1 - (uint32_t)pp.after_back) << 16, lane, 32, status);
  }

  // Stage chunk c of the activations: all threads.  Destination order [block][run t][octet][8 values],
  // 16 bytes per octet, so a lane's run of a block is 128 contiguous bytes.
  auto stage_pass = [&](int c, int m, int S) -> float {
    const int n_oct = geo.chunk_sb * 32;
    uint4* xv = reinterpret_cast<uint4*>(smem + geo.off_x + m * geo.x_row_bytes);
    float* xs = xs_all + m * geo.xs_row_floats;
    const float sum_scale = pow2f(S - 133);
    float amax = 0.f;
    for (int o = tid; o < n_oct; o += kThreads) {
      const int blk = o >> 5, tt = (o >> 3) & 3, oo = o & 7;
      int qa, qb;
      F::src_quads(tt, oo, qa, qb);
      const int64_t k0 = ((int64_t)c * geo.chunk_sb + blk) * 256;
      uint2 va = make_uint2(0, 0), vb = make_uint2(0, 0);
      if (m < M && k0 < K) {
        if (F::kPairOrder == 0 && pp.x_tagged) {
          const uint4 v = peer_load8_tagged(pp.x_tagged, (int)((k0 + qa) >> 3), x_tag, status);
          va = make_uint2(v.x, v.y); vb = make_uint2(v.z, v.w);
        } else {
          const __nv_bfloat16* xr = x + (int64_t)m * K + k0;
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
      xv[o] = o4;
      float sum = ((a0 + a1) + (a2 + a3)) + ((b0 + b1) + (b2 + b3));
      const float asum = ((fabsf(a0) + fabsf(a1)) + (fabsf(a2) + fabsf(a3))) + ((fabsf(b0) + fabsf(b1)) + (fabsf(b2) + fabsf(b3)));
      amax = fmaxf(amax, asum);
      if constexpr (F::kSums) {
        if (F::kGroupOct >= 2) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
        if (F::kGroupOct >= 4) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
        if ((oo & (F::kGroupOct - 1)) == 0) xs[o / F::kGroupOct] = sum * sum_scale;
      }
    }
    return amax;
  };
  auto stage_chunk = [&](int c) {
    bar_sync(kBarStage, kThreads);          // nobody still reads the previous chunk's activations
    if (tid < 16) { misc[tid] = 96; misc[16 + tid] = 0; }
    bar_sync(kBarStage, kThreads);
    // Optimistic scale 2^96: right whenever the largest |x| of the chunk lies in about [2^-30, 2^24).
    for (int m = 0; m < geo.x_rows; m++) {
      const float amax = stage_pass(c, m, 96);
      if (m < M) atomicMax(&misc[16 + m], (int)__float_as_uint(amax));      // non-negative floats order like integers
    }
    bar_sync(kBarStage, kThreads);
    for (int m = 0; m < M; m++) {
      const int emax = min((misc[16 + m] >> 23) & 0xFF, 254);               // biased exponent of the largest octet sum of |x|
      if (emax > 156 || (emax < 97 && emax > 0)) {
        const int S = max(8, min(120, 247 - emax));
        stage_pass(c, m, S);
        if (tid == 0) misc[m] = S;
      }
    }
    bar_sync(kBarStage, kThreads);
  };

  const bool live = (g >> 1) == t;
  const uint32_t x_base = live ? smem_u32(smem + geo.off_x) + (g & 1) * geo.x_row_bytes : smem_u32(smem + geo.off_zero);
  const uint32_t x_pass = live ? 2u * geo.x_row_bytes : 0u, x_oct = live ? 16u : 0u, x_blk = live ? 512u : 0u;
  const uint32_t x_run0 = x_base + (live ? (uint32_t)(j * nb * 512 + t * 128) : 0u);
  constexpr int kGroups = 8 / F::kGroupOct;

  int c_cur = -1;
  if (tile_warp) {
    int slot = 0, flush_i = 0;
    for (int i = 0; i < n_units; i++) {
      const int64_t u = u_begin + i;
      const int c = (int)(u / RG);
      if (c != c_cur) { stage_chunk(c); c_cur = c; }
      issue_next();
      cp_async_wait_pending(depth - 1);
      __syncwarp();
      float out[MP][4];
#pragma unroll
      for (int p = 0; p < MP; p++) out[p][0] = out[p][1] = out[p][2] = out[p][3] = 0.f;
      const int sb0 = c * geo.chunk_sb + j * nb;
      const int nbh = min(nb, SB - sb0);
      const uint8_t* tile = smem + (size_t)warp * (depth * geo.slot_bytes) + slot * geo.slot_bytes + g * pitch + a_off;
      for (int blk = 0; blk < nbh; blk++) {
        const tf::BlockLd ld0{tile + blk * F::kTs}, ld1{tile + blk * F::kTs + 8 * pitch};
        const typename F::Run run0 = F::load_run(ld0, t), run1 = F::load_run(ld1, t);
        const uint32_t xr = x_run0 + blk * x_blk;
        const float* xs = xs_all + ((j * nb + blk) * 4 + t) * kGroups;
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
              const uint4 xv = *reinterpret_cast<const uint4*>(__cvta_shared_to_generic(xg + q * x_oct + p * x_pass));
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
              s0 = xs[(2 * p) * geo.xs_row_floats + grp];
              s1 = xs[(2 * p + 1) * geo.xs_row_floats + grp];
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
      // hand this warp's 16 x 2MP sums to the reducer
      const int pb = flush_i & 1;
      if (flush_i >= 2) bar_sync(kBarFree + pb, kThreads);
      float* rb = red + (pb * kWarps + warp) * 16 * geo.x_rows;
#pragma unroll
      for (int p = 0; p < MP; p++) {
#pragma unroll
        for (int q = 0; q < 4; q++) {
          float v = out[p][q];
          v += __shfl_xor_sync(0xFFFFFFFFu, v, 1);
          v += __shfl_xor_sync(0xFFFFFFFFu, v, 2);
          if (t == 0) rb[(g + 8 * (q >> 1)) * geo.x_rows + 2 * p + (q & 1)] = v;
        }
      }
      __threadfence_block();
      bar_arrive(kBarFull + pb, kThreads);
      ++flush_i;
    }
  } else {
    // The reducer: folds the tile warps' sums of a unit, leaves them in scratch and bumps the row
    // group's arrival counter.  The counter's old value is not needed before the *next* unit has been
    // folded, so the atomic's round trip to L2 never holds the reducer (and through the two
    // hand-off buffers, the tile warps) up.
    int pend_rg = -1;
    int pend_old = 0;
    auto emit = [&](int row, int m, float val) {
      if (pp.world == 0) store_out(y, y_dtype, (int64_t)m * N + row, val);
      else peer_emit(pp, y, y_dtype, row, val, out_tag);
    };
    auto settle = [&]() {       // the pending unit: if it completed its row group, add the chunks in order
      const int old = __shfl_sync(0xFFFFFFFFu, pend_old, 0);
      if (old == geo.C - 1) {
        float s[2 * MP];
#pragma unroll
        for (int m = 0; m < 2 * MP; m++) s[m] = 0.f;
        for (int cc = 0; cc < geo.C; cc++) {
          const float* theirs = partials + (((int64_t)cc * RG + pend_rg) * geo.x_rows) * 32 + lane;
#pragma unroll
          for (int m = 0; m < 2 * MP; m++)
            if (m < M) s[m] += __ldcg(theirs + m * 32);
        }
        const int row = pend_rg * kRowsPerUnit + lane;
        if (row < N) {
#pragma unroll
          for (int m = 0; m < 2 * MP; m++)
            if (m < M) emit(row, m, s[m]);
        }
        if (lane == 0) counters[pend_rg] = 0;
      }
      pend_rg = -1;
    };
    for (int i = 0; i < n_units; i++) {
      const int64_t u = u_begin + i;
      const int c = (int)(u / RG), rg = (int)(u - (int64_t)c * RG);
      if (c != c_cur) { stage_chunk(c); c_cur = c; }
      const int pb = i & 1;
      bar_sync(kBarFull + pb, kThreads);
      const float* rb = red + (pb * kWarps + (lane >> 4) * 8) * 16 * geo.x_rows + (lane & 15) * geo.x_rows;
      float v[2 * MP];
#pragma unroll
      for (int m = 0; m < 2 * MP; m++) {
        float s = 0.f;
#pragma unroll
        for (int jj = 0; jj < 8; jj++) s += rb[jj * 16 * geo.x_rows + m];
        v[m] = s * pow2f(133 - misc[m]);        // undo the power-of-two scaling of the activations
      }
      __syncwarp();
      bar_arrive(kBarFree + pb, kThreads);
      const int row = rg * kRowsPerUnit + lane;
      if (geo.C == 1) {
        if (row < N) {
#pragma unroll
          for (int m = 0; m < 2 * MP; m++)
            if (m < M) emit(row, m, v[m]);
        }
      } else {
        float* mine = partials + (u * geo.x_rows) * 32 + lane;
#pragma unroll
        for (int m = 0; m < 2 * MP; m++)
          if (m < M) __stcg(mine + m * 32, v[m]);
        __syncwarp();
        if (pend_rg >= 0) settle();
        // release: this warp's partial stores are visible to whoever sees the increment; acquire: if this
        // is the last arrival, the other units' partials are visible to this warp
        if (lane == 0)
          asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(pend_old) : "l"(counters + rg) : "memory");
        pend_rg = rg;
      }
    }
    if (pend_rg >= 0) settle();
  }
  cp_async_wait_pending(0);
  peer_publish(pp, tid, G);
}

// ---------------------------------------------------------------------------------------------
// host side

struct FormatInfo { int qt, ts, table_bytes, sum_groups; bool sums; };

template <class F>
constexpr FormatInfo info_of() { return {F::kQt, F::kTs, F::kTableBytes, 8 / F::kGroupOct, F::kSums}; }

static bool format_of(int qtype, FormatInfo* fi) {
  switch (qtype) {
    case QT_Q4_K: *fi = info_of<tf::Q4K>(); return true;
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

// Shared-memory layout and work split for one launch; false if nothing fits.
static bool plan(const FormatInfo& fi, int64_t N, int64_t K, int M, int sm_count, int nb_forced, Geo* out) {
  const int SB = (int)(K / 256);
  const int x_rows = 2 * passes_of(M);
  Geo best{};
  double best_cost = 1e30;
  for (int nb = 1; nb <= 4; nb *= 2) {
    if (nb_forced > 0 && nb != nb_forced) continue;
    Geo g{};
    g.nb = nb;
    g.chunk_sb = 8 * nb;
    g.C = (SB + g.chunk_sb - 1) / g.chunk_sb;
    g.RG = (int)((N + kRowsPerUnit - 1) / kRowsPerUnit);
    g.U = (int64_t)g.C * g.RG;
    g.x_rows = x_rows;
    g.x_row_bytes = g.chunk_sb * 512;
    g.xs_row_floats = fi.sums ? g.chunk_sb * 4 * fi.sum_groups : 0;
    const int pieces = (14 + nb * fi.ts + 15) / 16;
    g.pitch = 16 * pieces;
    if (g.pitch % 32 == 0) g.pitch += 16;          // odd multiple of 16: rows fall into different bank groups
    g.slot_bytes = 16 * g.pitch;
    const int fixed = x_rows * g.x_row_bytes + x_rows * g.xs_row_floats * 4 + 64 + 2 * kWarps * 16 * x_rows * 4 +
                      (fi.table_bytes + 15) / 16 * 16 + 128;
    const int room = kSmemLimit - fixed;
    if (room < 2 * kWarps * g.slot_bytes) continue;
    g.depth = std::min(kMaxDepth, room / (kWarps * g.slot_bytes));
    g.off_x = kWarps * g.depth * g.slot_bytes;
    g.off_xs = g.off_x + x_rows * g.x_row_bytes;
    g.off_zero = g.off_xs + x_rows * g.xs_row_floats * 4;
    g.off_red = g.off_zero + 64;
    g.off_tab = g.off_red + 2 * kWarps * 16 * x_rows * 4;
    g.off_misc = g.off_tab + (fi.table_bytes + 15) / 16 * 16;
    g.total = g.off_misc + 128;
    // time ~ steps of the busiest CTA x (blocks per step + a fixed cost per step); a shallow ring costs extra
    const int grid = (int)std::min<int64_t>(g.U, sm_count);
    const double steps = (double)((g.U + grid - 1) / grid);
    const double cost = steps * (nb + 0.35) * (g.depth >= 3 ? 1.0 : 1.08);
    if (cost < best_cost) { best_cost = cost; best = g; }
  }
  if (best_cost >= 1e30) return false;
  *out = best;
  return true;
}

static int forced_nb() {
  static const int v = [] { const char* s = getenv("GGQ_TILE_NB"); return s ? atoi(s) : 0; }();
  return v;
}

template <class F, int MP>
static cudaError_t launch(const Geo& geo, int grid, cudaStream_t st, const uint8_t* w, int N, int K, const void* x, int M,
                          void* y, int y_dtype, int* counters, float* partials, const PeerPublish& pp, int* status,
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
                               (const __nv_bfloat16*)x, M, y, y_dtype, counters, partials, geo, pp, status, tab);
  return err != cudaSuccess ? err : cudaPeekAtLastError();
}

template <class F>
static cudaError_t launch_passes(int MP, const Geo& geo, int grid, cudaStream_t st, const uint8_t* w, int N, int K,
                                 const void* x, int M, void* y, int y_dtype, int* counters, float* partials,
                                 const PeerPublish& pp, int* status, const uint8_t* tab) {
  switch (MP) {
    case 1: return launch<F, 1>(geo, grid, st, w, N, K, x, M, y, y_dtype, counters, partials, pp, status, tab);
    case 2: return launch<F, 2>(geo, grid, st, w, N, K, x, M, y, y_dtype, counters, partials, pp, status, tab);
    default: return launch<F, 4>(geo, grid, st, w, N, K, x, M, y, y_dtype, counters, partials, pp, status, tab);
  }
}

}  // namespace tile

bool gemv_tile_applicable(int qtype, int64_t N, int64_t K, int M, const void* w, const void* x) {
  tile::FormatInfo fi;
  if (!tile::format_of(qtype, &fi)) return false;
  if (M < 1 || M > tile::kMaxBatch || K <= 0 || K % 256 || N < 1 || N > (1ll << 24)) return false;
  if ((K / 256 * fi.ts) % 16 || (uintptr_t)w % 16 || (uintptr_t)x % 16 || (K * 2) % 16) return false;
  if (N * (K / 256 * fi.ts) >= (1ll << 40)) return false;
  tile::Geo geo;
  return tile::plan(fi, N, K, M, 148, 0, &geo);
}

// Scratch: the arrival counters (one per 32-row group) in the counter area every kernel shares, and
// one 32 x batch-row float slot per unit in the float area; sized for the finest split (nb = 1).
size_t gemv_tile_workspace_bytes(int qtype, int64_t N, int64_t K, int M) {
  tile::FormatInfo fi;
  if (!tile::format_of(qtype, &fi) || M < 1 || M > tile::kMaxBatch) return 0;
  const int64_t RG = (N + tile::kRowsPerUnit - 1) / tile::kRowsPerUnit;
  const int64_t C = (K / 256 + 7) / 8;
  const size_t partial = C > 1 ? (size_t)(RG * C) * 2 * tile::passes_of(M) * 32 * sizeof(float) : 0;
  return kWsGemmPartialOffset + (partial + 255) / 256 * 256;
}

cudaError_t gemv_tile(int qtype, const uint8_t* w, int64_t N, int64_t K, const void* x, int M, void* y, int y_dtype,
                      void* ws, size_t ws_bytes, int sm_count, int* status, const uint8_t* tab, cudaStream_t st,
                      const PeerPublish* peers) {
  using namespace tile;
  FormatInfo fi;
  if (!format_of(qtype, &fi)) return cudaErrorInvalidValue;
  Geo geo;
  if (!plan(fi, N, K, M, sm_count, forced_nb(), &geo) && !plan(fi, N, K, M, sm_count, 0, &geo)) return cudaErrorInvalidValue;
  if (!ws || ws_bytes < gemv_tile_workspace_bytes(qtype, N, K, M) || (uintptr_t)ws % 256) return cudaErrorInvalidValue;
  if (kWsCounterOffset + (size_t)geo.RG * sizeof(int) > kWsGemmPartialOffset) return cudaErrorInvalidValue;
  PeerPublish pp = {};
  if (peers) pp = *peers;
  int* counters = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(ws) + kWsCounterOffset);
  float* partials = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ws) + kWsGemmPartialOffset);
  const int grid = (int)std::min<int64_t>(geo.U, sm_count);
  const int MP = passes_of(M);
#define GGQ_TILE_CASE(QT, F) \
  case QT: return launch_passes<tf::F>(MP, geo, grid, st, w, (int)N, (int)K, x, M, y, y_dtype, counters, partials, pp, status, tab);
  switch (qtype) {
    GGQ_TILE_CASE(QT_Q4_K, Q4K)
    GGQ_TILE_CASE(QT_Q2_K, Q2K)
    GGQ_TILE_CASE(QT_IQ4_XS, IQ4XS)
    GGQ_TILE_CASE(QT_IQ2_XXS, IQ2XXS)
    GGQ_TILE_CASE(QT_IQ2_XS, IQ2XS)
    GGQ_TILE_CASE(QT_IQ2_S, IQ2S)
    GGQ_TILE_CASE(QT_IQ3_XXS, IQ3XXS)
    GGQ_TILE_CASE(QT_IQ3_S, IQ3S)
    GGQ_TILE_CASE(QT_IQ1_S, IQ1S)
    GGQ_TILE_CASE(QT_IQ1_M, IQ1M)
    default: return cudaErrorInvalidValue;
  }
#undef GGQ_TILE_CASE
}

}  // namespace ggq
