// Q4_K fused decode + multiply for batch 1, tuned for B200 HBM bandwidth.
//
// Data movement.  A persistent CTA per SM with sixteen tile warps (and a seventeenth that only
// reduces and publishes row sums, see the multiply side).  Every warp streams its own
// steps (16 weight rows x two adjacent 144-byte superblocks, 4.6 KB) from HBM into a private
// ring of shared-memory slots, one to three steps ahead of the
// one it is multiplying (as many as shared memory allows next to the staged activations; no
// registers are held by loads in flight); the warps of a CTA sit on adjacent superblocks of
// the same 32 rows, so each row is read as a contiguous run.  A step arrives either as one
// two-dimensional TMA box (cp.async.bulk.tensor: 16 rows x 304 bytes of a tensor map over the
// weight, issued by one lane, counted on a per-warp mbarrier) or, where the driver offers no
// tensor-map encoder, as nine 16-byte cp.async per lane.  One-dimensional bulk copies (one per
// row, ~300 bytes each) were measured first and lose to per-thread copies (about 50 cycles of fixed
// cost per bulk copy); the box, one instruction per 4.8 KB, beats them: 29.2 against 31.2 us on
// 8192 x 28672, 10.0 against 12.7 us on 14336 x 4096.  The row pitch of a slot (304 B =
// 48 mod 128; the box simply reads 16 bytes past the two superblocks) makes the 128-bit
// shared-memory reads of the MMA fragment layout conflict free.
//
// Arithmetic.  Per-element FMAs cannot keep up with HBM on this part (about 2.5 issued
// lane-instructions per weight at peak bandwidth), so the dot products run on the tensor
// cores with *exact integer* weights.  A bf16 whose upper byte is zero is linear in its
// lower byte: bits 0x00vv decode to v * 2^-133 for every v in 0..255 (subnormals for
// v < 128, the first normal binade above).  So the masked word (w & 0x000F000F) already IS
// a pair of bf16 weights q * 2^-133, and (w & 0x00F000F0) is the pair 16 q * 2^-133 of the
// high nibbles: one logic instruction per two weights, no conversion, no bias.
// mma.sync.m16n8k16 multiplies 16 rows x 16 codes by the bf16 activations with float32
// accumulation; the activations are pre-scaled by a power of two (2^S for the even
// sub-blocks, 2^(S-4) for the odd ones, which also absorbs the 16) so that the products sit
// in the normal float32 range, and the matching 2^(133-S) goes into the float32 scale.
// The scales are applied to the accumulators, not to the weights:
//     y += (d * sc) * u - (dmin * mn) * sum(x),      u = sum(q * x)
// so a weight never loses precision (a one-hot x returns bf16(float32 weight) exactly).
// mma.sync (not tcgen05) is deliberate: the kernel is HBM-bound with the tensor pipe ~12 %
// busy, and tcgen05 takes its operands from shared memory, which would add a decode->smem
// round trip of 4 B per weight against 0.56 B per weight of HBM traffic.
//
// The eight columns of the MMA's B operand are used as eight *sub-block channels*: lane
// group t of the warp holds the 32 bytes [32t, 32t+32) of a superblock's quants, i.e. the
// sub-block pair (2t, 2t+1); column c of B carries the activations of sub-block c in the
// k-slots of lane group c/2 and zeros elsewhere.  The accumulator tiles therefore collect
// all eight sub-block sums of 16 rows, and lane (g, t) ends up holding exactly the sums
// whose scales it unpacks: rows g and g+8, sub-blocks 2t and 2t+1.
//
// Work split.  Units of (32-row group, 8-superblock chunk) are dealt to the CTAs as
// contiguous ranges of equal length, so every SM streams the same number of bytes; inside
// a unit warp (rt, j) takes row tile rt and superblock j.  A row group cut by a range
// boundary is finished by whichever CTA arrives last: partial sums go to a small scratch
// buffer, a per-row-group counter tells the last arriver, which adds the partials in CTA
// order (deterministic) and leaves the counter at zero again.  No thread ever waits on
// another CTA.  The only spin loop is the bounded wait of the row-sharded variant for the
// peers' flags of the previous exchange (50 ms, then the status word is raised).
#include "gemv.cuh"

#include <cuda.h>

#include <cstdlib>
#include <cstring>

namespace ggq {
namespace q4k {

constexpr int kBlockBytes = 144;
constexpr int kRowTiles = 2;                   // 16-row tiles per unit
constexpr int kWarps = 8 * kRowTiles;          // one warp per (row tile, superblock pair of the chunk)
constexpr int kThreads = (kWarps + 1) * 32;    // sixteen tile warps and one reducer warp
constexpr int kBarFull = 1, kBarFree = 3;      // named barriers (two each, alternating) of the flush hand-off
constexpr int kRowsPerUnit = 16 * kRowTiles;
constexpr int kSbPerWarp = 2;                  // adjacent superblocks a warp multiplies per step
constexpr int kSbPerUnit = 8 * kSbPerWarp;
constexpr int kTileBytes = 16 * kBlockBytes;   // 2304
// Row pitch of a slot, chosen so that the 128-bit reads of a quarter-warp (two rows x four lanes)
// fall into distinct banks: 144 = 16 (mod 128) for one superblock per step, 304 = 48 (mod 128) for two.
constexpr int kSlotPitch = kSbPerWarp == 1 ? kBlockBytes : kSbPerWarp * kBlockBytes + 16;
constexpr int kSlotBytes = 16 * kSlotPitch;                // one warp's step: 16 rows of kSbPerWarp superblocks
constexpr int kSmemLimit = 232448;             // 227 KB opt-in limit per CTA

struct Smem {
  // ring: [16 warps][DEPTH slots][2304 B] precedes everything else
  int x;                                                                         // bf16[K], scaled + permuted
  __host__ __device__ explicit Smem(int depth) : x(kWarps * depth * kSlotBytes) {}
  __host__ __device__ int xs(int K) const { return x + 2 * K; }       // float[K/32] sub-block sums
  __host__ __device__ int zero(int K) const { return xs(K) + (K / 32) * 4; }  // 64 zero bytes
  __host__ __device__ int red(int K) const { return zero(K) + 64; }   // float[2][kWarps][16]
  __host__ __device__ int misc(int K) const { return red(K) + 2 * kWarps * 16 * 4; }
  __host__ __device__ int bars(int K) const { return misc(K) + 16; }   // uint64[kWarps][4]: per-warp slot barriers (tensor-map copies)
  __host__ __device__ int total(int K) const { return bars(K) + kWarps * 4 * 8; }
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// A plain (schedulable) 128-bit shared-memory load from a shared-window address.
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  return *reinterpret_cast<const uint4*>(__cvta_shared_to_generic(addr));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const uint8_t* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void bar_sync(int id, int count) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory"); }
__device__ __forceinline__ void bar_arrive(int id, int count) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory"); }
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// Not volatile: the instruction is a pure function of its operands, and leaving the compiler free
// to interleave independent accumulation chains and the next tile's loads is worth a lot here.
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// byte `SEL` (0..3) of x as a float, exact: bits 0x4B0000vv are 2^23 + v.
template <int SEL>
__device__ __forceinline__ float byte_to_float(uint32_t x) {
  return __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7440 + SEL)) - 8388608.0f;
}
__device__ __forceinline__ float bf16lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16hi(uint32_t u) { return __uint_as_float(u & 0xFFFF0000u); }

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

// Multiply one tile by its superblock's activations (at xa, sums at xsa) and add this lane's share of the
// 16 row sums to out0 (row g) / out1 (row g+8).
__device__ __forceinline__ void compute_tile(uint32_t tile, int g, int t, const LaneScale& lc, uint32_t xa,
                                             uint32_t x_step, uint32_t xsa, float& out0, float& out1) {
  // this lane's share of the tile: block header and 32 quant bytes of rows g and g+8
  const uint32_t base0 = tile + g * kSlotPitch, base1 = base0 + 8 * kSlotPitch;
  const uint4 h0 = lds128(base0), h1 = lds128(base1);
  const uint4 qa0 = lds128(base0 + 16 + 32 * t), qb0 = lds128(base0 + 32 + 32 * t);
  const uint4 qa1 = lds128(base1 + 16 + 32 * t), qb1 = lds128(base1 + 32 + 32 * t);
  // A lane feeds column g of the B operand; that column is live only in the k-slots of lane
  // group g/2, so every other lane reads the zero page (base = zero page, strides = 0).
  const uint4 x0 = lds128(xa), x1 = lds128(xa + x_step), x2 = lds128(xa + 2 * x_step), x3 = lds128(xa + 3 * x_step);
  const float2 sx = *reinterpret_cast<const float2*>(__cvta_shared_to_generic(xsa));   // X[2t], X[2t+1], scaled

  // Two accumulator tiles: the low-nibble pass and the high-nibble pass both multiply by this
  // lane's activations; only column 2t of the first and 2t+1 of the second are kept.
  float lo[4] = {0.f, 0.f, 0.f, 0.f}, hi[4] = {0.f, 0.f, 0.f, 0.f};
  const uint32_t w0[8] = {qa0.x, qa0.y, qa0.z, qa0.w, qb0.x, qb0.y, qb0.z, qb0.w};
  const uint32_t w1[8] = {qa1.x, qa1.y, qa1.z, qa1.w, qb1.x, qb1.y, qb1.z, qb1.w};
  const uint32_t xr[16] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w,
                           x2.x, x2.y, x2.z, x2.w, x3.x, x3.y, x3.z, x3.w};
#pragma unroll
  for (int i = 0; i < 8; i++) {
    // word i = bytes 4i..4i+3 of the lane's run: elements 4i..4i+3 of sub-block 2t (low
    // nibbles) and 2t+1 (high nibbles).  Bytes (0,2) fill k-slots 2t,2t+1; bytes (1,3) fill
    // k-slots 2t+8,2t+9, matching the pair-permuted activations.
    const uint32_t a = w0[i], b = w1[i];
    const uint32_t as = a >> 8, bs = b >> 8;   // (an integer-multiply shift on the FMA pipe measured 4 us slower)
    mma16816(lo, a & 0x000F000Fu, b & 0x000F000Fu, as & 0x000F000Fu, bs & 0x000F000Fu, xr[2 * i], xr[2 * i + 1]);
    mma16816(hi, a & 0x00F000F0u, b & 0x00F000F0u, as & 0x00F000F0u, bs & 0x00F000F0u, xr[2 * i], xr[2 * i + 1]);
  }
  float dla, dma, dlb, dmb;
  pair_scales(h0, lc, dla, dma, dlb, dmb);
  out0 = fmaf(dla, lo[0], out0); out0 = fmaf(dma, sx.x, out0);
  out0 = fmaf(dlb, hi[1], out0); out0 = fmaf(dmb, sx.y, out0);
  pair_scales(h1, lc, dla, dma, dlb, dmb);
  out1 = fmaf(dla, lo[2], out1); out1 = fmaf(dma, sx.x, out1);
  out1 = fmaf(dlb, hi[3], out1); out1 = fmaf(dmb, sx.y, out1);
}

// TMA: a step's 16 rows x 304 bytes arrive as one two-dimensional tensor-map box (cp.async.bulk.tensor) issued by one
// lane and counted on a per-warp, per-slot mbarrier, instead of nine cp.async instructions per lane.
template <int DEPTH, bool TMA>
__global__ void __launch_bounds__(kThreads, 1)
gemv_q4k_m1_kernel(const uint8_t* __restrict__ w, int N, int K, const __nv_bfloat16* __restrict__ x,
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
  if (TMA && warp < kWarps) {
    if (lane == 0) {
      for (int d = 0; d < DEPTH; d++) asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(my_bars + 8 * d), "r"(1u) : "memory");
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
  }

  // ---- copy side.  A step's slot holds 16 rows x 288 B (two adjacent superblocks per row) at a
  // row pitch of 304 B.  Nine cp.async instructions fill it: eight copy pieces 0..15 (256 B) of
  // two rows each (one row per half-warp), the ninth copies pieces 16..17 of all sixteen rows.
  // Source and destination are affine in the instruction index, so a lane keeps three offsets.
  // The last row group of a weight whose N is not a multiple of 32 takes a slower path that
  // clamps every row to N - 1 (copied, multiplied, never stored); a missing second superblock
  // (odd K/256) is never multiplied, its 144 bytes are simply not copied.
  // two-superblock steps: 8 instructions copy pieces 0..15 of two rows each, a ninth pieces 16..17
  // of all rows; one-superblock steps: 6 instructions copy the 9 pieces of three rows each.
  const int hl = lane >> 4, kl = lane & 15, r3 = lane / 9, k9 = lane - 9 * r3;
  const int32_t src_a = kSbPerWarp == 2 ? hl * row_bytes + 16 * kl : r3 * row_bytes + 16 * k9;
  const int32_t src_b = (lane >> 1) * row_bytes + 256 + 16 * (lane & 1);
  const uint32_t dst_a = kSbPerWarp == 2 ? hl * kSlotPitch + 16 * kl : r3 * kSlotPitch + 16 * k9;
  const uint32_t dst_b = (lane >> 1) * kSlotPitch + 256 + 16 * (lane & 1);
  const uint8_t* src = w;        // first source byte of the next step
  int rg_i = rg_begin, c_i = c_begin, issued = 0, slot_i = 0;
  auto seek_row_group = [&]() {
    src = w + (int64_t)(rg_i * kRowsPerUnit + 16 * rt) * row_bytes +
          (int64_t)(c_i * kSbPerUnit + kSbPerWarp * j) * kBlockBytes;
  };
  seek_row_group();
  auto issue_next = [&]() {
    if (TMA) {
      if (issued < n_units) {
        if (lane == 0) {
          const int sb0 = c_i * kSbPerUnit + kSbPerWarp * j;
          const int row0 = rg_i * kRowsPerUnit + 16 * rt;
          const uint32_t dst = my_ring + slot_i * kSlotBytes, bar = my_bars + 8 * slot_i;
          // the box is 76 32-bit words (304 bytes: the two superblocks and the 16 bytes behind them, which keep the slot's
          // row pitch) by 16 rows; words and rows outside the tensor arrive as zeros and count towards the bytes
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // the slot's last reads precede the copy
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)kSlotBytes) : "memory");
          asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                       ::"r"(dst), "l"(&w_map), "r"(sb0 * (kBlockBytes / 4)), "r"(row0), "r"(bar) : "memory");
        }
        ++issued;
        if (++slot_i == DEPTH) slot_i = 0;
        if (++c_i == C) { c_i = 0; ++rg_i; }
      }
      return;
    }
    if (issued < n_units) {
      const int sb0 = c_i * kSbPerUnit + kSbPerWarp * j;
      const uint32_t dst = my_ring + slot_i * kSlotBytes;
      const int row0 = rg_i * kRowsPerUnit + 16 * rt;
      if (sb0 + kSbPerWarp <= SB && row0 + 16 <= N) {
        // common case: every superblock of the step and all sixteen rows exist
        const uint8_t* pa = src + src_a;
        if constexpr (kSbPerWarp == 2) {
#pragma unroll
          for (int i = 0; i < 8; i++) cp_async16(dst + dst_a + i * (2 * kSlotPitch), pa + (int64_t)i * (2 * row_bytes));
          cp_async16(dst + dst_b, src + src_b);
        } else {
          if (lane < 27) {
#pragma unroll
            for (int i = 0; i < 5; i++) cp_async16(dst + dst_a + i * (3 * kSlotPitch), pa + (int64_t)i * (3 * row_bytes));
          }
          if (lane < 9) cp_async16(dst + dst_a + 15 * kSlotPitch, pa + (int64_t)15 * row_bytes);
        }
      } else if (sb0 < SB) {
        const int nsb = min(kSbPerWarp, SB - sb0);
        for (int p = lane; p < 16 * 9 * nsb; p += 32) {
          const int row = p / (9 * nsb), k = p - row * (9 * nsb);
          const int64_t roff = (int64_t)(min(row0 + row, N - 1) - row0) * row_bytes;
          cp_async16(dst + row * kSlotPitch + 16 * k, src + roff + 16 * k);
        }
      }
      ++issued;
      if (++slot_i == DEPTH) slot_i = 0;
      src += kSbPerUnit * kBlockBytes;
      if (++c_i == C) { c_i = 0; ++rg_i; seek_row_group(); }
    }
    cp_async_commit();
  };
  // Fill the pipeline before the activation prologue so HBM is busy from the first cycle.
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
    // Once per CTA: zero page, per-sub-block sums X, largest |x|, then x written to shared
    // memory as scaled, pair-permuted bf16: word 2i = (x[4i], x[4i+2]), word 2i+1 = (x[4i+1], x[4i+3]).
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
    // One pass: read x once, accumulate the sub-block sum and the largest magnitude, and store the
    // activations scaled by 2^S_ (2^(S_-4) for odd sub-blocks) in pair-permuted order.
    auto stage_x = [&](int S_) -> float {
      const float up_even = __uint_as_float((uint32_t)(127 + S_) << 23);
      const float up_odd = __uint_as_float((uint32_t)(127 + S_ - 4) << 23);
      const float xs_scale = __uint_as_float((uint32_t)(127 + S_ - 133) << 23);   // sums follow the accumulators' scale
      float amax = 0.f;   // largest sum of |x| over a sub-block: within a factor 32 of the largest |x|
      // Every CTA needs all of x; start each one at a different place so that the CTAs do not read
      // the same L2 lines in lockstep.
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
          // raw words (x[4i], x[4i+1]), (x[4i+2], x[4i+3]), i = 2q, 2q+1
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
    // Optimistic scale 2^96: right whenever the largest |x| lies in about [2^-30, 2^24), i.e. for
    // any sane activation tensor.  Otherwise the tensor is staged a second time with a scale that
    // puts its largest magnitude near 2^120 (S limited to 8..120, which covers largest magnitudes
    // from about 2^-80 to 2^112 at full precision; beyond that the products over- or underflow).
    // The magnitude is judged from the largest sub-block sum of |x| (cheap: one add per element),
    // which overestimates the largest |x| by at most a factor 32.
    S = 96;
    atomicMax(xmax, (int)__float_as_uint(stage_x(S)));    // non-negative floats order like integers
    __syncthreads();
    const int emax = min((*xmax >> 23) & 0xFF, 254);       // biased exponent of that bound (NaN/inf: 255)
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
  float* red = reinterpret_cast<float*>(smem + L.red(K));

  auto emit = [&](int row, float v) { peer_emit(pp, y, y_dtype, row, v, out_tag); };

  // ---- multiply side: the tile warps walk the CTA's units row group by row group; at the end of a
  // row group they leave their row sums in shared memory and go on, and the reducer warp folds
  // them, settles split row groups with the other CTAs and stores the outputs.  The hand-off is
  // two pairs of named barriers (buffer full / buffer free), so a tile warp never waits for the
  // global-memory round trips of the reduction and the reducer never delays a tile.
  if (tile_warp) {
    int rg = rg_begin, c = c_begin, done = 0, slot = 0, flush_i = 0;
    uint32_t ring_round = 0;                               // how often the ring has wrapped: the parity the slot's barrier shows
    while (done < n_units) {
      const int c_first = c;
      const int c_stop = min(C, c + (n_units - done));     // chunks [c, c_stop) of row group rg are mine
      float out0 = 0.f, out1 = 0.f;                        // rows g and g+8 of this warp's tile, this lane's share
      int sbg = c * kSbPerUnit + kSbPerWarp * j;
      uint32_t xa = x_lane_base + (uint32_t)sbg * x_sb_stride;
      uint32_t xsa = xs_lane_base + (uint32_t)sbg * 32u;
      for (; c < c_stop; ++c) {
        issue_next();                                      // keeps DEPTH - 1 steps in flight
        if (TMA) {
          // bounded wait for the box of this slot; a wait that runs out raises the status word and goes on
          const uint32_t bar = my_bars + 8 * slot, parity = ring_round & 1;
          uint32_t ok = 0;
          for (uint32_t spin = 0; spin < (1u << 20) && !ok; spin++)
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
          if (!ok && status && lane == 0) atomicOr(status, STATUS_WAIT_EXPIRED);
        } else {
          cp_async_wait<DEPTH - 1>();                      // the oldest one has landed
        }
        __syncwarp();
        const uint32_t tile = my_ring + slot * kSlotBytes;
        if (sbg < SB) compute_tile(tile, g, t, lc, xa, x_step, xsa, out0, out1);
        if constexpr (kSbPerWarp == 2) {
          if (sbg + 1 < SB) compute_tile(tile + kBlockBytes, g, t, lc, xa + x_sb_stride, x_step, xsa + 32u, out0, out1);
        }
        __syncwarp();   // every lane is done with the slot before a later copy overwrites it
        if (++slot == DEPTH) { slot = 0; ++ring_round; }
        sbg += kSbPerUnit;
        xa += kSbPerUnit * x_sb_stride;
        xsa += kSbPerUnit * 32u;
      }
      done += c_stop - c_first;
      // fold the four lanes of a quad, then hand the 16 row sums of this warp to the reducer
      float v0 = out0, v1 = out1;
      v0 += __shfl_xor_sync(0xFFFFFFFFu, v0, 1); v0 += __shfl_xor_sync(0xFFFFFFFFu, v0, 2);
      v1 += __shfl_xor_sync(0xFFFFFFFFu, v1, 1); v1 += __shfl_xor_sync(0xFFFFFFFFu, v1, 2);
      const int p = flush_i & 1;
      if (flush_i >= 2) bar_sync(kBarFree + p, kThreads);  // the reducer has read this buffer's previous content
      float* redbuf = red + p * (kWarps * 16);
      if (t == 0) {
        redbuf[warp * 16 + g] = v0 * d_up;      // undo the power-of-two scaling of the activations
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
      float v[2];
#pragma unroll
      for (int h = 0; h < 2; h++) {
        const int r = lane + 32 * h;            // row within the unit
        v[h] = 0.f;
        if (r < kRowsPerUnit) {
#pragma unroll
          for (int jj = 0; jj < 8; jj++) v[h] += redbuf[((r >> 4) * 8 + jj) * 16 + (r & 15)];
        }
      }
      __syncwarp();
      bar_arrive(kBarFree + p, kThreads);                  // the buffer may be overwritten
      ++flush_i;
      if (complete) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
          const int r = lane + 32 * h, row = rg * kRowsPerUnit + r;
          if (r < kRowsPerUnit && row < N) emit(row, v[h]);
        }
      } else {
        const int slot_p = (rg == rg_begin) ? 0 : 1;
        float* mine = partials + ((int64_t)b * 2 + slot_p) * 64;
        __stcg(&mine[lane], v[0]);
        __stcg(&mine[lane + 32], v[1]);
        __threadfence();
        __syncwarp();
        const int bf = owner_of(rg_first_unit, U, G), bl = owner_of(rg_last_unit, U, G);
        int old = 0;
        if (lane == 0) old = atomicAdd(&counters[rg], 1);
        old = __shfl_sync(0xFFFFFFFFu, old, 0);
        if (old == bl - bf) {   // last of the bl - bf + 1 contributors: add the partials in CTA order
          __threadfence();
          float s0 = 0.f, s1 = 0.f;
          for (int bb = bf; bb <= bl; bb++) {
            const int sl = (rg == (int)((U * bb / G) / C)) ? 0 : 1;
            const float* theirs = partials + ((int64_t)bb * 2 + sl) * 64;
            s0 += __ldcg(&theirs[lane]);
            s1 += __ldcg(&theirs[lane + 32]);
          }
          const int row0 = rg * kRowsPerUnit + lane, row1 = row0 + 32;
          if (row0 < N) emit(row0, s0);
          if (lane + 32 < kRowsPerUnit && row1 < N) emit(row1, s1);
          if (lane == 0) counters[rg] = 0;
        }
      }
      if (c == C) { c = 0; ++rg; }
    }
  }
  if (!TMA) cp_async_wait<0>();
  peer_publish(pp, tid, G);
}

}  // namespace q4k

bool gemv_q4k_applicable(int64_t N, int64_t K, int M, const void* w, const void* x) {
  return M == 1 && K % 256 == 0 && q4k::Smem(2).total((int)K) <= q4k::kSmemLimit && N >= 1 &&
         N <= (1ll << 24) && N * (K / 256 * 144) < (1ll << 40) && (uintptr_t)w % 16 == 0 && (uintptr_t)x % 16 == 0;
}

// Scratch layout: [partial slots: kMaxSmCount CTAs x 2 x 64 floats][arrival counters: one int per
// row group].  The partial area has a fixed size and comes first, so that the counters of every
// call, whatever its shape, live in bytes that only ever hold counters (which each launch leaves
// at zero); partial slots may hold stale floats, they are always written before they are read.
static constexpr size_t kPartialBytes = (size_t)kMaxSmCount * 2 * 64 * sizeof(float);
static_assert(kPartialBytes == kWsCounterOffset, "the counters of every kernel share one area");

size_t gemv_q4k_workspace_bytes(int64_t N, int sm_count) {
  (void)sm_count;
  const int64_t RG = (N + q4k::kRowsPerUnit - 1) / q4k::kRowsPerUnit;
  return kPartialBytes + ((size_t)RG * sizeof(int) + 255) / 256 * 256;
}

cudaError_t gemv_q4k(const uint8_t* w, int64_t N, int64_t K, const void* x, void* y, int y_dtype, void* ws,
                     size_t ws_bytes, int sm_count, int* status, cudaStream_t st, const PeerPublish* peers) {
  using namespace q4k;
  PeerPublish pp = {};
  if (peers) pp = *peers;
  if (ws_bytes < gemv_q4k_workspace_bytes(N, sm_count) || !ws) return cudaErrorInvalidValue;
  const int64_t RG = (N + kRowsPerUnit - 1) / kRowsPerUnit;
  const int SB = (int)(K / 256);
  const int64_t U = RG * ((SB + kSbPerUnit - 1) / kSbPerUnit);
  const int grid = (int)(U < sm_count ? U : sm_count);
  int depth = 4;
  while (depth > 2 && Smem(depth).total((int)K) > kSmemLimit) depth--;
  const int smem = Smem(depth).total((int)K);
  if (smem > kSmemLimit) return cudaErrorInvalidValue;
  static std::atomic<bool> attr_done[64];   // setting the attribute twice is harmless, so a flag per device suffices
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(gemv_q4k_m1_kernel<4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_q4k_m1_kernel<3, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_q4k_m1_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_q4k_m1_kernel<4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_q4k_m1_kernel<3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_q4k_m1_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e != cudaSuccess) return e;
    attr_done[dev].store(true, std::memory_order_release);
  }
  float* partials = reinterpret_cast<float*>(ws);
  int* counters = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(ws) + kPartialBytes);
  if (sm_count > kMaxSmCount) return cudaErrorInvalidValue;
  const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
  // Copy path: the weight as a tensor map of 32-bit words [N rows, row bytes / 4], box 76 words x 16 rows, where the
  // driver offers the encoder (measured on B200: 29.2 against 31.2 us on 8192 x 28672, 10.0 against 12.7 us on
  // 14336 x 4096); GGQ_Q4K_TMA=0 keeps the cp.async path, which is also the fallback.
  alignas(64) CUtensorMap w_map;
  memset(&w_map, 0, sizeof(w_map));
  static const bool want_tma = [] { const char* e = getenv("GGQ_Q4K_TMA"); return !(e && e[0] == '0'); }();
  bool tma = false;
  if (want_tma && kSbPerWarp == 2) tma = make_weight_map(&w_map, w, N, (int64_t)SB * kBlockBytes, kSlotPitch / 4);
  cudaError_t err;
#define GGQ_Q4K_LAUNCH(D, T) launch_pdl(gemv_q4k_m1_kernel<D, T>, grid, kThreads, smem, st, w, (int)N, (int)K, xb, y, y_dtype, counters, partials, pp, status, w_map)
  if (tma) err = depth == 4 ? GGQ_Q4K_LAUNCH(4, true) : depth == 3 ? GGQ_Q4K_LAUNCH(3, true) : GGQ_Q4K_LAUNCH(2, true);
  else err = depth == 4 ? GGQ_Q4K_LAUNCH(4, false) : depth == 3 ? GGQ_Q4K_LAUNCH(3, false) : GGQ_Q4K_LAUNCH(2, false);
#undef GGQ_Q4K_LAUNCH
  return err != cudaSuccess ? err : cudaPeekAtLastError();
}


// ---------------------------------------------------------------------------------------------
// ggq_gemv_q4k_static: the same batch-1 Q4_K kernel for callers that cannot hand over scratch.
//
// Some hosts of this library are not allowed to allocate device memory around a call: a
// custom-call handler whose framework owns every buffer and passes only operands and results, a
// serving loop with a fixed memory plan.  For them the partial-sum slots and arrival counters
// live in the file-scope device array below instead of a caller buffer.  Every GPU that loads
// the library carries these 192 KB until the process exits.
//
// In host code the array's name is only a host-side handle; the device address is obtained per
// device with cudaGetSymbolAddress (with that device current) the first time the entry point
// runs there (a synchronous runtime query).
// All calls on a device share the one array: calls whose kernels may overlap on the GPU
// (different streams without an ordering between them) would mix their partial sums and must be
// serialised by the caller.  The counters are cleared on the stream before every launch, so a
// call never depends on what the previous one left behind.
namespace q4k {
constexpr int64_t kStaticMaxRows = 524288;                                      // output rows it can take
static_assert(kRowsPerUnit >= 32, "the built-in scratch holds one counter per 32 rows");
constexpr size_t kStaticCounterBytes = (size_t)(kStaticMaxRows / 32) * sizeof(int);
constexpr size_t kStaticBytes = kPartialBytes + kStaticCounterBytes;             // 128 KB + 64 KB
static __device__ __align__(256) uint8_t g_static_scratch[kStaticBytes];
}  // namespace q4k

int32_t gemv_q4k_static(const void* w, int64_t N, int64_t K, const void* x, void* y, int32_t y_dtype,
                        int sm_count, cudaStream_t st) {
  using namespace q4k;
  if (N < 1 || N > kStaticMaxRows)
    return fail(GGQ_BAD_SHAPE, "ggq_gemv_q4k_static: N=%lld outside 1..%lld (the built-in scratch holds one "
                "arrival counter per %d rows)", (long long)N, (long long)kStaticMaxRows, kRowsPerUnit);
  if (!gemv_q4k_applicable(N, K, 1, w, x))
    return fail(GGQ_BAD_SHAPE, "ggq_gemv_q4k_static: needs K a multiple of 256 with K <= %d and 16-byte aligned "
                "w and x (got K=%lld)", (kSmemLimit - Smem(2).total(0)) / 2 / 256 * 256, (long long)K);
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess || dev < 0 || dev >= 64) return fail(GGQ_LAUNCH_FAILED, "ggq_gemv_q4k_static: no current device");
  static std::atomic<uint8_t*> dev_ptr[64];
  if (!dev_ptr[dev].load(std::memory_order_acquire)) {
    // once per device, with that device current: translate the symbol into a device address
    uint8_t* p = nullptr;
    err = cudaGetSymbolAddress((void**)&p, g_static_scratch);
    if (err != cudaSuccess || !p)
      return fail(GGQ_LAUNCH_FAILED, "ggq_gemv_q4k_static: cudaGetSymbolAddress: %s", cudaGetErrorString(err));
    dev_ptr[dev].store(p, std::memory_order_release);
  }
  uint8_t* scratch = dev_ptr[dev].load(std::memory_order_acquire);
  const int64_t RG = (N + kRowsPerUnit - 1) / kRowsPerUnit;
  err = cudaMemsetAsync(scratch + kPartialBytes, 0, (size_t)RG * sizeof(int), st);   // counters start at zero
  if (err == cudaSuccess)
    err = gemv_q4k((const uint8_t*)w, N, K, x, y, y_dtype, scratch, kStaticBytes, sm_count, nullptr, st);
  if (err != cudaSuccess) return fail(GGQ_LAUNCH_FAILED, "ggq_gemv_q4k_static: %s", cudaGetErrorString(err));
  return GGQ_OK;
}

}  // namespace ggq
