// Q4_K fused decode + multiply for batch 1, tuned for B200 HBM bandwidth.
//
// Data movement.  A persistent CTA per SM with sixteen warps.  Every warp streams its own
// tiles (16 weight rows x one 144-byte superblock) straight from HBM into registers with
// 128-bit read-only loads, one tile ahead of the one it is multiplying; the sixteen warps
// of a CTA sit on adjacent superblocks of the same 32 rows, so each row is read as a
// contiguous run.  Plain loads are used rather than TMA on purpose: measured on this part, a
// ring fed by cp.async.bulk copies of ~1 KB per row stops at 3.4 TB/s (about 50 cycles of
// fixed cost per bulk copy, one TMA unit per SM), copies of 16 KB reach 5.7 TB/s, while
// 128-bit loads issued by all warps stream 5.8-6.4 TB/s.  The GGUF row-major block layout
// only offers ~1 KB contiguous per row per 16-row tile, so the loads win.
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
// another CTA or on an asynchronous copy, so there is no spin loop in this kernel.
#include "gemv.cuh"

namespace ggq {
namespace q4k {

constexpr int kBlockBytes = 144;
constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr int kRowsPerUnit = 32;
constexpr int kSbPerUnit = 8;
constexpr int kMaxK = 98304;   // bf16 activations (2 B each) + their sums stay resident in shared memory

struct Smem {
  static constexpr int x = 0;                                                   // bf16[K], scaled + permuted
  static __host__ __device__ constexpr int xs(int K) { return x + 2 * K; }       // float[K/32] sub-block sums
  static __host__ __device__ constexpr int zero(int K) { return xs(K) + (K / 32) * 4; }  // 64 zero bytes
  static __host__ __device__ constexpr int red(int K) { return zero(K) + 64; }   // float[2][16 warps][16]
  static __host__ __device__ constexpr int misc(int K) { return red(K) + 2 * kWarps * 16 * 4; }
  static __host__ __device__ constexpr int total(int K) { return misc(K) + 16; }
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
// Streaming 128-bit load: read-only path, no L1 allocation priority (each byte is used once).
__device__ __forceinline__ uint4 ldg_stream(const uint8_t* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float bf16lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16hi(uint32_t u) { return __uint_as_float(u & 0xFFFF0000u); }

// Which CTA owns unit u when U units are dealt to G CTAs as ranges [U*b/G, U*(b+1)/G).
__device__ __forceinline__ int owner_of(int64_t u, int64_t U, int G) { return (int)(((u + 1) * G - 1) / U); }

// Scales of the sub-block pair (2t, 2t+1) from a block header (d|dmin, s0-3, s4-7, s8-11):
// dl = d * sc, dm = dmin * mn, the products exact in float32 (src/gguf_jax/quants.py:275-305).
// d is additionally multiplied by the power of two `d_up` that undoes the activation scaling.
__device__ __forceinline__ void pair_scales(const uint4& h, int t, float d_up, float& dl_a, float& dm_a,
                                            float& dl_b, float& dm_b) {
  const __half2 dd = *reinterpret_cast<const __half2*>(&h.x);
  const float d = __fmul_rn(__low2float(dd), d_up), dmin = __high2float(dd);
  const int sh = 16 * (t & 1);
  const uint32_t u1 = h.y >> sh, u2 = h.z >> sh, u3 = h.w >> sh;
  uint32_t scp, mnp;
  if (t < 2) {
    scp = u1 & 0x3F3Fu;
    mnp = u2 & 0x3F3Fu;
  } else {
    scp = (u3 & 0x0F0Fu) | ((u1 >> 2) & 0x3030u);
    mnp = ((u3 >> 4) & 0x0F0Fu) | ((u2 >> 2) & 0x3030u);
  }
  dl_a = __fmul_rn(d, (float)(scp & 0xFF));
  dl_b = __fmul_rn(d, (float)(scp >> 8));
  dm_a = __fmul_rn(dmin, (float)(mnp & 0xFF));
  dm_b = __fmul_rn(dmin, (float)(mnp >> 8));
}

// One lane's share of a tile: block header and 32 quant bytes of rows g and g+8.
struct TileRegs {
  uint4 h0, h1, qa0, qb0, qa1, qb1;
};

__device__ __forceinline__ void load_tile(TileRegs& r, const uint8_t* p0, const uint8_t* p1, int t) {
  r.h0 = ldg_stream(p0);
  r.h1 = ldg_stream(p1);
  r.qa0 = ldg_stream(p0 + 16 + 32 * t);
  r.qb0 = ldg_stream(p0 + 32 + 32 * t);
  r.qa1 = ldg_stream(p1 + 16 + 32 * t);
  r.qb1 = ldg_stream(p1 + 32 + 32 * t);
}

// Multiply one tile by the activations of superblock `sbg` and add this lane's share of the
// 16 row sums to out0 (row g) / out1 (row g+8).
__device__ __forceinline__ void compute_tile(const TileRegs& r, int sbg, int g, int t, bool live, uint32_t x_base,
                                             uint32_t zero_base, const float* xs, float d_up, float& out0,
                                             float& out1) {
  // A lane feeds column g of the B operand; that column is live only in the k-slots of lane
  // group g/2, so every other lane reads zeros.
  const uint32_t xa = live ? x_base + (uint32_t)(sbg * 8 + g) * 64 : zero_base;
  const uint32_t xstep = live ? 16u : 0u;
  const uint4 x0 = lds128(xa), x1 = lds128(xa + xstep), x2 = lds128(xa + 2 * xstep), x3 = lds128(xa + 3 * xstep);
  const float2 sx = *reinterpret_cast<const float2*>(xs + sbg * 8 + 2 * t);   // X[2t], X[2t+1]

  // Two accumulator tiles: the low-nibble pass and the high-nibble pass both multiply by this
  // lane's activations; only column 2t of the first and 2t+1 of the second are kept.
  float lo[4] = {0.f, 0.f, 0.f, 0.f}, hi[4] = {0.f, 0.f, 0.f, 0.f};
  const uint32_t w0[8] = {r.qa0.x, r.qa0.y, r.qa0.z, r.qa0.w, r.qb0.x, r.qb0.y, r.qb0.z, r.qb0.w};
  const uint32_t w1[8] = {r.qa1.x, r.qa1.y, r.qa1.z, r.qa1.w, r.qb1.x, r.qb1.y, r.qb1.z, r.qb1.w};
  const uint32_t xr[16] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w,
                           x2.x, x2.y, x2.z, x2.w, x3.x, x3.y, x3.z, x3.w};
#pragma unroll
  for (int i = 0; i < 8; i++) {
    // word i = bytes 4i..4i+3 of the lane's run: elements 4i..4i+3 of sub-block 2t (low
    // nibbles) and 2t+1 (high nibbles).  Bytes (0,2) fill k-slots 2t,2t+1; bytes (1,3) fill
    // k-slots 2t+8,2t+9, matching the pair-permuted activations.
    const uint32_t a = w0[i], b = w1[i];
    const uint32_t as = a >> 8, bs = b >> 8;
    mma16816(lo, a & 0x000F000Fu, b & 0x000F000Fu, as & 0x000F000Fu, bs & 0x000F000Fu, xr[2 * i], xr[2 * i + 1]);
    mma16816(hi, a & 0x00F000F0u, b & 0x00F000F0u, as & 0x00F000F0u, bs & 0x00F000F0u, xr[2 * i], xr[2 * i + 1]);
  }
  float dla, dma, dlb, dmb;
  pair_scales(r.h0, t, d_up, dla, dma, dlb, dmb);
  out0 = fmaf(dla, lo[0], out0); out0 = fmaf(-dma, sx.x, out0);
  out0 = fmaf(dlb, hi[1], out0); out0 = fmaf(-dmb, sx.y, out0);
  pair_scales(r.h1, t, d_up, dla, dma, dlb, dmb);
  out1 = fmaf(dla, lo[2], out1); out1 = fmaf(-dma, sx.x, out1);
  out1 = fmaf(dlb, hi[3], out1); out1 = fmaf(-dmb, sx.y, out1);
}

__global__ void __launch_bounds__(kThreads, 1)
gemv_q4k_m1_kernel(const uint8_t* __restrict__ w, int N, int K, const __nv_bfloat16* __restrict__ x,
                   void* __restrict__ y, int y_dtype, int* __restrict__ counters, float* __restrict__ partials) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int SB = K / 256;                        // superblocks per row
  const int64_t row_bytes = (int64_t)SB * kBlockBytes;
  const int C = (SB + kSbPerUnit - 1) / kSbPerUnit;   // chunks per row group
  const int RG = (N + kRowsPerUnit - 1) / kRowsPerUnit;
  const int64_t U = (int64_t)RG * C;
  const int G = gridDim.x, b = blockIdx.x;
  const int64_t u_begin = U * b / G, u_end = U * (b + 1) / G;
  const int n_units = (int)(u_end - u_begin);

  const int g = lane >> 2, t = lane & 3;
  const int rt = warp >> 3, j = warp & 7;        // row tile (16 rows) and superblock slot of this warp
  int rg = (int)(u_begin / C), c = (int)(u_begin - (int64_t)(u_begin / C) * C);

  // Address of this lane's rows for a unit; rows past N are clamped (loaded, never stored).
  auto tile_ptrs = [&](int rg_, int c_, const uint8_t*& p0, const uint8_t*& p1) -> bool {
    const int sbg = c_ * kSbPerUnit + j;
    const int r0 = min(rg_ * kRowsPerUnit + 16 * rt + g, N - 1), r1 = min(rg_ * kRowsPerUnit + 16 * rt + g + 8, N - 1);
    const int sbc = min(sbg, SB - 1);
    p0 = w + (int64_t)r0 * row_bytes + (int64_t)sbc * kBlockBytes;
    p1 = w + (int64_t)r1 * row_bytes + (int64_t)sbc * kBlockBytes;
    return sbg < SB;
  };

  // Start the first tile's loads before the activation prologue so HBM is busy from cycle one.
  TileRegs cur, nxt;
  {
    const uint8_t *p0, *p1;
    if (n_units > 0) { tile_ptrs(rg, c, p0, p1); load_tile(cur, p0, p1, t); }
  }

  float* xs = reinterpret_cast<float*>(smem + Smem::xs(K));
  int* xmax = reinterpret_cast<int*>(smem + Smem::misc(K));
  int S;  // activations are held as x * 2^S (even sub-blocks) / x * 2^(S-4) (odd sub-blocks)
  {
    // Once per CTA: zero page, per-sub-block sums X, largest |x|, then x written to shared
    // memory as scaled, pair-permuted bf16: word 2i = (x[4i], x[4i+2]), word 2i+1 = (x[4i+1], x[4i+3]).
    if (tid < 16) reinterpret_cast<uint32_t*>(smem + Smem::zero(K))[tid] = 0;
    if (tid == 0) *xmax = 0;
    __syncthreads();
    const uint4* xg = reinterpret_cast<const uint4*>(x);
    uint4* xv = reinterpret_cast<uint4*>(smem + Smem::x);
    uint32_t mx = 0;
    for (int sblk = tid; sblk < K / 32; sblk += kThreads) {
      float sum = 0.f;
#pragma unroll
      for (int q = 0; q < 4; q++) {
        const uint4 v = __ldg(xg + sblk * 4 + q);
        sum += bf16lo(v.x); sum += bf16hi(v.x); sum += bf16lo(v.y); sum += bf16hi(v.y);
        sum += bf16lo(v.z); sum += bf16hi(v.z); sum += bf16lo(v.w); sum += bf16hi(v.w);
        mx = max(mx, max(max(v.x & 0x7FFFu, (v.x >> 16) & 0x7FFFu), max(v.y & 0x7FFFu, (v.y >> 16) & 0x7FFFu)));
        mx = max(mx, max(max(v.z & 0x7FFFu, (v.z >> 16) & 0x7FFFu), max(v.w & 0x7FFFu, (v.w >> 16) & 0x7FFFu)));
      }
      xs[sblk] = sum;
    }
    atomicMax(xmax, (int)mx);
    __syncthreads();
    // biased exponent of the largest |x|; keep x * 2^S below 2^126 and 2^(133-S) a normal float
    const int emax = min((*xmax >> 7) & 0xFF, 254);
    S = max(8, min(64, 252 - emax));
    const float up_even = __uint_as_float((uint32_t)(127 + S) << 23);
    const float up_odd = __uint_as_float((uint32_t)(127 + S - 4) << 23);
    for (int sblk = tid; sblk < K / 32; sblk += kThreads) {
      const float up = (sblk & 1) ? up_odd : up_even;
#pragma unroll
      for (int q = 0; q < 4; q++) {
        const uint4 v = __ldg(xg + sblk * 4 + q);   // raw words (x[4i], x[4i+1]), (x[4i+2], x[4i+3]), i = 2q, 2q+1
        __nv_bfloat162 p0 = __floats2bfloat162_rn(bf16lo(v.x) * up, bf16lo(v.y) * up);
        __nv_bfloat162 p1 = __floats2bfloat162_rn(bf16hi(v.x) * up, bf16hi(v.y) * up);
        __nv_bfloat162 p2 = __floats2bfloat162_rn(bf16lo(v.z) * up, bf16lo(v.w) * up);
        __nv_bfloat162 p3 = __floats2bfloat162_rn(bf16hi(v.z) * up, bf16hi(v.w) * up);
        xv[sblk * 4 + q] = make_uint4(*reinterpret_cast<uint32_t*>(&p0), *reinterpret_cast<uint32_t*>(&p1),
                                      *reinterpret_cast<uint32_t*>(&p2), *reinterpret_cast<uint32_t*>(&p3));
      }
    }
    __syncthreads();
  }
  const float d_up = __uint_as_float((uint32_t)(127 + 133 - S) << 23);   // 2^(133-S)
  const uint32_t x_base = smem_u32(smem + Smem::x);
  const uint32_t zero_base = smem_u32(smem + Smem::zero(K));
  const bool live = (g >> 1) == t;
  float* red = reinterpret_cast<float*>(smem + Smem::red(K));

  float out0 = 0.f, out1 = 0.f;   // rows g and g+8 of this warp's tile, this lane's share
  int flush_parity = 0;
  for (int it = 0; it < n_units; ++it) {
    // next unit's position and loads (one tile ahead)
    int rg_n = rg, c_n = c + 1;
    if (c_n == C) { c_n = 0; ++rg_n; }
    if (it + 1 < n_units) {
      const uint8_t *p0, *p1;
      tile_ptrs(rg_n, c_n, p0, p1);
      load_tile(nxt, p0, p1, t);
    }
    const int sbg = c * kSbPerUnit + j;
    if (sbg < SB) compute_tile(cur, sbg, g, t, live, x_base, zero_base, xs, d_up, out0, out1);
    cur = nxt;

    const bool last_of_rg = (c == C - 1) || (it + 1 == n_units);
    const int rg_now = rg;
    rg = rg_n; c = c_n;
    if (!last_of_rg) continue;

    // ---- flush the row group: fold lanes, fold the warps that shared a row tile, publish ----
    float v0 = out0, v1 = out1;
    v0 += __shfl_xor_sync(0xFFFFFFFFu, v0, 1); v0 += __shfl_xor_sync(0xFFFFFFFFu, v0, 2);
    v1 += __shfl_xor_sync(0xFFFFFFFFu, v1, 1); v1 += __shfl_xor_sync(0xFFFFFFFFu, v1, 2);
    float* redbuf = red + flush_parity * (kWarps * 16);
    if (t == 0) {
      redbuf[warp * 16 + g] = v0;
      redbuf[warp * 16 + g + 8] = v1;
    }
    out0 = out1 = 0.f;
    flush_parity ^= 1;
    __syncthreads();
    if (warp == 0) {
      const int tile = lane >> 4, r = lane & 15;
      float v = 0.f;
#pragma unroll
      for (int jj = 0; jj < 8; jj++) v += redbuf[(tile * 8 + jj) * 16 + r];
      const int row = rg_now * kRowsPerUnit + lane;
      const int64_t rg_first_unit = (int64_t)rg_now * C, rg_last_unit = rg_first_unit + C - 1;
      const bool complete = (u_begin <= rg_first_unit) && (u_end > rg_last_unit);
      if (complete) {
        if (row < N) store_out(y, y_dtype, row, v);
      } else {
        const int slot = (rg_now == (int)(u_begin / C)) ? 0 : 1;
        __stcg(&partials[((int64_t)b * 2 + slot) * kRowsPerUnit + lane], v);
        __threadfence();
        __syncwarp();
        const int bf = owner_of(rg_first_unit, U, G), bl = owner_of(rg_last_unit, U, G);
        int old = 0;
        if (lane == 0) old = atomicAdd(&counters[rg_now], 1);
        old = __shfl_sync(0xFFFFFFFFu, old, 0);
        if (old == bl - bf) {   // last of the bl - bf + 1 contributors
          __threadfence();
          float sum = 0.f;
          for (int bb = bf; bb <= bl; bb++) {
            const int sl = (rg_now == (int)((U * bb / G) / C)) ? 0 : 1;
            sum += __ldcg(&partials[((int64_t)bb * 2 + sl) * kRowsPerUnit + lane]);
          }
          if (row < N) store_out(y, y_dtype, row, sum);
          if (lane == 0) counters[rg_now] = 0;
        }
      }
    }
  }
}

}  // namespace q4k

bool gemv_q4k_applicable(int64_t N, int64_t K, int M, const void* w, const void* x) {
  return M == 1 && K % 256 == 0 && K <= q4k::kMaxK && N >= 1 && N < (1ll << 31) - 64 &&
         (uintptr_t)w % 16 == 0 && (uintptr_t)x % 16 == 0;
}

size_t gemv_q4k_workspace_bytes(int64_t N, int sm_count) {
  const int64_t RG = (N + q4k::kRowsPerUnit - 1) / q4k::kRowsPerUnit;
  size_t counters = ((size_t)RG * sizeof(int) + 255) / 256 * 256;
  size_t partials = (size_t)sm_count * 2 * q4k::kRowsPerUnit * sizeof(float);
  return counters + partials;
}

cudaError_t gemv_q4k(const uint8_t* w, int64_t N, int64_t K, const void* x, void* y, int y_dtype, void* ws,
                     size_t ws_bytes, int sm_count, int* status, cudaStream_t st) {
  using namespace q4k;
  (void)status;
  if (ws_bytes < gemv_q4k_workspace_bytes(N, sm_count) || !ws) return cudaErrorInvalidValue;
  const int64_t RG = (N + kRowsPerUnit - 1) / kRowsPerUnit;
  const int SB = (int)(K / 256);
  const int64_t U = RG * ((SB + kSbPerUnit - 1) / kSbPerUnit);
  const int grid = (int)(U < sm_count ? U : sm_count);
  const int smem = Smem::total((int)K);
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemv_q4k_m1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Smem::total(kMaxK));
    if (e != cudaSuccess) return e;
    attr_done[dev] = true;
  }
  int* counters = reinterpret_cast<int*>(ws);
  float* partials = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ws) + ((size_t)RG * sizeof(int) + 255) / 256 * 256);
  gemv_q4k_m1_kernel<<<grid, kThreads, smem, st>>>(w, (int)N, (int)K, (const __nv_bfloat16*)x, y, y_dtype,
                                                  counters, partials);
  return cudaPeekAtLastError();
}

}  // namespace ggq
