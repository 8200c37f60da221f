// Q4_K fused decode + multiply for batch 1, tuned for B200 HBM bandwidth.
//
// Data movement.  A persistent CTA per SM streams the weight through a shared-memory ring
// with 1-D TMA bulk copies (cp.async.bulk, one per weight row per stage, completion on an
// mbarrier).  A stage holds 32 rows x 8 superblocks (36 KB); four stages give ~150 KB of
// loads in flight per SM, which is what it takes to cover HBM latency at 6-8 TB/s.  One
// producer warp issues the copies; sixteen consumer warps decode and multiply.
//
// Arithmetic.  Per-element FMAs cannot keep up with HBM on this part (about 2.5 issued
// lane-instructions per weight at peak bandwidth), so the dot products run on the tensor
// cores with *exact integer* weights: each 4-bit code q is turned into the bf16 value
// 128 + q by OR-ing it into the mantissa of 0x4300 (one byte-permute per two codes), and
// mma.sync.m16n8k16 multiplies 16 rows x 16 codes by the bf16 activations with float32
// accumulation.  The accumulator starts at -128 * sum(x) of the sub-block, which removes
// the bias, so it ends at u = sum(q * x) exactly as float32 sums of exact products.
// The float32 scales are applied to the accumulators, not to the weights:
//     y += (d * sc) * u - (dmin * mn) * sum(x)
// so a weight never loses precision (a one-hot x returns bf16(float32 weight) exactly).
//
// The eight columns of the MMA's B operand are used as eight *sub-block channels*: lane
// group t of the warp holds the 32 bytes [32t, 32t+32) of a superblock's quants, i.e. the
// sub-block pair (2t, 2t+1); column c of B carries the activations of sub-block c in the
// k-slots of lane group c/2 and zeros elsewhere.  One accumulator tile therefore collects
// all eight sub-block sums of 16 rows, and lane (g, t) ends up holding exactly the sums
// whose scales it unpacks: rows g and g+8, sub-blocks 2t and 2t+1.
//
// Work split.  Units of (32-row group, 8-superblock chunk) are dealt to the CTAs as
// contiguous ranges of equal length, so every SM streams the same number of bytes.  A row
// group cut by a range boundary is finished by whichever CTA arrives last: partial sums go
// to a small scratch buffer, a per-row-group counter tells the last arriver, which adds the
// partials in CTA order (deterministic) and leaves the counter at zero again.
#include "gemv.cuh"

namespace ggq {
namespace q4k {

constexpr int kBlockBytes = 144;
constexpr int kConsumerWarps = 16;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kRowsPerStage = 32;
constexpr int kSbPerStage = 8;
constexpr int kRowPitch = kSbPerStage * kBlockBytes + 16;  // 1168: == 16 (mod 128), conflict-free LDS.128
constexpr int kStageBytes = kRowsPerStage * kRowPitch;      // 37376
constexpr int kStages = 4;
constexpr int kMaxK = 28672;                                // activations stay resident in shared memory
constexpr uint32_t kSpinLimit = 1u << 22;

struct Smem {
  // offsets into dynamic shared memory
  static constexpr int ring = 0;
  static constexpr int x = ring + kStages * kStageBytes;          // bf16[K]
  static __host__ __device__ constexpr int xs(int K) { return x + 2 * K; }             // float4[K/64]
  static __host__ __device__ constexpr int zero(int K) { return xs(K) + (K / 256) * 64; }  // 64 zero bytes
  static __host__ __device__ constexpr int red(int K) { return zero(K) + 64; }         // float[2][16 warps][16]
  static __host__ __device__ constexpr int bars(int K) { return red(K) + 2 * kConsumerWarps * 16 * 4; }
  static __host__ __device__ constexpr int flags(int K) { return bars(K) + 8 * (2 * kStages + 1); }
  static __host__ __device__ constexpr int total(int K) { return flags(K) + 16; }
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
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
// Bounded wait: gives up after kSpinLimit probes, raises the abort flag and the device
// status word, and lets the caller run on (the results are then garbage, the host sees
// GGQ_TIMEOUT through ggq_read_status).  Never spins forever.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status) {
  if (*abort_flag) return;
  for (uint32_t i = 0; i < kSpinLimit; i++) {
    if (mbar_try_wait(bar, parity)) return;
    if ((i & 1023) == 1023 && *abort_flag) return;
  }
  *abort_flag = 1;
  if (status) atomicOr(status, STATUS_WAIT_EXPIRED);
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void consumer_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
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
__device__ __forceinline__ void pair_scales(const uint4& h, int t, float& dl_a, float& dm_a, float& dl_b, float& dm_b) {
  const __half2 dd = *reinterpret_cast<const __half2*>(&h.x);
  const float d = __low2float(dd), dmin = __high2float(dd);
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

__global__ void __launch_bounds__(kThreads, 1)
gemv_q4k_m1_kernel(const uint8_t* __restrict__ w, int N, int K, const __nv_bfloat16* __restrict__ x,
                   void* __restrict__ y, int y_dtype, int* __restrict__ counters, float* __restrict__ partials,
                   int* __restrict__ status) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int SB = K / 256;                        // superblocks per row
  const int64_t row_bytes = (int64_t)SB * kBlockBytes;
  const int C = (SB + kSbPerStage - 1) / kSbPerStage;   // chunks per row group
  const int RG = (N + kRowsPerStage - 1) / kRowsPerStage;
  const int64_t U = (int64_t)RG * C;
  const int G = gridDim.x, b = blockIdx.x;
  const int64_t u_begin = U * b / G, u_end = U * (b + 1) / G;

  const uint32_t ring = smem_u32(smem + Smem::ring);
  const uint32_t bars = smem_u32(smem + Smem::bars(K));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Smem::flags(K));
  auto full_bar = [&](int s) { return bars + 8 * s; };
  auto empty_bar = [&](int s) { return bars + 8 * (kStages + s); };
  const uint32_t x_bar = bars + 8 * (2 * kStages);

  if (tid == 0) {
    for (int s = 0; s < kStages; s++) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), kConsumerWarps);
    }
    mbar_init(x_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  if (warp == kConsumerWarps) {
    // ------------------------------ producer warp ------------------------------
    if (lane == 0) {
      mbar_expect_tx(x_bar, 2u * K);
      bulk_g2s(smem_u32(smem + Smem::x), x, 2u * K, x_bar);
    }
    int it = 0;
    for (int64_t u = u_begin; u < u_end; ++u, ++it) {
      const int s = it % kStages, k = it / kStages;
      if (k > 0) mbar_wait(empty_bar(s), (k - 1) & 1, abort_flag, status);
      if (*abort_flag) break;
      const int rg = (int)(u / C), c = (int)(u - (int64_t)rg * C);
      const int nsb = min(kSbPerStage, SB - c * kSbPerStage);
      const int rows_valid = min(kRowsPerStage, N - rg * kRowsPerStage);
      const uint32_t bytes_row = (uint32_t)nsb * kBlockBytes;
      if (lane == 0) mbar_expect_tx(full_bar(s), bytes_row * rows_valid);
      __syncwarp();
      if (lane < rows_valid) {
        const uint8_t* src = w + ((int64_t)rg * kRowsPerStage + lane) * row_bytes + (int64_t)c * kSbPerStage * kBlockBytes;
        bulk_g2s(ring + s * kStageBytes + lane * kRowPitch, src, bytes_row, full_bar(s));
      }
    }
    return;
  }

  // -------------------------------- consumer warps --------------------------------
  const int g = lane >> 2, t = lane & 3;
  const int rt = warp >> 3, j = warp & 7;        // row tile (16 rows) and superblock slot of this warp
  float* xs = reinterpret_cast<float*>(smem + Smem::xs(K));
  {
    // zero page + per-sub-block activation sums {X, -128 X}, once per CTA
    if (tid < 16) reinterpret_cast<uint32_t*>(smem + Smem::zero(K))[tid] = 0;
    mbar_wait(x_bar, 0, abort_flag, status);
    const uint4* xv = reinterpret_cast<const uint4*>(smem + Smem::x);
    for (int sblk = tid; sblk < K / 32; sblk += kConsumerWarps * 32) {
      float sum = 0.f;
#pragma unroll
      for (int q = 0; q < 4; q++) {
        uint4 v = xv[sblk * 4 + q];
        sum += bf16lo(v.x); sum += bf16hi(v.x); sum += bf16lo(v.y); sum += bf16hi(v.y);
        sum += bf16lo(v.z); sum += bf16hi(v.z); sum += bf16lo(v.w); sum += bf16hi(v.w);
      }
      xs[2 * sblk] = sum;
      xs[2 * sblk + 1] = -128.0f * sum;
    }
    consumer_sync();
  }
  const uint32_t xs_base = smem_u32(xs);
  const uint32_t x_base = smem_u32(smem + Smem::x);
  const uint32_t zero_base = smem_u32(smem + Smem::zero(K));
  const bool act_lo = (g == 2 * t), act_hi = (g == 2 * t + 1);
  float* red = reinterpret_cast<float*>(smem + Smem::red(K));

  float out0 = 0.f, out1 = 0.f;   // rows g and g+8 of this warp's tile, this lane's share
  int flush_parity = 0;
  int it = 0;
  for (int64_t u = u_begin; u < u_end; ++u, ++it) {
    const int s = it % kStages, k = it / kStages;
    const int rg = (int)(u / C), c = (int)(u - (int64_t)rg * C);
    mbar_wait(full_bar(s), k & 1, abort_flag, status);
    const int sbg = c * kSbPerStage + j;         // superblock index within the row
    if (sbg < SB) {
      const uint32_t base0 = ring + s * kStageBytes + (16 * rt + g) * kRowPitch + j * kBlockBytes;
      const uint32_t base1 = base0 + 8 * kRowPitch;
      const uint4 h0 = lds128(base0), h1 = lds128(base1);
      const uint4 qa0 = lds128(base0 + 16 + 32 * t), qb0 = lds128(base0 + 32 + 32 * t);
      const uint4 qa1 = lds128(base1 + 16 + 32 * t), qb1 = lds128(base1 + 32 + 32 * t);
      // activations of sub-block g (natural order), only in the pass where this lane's column is live
      const uint32_t xsub = x_base + (uint32_t)(sbg * 8 + g) * 64;
      const uint32_t xl = act_lo ? xsub : zero_base, xh = act_hi ? xsub : zero_base;
      const uint4 xl0 = lds128(xl), xl1 = lds128(xl + 16), xl2 = lds128(xl + 32), xl3 = lds128(xl + 48);
      const uint4 xh0 = lds128(xh), xh1 = lds128(xh + 16), xh2 = lds128(xh + 32), xh3 = lds128(xh + 48);
      const uint4 sx = lds128(xs_base + (uint32_t)(sbg * 4 + t) * 16);  // X[2t], -128X[2t], X[2t+1], -128X[2t+1]
      const float Xa = __uint_as_float(sx.x), nXa = __uint_as_float(sx.y);
      const float Xb = __uint_as_float(sx.z), nXb = __uint_as_float(sx.w);

      float acc[4] = {nXa, nXb, nXa, nXb};
      const uint32_t w0[8] = {qa0.x, qa0.y, qa0.z, qa0.w, qb0.x, qb0.y, qb0.z, qb0.w};
      const uint32_t w1[8] = {qa1.x, qa1.y, qa1.z, qa1.w, qb1.x, qb1.y, qb1.z, qb1.w};
      const uint32_t xlo[16] = {xl0.x, xl0.y, xl0.z, xl0.w, xl1.x, xl1.y, xl1.z, xl1.w,
                                xl2.x, xl2.y, xl2.z, xl2.w, xl3.x, xl3.y, xl3.z, xl3.w};
      const uint32_t xhi[16] = {xh0.x, xh0.y, xh0.z, xh0.w, xh1.x, xh1.y, xh1.z, xh1.w,
                                xh2.x, xh2.y, xh2.z, xh2.w, xh3.x, xh3.y, xh3.z, xh3.w};
#pragma unroll
      for (int i = 0; i < 8; i++) {
        // word i = bytes 4i..4i+3 of the lane's run = elements 4i..4i+3 of sub-blocks 2t (low
        // nibbles) and 2t+1 (high nibbles)
        const uint32_t l0 = w0[i] & 0x0F0F0F0Fu, h0n = (w0[i] >> 4) & 0x0F0F0F0Fu;
        const uint32_t l1 = w1[i] & 0x0F0F0F0Fu, h1n = (w1[i] >> 4) & 0x0F0F0F0Fu;
        // bf16 pairs 0x4300|q = 128 + q: elements (4i, 4i+1) -> k-slots 2t, 2t+1; (4i+2, 4i+3) -> 2t+8, 2t+9
        mma16816(acc, __byte_perm(l0, 0x43434343u, 0x4140), __byte_perm(l1, 0x43434343u, 0x4140),
                 __byte_perm(l0, 0x43434343u, 0x4342), __byte_perm(l1, 0x43434343u, 0x4342),
                 xlo[2 * i], xlo[2 * i + 1]);
        mma16816(acc, __byte_perm(h0n, 0x43434343u, 0x4140), __byte_perm(h1n, 0x43434343u, 0x4140),
                 __byte_perm(h0n, 0x43434343u, 0x4342), __byte_perm(h1n, 0x43434343u, 0x4342),
                 xhi[2 * i], xhi[2 * i + 1]);
      }
      float dla, dma, dlb, dmb;
      pair_scales(h0, t, dla, dma, dlb, dmb);
      out0 = fmaf(dla, acc[0], out0); out0 = fmaf(-dma, Xa, out0);
      out0 = fmaf(dlb, acc[1], out0); out0 = fmaf(-dmb, Xb, out0);
      pair_scales(h1, t, dla, dma, dlb, dmb);
      out1 = fmaf(dla, acc[2], out1); out1 = fmaf(-dma, Xa, out1);
      out1 = fmaf(dlb, acc[3], out1); out1 = fmaf(-dmb, Xb, out1);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_bar(s));

    const bool last_of_rg = (c == C - 1) || (u + 1 == u_end);
    if (!last_of_rg) continue;

    // ---- flush the row group: fold lanes, fold the warps that shared a row tile, publish ----
    float v0 = out0, v1 = out1;
    v0 += __shfl_xor_sync(0xFFFFFFFFu, v0, 1); v0 += __shfl_xor_sync(0xFFFFFFFFu, v0, 2);
    v1 += __shfl_xor_sync(0xFFFFFFFFu, v1, 1); v1 += __shfl_xor_sync(0xFFFFFFFFu, v1, 2);
    float* redbuf = red + flush_parity * (kConsumerWarps * 16);
    if (t == 0) {
      redbuf[warp * 16 + g] = v0;
      redbuf[warp * 16 + g + 8] = v1;
    }
    out0 = out1 = 0.f;
    flush_parity ^= 1;
    consumer_sync();
    if (warp == 0) {
      const int tile = lane >> 4, r = lane & 15;
      float v = 0.f;
#pragma unroll
      for (int jj = 0; jj < 8; jj++) v += redbuf[(tile * 8 + jj) * 16 + r];
      const int row = rg * kRowsPerStage + lane;
      const int64_t rg_first_unit = (int64_t)rg * C, rg_last_unit = rg_first_unit + C - 1;
      const bool complete = (u_begin <= rg_first_unit) && (u_end > rg_last_unit);
      if (complete) {
        if (row < N) store_out(y, y_dtype, row, v);
      } else {
        const int slot = (rg == (int)(u_begin / C)) ? 0 : 1;
        __stcg(&partials[((int64_t)b * 2 + slot) * kRowsPerStage + lane], v);
        __threadfence();
        __syncwarp();
        const int bf = owner_of(rg_first_unit, U, G), bl = owner_of(rg_last_unit, U, G);
        int old = 0;
        if (lane == 0) old = atomicAdd(&counters[rg], 1);
        old = __shfl_sync(0xFFFFFFFFu, old, 0);
        if (old == bl - bf) {   // last of the bl - bf + 1 contributors
          __threadfence();
          float sum = 0.f;
          for (int bb = bf; bb <= bl; bb++) {
            const int sl = (rg == (int)((U * bb / G) / C)) ? 0 : 1;
            sum += __ldcg(&partials[((int64_t)bb * 2 + sl) * kRowsPerStage + lane]);
          }
          if (row < N) store_out(y, y_dtype, row, sum);
          if (lane == 0) counters[rg] = 0;
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
  const int64_t RG = (N + q4k::kRowsPerStage - 1) / q4k::kRowsPerStage;
  size_t counters = ((size_t)RG * sizeof(int) + 255) / 256 * 256;
  size_t partials = (size_t)sm_count * 2 * q4k::kRowsPerStage * sizeof(float);
  return counters + partials;
}

cudaError_t gemv_q4k(const uint8_t* w, int64_t N, int64_t K, const void* x, void* y, int y_dtype, void* ws,
                     size_t ws_bytes, int sm_count, int* status, cudaStream_t st) {
  using namespace q4k;
  if (ws_bytes < gemv_q4k_workspace_bytes(N, sm_count) || !ws) return cudaErrorInvalidValue;
  const int64_t RG = (N + kRowsPerStage - 1) / kRowsPerStage;
  const int SB = (int)(K / 256);
  const int64_t U = RG * ((SB + kSbPerStage - 1) / kSbPerStage);
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
                                                  counters, partials, status);
  return cudaPeekAtLastError();
}

}  // namespace ggq
