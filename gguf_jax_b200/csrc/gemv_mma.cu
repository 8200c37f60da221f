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
  cudaError_t err = cudaErrorInvalidValue;
  dispatch_block_qtype(ti->qtype, [&]<int QT>() { err = mmav::launch<QT>(w, N, K, x, M, y, y_dtype, tab, st); });
  return err;
}

}  // namespace ggq
