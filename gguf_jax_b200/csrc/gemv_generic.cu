// Generic fused decode + multiply for small batches: every block qtype, any K that is a
// multiple of the block, no alignment requirement on rows.
//
// One warp per output row.  Lane l decodes groups of eight consecutive weights with the
// same decode8 routines the decode kernel uses (so the weights are the bit-exact float32
// values), multiplies them with the matching eight activations of each batch row and
// accumulates in float32; a butterfly shuffle folds the 32 lanes.  This is the coverage
// kernel: the tuned per-qtype kernels (gemv_q4k.cu ...) take over where they apply.
#include "ggq_decode.cuh"
#include "gemv.cuh"

namespace ggq {

__device__ __forceinline__ void bf16x8_to_f32(const uint4& u, float* f) {
  f[0] = __uint_as_float(u.x << 16); f[1] = __uint_as_float(u.x & 0xFFFF0000u);
  f[2] = __uint_as_float(u.y << 16); f[3] = __uint_as_float(u.y & 0xFFFF0000u);
  f[4] = __uint_as_float(u.z << 16); f[5] = __uint_as_float(u.z & 0xFFFF0000u);
  f[6] = __uint_as_float(u.w << 16); f[7] = __uint_as_float(u.w & 0xFFFF0000u);
}

template <int QT, int BS, int TS, int MB>
__global__ void __launch_bounds__(256)
gemv_generic_kernel(const uint8_t* __restrict__ w, int64_t N, int64_t K, const __nv_bfloat16* __restrict__ x,
                    int M, void* __restrict__ y, int y_dtype, const uint8_t* __restrict__ tab) {
  constexpr int GPB = BS / 8;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t row = (int64_t)blockIdx.x * 8 + warp;
  if (row >= N) return;
  const int64_t n_groups = K / 8;
  const uint8_t* wrow = w + row * (K / BS) * TS;
  float acc[MB];
#pragma unroll
  for (int m = 0; m < MB; m++) acc[m] = 0.f;
  for (int64_t grp = lane; grp < n_groups; grp += 32) {
    int64_t blk = grp / GPB;
    int g = (int)(grp - blk * GPB);
    float wv[8];
    Dec<QT>::run(wrow + blk * TS, g, tab, wv);
#pragma unroll
    for (int m = 0; m < MB; m++) {
      if (m < M) {
        uint4 u = __ldg(reinterpret_cast<const uint4*>(x + (int64_t)m * K) + grp);
        float xv[8];
        bf16x8_to_f32(u, xv);
        float s = acc[m];
#pragma unroll
        for (int i = 0; i < 8; i++) s = fmaf(wv[i], xv[i], s);
        acc[m] = s;
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MB; m++) {
    float v = acc[m];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    if (lane == 0 && m < M) store_out(y, y_dtype, (int64_t)m * N + row, v);
  }
}

template <int QT, int BS, int TS>
static cudaError_t launch_generic(const uint8_t* w, int64_t N, int64_t K, const void* x, int M, void* y,
                                  int y_dtype, const uint8_t* tab, cudaStream_t st) {
  unsigned grid = (unsigned)((N + 7) / 8);
  const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
  if (M <= 1) gemv_generic_kernel<QT, BS, TS, 1><<<grid, 256, 0, st>>>(w, N, K, xb, M, y, y_dtype, tab);
  else if (M <= 2) gemv_generic_kernel<QT, BS, TS, 2><<<grid, 256, 0, st>>>(w, N, K, xb, M, y, y_dtype, tab);
  else if (M <= 4) gemv_generic_kernel<QT, BS, TS, 4><<<grid, 256, 0, st>>>(w, N, K, xb, M, y, y_dtype, tab);
  else if (M <= 8) gemv_generic_kernel<QT, BS, TS, 8><<<grid, 256, 0, st>>>(w, N, K, xb, M, y, y_dtype, tab);
  else gemv_generic_kernel<QT, BS, TS, 16><<<grid, 256, 0, st>>>(w, N, K, xb, M, y, y_dtype, tab);
  return cudaPeekAtLastError();
}

cudaError_t gemv_generic(const TypeInfo* ti, const uint8_t* w, int64_t N, int64_t K, const void* x, int M,
                         void* y, int y_dtype, const uint8_t* tab, cudaStream_t st) {
  cudaError_t err = cudaErrorInvalidValue;
  dispatch_block_qtype(ti->qtype, [&]<int QT>() {
    err = launch_generic<QT, block_elems_of(QT), block_bytes_of(QT)>(w, N, K, x, M, y, y_dtype, tab, st);
  });
  return err;
}

}  // namespace ggq
