// Batch-1 fused decode + multiply for every block qtype without a tuned kernel of its own.
//
// One warp per output row.  The row's raw block bytes are streamed through a small private ring in
// shared memory with 16-byte cp.async copies, three chunks of 256 weights ahead of the one being
// decoded, so that HBM latency is covered by copies in flight instead of by one dependent load
// per lane and step (which is what bounds gemv_generic.cu).  Rows of a GGUF tensor have no
// alignment beyond their block size, so a copy takes the 16-byte aligned window around the
// chunk and the decoder reads at the chunk's offset inside it (the address modulo 16 is the same
// as in global memory, which is all the decoders' alignment assumptions need).  Each lane then
// decodes eight consecutive weights with the shared bit-exact decode8 routines, multiplies them
// with the matching activations in float32, and a butterfly shuffle folds the lanes.
#define GGQ_DECODE_GENERIC_LOADS   // the decoders read staged blocks from shared memory
#include "ggq_decode.cuh"
#include "gemv.cuh"

namespace ggq {
namespace stream {

constexpr int kWarps = 8;
constexpr int kDepth = 4;
constexpr int kChunk = 256;

template <int QT> constexpr int raw_bytes() { return kChunk / block_elems_of(QT) * block_bytes_of(QT); }
template <int QT> constexpr int pitch() { return (raw_bytes<QT>() + 30) / 16 * 16; }

__device__ __forceinline__ void cp_async16(uint32_t dst, const uint8_t* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

template <int QT>
__global__ void __launch_bounds__(kWarps * 32)
gemv_stream_kernel(const uint8_t* __restrict__ w, int64_t N, int K, const __nv_bfloat16* __restrict__ x,
                   void* __restrict__ y, int y_dtype, const uint8_t* __restrict__ tab) {
  constexpr int BS = block_elems_of(QT), TS = block_bytes_of(QT), RB = raw_bytes<QT>(), PITCH = pitch<QT>();
  __shared__ __align__(16) uint8_t ring[kWarps][kDepth][PITCH];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t row = (int64_t)blockIdx.x * kWarps + warp;
  if (row >= N) return;
  const int n_chunks = K / kChunk;
  const uint8_t* wrow = w + row * (int64_t)(K / BS) * TS;
  // reads stop at the 16-byte boundary at or after the end of the tensor
  const uint8_t* const w_stop = w + ((N * (int64_t)(K / BS) * TS + 15) & ~(int64_t)15);
  const uint32_t my_ring = (uint32_t)__cvta_generic_to_shared(&ring[warp][0][0]);

  auto issue = [&](int c) {
    if (c < n_chunks) {
      const uint8_t* p = wrow + (int64_t)c * RB;
      const int skew = (int)((uintptr_t)p & 15);
      const uint8_t* src = p - skew + 16 * lane;
      if (16 * lane < skew + RB && src + 16 <= w_stop) cp_async16(my_ring + (c % kDepth) * PITCH + 16 * lane, src);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
#pragma unroll
  for (int d = 0; d < kDepth - 1; d++) issue(d);

  // lane l owns weights 8l .. 8l+7 of every chunk
  constexpr int kBlockOfLane_den = BS / 8;               // groups of eight per block
  const int blk_in_chunk = lane / kBlockOfLane_den, grp = lane % kBlockOfLane_den;
  const uint4* xv = reinterpret_cast<const uint4*>(x) + lane;
  float acc = 0.f;
  for (int c = 0; c < n_chunks; c++) {
    issue(c + kDepth - 1);
    asm volatile("cp.async.wait_group %0;" ::"n"(kDepth - 1) : "memory");
    __syncwarp();
    const uint4 u = __ldg(xv + (int64_t)c * (kChunk / 8));
    const int skew = (int)((uintptr_t)(wrow + (int64_t)c * RB) & 15);
    float wv[8];
    Dec<QT>::run(&ring[warp][c % kDepth][skew + blk_in_chunk * TS], grp, tab, wv);
    acc = fmaf(wv[0], __uint_as_float(u.x << 16), acc);
    acc = fmaf(wv[1], __uint_as_float(u.x & 0xFFFF0000u), acc);
    acc = fmaf(wv[2], __uint_as_float(u.y << 16), acc);
    acc = fmaf(wv[3], __uint_as_float(u.y & 0xFFFF0000u), acc);
    acc = fmaf(wv[4], __uint_as_float(u.z << 16), acc);
    acc = fmaf(wv[5], __uint_as_float(u.z & 0xFFFF0000u), acc);
    acc = fmaf(wv[6], __uint_as_float(u.w << 16), acc);
    acc = fmaf(wv[7], __uint_as_float(u.w & 0xFFFF0000u), acc);
    __syncwarp();   // every lane is done with the slot before a later copy overwrites it
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
  if (lane == 0) store_out(y, y_dtype, row, acc);
}

}  // namespace stream

bool gemv_stream_applicable(const TypeInfo* ti, int64_t N, int64_t K, int M, const void* w, const void* x) {
  return ti && M == 1 && K % stream::kChunk == 0 && K < (1ll << 31) && N >= 1 && (uintptr_t)w % 16 == 0 &&
         (uintptr_t)x % 16 == 0;
}

cudaError_t gemv_stream(const TypeInfo* ti, const uint8_t* w, int64_t N, int64_t K, const void* x, void* y,
                        int y_dtype, const uint8_t* tab, cudaStream_t st) {
  cudaError_t err = cudaErrorInvalidValue;
  dispatch_block_qtype(ti->qtype, [&]<int QT>() {
    const unsigned grid = (unsigned)((N + stream::kWarps - 1) / stream::kWarps);
    stream::gemv_stream_kernel<QT><<<grid, stream::kWarps * 32, 0, st>>>(w, N, (int)K, (const __nv_bfloat16*)x, y,
                                                                        y_dtype, tab);
    err = cudaPeekAtLastError();
  });
  return err;
}

}  // namespace ggq
