// Block-decode kernels: quantized bytes -> float32 / bfloat16 / float16.
//
// HBM-bound on the WRITE side (a Q4_K block is 144 bytes in, 1024 bytes of float32 out),
// so the mapping is chosen for the stores: one thread produces eight consecutive output
// elements and writes them as one (bf16/f16) or two (f32) 16-byte stores; consecutive
// threads own consecutive groups, so a warp writes 512 B / 1 KiB contiguous.  The block
// bytes come through the read-only path and are reused by the 32 threads of a superblock
// out of L1.
#include "ggq_decode.cuh"

namespace ggq {

template <int OUT> struct OutT;
template <> struct OutT<GGQ_F32> { using type = float; };
template <> struct OutT<GGQ_BF16> { using type = __nv_bfloat16; };
template <> struct OutT<GGQ_F16> { using type = __half; };

template <int OUT>
__device__ __forceinline__ void store8(void* out, int64_t group, const float* v) {
  if constexpr (OUT == GGQ_F32) {
    float4* p = reinterpret_cast<float4*>(out) + 2 * group;
    p[0] = make_float4(v[0], v[1], v[2], v[3]);
    p[1] = make_float4(v[4], v[5], v[6], v[7]);
  } else if constexpr (OUT == GGQ_BF16) {
    uint4 u;
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    __nv_bfloat162 c = __floats2bfloat162_rn(v[4], v[5]), d = __floats2bfloat162_rn(v[6], v[7]);
    u.x = *reinterpret_cast<uint32_t*>(&a); u.y = *reinterpret_cast<uint32_t*>(&b);
    u.z = *reinterpret_cast<uint32_t*>(&c); u.w = *reinterpret_cast<uint32_t*>(&d);
    reinterpret_cast<uint4*>(out)[group] = u;
  } else {
    uint4 u;
    __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
    __half2 c = __floats2half2_rn(v[4], v[5]), d = __floats2half2_rn(v[6], v[7]);
    u.x = *reinterpret_cast<uint32_t*>(&a); u.y = *reinterpret_cast<uint32_t*>(&b);
    u.z = *reinterpret_cast<uint32_t*>(&c); u.w = *reinterpret_cast<uint32_t*>(&d);
    reinterpret_cast<uint4*>(out)[group] = u;
  }
}

template <int QT, int BS, int TS, int OUT>
__global__ void __launch_bounds__(256)
dequant_kernel(const uint8_t* __restrict__ blocks, int64_t n_groups, void* __restrict__ out,
               const uint8_t* __restrict__ tab) {
  constexpr int GPB = BS / 8;  // groups of 8 elements per block
  int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= n_groups) return;
  int64_t blk = gid / GPB;
  int g = (int)(gid - blk * GPB);
  float v[8];
  Dec<QT>::run(blocks + blk * TS, g, tab, v);
  store8<OUT>(out, gid, v);
}

// F32 / F16 / BF16 "qtypes": widen (or copy) element-wise, bit-exact
// (src/gguf_jax/quants.py:125-138).
template <int QT, int OUT>
__global__ void __launch_bounds__(256)
passthrough_kernel(const uint8_t* __restrict__ in, int64_t n, void* __restrict__ out) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v;
  if constexpr (QT == QT_F32) v = __uint_as_float(ld32(in + 4 * i));
  else if constexpr (QT == QT_F16) v = h2f(ld16(in + 2 * i));
  else v = __uint_as_float(ld16(in + 2 * i) << 16);
  if constexpr (OUT == GGQ_F32) reinterpret_cast<float*>(out)[i] = v;
  else if constexpr (OUT == GGQ_BF16) reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half*>(out)[i] = __float2half_rn(v);
}

template <int QT, int OUT>
static cudaError_t launch_block(const TypeInfo* ti, const uint8_t* blocks, int64_t n_blocks, void* out,
                                const uint8_t* tab, cudaStream_t st) {
  constexpr int BS = block_elems_of(QT), TS = block_bytes_of(QT);
  if (ti->block_elems != BS || ti->block_bytes != TS) return cudaErrorInvalidValue;
  int64_t n_groups = n_blocks * (BS / 8);
  if (n_groups == 0) return cudaSuccess;
  int64_t grid = (n_groups + 255) / 256;
  dequant_kernel<QT, BS, TS, OUT><<<(unsigned)grid, 256, 0, st>>>(blocks, n_groups, out, tab);
  return cudaPeekAtLastError();
}

template <int OUT>
static cudaError_t launch_out(const TypeInfo* ti, const uint8_t* blocks, int64_t n_blocks, void* out,
                              const uint8_t* tab, cudaStream_t st) {
  int qt = ti->qtype;
  if (qt == QT_F32 || qt == QT_F16 || qt == QT_BF16) {
    if (n_blocks == 0) return cudaSuccess;
    unsigned grid = (unsigned)((n_blocks + 255) / 256);
    if (qt == QT_F32) passthrough_kernel<QT_F32, OUT><<<grid, 256, 0, st>>>(blocks, n_blocks, out);
    else if (qt == QT_F16) passthrough_kernel<QT_F16, OUT><<<grid, 256, 0, st>>>(blocks, n_blocks, out);
    else passthrough_kernel<QT_BF16, OUT><<<grid, 256, 0, st>>>(blocks, n_blocks, out);
    return cudaPeekAtLastError();
  }
  cudaError_t err = cudaErrorInvalidValue;
  dispatch_block_qtype(qt, [&]<int QT>() { err = launch_block<QT, OUT>(ti, blocks, n_blocks, out, tab, st); });
  return err;
}

}  // namespace ggq

extern "C" int32_t ggq_dequant(int32_t qtype, const void* blocks, int64_t n_blocks, void* out,
                               int32_t out_dtype, void* stream) {
  using namespace ggq;
  const TypeInfo* ti = type_info(qtype);
  if (!ti) return fail(GGQ_BAD_QTYPE, "ggq_dequant: qtype %d is not decodable", qtype);
  if (n_blocks < 0) return fail(GGQ_BAD_SHAPE, "ggq_dequant: n_blocks %lld < 0", (long long)n_blocks);
  if (n_blocks * (int64_t)(ti->block_elems >= 8 ? ti->block_elems / 8 : 1) > (int64_t)0x7FFFFFFF * 256)
    return fail(GGQ_BAD_SHAPE, "ggq_dequant: %lld blocks exceed one launch", (long long)n_blocks);
  if (n_blocks == 0) return GGQ_OK;
  if (!blocks || !out) return fail(GGQ_MISALIGNED, "ggq_dequant: null pointer");
  if ((uintptr_t)out % 16) return fail(GGQ_MISALIGNED, "ggq_dequant: out must be 16-byte aligned");
  if ((uintptr_t)blocks % block_alignment(ti))
    return fail(GGQ_MISALIGNED, "ggq_dequant: blocks must be %d-byte aligned for qtype %d", block_alignment(ti), qtype);
  int dev = 0;
  cudaGetDevice(&dev);
  const uint8_t* tab = device_tables(dev);
  if (ti->needs_tables && !tab)
    return fail(GGQ_NO_TABLES, "ggq_dequant: call ggq_set_tables(%d, ...) before decoding qtype %d", dev, qtype);
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t err;
  switch (out_dtype) {
    case GGQ_F32: err = launch_out<GGQ_F32>(ti, (const uint8_t*)blocks, n_blocks, out, tab, st); break;
    case GGQ_BF16: err = launch_out<GGQ_BF16>(ti, (const uint8_t*)blocks, n_blocks, out, tab, st); break;
    case GGQ_F16: err = launch_out<GGQ_F16>(ti, (const uint8_t*)blocks, n_blocks, out, tab, st); break;
    default: return fail(GGQ_BAD_DTYPE, "ggq_dequant: out_dtype %d", out_dtype);
  }
  if (err != cudaSuccess) return fail(GGQ_LAUNCH_FAILED, "ggq_dequant: %s", cudaGetErrorString(err));
  return GGQ_OK;
}
