// Internal interface between the multiply kernels and the ggq_gemv / ggq_gemm entry points.
#pragma once

#include "ggq_common.cuh"

namespace ggq {

// Single rounding of a float32 result to the caller's output dtype.
__device__ __forceinline__ void store_out(void* y, int y_dtype, int64_t idx, float v) {
  if (y_dtype == GGQ_F32) reinterpret_cast<float*>(y)[idx] = v;
  else if (y_dtype == GGQ_BF16) reinterpret_cast<__nv_bfloat16*>(y)[idx] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half*>(y)[idx] = __float2half_rn(v);
}

// Coverage kernel: any block qtype, any M <= 16 (gemv_generic.cu).
cudaError_t gemv_generic(const TypeInfo* ti, const uint8_t* w, int64_t N, int64_t K, const void* x, int M,
                         void* y, int y_dtype, const uint8_t* tab, cudaStream_t st);

// Q4_K, batch 1: TMA-staged tensor-core kernel (gemv_q4k.cu).
bool gemv_q4k_applicable(int64_t N, int64_t K, int M, const void* w, const void* x);
size_t gemv_q4k_workspace_bytes(int64_t N, int sm_count);
cudaError_t gemv_q4k(const uint8_t* w, int64_t N, int64_t K, const void* x, void* y, int y_dtype, void* ws,
                     size_t ws_bytes, int sm_count, int* status, cudaStream_t st);

// Same kernel with the scratch in a file-scope device array (no caller buffer); returns a ggq_status.
int32_t gemv_q4k_static(const void* w, int64_t N, int64_t K, const void* x, void* y, int32_t y_dtype,
                        int sm_count, cudaStream_t st);

// Any block qtype, M <= 16, K a multiple of 32: tensor-core kernel with exact three-way bf16 split
// of the decoded weights (gemv_mma.cu).
bool gemv_mma_applicable(const TypeInfo* ti, int64_t N, int64_t K, int M);
cudaError_t gemv_mma(const TypeInfo* ti, const uint8_t* w, int64_t N, int64_t K, const void* x, int M, void* y,
                     int y_dtype, const uint8_t* tab, cudaStream_t st);

// Larger batches: tcgen05 / TMEM tensor-core kernel with tf32 operands (gemm_tcgen05.cu).
bool gemm_applicable(const TypeInfo* ti, int64_t N, int64_t K, int M);
cudaError_t gemm_tf32(const TypeInfo* ti, const uint8_t* w, int64_t N, int64_t K, const void* x, int M, void* y,
                      int y_dtype, const uint8_t* tab, int* status, cudaStream_t st);

// Upper bound on the SM count used when sizing scratch (the kernels use the real count).
constexpr int kMaxSmCount = 256;

}  // namespace ggq
