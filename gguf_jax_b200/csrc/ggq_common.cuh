// Shared definitions for the sm_100a kernels behind the C ABI in include/ggq.h.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/ggq.h"

namespace ggq {

// GGMLQuantizationType values (gguf/constants.py), the qtype codes of the ABI.
enum QType : int {
  QT_F32 = 0, QT_F16 = 1, QT_Q4_0 = 2, QT_Q4_1 = 3, QT_Q5_0 = 6, QT_Q5_1 = 7, QT_Q8_0 = 8,
  QT_Q2_K = 10, QT_Q3_K = 11, QT_Q4_K = 12, QT_Q5_K = 13, QT_Q6_K = 14,
  QT_IQ2_XXS = 16, QT_IQ2_XS = 17, QT_IQ3_XXS = 18, QT_IQ1_S = 19, QT_IQ4_NL = 20,
  QT_IQ3_S = 21, QT_IQ2_S = 22, QT_IQ4_XS = 23, QT_IQ1_M = 29, QT_BF16 = 30,
  QT_TQ1_0 = 34, QT_TQ2_0 = 35, QT_MXFP4 = 39, QT_NVFP4 = 40
};

// Codebook blob layout (bytes), documented at ggq_tables_bytes in include/ggq.h.
enum TableOffsets : int {
  TAB_IQ2_XXS = 0,
  TAB_IQ2_XS = TAB_IQ2_XXS + 256 * 8,
  TAB_IQ2_S = TAB_IQ2_XS + 512 * 8,
  TAB_IQ3_XXS = TAB_IQ2_S + 1024 * 8,
  TAB_IQ3_S = TAB_IQ3_XXS + 256 * 4,
  TAB_IQ1 = TAB_IQ3_S + 512 * 4,
  TAB_KV_IQ4 = TAB_IQ1 + 2048 * 8,
  TAB_KV_MXFP4 = TAB_KV_IQ4 + 16,
  TAB_BYTES = TAB_KV_MXFP4 + 16
};

struct TypeInfo { int qtype, block_elems, block_bytes; bool needs_tables; bool fused; };

// Returns nullptr for a qtype outside the 26 decodable ones.
const TypeInfo* type_info(int qtype);

// Alignment every block of a tensor has when the tensor starts 16-byte aligned: gcd(block bytes, 16).
// The decoders load with this width, so quantized pointers handed to the ABI must honour it.
inline int block_alignment(const TypeInfo* ti) {
  int a = 16;
  while (ti->block_bytes % a) a >>= 1;
  return a;
}

// Per-device immutable state owned by the library (capi.cu).
const uint8_t* device_tables(int device);    // nullptr until ggq_set_tables(device, ...)
int* device_status_word(int device);         // allocated on first use (or by ggq_init), nullptr if that failed
int* device_status_word_if_any(int device);  // the same word if it exists already; never allocates (safe under stream capture)
int device_sm_count(int device);             // multiprocessor count, cached per device; 0 if unknown

// Thread-local error text (capi.cu).
int32_t fail(int32_t status, const char* fmt, ...);

// Bit in the device status word set when a bounded wait gave up.
constexpr int STATUS_WAIT_EXPIRED = 1;

}  // namespace ggq
