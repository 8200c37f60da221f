// Per-qtype block decoders: decode8<QT>(block, g, tables, out) writes the eight
// consecutive elements 8g .. 8g+7 of one block as float32.
//
// The arithmetic is the float32 arithmetic of gguf.quants / gguf-jax
// (src/gguf_jax/quants.py:125-712) in the same association, written with __fmul_rn /
// __fadd_rn / __fsub_rn so the compiler can neither contract nor reassociate it.  Every
// product is exact in float32 (f16 scale x small integer), so the only rounding is the
// final add/sub of Q4_1, Q5_1, Q2_K, Q4_K and Q5_K -- which is why the result is
// bit-identical to the numpy decode.  No flush-to-zero: MXFP4 scales below 2^-126 are
// float32 subnormals.
//
// Blocks are read byte-wise: most block sizes (17, 18, 22, 34, 50, 66, 110, 210 ...) give
// no alignment beyond one or two bytes.
#pragma once

#include "ggq_common.cuh"

// Where the block bytes live.  By default they are read from global memory through the
// read-only path (__ldg).  A translation unit that stages raw blocks in shared memory first
// (gemm_tcgen05.cu) defines GGQ_DECODE_GENERIC_LOADS before including this header and gets the
// same decoders with plain generic loads, which work on shared and global addresses alike.
// The two flavours live in different inline namespaces, so they are different entities.
#ifdef GGQ_DECODE_GENERIC_LOADS
#define GGQ_LD(p) (*(p))
#define GGQ_DEC_NS dec_generic_loads
#else
#define GGQ_LD(p) __ldg(p)
#define GGQ_DEC_NS dec_global_loads
#endif

namespace ggq {
inline namespace GGQ_DEC_NS {

__device__ __forceinline__ uint32_t ldb(const uint8_t* p) { return GGQ_LD(p); }
__device__ __forceinline__ uint32_t ld16(const uint8_t* p) { return ldb(p) | (ldb(p + 1) << 8); }
__device__ __forceinline__ uint32_t ld32(const uint8_t* p) {
  return ldb(p) | (ldb(p + 1) << 8) | (ldb(p + 2) << 16) | (ldb(p + 3) << 24);
}
// Eight consecutive block bytes as two little-endian words, with loads as wide as the block's
// alignment allows.  ALIGN is the guaranteed alignment of p: a tensor starts 16-byte aligned and
// every block starts a multiple of its size further on, so ALIGN = gcd(block bytes, 16) combined
// with the (even) offset inside the block.
template <int ALIGN>
__device__ __forceinline__ uint2 ld8(const uint8_t* p) {
  if constexpr (ALIGN >= 8) {
    return GGQ_LD(reinterpret_cast<const uint2*>(p));
  } else if constexpr (ALIGN >= 4) {
    const uint32_t* q = reinterpret_cast<const uint32_t*>(p);
    return make_uint2(GGQ_LD(q), GGQ_LD(q + 1));
  } else if constexpr (ALIGN >= 2) {
    const unsigned short* q = reinterpret_cast<const unsigned short*>(p);
    return make_uint2((uint32_t)GGQ_LD(q) | ((uint32_t)GGQ_LD(q + 1) << 16),
                      (uint32_t)GGQ_LD(q + 2) | ((uint32_t)GGQ_LD(q + 3) << 16));
  } else {
    return make_uint2(ld32(p), ld32(p + 4));
  }
}
__device__ __forceinline__ uint32_t byte_of(const uint2& v, int i) { return ((i < 4 ? v.x : v.y) >> (8 * (i & 3))) & 0xFF; }

// IEEE half bits -> float (exact; cvt.f32.f16 keeps subnormals).
__device__ __forceinline__ float h2f(uint32_t bits) {
  return __half2float(__ushort_as_half((unsigned short)bits));
}
__device__ __forceinline__ float i2f(int v) { return (float)v; }
// ksigns[i] = i | parity(i) << 7 (gguf/quants.py IQ2_XXS.ksigns).
__device__ __forceinline__ uint32_t ksign(uint32_t i) { return i | ((__popc(i) & 1) << 7); }
__device__ __forceinline__ float sgnf(uint32_t signs, int j) { return ((signs >> j) & 1) ? -1.0f : 1.0f; }

// 6-bit (scale, min) of sub-block k in the 12 packed bytes of Q4_K / Q5_K
// (src/gguf_jax/quants.py:275-283).
__device__ __forceinline__ void scale_min_k4(const uint8_t* s, int k, int& sc, int& mn) {
  if (k < 4) {
    sc = ldb(s + k) & 63;
    mn = ldb(s + 4 + k) & 63;
  } else {
    uint32_t md = ldb(s + 4 + k);
    sc = (md & 15) | ((ldb(s + k - 4) >> 6) << 4);
    mn = (md >> 4) | ((ldb(s + k) >> 6) << 4);
  }
}

// Compile-time block geometry (elements, bytes) of the block qtypes.
constexpr int block_elems_of(int qt) {
  return (qt == QT_Q4_0 || qt == QT_Q4_1 || qt == QT_Q5_0 || qt == QT_Q5_1 || qt == QT_Q8_0 ||
          qt == QT_IQ4_NL || qt == QT_MXFP4) ? 32 : (qt == QT_NVFP4 ? 64 : 256);
}
constexpr int block_bytes_of(int qt) {
  return qt == QT_Q4_0 ? 18 : qt == QT_Q4_1 ? 20 : qt == QT_Q5_0 ? 22 : qt == QT_Q5_1 ? 24 : qt == QT_Q8_0 ? 34 :
         qt == QT_Q2_K ? 84 : qt == QT_Q3_K ? 110 : qt == QT_Q4_K ? 144 : qt == QT_Q5_K ? 176 : qt == QT_Q6_K ? 210 :
         qt == QT_IQ2_XXS ? 66 : qt == QT_IQ2_XS ? 74 : qt == QT_IQ3_XXS ? 98 : qt == QT_IQ1_S ? 50 :
         qt == QT_IQ4_NL ? 18 : qt == QT_IQ3_S ? 110 : qt == QT_IQ2_S ? 82 : qt == QT_IQ4_XS ? 136 :
         qt == QT_IQ1_M ? 56 : qt == QT_TQ1_0 ? 54 : qt == QT_TQ2_0 ? 66 : qt == QT_MXFP4 ? 17 : 36;
}

template <int QT>
struct Dec;  // Dec<QT>::run(block, g, tables, out[8])

// ---- legacy 32-element blocks ------------------------------------------------------
// nibble order: elements 0-15 = low nibbles of qs[0..15], 16-31 = high nibbles.
template <> struct Dec<QT_Q4_0> {
  __device__ static void run(const uint8_t* b, int g, const uint8_t*, float* o) {
    float d = h2f(ld16(b));
    const uint8_t* qs = b + 2 + 8 * (g & 1);
    int sh = 4 * (g >> 1);
#pragma unroll
    for (int i = 0; i < 8; i++) o[i] = __fmul_rn(d, i2f((int)((ldb(qs + i) >> sh) & 15) - 8));
  }
};
template <> struct Dec<QT_Q4_1> {
  __device__ static void run(const uint8_t* b, int g, const uint8_t*, float* o) {
    float d = h2f(ld16(b)), m = h2f(ld16(b + 2));
    const uint8_t* qs = b + 4 + 8 * (g & 1);
    int sh = 4 * (g >> 1);
#pragma unroll
    for (int i = 0; i < 8; i++) o[i] = __fadd_rn(__fmul_rn(d, i2f((ldb(qs + i) >> sh) & 15)), m);
  }
};
template <> struct Dec<QT_Q5_0> {
  __device__ static void run(const uint8_t* b, int g, const uint8_t*, float* o) {
    float d = h2f(ld16(b));
    uint32_t qh = ld32(b + 2) >> (8 * g);
    const uint8_t* qs = b + 6 + 8 * (g & 1);
    int sh = 4 * (g >> 1);
#pragma unroll
    for (int i = 0; i < 8; i++) {
      int q = ((ldb(qs + i) >> sh) & 15) | (((qh >> i) & 1) << 4);
      o[i] = __fmul_rn(d, i2f(q - 16));
    }
  }
};
template <> struct Dec<QT_Q5_1> {
  __device__ static void run(const uint8_t* b, int g, const uint8_t*, float* o) {
    float d = h2f(ld16(b)), m = h2f(ld16(b + 2));
    uint32_t qh = ld32(b + 4) >> (8 * g);
    const uint8_t* qs = b + 8 + 8 * (g & 1);
    int sh = 4 * (g >> 1);
#pragma unroll
    for (int i = 0; i < 8; i++) {
      int q = ((ldb(qs + i) >> sh) & 15) | (((qh >> i) & 1) << 4);
      o[i] = __fadd_rn(__fmul_rn(d, i2f(q)), m);
    }
  }
};
template <> struct Dec<QT_Q8_0> {
  __device__ static void run(const uint8_t* b, int g, const uint8_t*, float* o) {
    float d = h2f(GGQ_LD(reinterpret_cast<const unsigned short*>(b)));
    const uint2 q = ld8<2>(b + 2 + 8 * g);
#pragma unroll
    for (int i = 0; i < 8; i++) o[i] = __fmul_rn(i2f((int8_t)byte_of(q, i)), d);
  }
};
template <> struct Dec<QT_IQ4_NL> {
  __device__ static void run(const uint8_t* b, int g, const uint8_t* tab, float* o) {
    const int8_t* kv = (const int8_t*)(tab + TAB_KV_IQ4);
    float d = h2f(ld16(b));
    const uint8_t* qs = b + 2 + 8 * (g & 1);
    int sh = 4 * (g >> 1);
#pragma unroll
    for (int i = 0; i < 8; i++) o[i] = __fmul_rn(d, i2f(kv[(ldb(qs + i) >> sh) & 15]));
  }
};
template <> struct Dec<QT_MXFP4> {
  __device__ static void run(const uint8_t* b, int g, const uint8_t* tab, float* o) {
    const int8_t* kv = (const int8_t*)(tab + TAB_KV_MXFP4);
    uint32_t e = ldb(b);
    float d = __uint_as_float(e < 2 ? (0x00200000u << e) : ((e - 1) << 23));
    const uint8_t* qs = b + 1 + 8 * (g & 1);
    int sh = 4 * (g >> 1);
#pragma unroll
    for (int i = 0; i < 8; i++) o[i] = __fmul_rn(d, i2f(kv[(ldb(qs + i) >> sh) & 15]));
  }
};
// NVFP4: 64 elements, four UE4M3 sub-scales; elements 16s+j (low nibble of qs[8s+j]) and
// 16s+8+j (high nibble).
template <> struct Dec<QT_NVFP4> {
  __device__ static void run(const uint8_t* b, int g, const uint8_t* tab, float* o) {
    const int8_t* kv = (const int8_t*)(tab + TAB_KV_MXFP4);
    int s = g >> 1;
    uint32_t x = ldb(b + s);
    int ex = (x >> 3) & 15;
    float man = i2f(x & 7);
    float raw = ex == 0 ? __fmul_rn(man, 0.001953125f)
                        : __fmul_rn(__fadd_rn(1.0f, __fmul_rn(man, 0.125f)),
                                    __uint_as_float((uint32_t)(ex - 7 + 127) << 23));
    float d = (x == 0 || x == 0x7F) ? 0.0f : __fmul_rn(raw, 0.5f);
    const uint8_t* qs = b + 4 + 8 * s;
    int sh = 4 * (g & 1);
#pragma unroll
    for (int i = 0; i < 8; i++) o[i] = __fmul_rn(d, i2f(kv[(ldb(qs + i) >> sh) & 15]));
  }
};

// ---- K-quants -----------------------------------------------------------------------
template <> struct Dec<QT_Q2_K> {
  __device__ static void run(const uint8_t* b, int g, const uint8_t*, float* o) {
    float d = h2f(ld16(b + 80)), dmin = h2f(ld16(b + 82));
    uint32_t sc = ldb(b + (g >> 1));
    float dl = __fmul_rn(d, i2f(sc & 15)), ml = __fmul_rn(dmin, i2f(sc >> 4));
    const uint8_t* qs = b + 16 + 32 * (g >> 4) + 8 * (g & 3);
    int sh = 2 * ((g >> 2) & 3);
#pragma unroll
    for (int i = 0; i < 8; i++) o[i] = __fsub_rn(__fmul_rn(dl, i2f((ldb(qs + i) >> sh) & 3)), ml);
  }
};
template <> struct Dec<QT_Q3_K> {
  __device__ static void run(const uint8_t* b, int g, const uint8_t*, float* o) {
    const uint8_t* s = b + 96;
    float d = h2f(ld16(b + 108));
    int i16 = g >> 1;
    int lo = i16 < 8 ? (ldb(s + i16) & 15) : (ldb(s + i16 - 8) >> 4);
    int hi = (ldb(s + 8 + (i16 & 3)) >> (2 * (i16 >> 2))) & 3;
    float dl = __fmul_rn(d, i2f((lo | (hi << 4)) - 32));
    const uint8_t* qs = b + 32 + 32 * (g >> 4) + 8 * (g & 3);
    const uint8_t* hm = b + 8 * (g & 3);
    int sh = 2 * ((g >> 2) & 3), hb = g >> 2;
#pragma unroll
    for (int i = 0; i < 8; i++) {
      int ql = (ldb(qs + i) >> sh) & 3;
      int qh = ((ldb(hm + i) >> hb) & 1) ^ 1;
      o[i] = __fmul_rn(dl, i2f(ql - (qh << 2)));
    }
  }
};
// Q4_K / Q5_K blocks are 144 / 176 bytes: always 16-byte aligned, so the header is one
// 128-bit load and the eight quant bytes one 64-bit load.
__device__ __forceinline__ void scale_min_k4_words(const uint4& h, int k, int& sc, int& mn) {
  // h = (d|dmin, s0-3, s4-7, s8-11); same unpack as scale_min_k4
  const int sh = 8 * (k & 3);
  const uint32_t a = (h.y >> sh) & 0xFF, m = (h.z >> sh) & 0xFF, md = (h.w >> sh) & 0xFF;
  if (k < 4) { sc = a & 63; mn = m & 63; }
  else { sc = (md & 15) | ((a >> 6) << 4); mn = (md >> 4) | ((m >> 6) << 4); }
}
template <> struct Dec<QT_Q4_K> {
  __device__ static void run(const uint8_t* b, int g, const uint8_t*, float* o) {
    const uint4 h = GGQ_LD(reinterpret_cast<const uint4*>(b));
    const float d = h2f(h.x & 0xFFFF), dmin = h2f(h.x >> 16);
    int k = g >> 2, sc, mn;
    scale_min_k4_words(h, k, sc, mn);
    float dl = __fmul_rn(d, i2f(sc)), dm = __fmul_rn(dmin, i2f(mn));
    const uint2 q = ld8<8>(b + 16 + 32 * (k >> 1) + 8 * (g & 3));
    int sh = 4 * (k & 1);
#pragma unroll
    for (int i = 0; i < 8; i++) o[i] = __fsub_rn(__fmul_rn(dl, i2f((byte_of(q, i) >> sh) & 15)), dm);
  }
};
template <> struct Dec<QT_Q5_K> {
  __device__ static void run(const uint8_t* b, int g, const uint8_t*, float* o) {
    const uint4 h = GGQ_LD(reinterpret_cast<const uint4*>(b));
    const float d = h2f(h.x & 0xFFFF), dmin = h2f(h.x >> 16);
    int k = g >> 2, sc, mn;
    scale_min_k4_words(h, k, sc, mn);
    float dl = __fmul_rn(d, i2f(sc)), dm = __fmul_rn(dmin, i2f(mn));
    const uint2 qh = ld8<8>(b + 16 + 8 * (g & 3));
    const uint2 qs = ld8<8>(b + 48 + 32 * (k >> 1) + 8 * (g & 3));
    int sh = 4 * (k & 1);
#pragma unroll
    for (int i = 0; i < 8; i++) {
      int q = ((byte_of(qs, i) >> sh) & 15) | (((byte_of(qh, i) >> k) & 1) << 4);
      o[i] = __fsub_rn(__fmul_rn(dl, i2f(q)), dm);
    }
  }
};
// Q6_K blocks are 210 bytes: 2-byte aligned, all offsets below are even.
template <> struct Dec<QT_Q6_K> {
  __device__ static void run(const uint8_t* b, int g, const uint8_t*, float* o) {
    float d = h2f(GGQ_LD(reinterpret_cast<const unsigned short*>(b + 208)));
    float dl = __fmul_rn(d, i2f((int8_t)ldb(b + 192 + (g >> 1))));
    int c = g >> 2, t0 = 8 * (g & 3);
    const uint2 ql = ld8<2>(b + 64 * (c >> 2) + 32 * (c & 1) + t0);
    const uint2 qh = ld8<2>(b + 128 + 32 * (c >> 2) + t0);
    int shl = 4 * ((c >> 1) & 1), shh = 2 * (c & 3);
#pragma unroll
    for (int i = 0; i < 8; i++) {
      int q = ((byte_of(ql, i) >> shl) & 15) | (((byte_of(qh, i) >> shh) & 3) << 4);
      o[i] = __fmul_rn(dl, i2f(q - 32));
    }
  }
};

// ---- ternary --------------------------------------------------------------------------
template <> struct Dec<QT_TQ1_0> {
  __device__ static void run(const uint8_t* b, int g, const uint8_t*, float* o) {
    float d = h2f(ld16(b + 52));
    const uint32_t pow3[5] = {1, 3, 9, 27, 81};
#pragma unroll
    for (int i = 0; i < 8; i++) {
      uint32_t v;
      if (g < 20) v = ldb(b + 8 * (g & 3) + i) * pow3[g >> 2];
      else if (g < 30) v = ldb(b + 32 + 8 * ((g - 20) & 1) + i) * pow3[(g - 20) >> 1];
      else v = ldb(b + 48 + (i & 3)) * pow3[2 * (g - 30) + (i >> 2)];
      v &= 0xFF;
      o[i] = __fmul_rn(d, i2f((int)((v * 3) >> 8) - 1));
    }
  }
};
template <> struct Dec<QT_TQ2_0> {
  __device__ static void run(const uint8_t* b, int g, const uint8_t*, float* o) {
    float d = h2f(ld16(b + 64));
    const uint8_t* qs = b + 32 * (g >> 4) + 8 * (g & 3);
    int sh = 2 * ((g >> 2) & 3);
#pragma unroll
    for (int i = 0; i < 8; i++) o[i] = __fmul_rn(d, i2f((int)((ldb(qs + i) >> sh) & 3) - 1));
  }
};

// ---- codebook (I-quant) types ------------------------------------------------------------
template <> struct Dec<QT_IQ2_XXS> {
  __device__ static void run(const uint8_t* b, int g, const uint8_t* tab, float* o) {
    float d = h2f(ld16(b));
    int ib = g >> 2, l = g & 3;
    uint32_t aux = ld32(b + 2 + 8 * ib + 4);
    float db = __fmul_rn(__fmul_rn(d, __fadd_rn(0.5f, i2f(aux >> 28))), 0.25f);
    uint32_t signs = ksign((aux >> (7 * l)) & 127);
    const uint8_t* gr = tab + TAB_IQ2_XXS + 8 * ldb(b + 2 + 8 * ib + l);
#pragma unroll
    for (int j = 0; j < 8; j++) o[j] = __fmul_rn(__fmul_rn(db, i2f(gr[j])), sgnf(signs, j));
  }
};
template <> struct Dec<QT_IQ2_XS> {
  __device__ static void run(const uint8_t* b, int g, const uint8_t* tab, float* o) {
    float d = h2f(ld16(b));
    uint32_t q = ld16(b + 2 + 2 * g);
    uint32_t s = (ldb(b + 66 + (g >> 2)) >> (4 * ((g >> 1) & 1))) & 15;
    float db = __fmul_rn(__fmul_rn(d, __fadd_rn(0.5f, i2f(s))), 0.25f);
    uint32_t signs = ksign(q >> 9);
    const uint8_t* gr = tab + TAB_IQ2_XS + 8 * (q & 511);
#pragma unroll
    for (int j = 0; j < 8; j++) o[j] = __fmul_rn(__fmul_rn(db, i2f(gr[j])), sgnf(signs, j));
  }
};
template <> struct Dec<QT_IQ2_S> {
  __device__ static void run(const uint8_t* b, int g, const uint8_t* tab, float* o) {
    float d = h2f(ld16(b));
    uint32_t s = (ldb(b + 74 + (g >> 2)) >> (4 * ((g >> 1) & 1))) & 15;
    float db = __fmul_rn(__fmul_rn(d, __fadd_rn(0.5f, i2f(s))), 0.25f);
    uint32_t idx = ldb(b + 2 + g) | (((ldb(b + 66 + (g >> 2)) >> (2 * (g & 3))) & 3) << 8);
    uint32_t signs = ldb(b + 34 + g);
    const uint8_t* gr = tab + TAB_IQ2_S + 8 * idx;
#pragma unroll
    for (int j = 0; j < 8; j++) o[j] = __fmul_rn(__fmul_rn(db, i2f(gr[j])), sgnf(signs, j));
  }
};
template <> struct Dec<QT_IQ3_XXS> {
  __device__ static void run(const uint8_t* b, int g, const uint8_t* tab, float* o) {
    float d = h2f(ld16(b));
    int ib = g >> 2, l = g & 3;
    uint32_t aux = ld32(b + 66 + 4 * ib);
    float db = __fmul_rn(__fmul_rn(d, __fadd_rn(0.5f, i2f(aux >> 28))), 0.5f);
    uint32_t signs = ksign((aux >> (7 * l)) & 127);
    const uint8_t* g0 = tab + TAB_IQ3_XXS + 4 * ldb(b + 2 + 8 * ib + 2 * l);
    const uint8_t* g1 = tab + TAB_IQ3_XXS + 4 * ldb(b + 2 + 8 * ib + 2 * l + 1);
#pragma unroll
    for (int j = 0; j < 8; j++)
      o[j] = __fmul_rn(__fmul_rn(db, i2f(j < 4 ? g0[j] : g1[j - 4])), sgnf(signs, j));
  }
};
template <> struct Dec<QT_IQ3_S> {
  __device__ static void run(const uint8_t* b, int g, const uint8_t* tab, float* o) {
    float d = h2f(ld16(b));
    uint32_t s = (ldb(b + 106 + (g >> 3)) >> (4 * ((g >> 2) & 1))) & 15;
    float db = __fmul_rn(d, i2f(1 + 2 * s));
    uint32_t qh = ldb(b + 66 + (g >> 2)) >> (2 * (g & 3));
    uint32_t i0 = ldb(b + 2 + 2 * g) | ((qh & 1) << 8);
    uint32_t i1 = ldb(b + 2 + 2 * g + 1) | (((qh >> 1) & 1) << 8);
    uint32_t signs = ldb(b + 74 + g);
    const uint8_t* g0 = tab + TAB_IQ3_S + 4 * i0;
    const uint8_t* g1 = tab + TAB_IQ3_S + 4 * i1;
#pragma unroll
    for (int j = 0; j < 8; j++)
      o[j] = __fmul_rn(__fmul_rn(db, i2f(j < 4 ? g0[j] : g1[j - 4])), sgnf(signs, j));
  }
};
template <> struct Dec<QT_IQ1_S> {
  __device__ static void run(const uint8_t* b, int g, const uint8_t* tab, float* o) {
    float d = h2f(ld16(b));
    int ib = g >> 2, l = g & 3;
    uint32_t qh = ld16(b + 34 + 2 * ib);
    float dl = __fmul_rn(d, i2f(2 * ((qh >> 12) & 7) + 1));
    float delta = (qh & 0x8000) ? -0.125f : 0.125f;
    uint32_t idx = ldb(b + 2 + 4 * ib + l) | (((qh >> (3 * l)) & 7) << 8);
    const int8_t* gr = (const int8_t*)(tab + TAB_IQ1 + 8 * idx);
#pragma unroll
    for (int j = 0; j < 8; j++) o[j] = __fmul_rn(dl, __fadd_rn(i2f(gr[j]), delta));
  }
};
template <> struct Dec<QT_IQ1_M> {
  __device__ static void run(const uint8_t* b, int g, const uint8_t* tab, float* o) {
    uint32_t w0 = ld16(b + 48), w1 = ld16(b + 50), w2 = ld16(b + 52), w3 = ld16(b + 54);
    uint32_t dbits = (w0 >> 12) | ((w1 >> 8) & 0x00F0) | ((w2 >> 4) & 0x0F00) | (w3 & 0xF000);
    float d = h2f(dbits);
    int e = 8 * g;
    uint32_t w = (e >> 6) == 0 ? w0 : (e >> 6) == 1 ? w1 : (e >> 6) == 2 ? w2 : w3;
    uint32_t s = (w >> (3 * ((e >> 4) & 3))) & 7;
    float dl = __fmul_rn(d, i2f(2 * s + 1));
    uint32_t n = (ldb(b + 32 + (g >> 1)) >> (4 * (g & 1))) & 15;
    uint32_t idx = ldb(b + g) | ((n & 7) << 8);
    float delta = (n & 8) ? -0.125f : 0.125f;
    const int8_t* gr = (const int8_t*)(tab + TAB_IQ1 + 8 * idx);
#pragma unroll
    for (int j = 0; j < 8; j++) o[j] = __fmul_rn(dl, __fadd_rn(i2f(gr[j]), delta));
  }
};
template <> struct Dec<QT_IQ4_XS> {
  __device__ static void run(const uint8_t* b, int g, const uint8_t* tab, float* o) {
    const int8_t* kv = (const int8_t*)(tab + TAB_KV_IQ4);
    float d = h2f(ld16(b));
    uint32_t sh = ld16(b + 2);
    int j = g >> 2;
    int sc = (int)(((ldb(b + 4 + (j >> 1)) >> (4 * (j & 1))) & 15) | (((sh >> (2 * j)) & 3) << 4)) - 32;
    float dl = __fmul_rn(d, i2f(sc));
    const uint8_t* qs = b + 8 + 16 * j + 8 * (g & 1);
    int s4 = 4 * ((g >> 1) & 1);
#pragma unroll
    for (int i = 0; i < 8; i++) o[i] = __fmul_rn(dl, i2f(kv[(ldb(qs + i) >> s4) & 15]));
  }
};

// Calls f.template operator()<QT>() for the block qtype `qtype`; returns false for the
// float passthrough types and unknown codes.
template <class F>
inline bool dispatch_block_qtype(int qtype, F&& f) {
  switch (qtype) {
#define GGQ_CASE(T) case T: f.template operator()<T>(); return true;
    GGQ_CASE(QT_Q4_0) GGQ_CASE(QT_Q4_1) GGQ_CASE(QT_Q5_0) GGQ_CASE(QT_Q5_1) GGQ_CASE(QT_Q8_0)
    GGQ_CASE(QT_Q2_K) GGQ_CASE(QT_Q3_K) GGQ_CASE(QT_Q4_K) GGQ_CASE(QT_Q5_K) GGQ_CASE(QT_Q6_K)
    GGQ_CASE(QT_IQ2_XXS) GGQ_CASE(QT_IQ2_XS) GGQ_CASE(QT_IQ3_XXS) GGQ_CASE(QT_IQ1_S)
    GGQ_CASE(QT_IQ4_NL) GGQ_CASE(QT_IQ3_S) GGQ_CASE(QT_IQ2_S) GGQ_CASE(QT_IQ4_XS)
    GGQ_CASE(QT_IQ1_M) GGQ_CASE(QT_TQ1_0) GGQ_CASE(QT_TQ2_0) GGQ_CASE(QT_MXFP4) GGQ_CASE(QT_NVFP4)
#undef GGQ_CASE
    default: return false;
  }
}

}  // inline namespace
}  // namespace ggq
