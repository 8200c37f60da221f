/*
 * ggq_oracle.c -- TEST INFRASTRUCTURE, not product code.
 *
 * A plain-C, scalar restatement of the dequantize-and-multiply path of gguf-jax, used
 * only as the checker in tests/, in the smoke test and as the timed CPU baseline of
 * bench.py.  The product (gguf_jax_b200 + libggq_b200.so) never links, imports or calls
 * anything in this file.
 *
 * What it restates: gguf-jax's decoders (src/gguf_jax/quants.py:125-712) mirror the numpy
 * decoders of the third-party package gguf 0.19.0 (gguf/quants.py) operation for
 * operation; every function below cites both.  All arithmetic is float32 with the
 * association written in the reference, so the output is meant to be bit-identical.
 * The matmul follows _dequant_forward (src/gguf_jax/_matmul.py:195-201) with float32
 * weights: y = x @ dequantize(w).T.
 *
 * Pinning: tests/test_oracle.py checks every decoder here against gguf.quants.dequantize
 * (the oracle the reference's own tests use, tests/test_bitwise.py:65-101) on random
 * bytes, on quantizer round trips and on the committed fixtures in tests/golden/.
 *
 * Codebook tables are never transcribed: the caller passes the blob built from
 * gguf.quants at run time (layout in include/ggq.h, ggq_tables_bytes).
 *
 * Build: make -C oracle   (gcc -O2 -fopenmp -ffp-contract=off -shared -fPIC)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define QK_K 256

/* ---- table blob ----------------------------------------------------------------- */
enum {
  OFF_IQ2_XXS = 0,
  OFF_IQ2_XS = OFF_IQ2_XXS + 256 * 8,
  OFF_IQ2_S = OFF_IQ2_XS + 512 * 8,
  OFF_IQ3_XXS = OFF_IQ2_S + 1024 * 8,
  OFF_IQ3_S = OFF_IQ3_XXS + 256 * 4,
  OFF_IQ1 = OFF_IQ3_S + 512 * 4,
  OFF_KV_IQ4 = OFF_IQ1 + 2048 * 8,
  OFF_KV_MXFP4 = OFF_KV_IQ4 + 16,
  TABLE_BYTES = OFF_KV_MXFP4 + 16
};
static uint8_t g_tab[TABLE_BYTES];
static int g_tab_set = 0;

int ggq_oracle_tables_bytes(void) { return TABLE_BYTES; }

int ggq_oracle_set_tables(const void* blob, size_t bytes) {
  if (bytes != TABLE_BYTES) return 1;
  memcpy(g_tab, blob, TABLE_BYTES);
  g_tab_set = 1;
  return 0;
}

/* ---- scalar helpers ------------------------------------------------------------- */
static inline uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }
static inline uint32_t rd32(const uint8_t* p) {
  return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* IEEE half -> float, exact, NaN payload shifted up as numpy does
 * (src/gguf_jax/quants.py:91-101). */
static float f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000) << 16;
  uint32_t exp = (h >> 10) & 0x1F;
  uint32_t man = h & 0x3FF;
  if (exp == 31) return bits_f32(sign | 0x7F800000u | (man << 13));
  if (exp == 0) {
    if (man == 0) return bits_f32(sign);
    /* subnormal half: man * 2^-24 */
    float v = (float)man * bits_f32(0x33800000u); /* 2^-24 */
    return sign ? -v : v;
  }
  return bits_f32(sign | ((exp + 112) << 23) | (man << 13));
}

/* ksigns[i] = i | parity(i) << 7  (gguf/quants.py IQ2_XXS.ksigns; checked in tests). */
static inline uint8_t ksign(uint32_t i) {
  uint32_t p = i ^ (i >> 4); p ^= p >> 2; p ^= p >> 1;
  return (uint8_t)(i | ((p & 1) << 7));
}
static inline float sgn(uint8_t signs, int j) { return ((signs >> j) & 1) ? -1.0f : 1.0f; }

/* ---- block decoders: one block in, block_elems floats out ------------------------ */

/* Q4_0: quants.py:144-154; gguf/quants.py Q4_0.dequantize_blocks */
static void dq_q4_0(const uint8_t* b, float* o) {
  float d = f16_to_f32(rd16(b));
  for (int e = 0; e < 32; e++) {
    int nib = e < 16 ? (b[2 + e] & 15) : (b[2 + e - 16] >> 4);
    o[e] = d * (float)(int8_t)(nib - 8);
  }
}
/* Q4_1: quants.py:157-168 */
static void dq_q4_1(const uint8_t* b, float* o) {
  float d = f16_to_f32(rd16(b)), m = f16_to_f32(rd16(b + 2));
  for (int e = 0; e < 32; e++) {
    int nib = e < 16 ? (b[4 + e] & 15) : (b[4 + e - 16] >> 4);
    float p = d * (float)nib;
    o[e] = p + m;
  }
}
/* Q5_0: quants.py:171-186 */
static void dq_q5_0(const uint8_t* b, float* o) {
  float d = f16_to_f32(rd16(b));
  uint32_t qh = rd32(b + 2);
  for (int e = 0; e < 32; e++) {
    int nib = e < 16 ? (b[6 + e] & 15) : (b[6 + e - 16] >> 4);
    int q = nib | (((qh >> e) & 1) << 4);
    o[e] = d * (float)(int8_t)(q - 16);
  }
}
/* Q5_1: quants.py:189-205 */
static void dq_q5_1(const uint8_t* b, float* o) {
  float d = f16_to_f32(rd16(b)), m = f16_to_f32(rd16(b + 2));
  uint32_t qh = rd32(b + 4);
  for (int e = 0; e < 32; e++) {
    int nib = e < 16 ? (b[8 + e] & 15) : (b[8 + e - 16] >> 4);
    int q = nib | (((qh >> e) & 1) << 4);
    float p = d * (float)q;
    o[e] = p + m;
  }
}
/* Q8_0: quants.py:208-213 */
static void dq_q8_0(const uint8_t* b, float* o) {
  float d = f16_to_f32(rd16(b));
  for (int e = 0; e < 32; e++) o[e] = (float)(int8_t)b[2 + e] * d;
}
/* Q2_K: quants.py:219-239 */
static void dq_q2_k(const uint8_t* b, float* o) {
  const uint8_t* sc = b; const uint8_t* qs = b + 16;
  float d = f16_to_f32(rd16(b + 80)), dmin = f16_to_f32(rd16(b + 82));
  for (int e = 0; e < 256; e++) {
    int h = e / 128, s = (e % 128) / 32, t = e % 32;
    float dl = d * (float)(sc[e / 16] & 15);
    float ml = dmin * (float)(sc[e / 16] >> 4);
    float q = (float)((qs[32 * h + t] >> (2 * s)) & 3);
    float p = dl * q;
    o[e] = p - ml;
  }
}
/* Q3_K: quants.py:242-269 */
static void dq_q3_k(const uint8_t* b, float* o) {
  const uint8_t* hmask = b; const uint8_t* qs = b + 32; const uint8_t* s = b + 96;
  float d = f16_to_f32(rd16(b + 108));
  for (int e = 0; e < 256; e++) {
    int i = e / 16;
    int lo = i < 8 ? (s[i] & 15) : (s[i - 8] >> 4);
    int hi = (s[8 + (i % 4)] >> (2 * (i / 4))) & 3;
    int scv = (int8_t)(lo | (hi << 4)) - 32;
    float dl = d * (float)scv;
    int h = e / 128, sh = (e % 128) / 32, t = e % 32;
    int ql = (qs[32 * h + t] >> (2 * sh)) & 3;
    int qh = ((hmask[t] >> (e / 32)) & 1) ^ 1;
    int q = (int8_t)ql - (int8_t)(qh << 2);
    o[e] = dl * (float)q;
  }
}
/* 6-bit scale/min unpack shared by Q4_K and Q5_K: quants.py:275-283 */
static void scale_min_k4(const uint8_t* s, int k, int* sc, int* mn) {
  if (k < 4) { *sc = s[k] & 63; *mn = s[4 + k] & 63; }
  else {
    *sc = (s[4 + k] & 15) | ((s[k - 4] >> 6) << 4);
    *mn = (s[4 + k] >> 4) | ((s[k] >> 6) << 4);
  }
}
/* Q4_K: quants.py:286-305 */
static void dq_q4_k(const uint8_t* b, float* o) {
  float d = f16_to_f32(rd16(b)), dmin = f16_to_f32(rd16(b + 2));
  const uint8_t* s = b + 4; const uint8_t* qs = b + 16;
  for (int e = 0; e < 256; e++) {
    int k = e / 32, t = e % 32, sc, mn;
    scale_min_k4(s, k, &sc, &mn);
    float dl = d * (float)sc, dm = dmin * (float)mn;
    float q = (float)((qs[32 * (k / 2) + t] >> (4 * (k % 2))) & 15);
    float p = dl * q;
    o[e] = p - dm;
  }
}
/* Q5_K: quants.py:308-331 */
static void dq_q5_k(const uint8_t* b, float* o) {
  float d = f16_to_f32(rd16(b)), dmin = f16_to_f32(rd16(b + 2));
  const uint8_t* s = b + 4; const uint8_t* qh = b + 16; const uint8_t* qs = b + 48;
  for (int e = 0; e < 256; e++) {
    int k = e / 32, t = e % 32, sc, mn;
    scale_min_k4(s, k, &sc, &mn);
    float dl = d * (float)sc, dm = dmin * (float)mn;
    int q = ((qs[32 * (k / 2) + t] >> (4 * (k % 2))) & 15) | (((qh[t] >> k) & 1) << 4);
    float p = dl * (float)q;
    o[e] = p - dm;
  }
}
/* Q6_K: quants.py:334-353 */
static void dq_q6_k(const uint8_t* b, float* o) {
  const uint8_t* ql = b; const uint8_t* qh = b + 128; const int8_t* sc = (const int8_t*)(b + 192);
  float d = f16_to_f32(rd16(b + 208));
  for (int e = 0; e < 256; e++) {
    int c = e / 32, t = e % 32;
    int lo = (ql[64 * (c / 4) + 32 * (c % 2) + t] >> (4 * ((c / 2) % 2))) & 15;
    int hi = (qh[32 * (c / 4) + t] >> (2 * (c % 4))) & 3;
    int q = (int8_t)(lo | (hi << 4)) - 32;
    float dl = d * (float)sc[e / 16];
    o[e] = dl * (float)q;
  }
}
/* TQ1_0: quants.py:359-378 */
static void dq_tq1_0(const uint8_t* b, float* o) {
  static const uint8_t pow3[5] = {1, 3, 9, 27, 81};
  float d = f16_to_f32(rd16(b + 52));
  for (int e = 0; e < 256; e++) {
    uint8_t v;
    if (e < 160) v = (uint8_t)(b[e % 32] * pow3[e / 32]);
    else if (e < 240) v = (uint8_t)(b[32 + (e - 160) % 16] * pow3[(e - 160) / 16]);
    else v = (uint8_t)(b[48 + (e - 240) % 4] * pow3[(e - 240) / 4]);
    int q = (int8_t)(((uint16_t)v * 3) >> 8) - 1;
    o[e] = d * (float)q;
  }
}
/* TQ2_0: quants.py:381-391 */
static void dq_tq2_0(const uint8_t* b, float* o) {
  float d = f16_to_f32(rd16(b + 64));
  for (int e = 0; e < 256; e++) {
    int h = e / 128, s = (e % 128) / 32, t = e % 32;
    int q = (int8_t)((b[32 * h + t] >> (2 * s)) & 3) - 1;
    o[e] = d * (float)q;
  }
}
/* E8M0 -> float "half scale": quants.py:400-403 */
static float e8m0_half(uint8_t e) {
  uint32_t x = e;
  return bits_f32(x < 2 ? (0x00200000u << x) : ((x - 1) << 23));
}
/* MXFP4: quants.py:406-434 (numpy keeps subnormals, so the plain product is right) */
static void dq_mxfp4(const uint8_t* b, float* o) {
  const int8_t* kv = (const int8_t*)(g_tab + OFF_KV_MXFP4);
  float d = e8m0_half(b[0]);
  for (int e = 0; e < 32; e++) {
    int nib = e < 16 ? (b[1 + e] & 15) : (b[1 + e - 16] >> 4);
    o[e] = d * (float)kv[nib];
  }
}
/* UE4M3 -> float: quants.py:442-449 */
static float ue4m3(uint8_t x) {
  int ex = (x >> 3) & 15; float man = (float)(x & 7);
  float raw;
  if (ex == 0) raw = man * bits_f32(0x3B000000u); /* 2^-9 */
  else raw = (1.0f + man / 8.0f) * bits_f32((uint32_t)(ex - 7 + 127) << 23);
  if (x == 0 || x == 0x7F) return 0.0f;
  return raw * 0.5f;
}
/* NVFP4: quants.py:452-467 */
static void dq_nvfp4(const uint8_t* b, float* o) {
  const int8_t* kv = (const int8_t*)(g_tab + OFF_KV_MXFP4);
  for (int s = 0; s < 4; s++) {
    float d = ue4m3(b[s]);
    for (int j = 0; j < 8; j++) {
      uint8_t q = b[4 + 8 * s + j];
      o[16 * s + j] = d * (float)kv[q & 15];
      o[16 * s + 8 + j] = d * (float)kv[q >> 4];
    }
  }
}
/* IQ2_XXS: quants.py:493-511 */
static void dq_iq2_xxs(const uint8_t* b, float* o) {
  const uint8_t* grid = g_tab + OFF_IQ2_XXS;
  float d = f16_to_f32(rd16(b));
  for (int ib = 0; ib < 8; ib++) {
    uint32_t aux = rd32(b + 2 + 8 * ib + 4);
    float db = d * (0.5f + (float)(aux >> 28)) * 0.25f;
    for (int l = 0; l < 4; l++) {
      uint8_t signs = ksign((aux >> (7 * l)) & 127);
      const uint8_t* g = grid + 8 * b[2 + 8 * ib + l];
      for (int j = 0; j < 8; j++) o[32 * ib + 8 * l + j] = db * (float)g[j] * sgn(signs, j);
    }
  }
}
/* IQ2_XS: quants.py:514-534 */
static void dq_iq2_xs(const uint8_t* b, float* o) {
  const uint8_t* grid = g_tab + OFF_IQ2_XS;
  float d = f16_to_f32(rd16(b));
  const uint8_t* sc = b + 66;
  for (int g8 = 0; g8 < 32; g8++) {
    uint16_t q = rd16(b + 2 + 2 * g8);
    int s = (sc[g8 / 4] >> (4 * ((g8 / 2) % 2))) & 15;
    float db = d * (0.5f + (float)s) * 0.25f;
    uint8_t signs = ksign(q >> 9);
    const uint8_t* g = grid + 8 * (q & 511);
    for (int j = 0; j < 8; j++) o[8 * g8 + j] = db * (float)g[j] * sgn(signs, j);
  }
}
/* IQ2_S: quants.py:537-560 */
static void dq_iq2_s(const uint8_t* b, float* o) {
  const uint8_t* grid = g_tab + OFF_IQ2_S;
  float d = f16_to_f32(rd16(b));
  const uint8_t* qs = b + 2; const uint8_t* signs = b + 34; const uint8_t* qh = b + 66;
  const uint8_t* sc = b + 74;
  for (int g8 = 0; g8 < 32; g8++) {
    int s = (sc[g8 / 4] >> (4 * ((g8 / 2) % 2))) & 15;
    float db = d * (0.5f + (float)s) * 0.25f;
    int idx = qs[g8] | (((qh[g8 / 4] >> (2 * (g8 % 4))) & 3) << 8);
    const uint8_t* g = grid + 8 * idx;
    for (int j = 0; j < 8; j++) o[8 * g8 + j] = db * (float)g[j] * sgn(signs[g8], j);
  }
}
/* IQ3_XXS: quants.py:563-582 */
static void dq_iq3_xxs(const uint8_t* b, float* o) {
  const uint8_t* grid = g_tab + OFF_IQ3_XXS;
  float d = f16_to_f32(rd16(b));
  const uint8_t* qs = b + 2;
  for (int ib = 0; ib < 8; ib++) {
    uint32_t aux = rd32(b + 66 + 4 * ib);
    float db = d * (0.5f + (float)(aux >> 28)) * 0.5f;
    for (int l = 0; l < 4; l++) {
      uint8_t signs = ksign((aux >> (7 * l)) & 127);
      for (int j = 0; j < 8; j++) {
        const uint8_t* g = grid + 4 * qs[8 * ib + 2 * l + j / 4];
        o[32 * ib + 8 * l + j] = db * (float)g[j % 4] * sgn(signs, j);
      }
    }
  }
}
/* IQ3_S: quants.py:585-609 */
static void dq_iq3_s(const uint8_t* b, float* o) {
  const uint8_t* grid = g_tab + OFF_IQ3_S;
  float d = f16_to_f32(rd16(b));
  const uint8_t* qs = b + 2; const uint8_t* qh = b + 66; const uint8_t* signs = b + 74;
  const uint8_t* sc = b + 106;
  for (int e = 0; e < 256; e++) {
    int s = (sc[e / 64] >> (4 * ((e / 32) % 2))) & 15;
    float db = d * (float)(1 + 2 * s);
    int k = e / 4;
    int idx = qs[k] | (((qh[k / 8] >> (k % 8)) & 1) << 8);
    o[e] = db * (float)grid[4 * idx + e % 4] * sgn(signs[e / 8], e % 8);
  }
}
/* IQ1_S: quants.py:612-635 */
static void dq_iq1_s(const uint8_t* b, float* o) {
  const int8_t* grid = (const int8_t*)(g_tab + OFF_IQ1);
  float d = f16_to_f32(rd16(b));
  const uint8_t* qs = b + 2;
  for (int ib = 0; ib < 8; ib++) {
    uint16_t qh = rd16(b + 34 + 2 * ib);
    float dl = d * (float)(2 * ((qh >> 12) & 7) + 1);
    float delta = (qh & 0x8000) ? -0.125f : 0.125f;
    for (int l = 0; l < 4; l++) {
      int idx = qs[4 * ib + l] | (((qh >> (3 * l)) & 7) << 8);
      for (int j = 0; j < 8; j++) {
        float gv = (float)grid[8 * idx + j] + delta;
        o[32 * ib + 8 * l + j] = dl * gv;
      }
    }
  }
}
/* IQ1_M: quants.py:638-664 */
static void dq_iq1_m(const uint8_t* b, float* o) {
  const int8_t* grid = (const int8_t*)(g_tab + OFF_IQ1);
  const uint8_t* qs = b; const uint8_t* qh = b + 32;
  uint16_t w[4];
  for (int j = 0; j < 4; j++) w[j] = rd16(b + 48 + 2 * j);
  uint16_t dbits = (uint16_t)((w[0] >> 12) | ((w[1] >> 8) & 0x00F0) | ((w[2] >> 4) & 0x0F00) | (w[3] & 0xF000));
  float d = f16_to_f32(dbits);
  for (int g8 = 0; g8 < 32; g8++) {
    int e = 8 * g8;
    int s = (w[e / 64] >> (3 * ((e / 16) % 4))) & 7;
    float dl = d * (float)(2 * s + 1);
    int n = (qh[g8 / 2] >> (4 * (g8 % 2))) & 15;
    int idx = qs[g8] | ((n & 7) << 8);
    float delta = (n & 8) ? -0.125f : 0.125f;
    for (int j = 0; j < 8; j++) {
      float gv = (float)grid[8 * idx + j] + delta;
      o[e + j] = dl * gv;
    }
  }
}
/* IQ4_NL: quants.py:667-683 */
static void dq_iq4_nl(const uint8_t* b, float* o) {
  const int8_t* kv = (const int8_t*)(g_tab + OFF_KV_IQ4);
  float d = f16_to_f32(rd16(b));
  for (int e = 0; e < 32; e++) {
    int nib = e < 16 ? (b[2 + e] & 15) : (b[2 + e - 16] >> 4);
    o[e] = d * (float)kv[nib];
  }
}
/* IQ4_XS: quants.py:686-712 */
static void dq_iq4_xs(const uint8_t* b, float* o) {
  const int8_t* kv = (const int8_t*)(g_tab + OFF_KV_IQ4);
  float d = f16_to_f32(rd16(b));
  uint16_t sh = rd16(b + 2);
  const uint8_t* sl = b + 4; const uint8_t* qs = b + 8;
  for (int e = 0; e < 256; e++) {
    int j = e / 32, t = e % 32;
    int scv = (int8_t)(((sl[j / 2] >> (4 * (j % 2))) & 15) | (((sh >> (2 * j)) & 3) << 4)) - 32;
    float dl = d * (float)scv;
    int idx = (qs[16 * j + t % 16] >> (4 * (t / 16))) & 15;
    o[e] = dl * (float)kv[idx];
  }
}
/* F32 / F16 / BF16 passthrough: quants.py:125-138 */
static void dq_f32(const uint8_t* b, float* o) { o[0] = bits_f32(rd32(b)); }
static void dq_f16(const uint8_t* b, float* o) { o[0] = f16_to_f32(rd16(b)); }
static void dq_bf16(const uint8_t* b, float* o) { o[0] = bits_f32((uint32_t)rd16(b) << 16); }

typedef void (*dq_fn)(const uint8_t*, float*);
typedef struct { int qtype, bs, ts; dq_fn fn; int needs_tables; } traits_t;
static const traits_t k_traits[] = {
  {0, 1, 4, dq_f32, 0},      {1, 1, 2, dq_f16, 0},      {30, 1, 2, dq_bf16, 0},
  {2, 32, 18, dq_q4_0, 0},   {3, 32, 20, dq_q4_1, 0},   {6, 32, 22, dq_q5_0, 0},
  {7, 32, 24, dq_q5_1, 0},   {8, 32, 34, dq_q8_0, 0},   {10, 256, 84, dq_q2_k, 0},
  {11, 256, 110, dq_q3_k, 0}, {12, 256, 144, dq_q4_k, 0}, {13, 256, 176, dq_q5_k, 0},
  {14, 256, 210, dq_q6_k, 0}, {16, 256, 66, dq_iq2_xxs, 1}, {17, 256, 74, dq_iq2_xs, 1},
  {18, 256, 98, dq_iq3_xxs, 1}, {19, 256, 50, dq_iq1_s, 1}, {20, 32, 18, dq_iq4_nl, 1},
  {21, 256, 110, dq_iq3_s, 1}, {22, 256, 82, dq_iq2_s, 1}, {23, 256, 136, dq_iq4_xs, 1},
  {29, 256, 56, dq_iq1_m, 1}, {34, 256, 54, dq_tq1_0, 0}, {35, 256, 66, dq_tq2_0, 0},
  {39, 32, 17, dq_mxfp4, 1}, {40, 64, 36, dq_nvfp4, 1},
};
static const traits_t* find(int qtype) {
  for (size_t i = 0; i < sizeof(k_traits) / sizeof(k_traits[0]); i++)
    if (k_traits[i].qtype == qtype) return &k_traits[i];
  return NULL;
}

int ggq_oracle_type_info(int qtype, int* bs, int* ts) {
  const traits_t* t = find(qtype);
  if (!t) return 1;
  *bs = t->bs; *ts = t->ts;
  return 0;
}

/* dequantize_blocks: quants.py:718-730.  out is float32[n_blocks * bs]. */
int ggq_oracle_dequant(int qtype, const uint8_t* blocks, int64_t n_blocks, float* out) {
  const traits_t* t = find(qtype);
  if (!t) return 1;
  if (t->needs_tables && !g_tab_set) return 7;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n_blocks; i++) t->fn(blocks + i * t->ts, out + i * t->bs);
  return 0;
}

static inline float bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

/* y[M,N] (float32) = x[M,K] (bf16) @ dequantize(w)[N,K].T with float32 weights:
 * _dequant_forward with blocks == 1 (_matmul.py:195-201) at dtype float32.  Each dot
 * product is accumulated in double and rounded to float32 once, so the checker carries
 * no summation-order noise of its own.  Decode is fused per row (one block buffer per
 * thread) so the 8192 x 28672 case needs no dense temporary. */
int ggq_oracle_matmul(int qtype, const uint8_t* w, int64_t N, int64_t K, const uint16_t* x_bf16,
                      int M, float* y) {
  const traits_t* t = find(qtype);
  if (!t || K % t->bs) return 1;
  if (t->needs_tables && !g_tab_set) return 7;
  int64_t nb = K / t->bs, row_bytes = nb * t->ts;
  float* xf = (float*)malloc(sizeof(float) * (size_t)M * K);
  for (int64_t i = 0; i < (int64_t)M * K; i++) xf[i] = bf16_to_f32(x_bf16[i]);
#pragma omp parallel
  {
    float blk[256];
    double* acc = (double*)malloc(sizeof(double) * M);
#pragma omp for schedule(static)
    for (int64_t n = 0; n < N; n++) {
      for (int m = 0; m < M; m++) acc[m] = 0.0;
      const uint8_t* row = w + n * row_bytes;
      for (int64_t bi = 0; bi < nb; bi++) {
        t->fn(row + bi * t->ts, blk);
        for (int m = 0; m < M; m++) {
          const float* xr = xf + (int64_t)m * K + bi * t->bs;
          double s = 0.0;
          for (int e = 0; e < t->bs; e++) s += (double)blk[e] * (double)xr[e];
          acc[m] += s;
        }
      }
      for (int m = 0; m < M; m++) y[(int64_t)m * N + n] = (float)acc[m];
    }
    free(acc);
  }
  free(xf);
  return 0;
}

/* Same product in plain float32 accumulation (the arithmetic a CPU BLAS would do); this
 * is the variant bench.py times as the CPU baseline. */
int ggq_oracle_matmul_f32(int qtype, const uint8_t* w, int64_t N, int64_t K, const uint16_t* x_bf16,
                          int M, float* y) {
  const traits_t* t = find(qtype);
  if (!t || K % t->bs) return 1;
  if (t->needs_tables && !g_tab_set) return 7;
  int64_t nb = K / t->bs, row_bytes = nb * t->ts;
  float* xf = (float*)malloc(sizeof(float) * (size_t)M * K);
  for (int64_t i = 0; i < (int64_t)M * K; i++) xf[i] = bf16_to_f32(x_bf16[i]);
#pragma omp parallel
  {
    float blk[256];
    float* acc = (float*)malloc(sizeof(float) * M);
#pragma omp for schedule(static)
    for (int64_t n = 0; n < N; n++) {
      for (int m = 0; m < M; m++) acc[m] = 0.0f;
      const uint8_t* row = w + n * row_bytes;
      for (int64_t bi = 0; bi < nb; bi++) {
        t->fn(row + bi * t->ts, blk);
        for (int m = 0; m < M; m++) {
          const float* xr = xf + (int64_t)m * K + bi * t->bs;
          float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
          int e = 0;
          for (; e + 3 < t->bs; e += 4) {
            s0 += blk[e] * xr[e]; s1 += blk[e + 1] * xr[e + 1];
            s2 += blk[e + 2] * xr[e + 2]; s3 += blk[e + 3] * xr[e + 3];
          }
          for (; e < t->bs; e++) s0 += blk[e] * xr[e];
          acc[m] += (s0 + s1) + (s2 + s3);
        }
      }
      for (int m = 0; m < M; m++) y[(int64_t)m * N + n] = acc[m];
    }
    free(acc);
  }
  free(xf);
  return 0;
}

int ggq_oracle_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Number of OpenMP threads later calls use (n < 1: leave as is).  Launchers such as torchrun
 * export OMP_NUM_THREADS=1 to their children; a timed CPU baseline sets the count explicitly. */
int ggq_oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n >= 1) omp_set_num_threads(n);
  return omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}
