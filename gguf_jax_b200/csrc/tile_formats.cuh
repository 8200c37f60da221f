// Block formats of the tiled fused multiply (gemv_tile.cuh): how one lane turns raw block bytes
// into tensor-core operands.
//
// The multiply uses mma.sync.m16n8k16 with *exact integer codes* as the A operand.  A bf16 whose
// upper byte is 0x00 (or 0x80) is linear in its lower byte: bits 0x00vv are +v * 2^-133, bits
// 0x80vv are -v * 2^-133, for every v in 0..255.  So a 32-bit register (v0 | s0 << 15 | v1 << 16 |
// s1 << 31) is a pair of bf16 weights without any conversion, and a masked field that was not
// shifted down (v << n) is the same weight times 2^n, which the activation side absorbs with an
// exact power-of-two scale.  Scales are applied to the float32 accumulators, once per scale group.
//
// A superblock of 256 weights is split into four lane runs of 64 weights; lane (g, t) of a warp
// owns run t of rows g and g + 8 of the warp's 16-row tile.  A run is eight octets of eight
// weights; an octet feeds two MMAs (four weights per row and MMA sit in the k-slots 2t, 2t+1,
// 2t+8, 2t+9).  Which weights form run t / octet oo, and in which order they enter the k-slots,
// is the format's choice (src_quads + kPairOrder): the activations are permuted to match when
// they are staged in shared memory.  A format provides
//
//   kTs, kQt            block bytes, qtype code
//   kOct                octets per run: 8, or 16 for the two-plane formats (Q5_K, Q6_K), whose codes are
//                       split into a nibble plane and a high-bit plane that are multiplied separately
//                       (every weight then appears in two octets, with its activation staged twice)
//   kGroupOct           octets per scale group inside a run (1, 2 or 4 = groups of 8, 16, 32)
//   kSums, kSumOct      the fold needs the activations' sum per scale group, taken over the group's first
//                       kSumOct octets (all of them, or the first plane of a two-plane format)
//   kPairOrder          0: an octet is 8 consecutive weights e..e+7 entering as (e, e+2), (e+1, e+3),
//                          (e+4, e+6), (e+5, e+7)    [byte pairs (0,2), (1,3) of two words]
//                       1: an octet is two quads a..a+3, b..b+3 entering as (a, a+1), (b, b+1),
//                          (a+2, a+3), (b+2, b+3)     [nibble pairs of one word]
//   src_quads(t, oo)    first weight of the octet's two quads
//   x_exp(t, oo)        exponent e <= 0: the octet's activations are staged times 2^e
//   kAlign              alignment of every block when rows start 16-byte aligned: gcd(kTs, 16)
//   kUnrollGroups       true for the bit-plane formats, whose groups share the same words (the run is
//                       loaded once and the group loop is unrolled); false for the grid formats, whose
//                       groups are loaded one at a time inside a real loop (keeps the loop body small)
//   Run, load_run(ld, t)             what is read once per run and row
//   Group, load_group(ld, run, t, grp)   the raw fields and the scale of group grp of the run
//   octet(group, q, tab, p)   the four A-operand registers of octet q of the group: p[0], p[1] = first
//                       MMA (k-slot pairs 2t.. and 2t+8..), p[2], p[3] = second MMA
//   fold(group, acc, xsum, out) -> float   out + the group's contribution given acc = sum(code * x)
//                       and xsum = sum(x) over the group (both in the same power-of-two scale)
//
// Everything here is plain integer and float32 arithmetic written for host and device, so the
// per-format logic is checked on the CPU against the block decoders (tests/test_tile_formats.py).
// Decode formulas: src/gguf_jax/quants.py:219-239 (Q2_K), :275-305 (Q4_K), :493-664 (IQ2/IQ3/IQ1),
// :686-712 (IQ4_XS) in the reference; gguf/quants.py for the same formats in gguf-py.
#pragma once

#include <stdint.h>
#include <string.h>

// Under nvcc everything here is device code (blocks and tables are addressed in shared memory);
// a plain C++ compiler gets the same functions over ordinary memory for the host-side check.
#if defined(__CUDACC__)
#define TF_HD __device__ __forceinline__
#define TF_DEVICE 1
#else
#define TF_HD inline
#define TF_DEVICE 0
#endif

namespace ggq {
namespace tf {

// ---- small portable helpers -----------------------------------------------------------------
TF_HD uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
#if TF_DEVICE
  return __byte_perm(a, b, sel);
#else
  const uint64_t v = (uint64_t)a | ((uint64_t)b << 32);
  uint32_t r = 0;
  for (int i = 0; i < 4; i++) r |= (uint32_t)((v >> (8 * ((sel >> (4 * i)) & 7))) & 0xFF) << (8 * i);
  return r;
#endif
}
TF_HD uint32_t popc(uint32_t v) {
#if TF_DEVICE
  return __popc(v);
#else
  return (uint32_t)__builtin_popcount(v);
#endif
}
TF_HD uint32_t funnel16(uint32_t lo, uint32_t hi) {   // bytes 2..5 of the eight bytes (lo, hi)
#if TF_DEVICE
  return __funnelshift_r(lo, hi, 16);
#else
  return (lo >> 16) | (hi << 16);
#endif
}
TF_HD float f16_bits_to_float(uint32_t h) {
#if TF_DEVICE
  return __half2float(__ushort_as_half((unsigned short)h));
#else
  const uint32_t s = (h >> 15) & 1, e = (h >> 10) & 31, m = h & 1023;
  uint32_t u;
  if (e == 0) {
    if (m == 0) u = s << 31;
    else { int k = 0; uint32_t mm = m; while (!(mm & 1024)) { mm <<= 1; k++; } u = (s << 31) | ((uint32_t)(113 - k) << 23) | ((mm & 1023) << 13); }
  } else if (e == 31) u = (s << 31) | 0x7F800000u | (m << 13);
  else u = (s << 31) | ((e + 112) << 23) | (m << 13);
  float f;
  memcpy(&f, &u, 4);
  return f;
#endif
}
TF_HD float mulf(float a, float b) {
#if TF_DEVICE
  return __fmul_rn(a, b);
#else
  volatile float r = a * b;
  return r;
#endif
}
TF_HD float fmaf_(float a, float b, float c) {
#if TF_DEVICE
  return __fmaf_rn(a, b, c);
#else
  return __builtin_fmaf(a, b, c);
#endif
}
TF_HD float u2f(uint32_t v) { return (float)v; }

// Pair registers from a word of four code bytes: bytes (0, 2) and bytes (1, 3), each byte widened
// to a bf16 with a zero upper byte.
TF_HD uint32_t pair02(uint32_t w) { return prmt(w, 0u, 0x4240u); }
TF_HD uint32_t pair13(uint32_t w) { return prmt(w, 0u, 0x4341u); }
// The same with sign bits: `s` holds 0x80 or 0x00 in byte j for the sign of code byte j.
TF_HD uint32_t pair02s(uint32_t w, uint32_t s) { return prmt(w, s, 0x6240u); }
TF_HD uint32_t pair13s(uint32_t w, uint32_t s) { return prmt(w, s, 0x7351u); }
// Four sign bits (bit j of `nib`, j = 0..3) spread to 0x80 in byte j.
TF_HD uint32_t spread_signs4(uint32_t nib) { return ((nib & 15u) * 0x00204081u) << 7 & 0x80808080u; }
// ksigns[i] = i | parity(i) << 7 (gguf/quants.py IQ2_XXS.ksigns)
TF_HD uint32_t ksigns(uint32_t i7) { return i7 | ((popc(i7) & 1u) << 7); }

// Reads 32-bit words starting at byte offset `off` of a block.  A is the alignment the caller
// guarantees for that address (16, 8, 4: vector or word loads; 2: aligned word loads plus funnel
// shifts when the address is 2 (mod 4) -- the branch is the same for every lane of a warp, since
// rows start 16-byte aligned and all rows of a tile see the block at the same offset).
// On the device a block lives in shared memory and is addressed by its 32-bit shared-window
// address, so that field offsets fold into the load instructions.
#if TF_DEVICE
__device__ __forceinline__ uint32_t lds_u16(uint32_t a) { uint16_t v; asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a)); return v; }
__device__ __forceinline__ uint32_t lds_u32(uint32_t a) { uint32_t v; asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a)); return v; }
__device__ __forceinline__ uint2 lds_v2(uint32_t a) { uint2 v; asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a)); return v; }
__device__ __forceinline__ uint4 lds_v4(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
struct BlockLd {
  uint32_t p;        // shared-window address of the block's first byte
  __device__ __forceinline__ uint32_t u16(int off) const { return lds_u16(p + off); }
  template <int NW, int A>
  __device__ __forceinline__ void words(int off, uint32_t (&out)[NW]) const {
    const uint32_t a = p + off;
    if constexpr (A >= 16 && NW % 4 == 0) {
#pragma unroll
      for (int i = 0; i < NW / 4; i++) {
        const uint4 v = lds_v4(a + 16 * i);
        out[4 * i] = v.x; out[4 * i + 1] = v.y; out[4 * i + 2] = v.z; out[4 * i + 3] = v.w;
      }
    } else if constexpr (A >= 8 && NW % 2 == 0) {
#pragma unroll
      for (int i = 0; i < NW / 2; i++) {
        const uint2 v = lds_v2(a + 8 * i);
        out[2 * i] = v.x; out[2 * i + 1] = v.y;
      }
    } else if constexpr (A >= 4) {
#pragma unroll
      for (int i = 0; i < NW; i++) out[i] = lds_u32(a + 4 * i);
    } else {
      // 2-byte aligned: NW + 1 aligned words and a funnel shift by 0 or 16 bits (no branch: a branch
      // here would leave the compiler unsure that the warp is converged at the next mma.sync)
      const uint32_t base = a & ~3u, sh = (a & 2u) << 3;
      uint32_t prev = lds_u32(base);
#pragma unroll
      for (int i = 0; i < NW; i++) { const uint32_t cur = lds_u32(base + 4 + 4 * i); out[i] = __funnelshift_r(prev, cur, sh); prev = cur; }
    }
  }
};
// Per-CTA lookup tables in shared memory.
struct Tables {
  uint32_t grid;           // shared-window address of the format's grid: 8 (IQ1, IQ2) or 4 (IQ3) code bytes per entry
  uint32_t kv[4];          // IQ4_XS: the sixteen codes kvalues + 128, four per register
};
#else
struct BlockLd {
  const uint8_t* p;
  uint32_t u16(int off) const { uint16_t v; memcpy(&v, p + off, 2); return v; }
  template <int NW, int A>
  void words(int off, uint32_t (&out)[NW]) const {
    for (int i = 0; i < NW; i++) memcpy(&out[i], p + off + 4 * i, 4);
  }
};
struct Tables {
  const uint8_t* grid;
  uint32_t kv[4];
};
#endif
struct NoRun {};

// =============================================================================================
// Q4_K  (144 B: d, dmin, 12 packed 6-bit scales/mins, 128 nibble bytes)
// run t = sub-blocks 2t (low nibbles of qs[32t..32t+32)) and 2t+1 (high nibbles); group 0 is the
// low-nibble sub-block, group 1 the high-nibble one (staged times 2^-4, the mask keeps the nibble
// in place).  Contribution of a sub-block: (d * sc) * acc - (dmin * mn) * sum(x).
struct Q4K {
  static constexpr int kQt = 12, kTs = 144, kAlign = 16, kOct = 8, kGroupOct = 4, kSumOct = 4, kPairOrder = 0;
  static constexpr bool kSums = true, kUnrollGroups = true;
  static constexpr int kTableBytes = 0;
  struct Run { uint32_t q[8]; float dl[2], ndm[2]; };
  struct Group { const Run* r; uint32_t mask; float dl, ndm; };
  TF_HD static void src_quads(int t, int oo, int& a, int& b) { a = 64 * t + 8 * oo; b = a + 4; }
  TF_HD static int x_exp(int, int oo) { return oo >= 4 ? -4 : 0; }
  TF_HD static Run load_run(const BlockLd& ld, int t) {
    Run r;
    uint32_t h[4];
    ld.words<4, 16>(0, h);
    ld.words<8, 16>(16 + 32 * t, r.q);
    const float d = f16_bits_to_float(h[0] & 0xFFFF), dmin = f16_bits_to_float(h[0] >> 16);
    // 6-bit scale / min of sub-blocks 2t, 2t+1: plain fields for t < 2, split fields for t >= 2
    const int sh = 16 * (t & 1);
    const uint32_t a = h[1] >> sh, m = h[2] >> sh, md = h[3] >> sh;
    const bool low = t < 2;       // selects, not a branch: the warp stays converged for the MMAs
    const uint32_t scp = low ? (a & 0x3F3F) : ((md & 0x0F0F) | ((a >> 2) & 0x3030));
    const uint32_t mnp = low ? (m & 0x3F3F) : (((md >> 4) & 0x0F0F) | ((m >> 2) & 0x3030));
    r.dl[0] = mulf(d, u2f(scp & 0xFF)); r.dl[1] = mulf(d, u2f(scp >> 8));
    r.ndm[0] = -mulf(dmin, u2f(mnp & 0xFF)); r.ndm[1] = -mulf(dmin, u2f(mnp >> 8));
    return r;
  }
  TF_HD static Group load_group(const BlockLd&, const Run& r, int, int grp) {
    return Group{&r, grp ? 0x00F000F0u : 0x000F000Fu, r.dl[grp], r.ndm[grp]};
  }
  TF_HD static void octet(const Group& g, int q, const Tables&, uint32_t (&p)[4]) {
    const uint32_t w0 = g.r->q[2 * q], w1 = g.r->q[2 * q + 1];
    p[0] = w0 & g.mask; p[1] = (w0 >> 8) & g.mask; p[2] = w1 & g.mask; p[3] = (w1 >> 8) & g.mask;
  }
  TF_HD static float fold(const Group& g, float acc, float xsum, float out) {
    return fmaf_(g.ndm, xsum, fmaf_(g.dl, acc, out));
  }
};

// =============================================================================================
// Q2_K  (84 B: 16 scale|min bytes, 64 quant bytes, d, dmin)
// weight e = 128 h + 32 s + p: code = (qs[32 h + p] >> 2 s) & 3, scale byte e / 16.
// run t = (h, u) = (t >> 1, t & 1): the sixteen bytes qs[32 h + 16 u ..+16) at all four shifts;
// group = shift s (16 weights, two octets = the two word pairs), staged times 2^-2s.
struct Q2K {
  static constexpr int kQt = 10, kTs = 84, kAlign = 4, kOct = 8, kGroupOct = 2, kSumOct = 2, kPairOrder = 0;
  static constexpr bool kSums = true, kUnrollGroups = true;
  static constexpr int kTableBytes = 0;
  struct Run { uint32_t q[4]; uint32_t sc[4]; float d, ndmin; };
  struct Group { const Run* r; uint32_t mask; float dl, ndm; };
  TF_HD static void src_quads(int t, int oo, int& a, int& b) {
    a = 128 * (t >> 1) + 32 * (oo >> 1) + 16 * (t & 1) + 8 * (oo & 1);
    b = a + 4;
  }
  TF_HD static int x_exp(int, int oo) { return -2 * (oo >> 1); }
  TF_HD static Run load_run(const BlockLd& ld, int t) {
    Run r;
    ld.words<4, 4>(16 + 16 * t, r.q);
    uint32_t dd[1], s2[2];
    ld.words<1, 4>(80, dd);
    r.d = f16_bits_to_float(dd[0] & 0xFFFF);
    r.ndmin = -f16_bits_to_float(dd[0] >> 16);
    // scale byte of group s: index 8 h + 2 s + u -> byte (2 s + u) of the eight bytes at 8 h
    ld.words<2, 4>(8 * (t >> 1), s2);
    const int u = t & 1;
    r.sc[0] = (s2[0] >> (8 * u)) & 0xFF; r.sc[1] = (s2[0] >> (16 + 8 * u)) & 0xFF;
    r.sc[2] = (s2[1] >> (8 * u)) & 0xFF; r.sc[3] = (s2[1] >> (16 + 8 * u)) & 0xFF;
    return r;
  }
  TF_HD static Group load_group(const BlockLd&, const Run& r, int, int grp) {
    return Group{&r, 0x00030003u << (2 * grp), mulf(r.d, u2f(r.sc[grp] & 15)), mulf(r.ndmin, u2f(r.sc[grp] >> 4))};
  }
  TF_HD static void octet(const Group& g, int q, const Tables&, uint32_t (&p)[4]) {
    const uint32_t w0 = g.r->q[2 * q], w1 = g.r->q[2 * q + 1];
    p[0] = w0 & g.mask; p[1] = (w0 >> 8) & g.mask; p[2] = w1 & g.mask; p[3] = (w1 >> 8) & g.mask;
  }
  TF_HD static float fold(const Group& g, float acc, float xsum, float out) {
    return fmaf_(g.ndm, xsum, fmaf_(g.dl, acc, out));
  }
};

// =============================================================================================
// Q5_K  (176 B: d, dmin, 12 packed 6-bit scales/mins, 32 bytes of fifth bits, 128 nibble bytes)
// code = nibble | bit k of qh[p] << 4 for sub-block k, element p.  Two planes per sub-block: the
// nibbles (as Q4_K) and the fifth bits, kept in place as qh & (0x00010001 << k) = bit * 2^k and
// staged times 2^(4 - k), so that nibble and bit products add up in one accumulator to sum(code * x).
// run t = sub-blocks 2t, 2t+1 = groups 0, 1 of eight octets: four of nibbles, four of fifth bits.
struct Q5K {
  static constexpr int kQt = 13, kTs = 176, kAlign = 16, kOct = 16, kGroupOct = 8, kSumOct = 4, kPairOrder = 0;
  static constexpr bool kSums = true, kUnrollGroups = true;
  static constexpr int kTableBytes = 0;
  struct Run { uint32_t q[8], h[8]; float dl[2], ndm[2]; int t; };
  struct Group { const Run* r; uint32_t mask_q, mask_h; float dl, ndm; };
  TF_HD static void src_quads(int t, int oo, int& a, int& b) { a = 64 * t + 32 * (oo >> 3) + 8 * (oo & 3); b = a + 4; }
  TF_HD static int x_exp(int t, int oo) {
    const int k = 2 * t + (oo >> 3);
    return (oo & 4) ? 4 - k : ((oo >> 3) ? -4 : 0);
  }
  TF_HD static Run load_run(const BlockLd& ld, int t) {
    Run r;
    uint32_t h[4];
    ld.words<4, 16>(0, h);
    ld.words<8, 16>(16, r.h);
    ld.words<8, 16>(48 + 32 * t, r.q);
    r.t = t;
    const float d = f16_bits_to_float(h[0] & 0xFFFF), dmin = f16_bits_to_float(h[0] >> 16);
    const int sh = 16 * (t & 1);
    const uint32_t a = h[1] >> sh, m = h[2] >> sh, md = h[3] >> sh;
    const bool low = t < 2;
    const uint32_t scp = low ? (a & 0x3F3F) : ((md & 0x0F0F) | ((a >> 2) & 0x3030));
    const uint32_t mnp = low ? (m & 0x3F3F) : (((md >> 4) & 0x0F0F) | ((m >> 2) & 0x3030));
    r.dl[0] = mulf(d, u2f(scp & 0xFF)); r.dl[1] = mulf(d, u2f(scp >> 8));
    r.ndm[0] = -mulf(dmin, u2f(mnp & 0xFF)); r.ndm[1] = -mulf(dmin, u2f(mnp >> 8));
    return r;
  }
  TF_HD static Group load_group(const BlockLd&, const Run& r, int, int grp) {
    return Group{&r, grp ? 0x00F000F0u : 0x000F000Fu, 0x00010001u << (2 * r.t + grp), r.dl[grp], r.ndm[grp]};
  }
  // octets 0-3: the nibbles of the sub-block, octets 4-7: its fifth bits (both add into one accumulator)
  TF_HD static void octet(const Group& g, int q, const Tables&, uint32_t (&p)[4]) {
    const uint32_t* w = q < 4 ? g.r->q : g.r->h;
    const uint32_t m = q < 4 ? g.mask_q : g.mask_h;
    const uint32_t w0 = w[2 * (q & 3)], w1 = w[2 * (q & 3) + 1];
    p[0] = w0 & m; p[1] = (w0 >> 8) & m; p[2] = w1 & m; p[3] = (w1 >> 8) & m;
  }
  TF_HD static float fold(const Group& g, float acc, float xsum, float out) {
    return fmaf_(g.ndm, xsum, fmaf_(g.dl, acc, out));
  }
};

// =============================================================================================
// Q6_K  (210 B: 128 low-nibble bytes, 64 bytes of 2-bit highs, 16 int8 scales, d)
// element e = 128 h + 32 c + p: low = nibble (c >> 1) of ql[64 h + 32 (c & 1) + p], high = bits 2c, 2c+1 of
// qh[32 h + p], weight = d * sc[8 h + 2 c + (p >> 4)] * (low + 16 high - 32).
// run t = (h, u) = (t >> 1, t & 1): elements p in [16 u, 16 u + 16) of every c, i.e. four scale groups
// of 16.  Two planes per group: the nibbles and the 2-bit highs kept in place (high * 4^c, staged times
// 2^(4 - 2c)) add up in one accumulator to sum((low + 16 high) * x); group c = two octets of nibbles,
// then two of highs.
struct Q6K {
  static constexpr int kQt = 14, kTs = 210, kAlign = 2, kOct = 16, kGroupOct = 4, kSumOct = 2, kPairOrder = 0;
  static constexpr bool kSums = true, kUnrollGroups = true;
  static constexpr int kTableBytes = 0;
  struct Run { uint32_t qa[4], qb[4], qh[4]; float dl[4]; };
  struct Group { const uint32_t* lo; const uint32_t* hi; uint32_t mask_lo, mask_hi; float dl; };
  TF_HD static void src_quads(int t, int oo, int& a, int& b) {
    a = 128 * (t >> 1) + 32 * (oo >> 2) + 16 * (t & 1) + 8 * (oo & 1);
    b = a + 4;
  }
  TF_HD static int x_exp(int, int oo) {
    const int c = oo >> 2;
    return (oo & 2) ? 4 - 2 * c : ((c >> 1) ? -4 : 0);
  }
  TF_HD static Run load_run(const BlockLd& ld, int t) {
    Run r;
    const int h = t >> 1, u = t & 1;
    ld.words<4, 2>(64 * h + 16 * u, r.qa);
    ld.words<4, 2>(64 * h + 32 + 16 * u, r.qb);
    ld.words<4, 2>(128 + 32 * h + 16 * u, r.qh);
    uint32_t sc[2];
    ld.words<2, 2>(192 + 8 * h, sc);
    const float d = f16_bits_to_float(ld.u16(208));
    for (int c = 0; c < 4; c++) {
      const uint32_t byte = (sc[c >> 1] >> (16 * (c & 1) + 8 * u)) & 0xFF;
      r.dl[c] = mulf(d, (float)(int)(int8_t)byte);
    }
    return r;
  }
  TF_HD static Group load_group(const BlockLd&, const Run& r, int, int grp) {
    return Group{(grp & 1) ? r.qb : r.qa, r.qh, (grp >> 1) ? 0x00F000F0u : 0x000F000Fu, 0x00030003u << (2 * grp), r.dl[grp]};
  }
  // octets 0-1: the nibbles of the group's sixteen weights, octets 2-3: their 2-bit highs
  TF_HD static void octet(const Group& g, int q, const Tables&, uint32_t (&p)[4]) {
    const uint32_t* w = q < 2 ? g.lo : g.hi;
    const uint32_t m = q < 2 ? g.mask_lo : g.mask_hi;
    const uint32_t w0 = w[2 * (q & 1)], w1 = w[2 * (q & 1) + 1];
    p[0] = w0 & m; p[1] = (w0 >> 8) & m; p[2] = w1 & m; p[3] = (w1 >> 8) & m;
  }
  TF_HD static float fold(const Group& g, float acc, float xsum, float out) {
    return fmaf_(g.dl, fmaf_(-32.0f, xsum, acc), out);
  }
};

// =============================================================================================
// IQ4_XS  (136 B: d, scales_h, 4 scales_l bytes, 128 nibble bytes)
// sub-block j (32 weights): low nibbles of qs[16 j ..+16) are weights 0-15, high nibbles 16-31;
// weight = d * (ls - 32) * kvalues[nibble].  Codes are kvalues + 128 (1..241), looked up with byte
// permutes from four registers; the fold takes the 128 * sum(x) back out.
// run t = sub-blocks 2t, 2t+1 = groups 0, 1; octet q of a group = word q of the sub-block: its four
// low nibbles (weights 4q..4q+3) and four high nibbles (16+4q..): MMA 1 takes the first two bytes
// of the word, MMA 2 the last two (pair order 1).
struct IQ4XS {
  static constexpr int kQt = 23, kTs = 136, kAlign = 8, kOct = 8, kGroupOct = 4, kSumOct = 4, kPairOrder = 1;
  static constexpr bool kSums = true, kUnrollGroups = false;
  static constexpr int kTableBytes = 0;
  typedef NoRun Run;
  struct Group { uint32_t q[4]; float dl; };
  TF_HD static void src_quads(int t, int oo, int& a, int& b) {
    a = 64 * t + 32 * (oo >> 2) + 4 * (oo & 3);
    b = a + 16;
  }
  TF_HD static int x_exp(int, int) { return 0; }
  TF_HD static Run load_run(const BlockLd&, int) { return Run{}; }
  TF_HD static Group load_group(const BlockLd& ld, const Run&, int t, int grp) {
    Group g;
    ld.words<4, 8>(8 + 32 * t + 16 * grp, g.q);
    uint32_t h[2];
    ld.words<2, 8>(0, h);                    // d | scales_h << 16, scales_l[0..3]
    const int j = 2 * t + grp;
    const int ls = (int)(((h[1] >> (4 * j)) & 15) | (((h[0] >> (16 + 2 * j)) & 3) << 4)) - 32;
    g.dl = mulf(f16_bits_to_float(h[0] & 0xFFFF), (float)ls);
    return g;
  }
  // Sixteen-entry lookup of the four nibbles held in the low 16 bits of `sel`: result bytes in
  // nibble order (byte0.lo, byte0.hi, byte1.lo, byte1.hi).
  TF_HD static uint32_t lookup4(const Tables& tb, uint32_t sel) {
    const uint32_t s7 = sel & 0x7777u;
    const uint32_t lo = prmt(tb.kv[0], tb.kv[1], s7), hi = prmt(tb.kv[2], tb.kv[3], s7);
    return prmt(lo, hi, ((sel >> 1) & 0x4444u) | 0x3210u);
  }
  TF_HD static void octet(const Group& g, int q, const Tables& tb, uint32_t (&p)[4]) {
    const uint32_t w = g.q[q];
    const uint32_t c0 = lookup4(tb, w), c1 = lookup4(tb, w >> 16);
    p[0] = pair02(c0); p[1] = pair13(c0); p[2] = pair02(c1); p[3] = pair13(c1);
  }
  TF_HD static float fold(const Group& g, float acc, float xsum, float out) {
    return fmaf_(g.dl, fmaf_(-128.0f, xsum, acc), out);
  }
};

// =============================================================================================
// Grid formats.  Common shape: an octet is one 8-byte grid entry (IQ2, IQ1) or two 4-byte entries
// (IQ3) of unsigned code bytes, times eight sign bits.
template <int ENTRY_BYTES>
TF_HD void grid_words(const Tables& tb, uint32_t i0, uint32_t i1, uint32_t& w0, uint32_t& w1) {
#if TF_DEVICE
  if (ENTRY_BYTES == 8) {
    const uint2 v = lds_v2(tb.grid + 8 * i0);
    w0 = v.x; w1 = v.y;
  } else {
    w0 = lds_u32(tb.grid + 4 * i0);
    w1 = lds_u32(tb.grid + 4 * i1);
  }
#else
  if (ENTRY_BYTES == 8) { memcpy(&w0, tb.grid + 8 * i0, 4); memcpy(&w1, tb.grid + 8 * i0 + 4, 4); }
  else { memcpy(&w0, tb.grid + 4 * i0, 4); memcpy(&w1, tb.grid + 4 * i1, 4); }
#endif
}
TF_HD void signed_octet(uint32_t w0, uint32_t w1, uint32_t signs8, uint32_t (&p)[4]) {
  const uint32_t s0 = spread_signs4(signs8), s1 = spread_signs4(signs8 >> 4);
  p[0] = pair02s(w0, s0); p[1] = pair13s(w0, s0); p[2] = pair02s(w1, s1); p[3] = pair13s(w1, s1);
}
TF_HD void plain_octet(uint32_t w0, uint32_t w1, uint32_t (&p)[4]) {
  p[0] = pair02(w0); p[1] = pair13(w0); p[2] = pair02(w1); p[3] = pair13(w1);
}

// IQ2_XXS (66 B: d, 8 x {4 index bytes, u32 = 4 x 7-bit sign index | 4-bit scale << 28}); group = one of them
struct IQ2XXS {
  static constexpr int kQt = 16, kTs = 66, kAlign = 2, kOct = 8, kGroupOct = 4, kSumOct = 4, kPairOrder = 0;
  static constexpr bool kSums = false, kUnrollGroups = false;
  static constexpr int kTableBytes = 256 * 8;
  typedef NoRun Run;
  struct Group { uint32_t q[2]; float db; };
  TF_HD static void src_quads(int t, int oo, int& a, int& b) { a = 64 * t + 8 * oo; b = a + 4; }
  TF_HD static int x_exp(int, int) { return 0; }
  TF_HD static Run load_run(const BlockLd&, int) { return Run{}; }
  TF_HD static Group load_group(const BlockLd& ld, const Run&, int t, int grp) {
    Group g;
    ld.words<2, 2>(2 + 16 * t + 8 * grp, g.q);
    g.db = mulf(mulf(f16_bits_to_float(ld.u16(0)), 0.5f + u2f(g.q[1] >> 28)), 0.25f);
    return g;
  }
  TF_HD static void octet(const Group& g, int q, const Tables& tb, uint32_t (&p)[4]) {
    uint32_t w0, w1;
    grid_words<8>(tb, (g.q[0] >> (8 * q)) & 0xFF, 0, w0, w1);
    signed_octet(w0, w1, ksigns((g.q[1] >> (7 * q)) & 127), p);
  }
  TF_HD static float fold(const Group& g, float acc, float, float out) { return fmaf_(g.db, acc, out); }
};

// IQ2_XS (74 B: d, 32 x u16 = 9-bit grid index | 7-bit sign index << 9, 8 scale bytes of two nibbles)
struct IQ2XS {
  static constexpr int kQt = 17, kTs = 74, kAlign = 2, kOct = 8, kGroupOct = 2, kSumOct = 2, kPairOrder = 0;
  static constexpr bool kSums = false, kUnrollGroups = false;
  static constexpr int kTableBytes = 512 * 8;
  typedef NoRun Run;
  struct Group { uint32_t q; float db; };
  TF_HD static void src_quads(int t, int oo, int& a, int& b) { a = 64 * t + 8 * oo; b = a + 4; }
  TF_HD static int x_exp(int, int) { return 0; }
  TF_HD static Run load_run(const BlockLd&, int) { return Run{}; }
  TF_HD static Group load_group(const BlockLd& ld, const Run&, int t, int grp) {
    Group g;
    g.q = ld.u16(2 + 16 * t + 4 * grp) | (ld.u16(4 + 16 * t + 4 * grp) << 16);
    const uint32_t sc = (ld.u16(66 + 2 * t) >> (4 * grp)) & 15;
    g.db = mulf(mulf(f16_bits_to_float(ld.u16(0)), 0.5f + u2f(sc)), 0.25f);
    return g;
  }
  TF_HD static void octet(const Group& g, int q, const Tables& tb, uint32_t (&p)[4]) {
    const uint32_t q16 = (g.q >> (16 * q)) & 0xFFFF;
    uint32_t w0, w1;
    grid_words<8>(tb, q16 & 511, 0, w0, w1);
    signed_octet(w0, w1, ksigns(q16 >> 9), p);
  }
  TF_HD static float fold(const Group& g, float acc, float, float out) { return fmaf_(g.db, acc, out); }
};

// IQ2_S (82 B: d, 32 index bytes, 32 sign bytes, 8 bytes of 2 high index bits, 8 scale bytes)
struct IQ2S {
  static constexpr int kQt = 22, kTs = 82, kAlign = 2, kOct = 8, kGroupOct = 2, kSumOct = 2, kPairOrder = 0;
  static constexpr bool kSums = false, kUnrollGroups = false;
  static constexpr int kTableBytes = 1024 * 8;
  typedef NoRun Run;
  struct Group { uint32_t qs, sg, qh; float db; };
  TF_HD static void src_quads(int t, int oo, int& a, int& b) { a = 64 * t + 8 * oo; b = a + 4; }
  TF_HD static int x_exp(int, int) { return 0; }
  TF_HD static Run load_run(const BlockLd&, int) { return Run{}; }
  TF_HD static Group load_group(const BlockLd& ld, const Run&, int t, int grp) {
    Group g;
    g.qs = ld.u16(2 + 8 * t + 2 * grp);
    g.sg = ld.u16(34 + 8 * t + 2 * grp);
    g.qh = ld.u16(66 + 2 * t) >> (4 * grp);
    const uint32_t sc = (ld.u16(74 + 2 * t) >> (4 * grp)) & 15;
    g.db = mulf(mulf(f16_bits_to_float(ld.u16(0)), 0.5f + u2f(sc)), 0.25f);
    return g;
  }
  TF_HD static void octet(const Group& g, int q, const Tables& tb, uint32_t (&p)[4]) {
    const uint32_t idx = ((g.qs >> (8 * q)) & 0xFF) | (((g.qh >> (2 * q)) & 3) << 8);
    uint32_t w0, w1;
    grid_words<8>(tb, idx, 0, w0, w1);
    signed_octet(w0, w1, (g.sg >> (8 * q)) & 0xFF, p);
  }
  TF_HD static float fold(const Group& g, float acc, float, float out) { return fmaf_(g.db, acc, out); }
};

// IQ3_XXS (98 B: d, 64 index bytes (one per 4 weights), 8 x u32 = 4 x 7-bit sign index | scale << 28)
struct IQ3XXS {
  static constexpr int kQt = 18, kTs = 98, kAlign = 2, kOct = 8, kGroupOct = 4, kSumOct = 4, kPairOrder = 0;
  static constexpr bool kSums = false, kUnrollGroups = false;
  static constexpr int kTableBytes = 256 * 4;
  typedef NoRun Run;
  struct Group { uint32_t q[2], aux; float db; };
  TF_HD static void src_quads(int t, int oo, int& a, int& b) { a = 64 * t + 8 * oo; b = a + 4; }
  TF_HD static int x_exp(int, int) { return 0; }
  TF_HD static Run load_run(const BlockLd&, int) { return Run{}; }
  TF_HD static Group load_group(const BlockLd& ld, const Run&, int t, int grp) {
    Group g;
    ld.words<2, 2>(2 + 16 * t + 8 * grp, g.q);
    uint32_t a[1];
    ld.words<1, 2>(66 + 8 * t + 4 * grp, a);
    g.aux = a[0];
    g.db = mulf(mulf(f16_bits_to_float(ld.u16(0)), 0.5f + u2f(g.aux >> 28)), 0.5f);
    return g;
  }
  TF_HD static void octet(const Group& g, int q, const Tables& tb, uint32_t (&p)[4]) {
    const uint32_t q16 = (g.q[q >> 1] >> (16 * (q & 1))) & 0xFFFF;
    uint32_t w0, w1;
    grid_words<4>(tb, q16 & 0xFF, q16 >> 8, w0, w1);
    signed_octet(w0, w1, ksigns((g.aux >> (7 * q)) & 127), p);
  }
  TF_HD static float fold(const Group& g, float acc, float, float out) { return fmaf_(g.db, acc, out); }
};

// IQ3_S (110 B: d, 64 index bytes, 8 bytes of ninth index bits, 32 sign bytes, 4 scale bytes of two nibbles)
struct IQ3S {
  static constexpr int kQt = 21, kTs = 110, kAlign = 2, kOct = 8, kGroupOct = 4, kSumOct = 4, kPairOrder = 0;
  static constexpr bool kSums = false, kUnrollGroups = false;
  static constexpr int kTableBytes = 512 * 4;
  typedef NoRun Run;
  struct Group { uint32_t q[2], sg, qh; float db; };
  TF_HD static void src_quads(int t, int oo, int& a, int& b) { a = 64 * t + 8 * oo; b = a + 4; }
  TF_HD static int x_exp(int, int) { return 0; }
  TF_HD static Run load_run(const BlockLd&, int) { return Run{}; }
  TF_HD static Group load_group(const BlockLd& ld, const Run&, int t, int grp) {
    Group g;
    ld.words<2, 2>(2 + 16 * t + 8 * grp, g.q);
    uint32_t s[1];
    ld.words<1, 2>(74 + 8 * t + 4 * grp, s);
    g.sg = s[0];
    g.qh = ld.u16(66 + 2 * t) >> (8 * grp);
    const uint32_t sc = (ld.u16(106 + (t & 2)) >> (8 * (t & 1) + 4 * grp)) & 15;
    g.db = mulf(f16_bits_to_float(ld.u16(0)), u2f(1 + 2 * sc));
    return g;
  }
  TF_HD static void octet(const Group& g, int q, const Tables& tb, uint32_t (&p)[4]) {
    const uint32_t q16 = (g.q[q >> 1] >> (16 * (q & 1))) & 0xFFFF;
    const uint32_t i0 = (q16 & 0xFF) | (((g.qh >> (2 * q)) & 1) << 8);
    const uint32_t i1 = (q16 >> 8) | (((g.qh >> (2 * q + 1)) & 1) << 8);
    uint32_t w0, w1;
    grid_words<4>(tb, i0, i1, w0, w1);
    signed_octet(w0, w1, (g.sg >> (8 * q)) & 0xFF, p);
  }
  TF_HD static float fold(const Group& g, float acc, float, float out) { return fmaf_(g.db, acc, out); }
};

// IQ1_S (50 B: d, 32 index bytes, 8 x u16 = 4 x 3 high index bits | 3-bit scale << 12 | delta sign << 15)
// weight = d (2 s + 1) (grid + delta), grid in {-1, 0, 1}, delta = -+1/8.  The shared-memory table
// holds the codes 8 grid + 9 (1, 9, 17); adding or subtracting 1 in every byte applies delta, the
// fold removes the 9 and the factor 8:  (dl / 8) * (sum(code x) - 9 sum(x)).
struct IQ1S {
  static constexpr int kQt = 19, kTs = 50, kAlign = 2, kOct = 8, kGroupOct = 4, kSumOct = 4, kPairOrder = 0;
  static constexpr bool kSums = true, kUnrollGroups = false;
  static constexpr int kTableBytes = 2048 * 8;
  typedef NoRun Run;
  struct Group { uint32_t qs, qh, dlt; float dl8; };
  TF_HD static void src_quads(int t, int oo, int& a, int& b) { a = 64 * t + 8 * oo; b = a + 4; }
  TF_HD static int x_exp(int, int) { return 0; }
  TF_HD static Run load_run(const BlockLd&, int) { return Run{}; }
  TF_HD static Group load_group(const BlockLd& ld, const Run&, int t, int grp) {
    Group g;
    g.qs = ld.u16(2 + 8 * t + 4 * grp) | (ld.u16(4 + 8 * t + 4 * grp) << 16);
    g.qh = ld.u16(34 + 4 * t + 2 * grp);
    g.dlt = (g.qh & 0x8000) ? 0xFEFEFEFFu : 0x01010101u;      // -1 / +1 in every byte
    g.dl8 = mulf(mulf(f16_bits_to_float(ld.u16(0)), u2f(2 * ((g.qh >> 12) & 7) + 1)), 0.125f);
    return g;
  }
  TF_HD static void octet(const Group& g, int q, const Tables& tb, uint32_t (&p)[4]) {
    const uint32_t idx = ((g.qs >> (8 * q)) & 0xFF) | (((g.qh >> (3 * q)) & 7) << 8);
    uint32_t w0, w1;
    grid_words<8>(tb, idx, 0, w0, w1);
    plain_octet(w0 + g.dlt, w1 + g.dlt, p);
  }
  TF_HD static float fold(const Group& g, float acc, float xsum, float out) {
    return fmaf_(g.dl8, fmaf_(-9.0f, xsum, acc), out);
  }
};

// IQ1_M (56 B: 32 index bytes, 16 bytes of 2 x {3 high index bits, delta sign}, 4 x u16 = 4 x 3-bit scale |
// a nibble of the f16 super-scale << 12)
struct IQ1M {
  static constexpr int kQt = 29, kTs = 56, kAlign = 8, kOct = 8, kGroupOct = 2, kSumOct = 2, kPairOrder = 0;
  static constexpr bool kSums = true, kUnrollGroups = false;
  static constexpr int kTableBytes = 2048 * 8;
  typedef NoRun Run;
  struct Group { uint32_t qs, qh; float dl8; };
  TF_HD static void src_quads(int t, int oo, int& a, int& b) { a = 64 * t + 8 * oo; b = a + 4; }
  TF_HD static int x_exp(int, int) { return 0; }
  TF_HD static Run load_run(const BlockLd&, int) { return Run{}; }
  TF_HD static Group load_group(const BlockLd& ld, const Run&, int t, int grp) {
    Group g;
    g.qs = ld.u16(8 * t + 2 * grp);
    g.qh = (ld.u16(32 + 4 * t + (grp & 2)) >> (8 * (grp & 1))) & 0xFF;
    uint32_t sc[2];
    ld.words<2, 8>(48, sc);
    const uint32_t dbits = ((sc[0] >> 12) & 0x000F) | ((sc[0] >> 24) & 0x00F0) | ((sc[1] >> 4) & 0x0F00) | ((sc[1] >> 16) & 0xF000);
    const uint32_t w = (sc[t >> 1] >> (16 * (t & 1))) & 0xFFFF;
    g.dl8 = mulf(mulf(f16_bits_to_float(dbits), u2f(2 * ((w >> (3 * grp)) & 7) + 1)), 0.125f);
    return g;
  }
  TF_HD static void octet(const Group& g, int q, const Tables& tb, uint32_t (&p)[4]) {
    const uint32_t n = (g.qh >> (4 * q)) & 15;
    const uint32_t idx = ((g.qs >> (8 * q)) & 0xFF) | ((n & 7) << 8);
    uint32_t w0, w1;
    grid_words<8>(tb, idx, 0, w0, w1);
    const uint32_t dlt = (n & 8) ? 0xFEFEFEFFu : 0x01010101u;
    plain_octet(w0 + dlt, w1 + dlt, p);
  }
  TF_HD static float fold(const Group& g, float acc, float xsum, float out) {
    return fmaf_(g.dl8, fmaf_(-9.0f, xsum, acc), out);
  }
};

}  // namespace tf
}  // namespace ggq
