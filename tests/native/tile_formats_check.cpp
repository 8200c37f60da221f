// Host-side check of gguf_jax_b200/csrc/tile_formats.cuh: for every lane run and octet of random
// blocks, the A-operand registers, the activation map and the fold of a format must reproduce the
// decoded weights (given in a file written by the Python test from the CPU decoders).
//
// usage: tile_formats_check <qtype> <blocks.bin> <decoded_f32.bin> <table.bin> <n_blocks>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "../../gguf_jax_b200/csrc/tile_formats.cuh"

using namespace ggq::tf;

static std::vector<uint8_t> slurp(const char* path) {
  FILE* f = fopen(path, "rb");
  if (!f) { fprintf(stderr, "cannot open %s\n", path); exit(2); }
  fseek(f, 0, SEEK_END);
  long n = ftell(f);
  fseek(f, 0, SEEK_SET);
  std::vector<uint8_t> v(n);
  if (fread(v.data(), 1, n, f) != (size_t)n) exit(2);
  fclose(f);
  return v;
}

// value of one half of a pair register: +-v * 2^-133 stands for the integer +-v
static double code_of(uint32_t half) {
  if (half & 0x7F00) { fprintf(stderr, "pair register with exponent bits set: %04x\n", half); exit(1); }
  const double v = half & 0xFF;
  return (half & 0x8000) ? -v : v;
}

template <class F>
int check(const std::vector<uint8_t>& blocks, const float* want, const Tables& tb, int nb) {
  long bad = 0, seen = 0;
  std::vector<int> cover(256);
  for (int b = 0; b < nb; b++) {
    std::fill(cover.begin(), cover.end(), 0);
    // the kernel sees blocks at 2-byte aligned addresses: give the loader exactly that
    std::vector<uint8_t> buf(F::kTs + 48);
    uint8_t* p = buf.data() + 2 * (b % 3);
    memcpy(p, blocks.data() + (size_t)b * F::kTs, F::kTs);
    BlockLd ld{p};
    if ((uintptr_t)p % F::kAlign) p += F::kAlign - (uintptr_t)p % F::kAlign;
    memcpy(p, blocks.data() + (size_t)b * F::kTs, F::kTs);
    ld = BlockLd{p};
    for (int t = 0; t < 4; t++) {
      const typename F::Run run = F::load_run(ld, t);
      for (int grp = 0; grp < F::kOct / F::kGroupOct; grp++) {
        const typename F::Group raw = F::load_group(ld, run, t, grp);
        // one-hot activations, one weight at a time: the group's accumulator receives code * x from every
        // octet the weight appears in (one, or one per plane), the sum of x is 1
        std::vector<double> acc(256, 0.0);
        std::vector<int> in_group(256, 0), in_sum(256, 0);
        for (int oo = grp * F::kGroupOct; oo < (grp + 1) * F::kGroupOct; oo++) {
          uint32_t pr[4];
          F::octet(raw, oo - grp * F::kGroupOct, tb, pr);
          int qa, qb;
          F::src_quads(t, oo, qa, qb);
          const double xs = std::ldexp(1.0, F::x_exp(t, oo));    // staged activations carry this factor
          for (int m = 0; m < 2; m++) {          // MMA m: registers pr[2m] (k-slots 2t, 2t+1), pr[2m+1] (2t+8, 2t+9)
            for (int h = 0; h < 2; h++) {
              const uint32_t reg = pr[2 * m + h];
              int e0, e1;
              if (F::kPairOrder == 0) { e0 = (m ? qb : qa) + h; e1 = e0 + 2; }
              else { e0 = (h ? qb : qa) + 2 * m; e1 = e0 + 1; }
              acc[e0] += code_of(reg & 0xFFFF) * xs;
              acc[e1] += code_of(reg >> 16) * xs;
              in_group[e0]++; in_group[e1]++;
              if (oo - grp * F::kGroupOct < F::kSumOct) { in_sum[e0]++; in_sum[e1]++; }
              cover[e0]++; cover[e1]++;
            }
          }
        }
        for (int e = 0; e < 256; e++) {
          if (!in_group[e]) continue;
          if (in_sum[e] != 1) { fprintf(stderr, "weight %d enters the group's sum of x %d times\n", e, in_sum[e]); return 1; }
          const float got = F::fold(raw, (float)acc[e], 1.0f, 0.0f);
          const float ref = want[(size_t)b * 256 + e];
          seen++;
          if (!(got == ref) && !(std::isnan(got) && std::isnan(ref))) {
            if (bad < 10) fprintf(stderr, "block %d run %d group %d weight %d: got %.9g want %.9g\n", b, t, grp, e, got, ref);
            bad++;
          }
        }
      }
    }
    for (int i = 0; i < 256; i++)
      if (cover[i] != F::kOct / 8) { fprintf(stderr, "block %d: weight %d covered %d times\n", b, i, cover[i]); return 1; }
  }
  printf("qtype %d: %ld values checked, %ld mismatches\n", F::kQt, seen, bad);
  return bad ? 1 : 0;
}

int main(int argc, char** argv) {
  if (argc != 6) { fprintf(stderr, "usage: %s qtype blocks decoded table n_blocks\n", argv[0]); return 2; }
  const int qt = atoi(argv[1]), nb = atoi(argv[5]);
  const std::vector<uint8_t> blocks = slurp(argv[2]), dec = slurp(argv[3]), table = slurp(argv[4]);
  const float* want = reinterpret_cast<const float*>(dec.data());
  Tables tb{};
  tb.grid = table.data();
  if (qt == IQ4XS::kQt) memcpy(tb.kv, table.data(), 16);
  switch (qt) {
    case Q4K::kQt: return check<Q4K>(blocks, want, tb, nb);
    case Q2K::kQt: return check<Q2K>(blocks, want, tb, nb);
    case Q5K::kQt: return check<Q5K>(blocks, want, tb, nb);
    case Q6K::kQt: return check<Q6K>(blocks, want, tb, nb);
    case IQ4XS::kQt: return check<IQ4XS>(blocks, want, tb, nb);
    case IQ2XXS::kQt: return check<IQ2XXS>(blocks, want, tb, nb);
    case IQ2XS::kQt: return check<IQ2XS>(blocks, want, tb, nb);
    case IQ2S::kQt: return check<IQ2S>(blocks, want, tb, nb);
    case IQ3XXS::kQt: return check<IQ3XXS>(blocks, want, tb, nb);
    case IQ3S::kQt: return check<IQ3S>(blocks, want, tb, nb);
    case IQ1S::kQt: return check<IQ1S>(blocks, want, tb, nb);
    case IQ1M::kQt: return check<IQ1M>(blocks, want, tb, nb);
  }
  fprintf(stderr, "no tile format for qtype %d\n", qt);
  return 2;
}
