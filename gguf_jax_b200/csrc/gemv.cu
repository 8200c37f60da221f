// ggq_gemv: argument checking and kernel selection for the small-batch fused multiply.
#include "gemv.cuh"

#include <cstdlib>
#include <cstring>

using namespace ggq;

namespace {
constexpr int kGemvMaxBatch = 16;
// From this batch on the tensor-core small-batch kernel beats the per-element FMA kernel.
constexpr int kMmaMinBatch = 2;
// Up to this batch the tuned batch-1 kernels are simply launched once per batch row (only where the
// tiled kernel cannot run: no workspace, or rows that are not 16-byte aligned).
inline int tuned_max_repeat(int qtype, int64_t weight_bytes) {
  if (qtype == QT_Q6_K) return weight_bytes < (24ll << 20) ? 2 : weight_bytes < (100ll << 20) ? 3 : 4;
  return weight_bytes < (24ll << 20) ? 1 : weight_bytes < (80ll << 20) ? 2 : 3;
}
inline bool is_k_quant(int qtype) { return qtype == QT_Q4_K || qtype == QT_Q5_K || qtype == QT_Q6_K; }
// The batch-major kernel (gemv_wide.cu) costs two launches and a partial-sum settle, about 10 us on a weight
// of a few MB, and then very little per batch row; the integer-code MMA kernel (gemv_mma.cu) starts at 4 us
// and grows with the weight.  Measured crossover on B200 at 5..16 batch rows: about 20 MB for Q4_K / Q5_K
// (8192 x 2048 and 4096 x 4096, 9 MB: 10-12 us against 14-18 us; 14336 x 4096, 33 MB: 28-35 us against 24-27 us),
// about 10 MB for Q6_K (4096 x 4096, 14 MB: 20 us either way).
inline bool wide_pays(int qtype, int64_t weight_bytes) {
  return weight_bytes >= (qtype == QT_Q6_K ? (10ll << 20) : (20ll << 20));
}
// Above 16 batch rows the choice is between slices of 32 rows through the batch-major kernel and, in the
// caller, the decode kernel followed by a library GEMM.  One slice wins from about 20 MB on (Q4_K 8192 x 8192:
// 39 us against 76 us; Q6_K 14336 x 4096: 45 us against 66 us; Q5_K 4096 x 4096, 11.5 MB: 28 us against 23 us,
// its decoded copy stays in the L2); two slices or more lose, so the router's cap is 32 there and 16 elsewhere.
// The tcgen05 kernels behind ggq_gemm (integer-code and tf32 operands) are slower than both at every
// batch measured and are reached only by name, above 128 rows or for the other formats.
constexpr int kWideRouterBatch = 32;
// Above 32 rows the bf16-weight tcgen05 kernel (gemm_bf16w.cu; the fallback's own precision) is compared with the same
// fallback: on the large weights it wins up to 256 rows (Q6_K 14336 x 4096: 52 / 55 / 62 us at 64 / 128 / 256 rows against
// 67 / 68 / 75 us; Q6_K 4096 x 14336: 54 / 62 / 79 us against 70 / 73 / 80 us), and up to 512 rows where there are enough
// row tiles to fill the device without cutting K (14336 rows: 78 us against 92 us; 4096 rows: 118 us against 92 us);
// on weights of a few MB the fallback's library GEMM reads a decoded copy that stays in the L2 and wins from 64 rows on.
constexpr int kGemmRouterBatchWide = 512;      // at least 96 row tiles of 128 rows
constexpr int kGemmRouterBatch = 256;
}

extern "C" int32_t ggq_gemv_max_batch(void) { return kGemvMaxBatch; }

extern "C" int32_t ggq_fused_batch_limit(int32_t qtype, int64_t N, int64_t K) {
  const TypeInfo* ti = type_info(qtype);
  if (!ti || !ti->fused || N <= 0 || K <= 0 || K % ti->block_elems) return 0;
  if (is_k_quant(qtype) && K % 256 == 0 && (K / 256 * ti->block_bytes) % 16 == 0 &&
      wide_pays(qtype, N * (K / 256) * (int64_t)ti->block_bytes) && gemv_wide_applicable(qtype, N, K, kWideRouterBatch, nullptr, nullptr))
    return !gemm_bf16w_applicable(qtype, N, K, kGemmRouterBatch) ? kWideRouterBatch : N >= 96 * 128 ? kGemmRouterBatchWide : kGemmRouterBatch;
  return kGemvMaxBatch;
}

static int sm_count_of(int dev) { return device_sm_count(dev); }

extern "C" size_t ggq_workspace_bytes(int32_t qtype, int64_t N, int64_t K, int32_t M) {
  const TypeInfo* ti = type_info(qtype);
  if (!ti || N <= 0 || K <= 0) return 0;
  size_t need = 0;
  if (qtype == QT_Q4_K || qtype == QT_Q5_K || qtype == QT_Q6_K) need = gemv_q4k_workspace_bytes(N, kMaxSmCount);
  if (M <= kGemvMaxBatch) {
    const int tmax = gemv_tile_max_batch(qtype);
    const size_t tile = tmax ? gemv_tile_workspace_bytes(qtype, N, K, M < tmax ? M : tmax) : 0;
    if (tile > need && K % 256 == 0) need = tile;
  }
  if ((qtype == QT_Q4_K || qtype == QT_Q5_K || qtype == QT_Q6_K) && M >= 2 && K % 256 == 0) {
    const size_t wd = gemv_wide_workspace_bytes(qtype, N, K, M, kMaxSmCount);
    if (wd > need) need = wd;
  }
  if (M > kGemvMaxBatch && gemm_applicable(ti, N, K, M)) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) { dev = -1; (void)cudaGetLastError(); }
    const size_t g = gemm_workspace_bytes(N, K, M, sm_count_of(dev));
    if (g > need) need = g;
    if (gemm_codes_applicable(qtype, N, K, M)) {
      const size_t c = gemm_codes_workspace_bytes(qtype, N, K, M, sm_count_of(dev));
      if (c > need) need = c;
    }
    if (gemm_bf16w_applicable(qtype, N, K, M)) {
      const size_t c = gemm_bf16w_workspace_bytes(qtype, N, K, M, sm_count_of(dev));
      if (c > need) need = c;
    }
  }
  return need;
}

extern "C" int32_t ggq_gemv(int32_t qtype, const void* w, int64_t N, int64_t K, const void* x_bf16,
                            int32_t M, void* y, int32_t y_dtype, void* workspace, size_t workspace_bytes,
                            void* stream) {
  const TypeInfo* ti = type_info(qtype);
  if (!ti) return fail(GGQ_BAD_QTYPE, "ggq_gemv: qtype %d is not decodable", qtype);
  if (!ti->fused) return fail(GGQ_UNSUPPORTED, "ggq_gemv: no fused kernel for qtype %d", qtype);
  if (N <= 0 || K <= 0 || K % ti->block_elems)
    return fail(GGQ_BAD_SHAPE, "ggq_gemv: N=%lld K=%lld (K must be a positive multiple of %d)",
                (long long)N, (long long)K, ti->block_elems);
  if (M < 1 || M > kGemvMaxBatch)
    return fail(GGQ_BAD_SHAPE, "ggq_gemv: M=%d outside 1..%d", M, kGemvMaxBatch);
  if (y_dtype != GGQ_F32 && y_dtype != GGQ_BF16 && y_dtype != GGQ_F16)
    return fail(GGQ_BAD_DTYPE, "ggq_gemv: y_dtype %d", y_dtype);
  if (!w || !x_bf16 || !y) return fail(GGQ_MISALIGNED, "ggq_gemv: null pointer");
  if ((uintptr_t)x_bf16 % 16) return fail(GGQ_MISALIGNED, "ggq_gemv: x must be 16-byte aligned");
  if ((uintptr_t)w % block_alignment(ti))
    return fail(GGQ_MISALIGNED, "ggq_gemv: w must be %d-byte aligned for qtype %d", block_alignment(ti), qtype);
  int dev = 0;
  cudaGetDevice(&dev);
  const uint8_t* tab = device_tables(dev);
  if (ti->needs_tables && !tab)
    return fail(GGQ_NO_TABLES, "ggq_gemv: call ggq_set_tables(%d, ...) before using qtype %d", dev, qtype);
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t err;
  // The tuned batch-1 kernels (Q4_K, Q5_K, Q6_K).  A few batch rows are served by that many
  // launches of the batch-1 kernel, which is still faster than the small-batch kernel.
  const int y_item = y_dtype == GGQ_F32 ? 4 : 2;
  const bool scratch_ok = workspace && workspace_bytes >= gemv_q4k_workspace_bytes(N, kMaxSmCount) &&
                          (uintptr_t)workspace % 256 == 0 && sm_count_of(dev) > 0 && sm_count_of(dev) <= kMaxSmCount;
  const bool rows_ok = M <= tuned_max_repeat(qtype, N * (K / ti->block_elems) * ti->block_bytes) && (M == 1 || ((K * 2) % 16 == 0 && (N * y_item) % 2 == 0));
  using Tuned = cudaError_t (*)(const uint8_t*, int64_t, int64_t, const void*, void*, int, void*, size_t, int, int*,
                                cudaStream_t, const PeerPublish*);
  Tuned tuned = nullptr;
  if (scratch_ok && rows_ok) {
    if (qtype == QT_Q4_K && gemv_q4k_applicable(N, K, 1, w, x_bf16)) tuned = gemv_q4k;
    else if (qtype == QT_Q5_K && gemv_q5k_applicable(N, K, 1, w, x_bf16)) tuned = gemv_q5k;
    else if (qtype == QT_Q6_K && gemv_q6k_applicable(N, K, 1, w, x_bf16)) tuned = gemv_q6k;
  }
  static const bool m1_tiled = [] { const char* e = getenv("GGQ_Q4K_M1_TILED"); return e && e[0] == '1'; }();
  // Q4_K / Q5_K / Q6_K keep their batch-1 kernels; the tiled kernel takes their batches 2..4 (Q4_K 8192 x 28672:
  // 36 / 49 us at batch 2 / 4) and every batch of the formats that have nothing better; from five batch rows on
  // the batch-major kernel takes the larger weights (Q4_K 8192 x 28672: 68 / 77 us at batch 8 / 16 against
  // 100 / 153 us) and the integer-code MMA kernel (gemv_mma.cu) the smaller ones (see wide_pays).
  const bool k_quant = is_k_quant(qtype);
  const bool tile_first = !k_quant || (M >= 2 && M <= 4) || (M == 1 && m1_tiled);
  const int tile_max = gemv_tile_max_batch(qtype);
  const int tile_m = M < tile_max ? M : tile_max;
  const size_t tile_need = tile_max ? gemv_tile_workspace_bytes(qtype, N, K, tile_m) : 0;
  const bool tile_ok = tile_first && tile_need && workspace && workspace_bytes >= tile_need && (uintptr_t)workspace % 256 == 0 &&
                       sm_count_of(dev) > 0 && gemv_tile_applicable(qtype, N, K, tile_m, w, x_bf16);
  static const int wide_min = [] { const char* e = getenv("GGQ_WIDE_MIN"); return e ? atoi(e) : 5; }();
  const bool wide_ok = k_quant && M >= wide_min && wide_pays(qtype, N * (K / ti->block_elems) * (int64_t)ti->block_bytes) && workspace && (uintptr_t)workspace % 256 == 0 && sm_count_of(dev) > 0 &&
                       workspace_bytes >= gemv_wide_workspace_bytes(qtype, N, K, M, sm_count_of(dev)) &&
                       gemv_wide_applicable(qtype, N, K, M, w, x_bf16);
  if (wide_ok) {
    err = gemv_wide(qtype, (const uint8_t*)w, N, K, x_bf16, M, y, y_dtype, workspace, workspace_bytes, sm_count_of(dev), st, 0, nullptr,
                    device_status_word_if_any(dev));
  } else if (tile_ok) {
    // up to tile_max batch rows per launch; a larger batch reads the weight once per tile_max rows
    err = cudaSuccess;
    for (int m0 = 0; m0 < M && err == cudaSuccess; m0 += tile_max) {
      const int mb = M - m0 < tile_max ? M - m0 : tile_max;
      err = gemv_tile(qtype, (const uint8_t*)w, N, K, (const uint8_t*)x_bf16 + (size_t)m0 * K * 2, mb,
                      (uint8_t*)y + (size_t)m0 * N * y_item, y_dtype, workspace, workspace_bytes, sm_count_of(dev), nullptr, tab,
                      st, nullptr);
    }
  } else if (tuned) {
    err = cudaSuccess;
    for (int m = 0; m < M && err == cudaSuccess; m++)
      err = tuned((const uint8_t*)w, N, K, (const uint8_t*)x_bf16 + (size_t)m * K * 2,
                  (uint8_t*)y + (size_t)m * N * y_item, y_dtype, workspace, workspace_bytes, sm_count_of(dev),
                  device_status_word_if_any(dev), st, nullptr);   // the bounded waits for the TMA boxes report there once the word exists (ggq_init)
  } else if (gemv_mma_applicable(ti, N, K, M) && M >= kMmaMinBatch) {
    err = gemv_mma(ti, (const uint8_t*)w, N, K, x_bf16, M, y, y_dtype, tab, st);
  } else if (gemv_stream_applicable(ti, N, K, M, w, x_bf16)) {
    err = gemv_stream(ti, (const uint8_t*)w, N, K, x_bf16, y, y_dtype, tab, st);
  } else {
    err = gemv_generic(ti, (const uint8_t*)w, N, K, x_bf16, M, y, y_dtype, tab, st);
  }
  if (err != cudaSuccess) return fail(GGQ_LAUNCH_FAILED, "ggq_gemv: %s", cudaGetErrorString(err));
  return GGQ_OK;
}

// ---------------------------------------------------------------------------------------------
// ggq_stage_host: activations that live in pinned host memory.  A copy-engine transfer in front of a 30 us product
// costs about 12 us of latency; this kernel reads the (page-locked, device-visible) host buffer directly over the bus
// and the product behind it, a programmatic dependent, prefetches its weight tiles meanwhile.
__global__ void __launch_bounds__(256) stage_host_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t n16) {
  pdl_wait();            // the destination may still be read by the previous product
  pdl_trigger();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n16) {
    uint4 v;
    asm volatile("ld.global.relaxed.sys.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src + i) : "memory");
    dst[i] = v;
  }
}

extern "C" int32_t ggq_stage_host(const void* host_src, void* device_dst, size_t bytes, void* stream) {
  if (bytes == 0) return GGQ_OK;
  if (!host_src || !device_dst) return fail(GGQ_BAD_SHAPE, "ggq_stage_host: null pointer");
  if (bytes % 16 || (uintptr_t)host_src % 16 || (uintptr_t)device_dst % 16)
    return fail(GGQ_MISALIGNED, "ggq_stage_host: addresses and size must be multiples of 16 bytes");
  if (bytes > (64u << 20)) return fail(GGQ_BAD_SHAPE, "ggq_stage_host: %zu bytes; meant for activation vectors (<= 64 MB)", bytes);
  const size_t n16 = bytes / 16;
  cudaError_t err = launch_pdl(stage_host_kernel, (int)((n16 + 255) / 256), 256, 0, (cudaStream_t)stream,
                               reinterpret_cast<const uint4*>(host_src), reinterpret_cast<uint4*>(device_dst), n16);
  if (err == cudaSuccess) err = cudaPeekAtLastError();
  if (err != cudaSuccess) return fail(GGQ_LAUNCH_FAILED, "ggq_stage_host: %s", cudaGetErrorString(err));
  return GGQ_OK;
}

extern "C" int32_t ggq_gemv_sharded(int32_t qtype, const void* w, int64_t N_local, int64_t K, const void* x_bf16,
                                    int32_t M, void* const* y_peers, uint32_t* const* flag_peers, int32_t world,
                                    int32_t rank, int64_t n_total, int32_t y_dtype, int32_t wait_previous,
                                    void* workspace, size_t workspace_bytes, void* stream) {
  const TypeInfo* ti = type_info(qtype);
  if (!ti) return fail(GGQ_BAD_QTYPE, "ggq_gemv_sharded: qtype %d is not decodable", qtype);
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world)
    return fail(GGQ_BAD_SHAPE, "ggq_gemv_sharded: rank %d of %d (at most %d ranks)", rank, world, kMaxPeers);
  if (N_local <= 0 || K <= 0 || K % ti->block_elems || n_total < (int64_t)world * N_local)
    return fail(GGQ_BAD_SHAPE, "ggq_gemv_sharded: N_local=%lld K=%lld n_total=%lld", (long long)N_local,
                (long long)K, (long long)n_total);
  if (y_dtype != GGQ_F32 && y_dtype != GGQ_BF16 && y_dtype != GGQ_F16)
    return fail(GGQ_BAD_DTYPE, "ggq_gemv_sharded: y_dtype %d", y_dtype);
  if (!w || !x_bf16 || !y_peers || !flag_peers) return fail(GGQ_MISALIGNED, "ggq_gemv_sharded: null pointer");
  int dev = 0;
  cudaGetDevice(&dev);
  const bool ok4 = qtype == QT_Q4_K && gemv_q4k_applicable(N_local, K, M, w, x_bf16);
  const bool ok5 = qtype == QT_Q5_K && gemv_q5k_applicable(N_local, K, M, w, x_bf16);
  const bool ok6 = qtype == QT_Q6_K && gemv_q6k_applicable(N_local, K, M, w, x_bf16);
  if (!(ok4 || ok5 || ok6))
    return fail(GGQ_UNSUPPORTED, "ggq_gemv_sharded: only the Q4_K / Q5_K / Q6_K batch-1 kernels publish to peers so "
                "far; use ggq_gemv plus an all-gather for qtype %d, M=%d, K=%lld", qtype, M, (long long)K);
  if (!workspace || workspace_bytes < gemv_q4k_workspace_bytes(N_local, kMaxSmCount) || (uintptr_t)workspace % 256)
    return fail(GGQ_BAD_WORKSPACE, "ggq_gemv_sharded: workspace of %zu bytes needed", gemv_q4k_workspace_bytes(N_local, kMaxSmCount));
  PeerPublish pp = {};
  for (int p = 0; p < world; p++) {
    if (!y_peers[p] || !flag_peers[p]) return fail(GGQ_MISALIGNED, "ggq_gemv_sharded: null peer pointer %d", p);
    pp.y[p] = y_peers[p];
    pp.flags[p] = flag_peers[p];
  }
  pp.world = world;
  pp.rank = rank;
  pp.n_total = n_total;
  pp.row_offset = (int64_t)rank * N_local;
  pp.wait_previous = wait_previous ? 1 : 0;
  cudaError_t (*kernel)(const uint8_t*, int64_t, int64_t, const void*, void*, int, void*, size_t, int, int*,
                        cudaStream_t, const PeerPublish*) = ok4 ? gemv_q4k : ok5 ? gemv_q5k : gemv_q6k;
  cudaError_t err = kernel((const uint8_t*)w, N_local, K, x_bf16, nullptr, y_dtype, workspace, workspace_bytes,
                           sm_count_of(dev), device_status_word(dev), (cudaStream_t)stream, &pp);
  if (err != cudaSuccess) return fail(GGQ_LAUNCH_FAILED, "ggq_gemv_sharded: %s", cudaGetErrorString(err));
  return GGQ_OK;
}

extern "C" int32_t ggq_gemm_sharded(int32_t qtype, const void* w, int64_t N_local, int64_t K, const void* x_bf16, int64_t ldx,
                                    int32_t M, void* const* y_peers, uint32_t* const* flag_peers, int32_t world, int32_t rank,
                                    int64_t n_total, int32_t y_dtype, int32_t wait_previous, void* workspace,
                                    size_t workspace_bytes, void* stream) {
  if (M == 1)
    return ggq_gemv_sharded(qtype, w, N_local, K, x_bf16, 1, y_peers, flag_peers, world, rank, n_total, y_dtype, wait_previous,
                            workspace, workspace_bytes, stream);
  const TypeInfo* ti = type_info(qtype);
  if (!ti) return fail(GGQ_BAD_QTYPE, "ggq_gemm_sharded: qtype %d is not decodable", qtype);
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world)
    return fail(GGQ_BAD_SHAPE, "ggq_gemm_sharded: rank %d of %d (at most %d ranks)", rank, world, kMaxPeers);
  if (M < 1 || N_local <= 0 || K <= 0 || K % ti->block_elems || n_total < (int64_t)world * N_local || ldx < K || (ldx * 2) % 16)
    return fail(GGQ_BAD_SHAPE, "ggq_gemm_sharded: M=%d N_local=%lld K=%lld ldx=%lld n_total=%lld (ldx >= K, rows 16-byte aligned)", M,
                (long long)N_local, (long long)K, (long long)ldx, (long long)n_total);
  if (y_dtype != GGQ_F32 && y_dtype != GGQ_BF16 && y_dtype != GGQ_F16)
    return fail(GGQ_BAD_DTYPE, "ggq_gemm_sharded: y_dtype %d", y_dtype);
  if (!w || !x_bf16 || !y_peers || !flag_peers) return fail(GGQ_MISALIGNED, "ggq_gemm_sharded: null pointer");
  int dev = 0;
  cudaGetDevice(&dev);
  const int slice = gemv_wide_max_batch();
  const int first = M < slice ? M : slice;
  if (!is_k_quant(qtype) || !gemv_wide_applicable(qtype, N_local, K, first, w, x_bf16))
    return fail(GGQ_UNSUPPORTED, "ggq_gemm_sharded: only Q4_K / Q5_K / Q6_K weights with K a multiple of 256 and 16-byte aligned rows "
                "publish batches to peers; use ggq_gemm plus an all-gather for qtype %d, K=%lld", qtype, (long long)K);
  const size_t need = gemv_wide_workspace_bytes(qtype, N_local, K, first, sm_count_of(dev));
  if (!workspace || workspace_bytes < need || (uintptr_t)workspace % 256)
    return fail(GGQ_BAD_WORKSPACE, "ggq_gemm_sharded: workspace of %zu bytes needed", need);
  const int y_item = y_dtype == GGQ_F32 ? 4 : 2;
  // slices of up to 32 batch rows, one exchange each; only the first has to wait for the activations, and a consumer that waits
  // for the last one has the earlier ones too (a rank raises its flags in launch order, each behind a system-scope fence)
  for (int m0 = 0; m0 < M; m0 += slice) {
    const int mb = M - m0 < slice ? M - m0 : slice;
    PeerPublish pp = {};
    for (int p = 0; p < world; p++) {
      if (!y_peers[p] || !flag_peers[p]) return fail(GGQ_MISALIGNED, "ggq_gemm_sharded: null peer pointer %d", p);
      pp.y[p] = (uint8_t*)y_peers[p] + (size_t)m0 * n_total * y_item;
      pp.flags[p] = flag_peers[p];
    }
    pp.world = world;
    pp.rank = rank;
    pp.n_total = n_total;
    pp.row_offset = (int64_t)rank * N_local;
    pp.wait_previous = (wait_previous && m0 == 0) ? 1 : 0;
    cudaError_t err = gemv_wide(qtype, (const uint8_t*)w, N_local, K, (const uint8_t*)x_bf16 + (size_t)m0 * ldx * 2, mb, nullptr, y_dtype,
                                workspace, workspace_bytes, sm_count_of(dev), (cudaStream_t)stream, ldx, &pp, device_status_word(dev));
    if (err != cudaSuccess) return fail(GGQ_LAUNCH_FAILED, "ggq_gemm_sharded: %s", cudaGetErrorString(err));
  }
  return GGQ_OK;
}

extern "C" int32_t ggq_gemv_sharded_tagged(int32_t qtype, const void* w, int64_t N_local, int64_t K,
                                           const void* x_bf16, const uint32_t* x_tagged, int32_t x_back,
                                           const uint32_t* after_tagged, int64_t after_words, int32_t after_back,
                                           uint32_t* const* y_peers, uint32_t* state, int32_t world, int32_t rank,
                                           int64_t n_total, void* workspace, size_t workspace_bytes, void* stream) {
  const TypeInfo* ti = type_info(qtype);
  if (!ti) return fail(GGQ_BAD_QTYPE, "ggq_gemv_sharded_tagged: qtype %d is not decodable", qtype);
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world)
    return fail(GGQ_BAD_SHAPE, "ggq_gemv_sharded_tagged: rank %d of %d (at most %d ranks)", rank, world, kMaxPeers);
  if (N_local <= 0 || K <= 0 || K % ti->block_elems || n_total < (int64_t)world * N_local)
    return fail(GGQ_BAD_SHAPE, "ggq_gemv_sharded_tagged: N_local=%lld K=%lld n_total=%lld", (long long)N_local,
                (long long)K, (long long)n_total);
  if (!w || !y_peers || !state || (!x_bf16) == (!x_tagged))
    return fail(GGQ_MISALIGNED, "ggq_gemv_sharded_tagged: null pointer (give exactly one of x_bf16, x_tagged)");
  if (x_tagged && (x_back < 1 || x_back > 65534))
    return fail(GGQ_BAD_SHAPE, "ggq_gemv_sharded_tagged: x_back=%d", x_back);
  if (after_tagged && (after_back < 1 || after_back > 65534 || after_words < 0 || after_words % 4 ||
                       (uintptr_t)after_tagged % 16))
    return fail(GGQ_BAD_SHAPE, "ggq_gemv_sharded_tagged: after_back=%d after_words=%lld (a multiple of 4, 16-byte "
                "aligned)", after_back, (long long)after_words);
  const void* xa = x_bf16 ? x_bf16 : (const void*)x_tagged;
  const bool ok4 = qtype == QT_Q4_K && gemv_q4k_applicable(N_local, K, 1, w, xa);
  const bool ok5 = qtype == QT_Q5_K && gemv_q5k_applicable(N_local, K, 1, w, xa);
  const bool ok6 = qtype == QT_Q6_K && gemv_q6k_applicable(N_local, K, 1, w, xa);
  if (!(ok4 || ok5 || ok6))
    return fail(GGQ_UNSUPPORTED, "ggq_gemv_sharded_tagged: only the Q4_K / Q5_K / Q6_K batch-1 kernels take part in "
                "the tagged exchange (qtype %d, K=%lld)", qtype, (long long)K);
  if (!workspace || workspace_bytes < gemv_q4k_workspace_bytes(N_local, kMaxSmCount) || (uintptr_t)workspace % 256)
    return fail(GGQ_BAD_WORKSPACE, "ggq_gemv_sharded_tagged: workspace of %zu bytes needed",
                gemv_q4k_workspace_bytes(N_local, kMaxSmCount));
  int dev = 0;
  cudaGetDevice(&dev);
  PeerPublish pp = {};
  for (int p = 0; p < world; p++) {
    if (!y_peers[p]) return fail(GGQ_MISALIGNED, "ggq_gemv_sharded_tagged: null peer pointer %d", p);
    pp.y[p] = y_peers[p];
  }
  pp.flags[rank] = state;
  pp.world = world;
  pp.rank = rank;
  pp.n_total = n_total;
  pp.row_offset = (int64_t)rank * N_local;
  pp.tagged = 1;
  pp.x_tagged = x_tagged;
  pp.x_back = x_tagged ? x_back : 1;
  pp.after_tagged = after_tagged;
  pp.after_words = after_tagged ? after_words : 0;
  pp.after_back = after_tagged ? after_back : 1;
  cudaError_t (*kernel)(const uint8_t*, int64_t, int64_t, const void*, void*, int, void*, size_t, int, int*,
                        cudaStream_t, const PeerPublish*) = ok4 ? gemv_q4k : ok5 ? gemv_q5k : gemv_q6k;
  cudaError_t err = kernel((const uint8_t*)w, N_local, K, xa, nullptr, GGQ_BF16, workspace, workspace_bytes,
                           sm_count_of(dev), device_status_word(dev), (cudaStream_t)stream, &pp);
  if (err != cudaSuccess) return fail(GGQ_LAUNCH_FAILED, "ggq_gemv_sharded_tagged: %s", cudaGetErrorString(err));
  return GGQ_OK;
}

extern "C" int32_t ggq_gemv_q4k_static(const void* w, int64_t N, int64_t K, const void* x_bf16, void* y,
                                       int32_t y_dtype, void* stream) {
  if (y_dtype != GGQ_F32 && y_dtype != GGQ_BF16 && y_dtype != GGQ_F16)
    return fail(GGQ_BAD_DTYPE, "ggq_gemv_q4k_static: y_dtype %d", y_dtype);
  if (!w || !x_bf16 || !y) return fail(GGQ_MISALIGNED, "ggq_gemv_q4k_static: null pointer");
  int dev = 0;
  cudaGetDevice(&dev);
  const int sms = sm_count_of(dev);
  if (sms <= 0 || sms > kMaxSmCount) return fail(GGQ_LAUNCH_FAILED, "ggq_gemv_q4k_static: no usable CUDA device");
  return gemv_q4k_static(w, N, K, x_bf16, y, y_dtype, sms, (cudaStream_t)stream);
}

extern "C" int32_t ggq_gemm(int32_t qtype, const void* w, int64_t N, int64_t K, const void* x_bf16,
                            int32_t M, void* y, int32_t y_dtype, void* workspace, size_t workspace_bytes,
                            void* stream) {
  const TypeInfo* ti = type_info(qtype);
  if (!ti) return fail(GGQ_BAD_QTYPE, "ggq_gemm: qtype %d is not decodable", qtype);
  if (!ti->fused) return fail(GGQ_UNSUPPORTED, "ggq_gemm: no fused kernel for qtype %d", qtype);
  if (N <= 0 || K <= 0 || K % ti->block_elems || M < 1)
    return fail(GGQ_BAD_SHAPE, "ggq_gemm: N=%lld K=%lld M=%d (K must be a positive multiple of %d)",
                (long long)N, (long long)K, M, ti->block_elems);
  if (!gemm_applicable(ti, N, K, M))
    return fail(GGQ_UNSUPPORTED, "ggq_gemm: shape N=%lld K=%lld M=%d is outside the tensor-core kernel's range "
                "(K must be a multiple of 256)", (long long)N, (long long)K, M);
  if (y_dtype != GGQ_F32 && y_dtype != GGQ_BF16 && y_dtype != GGQ_F16)
    return fail(GGQ_BAD_DTYPE, "ggq_gemm: y_dtype %d", y_dtype);
  if (!w || !x_bf16 || !y) return fail(GGQ_MISALIGNED, "ggq_gemm: null pointer");
  if ((uintptr_t)x_bf16 % 16) return fail(GGQ_MISALIGNED, "ggq_gemm: x must be 16-byte aligned");
  if ((uintptr_t)w % 16) return fail(GGQ_MISALIGNED, "ggq_gemm: w must be 16-byte aligned");
  int dev = 0;
  cudaGetDevice(&dev);
  const uint8_t* tab = device_tables(dev);
  if (ti->needs_tables && !tab)
    return fail(GGQ_NO_TABLES, "ggq_gemm: call ggq_set_tables(%d, ...) before using qtype %d", dev, qtype);
  cudaError_t err;
  // Kernel choice for Q4_K / Q5_K / Q6_K (the other formats always take the tf32 tcgen05 kernel):
  //   up to 32 rows     the batch-major mma.sync kernel: exact integer codes, nothing rounded before the output;
  //   above             the bf16-weight tcgen05 kernel: weights rounded once to bf16, as the reference's GEMM does.
  // GGQ_GEMM_KERNEL = wide | bf16w | codes | tf32 pins one of them (read on every call, so a test can switch);
  // a pinned kernel that cannot take the call falls through to the next one in that order.
  enum { kAuto, kWide, kBf16w, kCodes, kTf32 };
  int pin = kAuto;
  if (const char* e = getenv("GGQ_GEMM_KERNEL")) {
    pin = !strcmp(e, "wide") ? kWide : !strcmp(e, "bf16w") ? kBf16w : !strcmp(e, "codes") ? kCodes : !strcmp(e, "tf32") ? kTf32 : kAuto;
  }
  const int wide_slice = gemv_wide_max_batch();
  const int y_item = y_dtype == GGQ_F32 ? 4 : 2;
  const int sms = sm_count_of(dev);
  const bool ws_ok = workspace && (uintptr_t)workspace % 256 == 0;
  const int slice_m = M < wide_slice ? M : wide_slice;
  const bool can_wide = ws_ok && gemv_wide_applicable(qtype, N, K, slice_m, w, x_bf16) &&
                        workspace_bytes >= gemv_wide_workspace_bytes(qtype, N, K, slice_m, sms);
  const bool can_bf16w = ws_ok && gemm_bf16w_applicable(qtype, N, K, M) &&
                         workspace_bytes >= gemm_bf16w_workspace_bytes(qtype, N, K, M, sms);
  const bool can_codes = ws_ok && gemm_codes_applicable(qtype, N, K, M) &&
                         workspace_bytes >= gemm_codes_workspace_bytes(qtype, N, K, M, sms);
  int pick = kTf32;
  if (pin == kAuto) pick = (can_wide && M <= wide_slice) ? kWide : can_bf16w ? kBf16w : can_wide ? kWide : can_codes ? kCodes : kTf32;
  else if (pin == kWide) pick = can_wide ? kWide : can_bf16w ? kBf16w : can_codes ? kCodes : kTf32;
  else if (pin == kBf16w) pick = can_bf16w ? kBf16w : can_codes ? kCodes : kTf32;
  else if (pin == kCodes) pick = can_codes ? kCodes : kTf32;
  if (pick == kWide) {
    // slices of up to 32 batch rows: the weight is read once per slice
    err = cudaSuccess;
    for (int m0 = 0; m0 < M && err == cudaSuccess; m0 += wide_slice) {
      const int mb = M - m0 < wide_slice ? M - m0 : wide_slice;
      err = gemv_wide(qtype, (const uint8_t*)w, N, K, (const uint8_t*)x_bf16 + (size_t)m0 * K * 2, mb,
                      (uint8_t*)y + (size_t)m0 * N * y_item, y_dtype, workspace, workspace_bytes, sms, (cudaStream_t)stream, 0, nullptr,
                      device_status_word(dev));
    }
  } else if (pick == kBf16w) {
    err = gemm_bf16w(qtype, (const uint8_t*)w, N, K, x_bf16, M, y, y_dtype, device_status_word(dev), workspace, workspace_bytes, sms,
                     (cudaStream_t)stream);
  } else if (pick == kCodes) {
    err = gemm_codes(qtype, (const uint8_t*)w, N, K, x_bf16, M, y, y_dtype, device_status_word(dev), workspace, workspace_bytes, sms,
                     (cudaStream_t)stream);
  } else {
    err = gemm_tf32(ti, (const uint8_t*)w, N, K, x_bf16, M, y, y_dtype, tab, device_status_word(dev), workspace, workspace_bytes, sms,
                    (cudaStream_t)stream);
  }
  if (err != cudaSuccess) return fail(GGQ_LAUNCH_FAILED, "ggq_gemm: %s", cudaGetErrorString(err));
  return GGQ_OK;
}
