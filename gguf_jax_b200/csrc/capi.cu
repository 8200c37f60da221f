// Library-level pieces of the C ABI: type table, error text, per-device codebook tables.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "ggq_common.cuh"

namespace ggq {

static const TypeInfo k_types[] = {
    // qtype, block elems, block bytes, needs codebook tables, has a fused multiply kernel
    {QT_F32, 1, 4, false, false},       {QT_F16, 1, 2, false, false},      {QT_BF16, 1, 2, false, false},
    {QT_Q4_0, 32, 18, false, true},    {QT_Q4_1, 32, 20, false, true},   {QT_Q5_0, 32, 22, false, true},
    {QT_Q5_1, 32, 24, false, true},    {QT_Q8_0, 32, 34, false, true},   {QT_Q2_K, 256, 84, false, true},
    {QT_Q3_K, 256, 110, false, true},   {QT_Q4_K, 256, 144, false, true},  {QT_Q5_K, 256, 176, false, true},
    {QT_Q6_K, 256, 210, false, true},   {QT_IQ2_XXS, 256, 66, true, true}, {QT_IQ2_XS, 256, 74, true, true},
    {QT_IQ3_XXS, 256, 98, true, true},  {QT_IQ1_S, 256, 50, true, true},   {QT_IQ4_NL, 32, 18, true, true},
    {QT_IQ3_S, 256, 110, true, true},   {QT_IQ2_S, 256, 82, true, true},   {QT_IQ4_XS, 256, 136, true, true},
    {QT_IQ1_M, 256, 56, true, true},    {QT_TQ1_0, 256, 54, false, true}, {QT_TQ2_0, 256, 66, false, true},
    {QT_MXFP4, 32, 17, true, true},    {QT_NVFP4, 64, 36, true, true},
};

const TypeInfo* type_info(int qtype) {
  for (const TypeInfo& t : k_types)
    if (t.qtype == qtype) return &t;
  return nullptr;
}

static thread_local char t_err[512] = "";

int32_t fail(int32_t status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_err, sizeof(t_err), fmt, ap);
  va_end(ap);
  return status;
}

constexpr int kMaxDevices = 64;
// Everything the library keeps per device.  Each member is created at most once (std::call_once)
// and never freed or moved afterwards, so readers need no lock.
struct DeviceState {
  std::once_flag status_once, sm_once;
  std::mutex tables_mu;
  std::atomic<uint8_t*> tables{nullptr};
  std::atomic<int*> status{nullptr};
  std::atomic<int> sm_count{0};
};
static DeviceState g_dev[kMaxDevices];

const uint8_t* device_tables(int device) {
  if (device < 0 || device >= kMaxDevices) return nullptr;
  return g_dev[device].tables.load(std::memory_order_acquire);
}

// The status word is allocated the first time a launcher that can raise it runs on the device
// (or by ggq_init), independently of the codebook tables.  That first call allocates device
// memory and must therefore be made outside stream capture.
int* device_status_word(int device) {
  if (device < 0 || device >= kMaxDevices) return nullptr;
  DeviceState& d = g_dev[device];
  std::call_once(d.status_once, [&] {
    int prev = 0;
    cudaGetDevice(&prev);
    int* s = nullptr;
    cudaError_t err = cudaSetDevice(device);
    if (err == cudaSuccess) err = cudaMalloc(&s, 256);
    if (err == cudaSuccess) err = cudaMemset(s, 0, 256);
    cudaSetDevice(prev);
    if (err != cudaSuccess) {
      if (s) cudaFree(s);
      (void)cudaGetLastError();
      s = nullptr;
    }
    d.status.store(s, std::memory_order_release);
  });
  return d.status.load(std::memory_order_acquire);
}

int* device_status_word_if_any(int device) {
  if (device < 0 || device >= kMaxDevices) return nullptr;
  return g_dev[device].status.load(std::memory_order_acquire);
}

int device_sm_count(int device) {
  if (device < 0 || device >= kMaxDevices) return 0;
  DeviceState& d = g_dev[device];
  std::call_once(d.sm_once, [&] {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) { n = 0; (void)cudaGetLastError(); }
    d.sm_count.store(n, std::memory_order_release);
  });
  return d.sm_count.load(std::memory_order_acquire);
}

}  // namespace ggq

using namespace ggq;

extern "C" int32_t ggq_version(void) { return 100; }

extern "C" const char* ggq_last_error(void) { return t_err; }

extern "C" int32_t ggq_type_info(int32_t qtype, int32_t* block_elems, int32_t* block_bytes) {
  const TypeInfo* ti = type_info(qtype);
  if (!ti) return fail(GGQ_BAD_QTYPE, "ggq_type_info: qtype %d is not decodable", qtype);
  if (block_elems) *block_elems = ti->block_elems;
  if (block_bytes) *block_bytes = ti->block_bytes;
  return GGQ_OK;
}

extern "C" size_t ggq_tables_bytes(void) { return TAB_BYTES; }

extern "C" int32_t ggq_set_tables(int32_t device, const void* host_blob, size_t bytes) {
  if (device < 0 || device >= kMaxDevices) return fail(GGQ_BAD_SHAPE, "ggq_set_tables: device %d", device);
  if (bytes != TAB_BYTES || !host_blob)
    return fail(GGQ_BAD_SHAPE, "ggq_set_tables: blob must be %d bytes, got %zu", (int)TAB_BYTES, bytes);
  DeviceState& d = g_dev[device];
  std::lock_guard<std::mutex> lock(d.tables_mu);
  if (d.tables.load(std::memory_order_acquire)) return GGQ_OK;
  int prev = 0;
  cudaGetDevice(&prev);
  cudaError_t err = cudaSetDevice(device);
  uint8_t* t = nullptr;
  if (err == cudaSuccess) err = cudaMalloc(&t, TAB_BYTES);
  if (err == cudaSuccess) err = cudaMemcpy(t, host_blob, TAB_BYTES, cudaMemcpyHostToDevice);
  cudaSetDevice(prev);
  if (err != cudaSuccess) {
    if (t) cudaFree(t);
    return fail(GGQ_LAUNCH_FAILED, "ggq_set_tables: %s", cudaGetErrorString(err));
  }
  d.tables.store(t, std::memory_order_release);
  return GGQ_OK;
}

extern "C" int32_t ggq_init(int32_t device) {
  if (device < 0 || device >= kMaxDevices) return fail(GGQ_BAD_SHAPE, "ggq_init: device %d", device);
  if (!device_status_word(device)) return fail(GGQ_LAUNCH_FAILED, "ggq_init: could not allocate the status word on device %d", device);
  if (device_sm_count(device) <= 0) return fail(GGQ_LAUNCH_FAILED, "ggq_init: device %d reports no multiprocessors", device);
  return GGQ_OK;
}

extern "C" int32_t ggq_has_fused(int32_t qtype) {
  const TypeInfo* ti = type_info(qtype);
  return ti && ti->fused ? 1 : 0;
}

extern "C" int32_t ggq_read_status(int32_t device, int32_t* status_word) {
  if (!status_word) return fail(GGQ_BAD_SHAPE, "ggq_read_status: null out pointer");
  *status_word = 0;
  if (device < 0 || device >= kMaxDevices) return fail(GGQ_BAD_SHAPE, "ggq_read_status: device %d", device);
  int* s = g_dev[device].status.load(std::memory_order_acquire);
  if (!s) return GGQ_OK;  // no launcher that can raise it has run on this device
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(device);
  cudaError_t err = cudaDeviceSynchronize();
  int v = 0;
  if (err == cudaSuccess) err = cudaMemcpy(&v, s, sizeof(int), cudaMemcpyDeviceToHost);
  if (err == cudaSuccess && v) err = cudaMemset(s, 0, sizeof(int));
  cudaSetDevice(prev);
  if (err != cudaSuccess) return fail(GGQ_LAUNCH_FAILED, "ggq_read_status: %s", cudaGetErrorString(err));
  *status_word = v;
  return v ? fail(GGQ_TIMEOUT, "a bounded device-side wait ran out (status word 0x%x)", v) : GGQ_OK;
}
