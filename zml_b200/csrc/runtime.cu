// Library runtime: per-device state (status word, scratch), launch counting.
#include <atomic>
#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "host_api.h"

#ifdef ZB_BOUNDS_CHECK
// one copy per device for the whole library (relocatable device code): see common.cuh
__device__ ZbStatus* zb_bc_status = nullptr;
__device__ ZbBcExtents zb_bc_ext = {0, 0};
#endif

namespace {
constexpr int kMaxDevices = 16;
ZbDeviceState g_state[kMaxDevices];
bool g_ready[kMaxDevices] = {};
std::mutex g_mu;
std::atomic<unsigned long long> g_launches{0};

constexpr size_t kGemmScratchBytes = 64ull << 20;
constexpr int kGemmCounters = 1 << 16;
constexpr size_t kAttnScratchBytes = 128ull << 20;
}  // namespace

ZbDeviceState* zb_device_state() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  if (!g_ready[dev]) {
    if (zb_init(dev) != 0) return nullptr;
  }
  return &g_state[dev];
}

static std::atomic<int> g_pdl{-1};
bool zb_pdl_enabled() {
  int v = g_pdl.load();
  if (v < 0) {
    const char* e = getenv("ZB_PDL");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
    g_pdl.store(v);
  }
  return v != 0;
}
extern "C" void zb_set_pdl(int on) { g_pdl.store(on ? 1 : 0); }

void zb_count_launch(int n) { g_launches.fetch_add(static_cast<unsigned long long>(n)); }

extern "C" {

int zb_init(int device) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (device < 0 || device >= kMaxDevices) return -1;
  if (g_ready[device]) return 0;
  int prev = -1;
  cudaGetDevice(&prev);
  if (cudaSetDevice(device) != cudaSuccess) return -2;
  ZbDeviceState& s = g_state[device];
  s.device = device;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return -3;
  s.num_sms = prop.multiProcessorCount;
  if (cudaMalloc(&s.status, sizeof(ZbStatus)) != cudaSuccess) return -4;
  cudaMemset(s.status, 0, sizeof(ZbStatus));
  s.gemm_scratch_bytes = kGemmScratchBytes;
  if (cudaMalloc(&s.gemm_scratch, s.gemm_scratch_bytes) != cudaSuccess) return -5;
  s.gemm_counters_len = kGemmCounters;
  if (cudaMalloc(&s.gemm_counters, sizeof(uint32_t) * kGemmCounters) != cudaSuccess) return -6;
  cudaMemset(s.gemm_counters, 0, sizeof(uint32_t) * kGemmCounters);
  s.attn_scratch_bytes = kAttnScratchBytes;
  if (cudaMalloc(&s.attn_scratch, s.attn_scratch_bytes) != cudaSuccess) return -7;
  s.attn_counters_len = 1 << 16;
  if (cudaMalloc(&s.attn_counters, sizeof(uint32_t) * s.attn_counters_len) != cudaSuccess) return -8;
  cudaMemset(s.attn_counters, 0, sizeof(uint32_t) * s.attn_counters_len);
#ifdef ZB_BOUNDS_CHECK
  if (cudaMemcpyToSymbol(zb_bc_status, &s.status, sizeof(s.status)) != cudaSuccess) return -9;
#endif
  cudaDeviceSynchronize();
  g_ready[device] = true;
  if (prev >= 0 && prev != device) cudaSetDevice(prev);
  return 0;
}

int zb_num_sms() {
  ZbDeviceState* s = zb_device_state();
  return s ? s->num_sms : 0;
}

ZbStatus* zb_status_ptr() {
  ZbDeviceState* s = zb_device_state();
  return s ? s->status : nullptr;
}

int zb_status_read(uint32_t* out4) {
  ZbDeviceState* s = zb_device_state();
  if (!s) return -1;
  cudaError_t e = cudaMemcpy(out4, s->status, sizeof(ZbStatus), cudaMemcpyDeviceToHost);
  return static_cast<int>(e);
}

int zb_status_reset() {
  ZbDeviceState* s = zb_device_state();
  if (!s) return -1;
  return static_cast<int>(cudaMemset(s->status, 0, sizeof(ZbStatus)));
}

// 1 in the bounds-checking build of the library, 0 in the normal one.
int zb_bc_enabled() {
#ifdef ZB_BOUNDS_CHECK
  return 1;
#else
  return 0;
#endif
}

// Declares the extents that kernel arguments do not carry (bounds-checking build; a no-op otherwise).
int zb_bc_set_extents(long long num_pages, long long num_state_slots) {
#ifdef ZB_BOUNDS_CHECK
  if (!zb_device_state()) return -1;
  ZbBcExtents e = {num_pages, num_state_slots};
  return static_cast<int>(cudaMemcpyToSymbol(zb_bc_ext, &e, sizeof(e)));
#else
  (void)num_pages;
  (void)num_state_slots;
  return 0;
#endif
}

unsigned long long zb_launch_count() { return g_launches.load(); }
void zb_launch_count_reset() { g_launches.store(0); }
void zb_launch_count_add(unsigned long long n) { g_launches.fetch_add(n); }

}  // extern "C"
