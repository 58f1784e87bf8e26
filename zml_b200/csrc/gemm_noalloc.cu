// zb_gemm_bf16_noalloc: the bf16 GEMM with its scratch in a fixed device array (see
// gemm_noalloc.h for who needs this and what the limits are).
#include "gemm_noalloc.h"

#include <stdio.h>

#include "common.cuh"
#include "host_api.h"

extern "C" {
int zb_gemm_plan(int m, int n, int k, int num_sms, int split_hint, int* swap, int* bn, int* grid,
                 int* units_per_cta, int* rr_tiles);
size_t zb_gemm_scratch_needed(int m, int n, int k, int num_sms);
int zb_gemm_bf16_ex(const void* a, const void* w, void* out, const void* residual, const void* bias,
                    int m, int n, int k, int lda, int ldw, int ldo, int out_f32, int split_hint,
                    float* scratch, size_t scratch_bytes, uint32_t* counters, int counters_len,
                    ZbStatus* status, int num_sms, cudaStream_t stream);
}

namespace {

constexpr int kCounters = 4096;          // one per output tile of a stream-K problem (< 600 in practice)
constexpr size_t kCounterBytes = kCounters * sizeof(uint32_t);
constexpr size_t kStatusBytes = 256;     // ZbStatus, padded to keep the partial tiles aligned
constexpr size_t kTotalBytes = kCounterBytes + kStatusBytes + ZB_NOALLOC_SCRATCH_BYTES;

// Layout: [tile counters | status word | partial tiles].  In host code this name is only a
// handle for cudaGetSymbolAddress; it is not a device address.
static __device__ __align__(256) unsigned char zb_noalloc_scratch[kTotalBytes];

constexpr int kMaxDevices = 16;
unsigned char* g_base[kMaxDevices] = {};
int g_sms[kMaxDevices] = {};

}  // namespace

extern "C" int zb_gemm_bf16_noalloc(const void* a, const void* w, void* out, const void* residual,
                                    const void* bias, int m, int n, int k, int lda, int ldw, int ldo,
                                    int out_f32, void* status_out, void* stream) {
  if (a == nullptr || w == nullptr || out == nullptr || m <= 0 || n <= 0 || k <= 0)
    return ZB_NOALLOC_ERR_BAD_ARG;
  // `out_f32` is a yes / no here; the kernel's entry point reads further bits of its flag word (weight prefetch
  // ahead of the stream dependency), which this entry point never sets
  const int f32 = out_f32 ? 1 : 0;
  if ((k % 8) != 0 || (lda % 8) != 0 || (ldw % 8) != 0 || (!f32 && (ldo % 8) != 0))
    return ZB_NOALLOC_ERR_BAD_ARG;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return ZB_NOALLOC_ERR_SETUP;
  if (g_base[dev] == nullptr) {
    // once per device, with that device current: device address of this device's copy of the array
    unsigned char* ptr = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), zb_noalloc_scratch) != cudaSuccess || ptr == nullptr)
      return ZB_NOALLOC_ERR_SETUP;
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      return ZB_NOALLOC_ERR_SETUP;
    g_sms[dev] = sms;
    g_base[dev] = ptr;
  }
  unsigned char* base = g_base[dev];
  uint32_t* counters = reinterpret_cast<uint32_t*>(base);
  ZbStatus* status = status_out ? reinterpret_cast<ZbStatus*>(status_out)
                                : reinterpret_cast<ZbStatus*>(base + kCounterBytes);
  float* partials = reinterpret_cast<float*>(base + kCounterBytes + kStatusBytes);

  int sw, bn, grid, upc, rr;
  const int tiles = zb_gemm_plan(m, n, k, g_sms[dev], 0, &sw, &bn, &grid, &upc, &rr);
  // scratch of the plan that will really launch (whole-tile and cluster plans write no partial tile to memory)
  const size_t need = rr > 0 ? 0 : zb_gemm_scratch_needed(m, n, k, g_sms[dev]);
  if (need > ZB_NOALLOC_SCRATCH_BYTES || (rr == 0 && tiles > kCounters)) {
    fprintf(stderr,
            "zb_gemm_bf16_noalloc: M=%d N=%d K=%d needs %zu bytes of scratch for partial tiles, the "
            "built-in array holds %u; use zb_gemm_bf16 or a smaller M\n",
            m, n, k, need, ZB_NOALLOC_SCRATCH_BYTES);
    return ZB_NOALLOC_ERR_TOO_LARGE;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // the array keeps the previous call's contents: counters (and the status word) must start at zero
  if (cudaMemsetAsync(counters, 0, kCounterBytes, s) != cudaSuccess) return ZB_NOALLOC_ERR_SETUP;
  if (cudaMemsetAsync(status, 0, sizeof(ZbStatus), s) != cudaSuccess) return ZB_NOALLOC_ERR_SETUP;
  // whole-tile (round-robin) problems write no partial tile, so their size is not bounded by the array
  const size_t bound = rr > 0 ? (static_cast<size_t>(1) << 40) : static_cast<size_t>(ZB_NOALLOC_SCRATCH_BYTES);
  const int rc = zb_gemm_bf16_ex(a, w, out, residual, bias, m, n, k, lda, ldw, ldo, f32, 0, partials, bound,
                                 counters, rr > 0 ? (1 << 30) : kCounters, status, g_sms[dev], s);
  // the kernel's own does-not-fit codes (scratch, counters) are this entry point's "too large"
  return (rc == -13 || rc == -14) ? ZB_NOALLOC_ERR_TOO_LARGE : rc;
}
