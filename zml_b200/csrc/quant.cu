// Quantisation kernels:
//   zb_nvfp4_quantize      bf16 -> packed e2m1 codes + one f8e4m3fn scale per 16 values
//                          (the dynamic activation quantiser of the NVFP4 recipe)
//   zb_nvfp4_dequantize    packed e2m1 + block scales (+ global scale) -> bf16
//   zb_fp8_group_quant     bf16 -> f8e4m3fn with one float scale per `group` values
//
// Numerics follow the tensor formulation the reference lowers through XLA
// (zml/nn.zig:246-279: scale = clamp(amax / 6, 2^-6, 448) rounded to f8e4m3fn, value / scale
// rounded to e2m1) with the intermediate roundings of a bf16 evaluation, so the device
// result equals the PyTorch restatement bit for bit.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "common.cuh"
#include "host_api.h"
#include "quant.cuh"

namespace {

// one thread per 16-value block
__global__ void __launch_bounds__(256) zb_nvfp4_quantize_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                                                uint8_t* __restrict__ codes, uint8_t* __restrict__ scales,
                                                                const float* __restrict__ global_scale, int rows, int kblocks) {
  zb_pdl_launch();
  zb_pdl_wait();
  const long long idx = blockIdx.x * 256ll + threadIdx.x;
  if (idx >= static_cast<long long>(rows) * kblocks) return;
  const int r = static_cast<int>(idx / kblocks), b = static_cast<int>(idx % kblocks);
  const uint4* src = reinterpret_cast<const uint4*>(x + r * ldx + b * 16);
  uint4 raw[2] = {src[0], src[1]};
  const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(raw);
  float v[16];
  const float gs = global_scale != nullptr ? bf16_round(*global_scale) : 1.f;
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    v[i] = __bfloat162float(e[i]);
    if (global_scale != nullptr) v[i] = bf16_round(v[i] / gs);
    amax = fmaxf(amax, fabsf(v[i]));
  }
  (void)amax;
  uint8_t s8;
  *reinterpret_cast<uint2*>(codes + (static_cast<size_t>(r) * kblocks + b) * 8) = zb_nvfp4_quantize_block(v, s8);
  scales[static_cast<size_t>(r) * kblocks + b] = s8;
}

__global__ void __launch_bounds__(256) zb_nvfp4_dequantize_kernel(const uint8_t* __restrict__ codes,
                                                                  const uint8_t* __restrict__ scales,
                                                                  const float* __restrict__ global_scale,
                                                                  __nv_bfloat16* __restrict__ out, long long ldo, int rows,
                                                                  int kblocks) {
  zb_pdl_launch();
  zb_pdl_wait();
  const long long idx = blockIdx.x * 256ll + threadIdx.x;
  if (idx >= static_cast<long long>(rows) * kblocks) return;
  const int r = static_cast<int>(idx / kblocks), b = static_cast<int>(idx % kblocks);
  const uint2 p = *reinterpret_cast<const uint2*>(codes + (static_cast<size_t>(r) * kblocks + b) * 8);
  const float s = fp8_e4m3_to_float(scales[static_cast<size_t>(r) * kblocks + b]) * (global_scale ? *global_scale : 1.f);
  const uint32_t w[2] = {p.x, p.y};
  __align__(16) __nv_bfloat16 o[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i] = __float2bfloat16(e2m1_value((w[i >> 3] >> (4 * (i & 7))) & 15u) * s);
  uint4* dst = reinterpret_cast<uint4*>(out + r * ldo + b * 16);
  dst[0] = reinterpret_cast<const uint4*>(o)[0];
  dst[1] = reinterpret_cast<const uint4*>(o)[1];
}

// one warp per group of `group` values (group a multiple of 32)
__global__ void __launch_bounds__(256) zb_fp8_group_quant_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                                                 uint8_t* __restrict__ q, float* __restrict__ scale, int rows,
                                                                 int groups, int group) {
  zb_pdl_launch();
  zb_pdl_wait();
  const long long w = (blockIdx.x * 256ll + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= static_cast<long long>(rows) * groups) return;
  const int r = static_cast<int>(w / groups), g = static_cast<int>(w % groups);
  const __nv_bfloat16* src = x + r * ldx + static_cast<long long>(g) * group;
  float amax = 0.f;
  for (int i = lane; i < group; i += 32) amax = fmaxf(amax, fabsf(__bfloat162float(src[i])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float s = fmaxf(amax / 448.f, 1e-10f);
  for (int i = lane; i < group; i += 32) {
    const float v = fminf(fmaxf(__bfloat162float(src[i]) / s, -448.f), 448.f);
    q[(static_cast<size_t>(r) * groups + g) * group + i] =
        static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
  }
  if (lane == 0) scale[static_cast<size_t>(r) * groups + g] = s;
}

}  // namespace

extern "C" {

// x [rows, k] bf16 (row stride ldx, 16-byte aligned rows), k a multiple of 16.
// codes: [rows, k/2] bytes, low nibble first; scales: [rows, k/16] f8e4m3fn bytes.
int zb_nvfp4_quantize(const void* x, long long ldx, void* codes, void* scales, const float* global_scale, int rows,
                      int k, void* stream) {
  if (rows <= 0 || k <= 0) return 0;
  if (k % 16 != 0 || ldx % 8 != 0) return -80;
  const long long total = static_cast<long long>(rows) * (k / 16);
  zb_launch(zb_nvfp4_quantize_kernel, dim3(static_cast<unsigned>((total + 255) / 256)), dim3(256), 0,
            reinterpret_cast<cudaStream_t>(stream), reinterpret_cast<const __nv_bfloat16*>(x), ldx,
            reinterpret_cast<uint8_t*>(codes), reinterpret_cast<uint8_t*>(scales), global_scale, rows, k / 16);
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

int zb_nvfp4_dequantize(const void* codes, const void* scales, const float* global_scale, void* out, long long ldo,
                        int rows, int k, void* stream) {
  if (rows <= 0 || k <= 0) return 0;
  if (k % 16 != 0 || ldo % 8 != 0) return -80;
  const long long total = static_cast<long long>(rows) * (k / 16);
  zb_launch(zb_nvfp4_dequantize_kernel, dim3(static_cast<unsigned>((total + 255) / 256)), dim3(256), 0,
            reinterpret_cast<cudaStream_t>(stream), reinterpret_cast<const uint8_t*>(codes),
            reinterpret_cast<const uint8_t*>(scales), global_scale, reinterpret_cast<__nv_bfloat16*>(out), ldo, rows,
            k / 16);
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

int zb_fp8_group_quant(const void* x, long long ldx, void* q, float* scale, int rows, int k, int group, void* stream) {
  if (rows <= 0 || k <= 0) return 0;
  if (group <= 0 || group % 32 != 0 || k % group != 0) return -81;
  const long long warps = static_cast<long long>(rows) * (k / group);
  zb_launch(zb_fp8_group_quant_kernel, dim3(static_cast<unsigned>((warps * 32 + 255) / 256)), dim3(256), 0,
            reinterpret_cast<cudaStream_t>(stream), reinterpret_cast<const __nv_bfloat16*>(x), ldx,
            reinterpret_cast<uint8_t*>(q), scale, rows, k / group, group);
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
