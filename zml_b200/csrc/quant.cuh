// Device helpers of the NVFP4 quantiser, shared by the stand-alone kernel (quant.cu) and the kernels that quantise
// on the way (the expert-parallel gather in moe.cu, the SwiGLU epilogue of the block-scaled grouped GEMM in
// moe_fp4.cu).  Numerics: see the head of quant.cu.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "common.cuh"

ZB_DEVICE float bf16_round(float x) { return __bfloat162float(__float2bfloat16(x)); }

// round-to-nearest-even onto {0, .5, 1, 1.5, 2, 3, 4, 6}, saturating; returns the 4-bit code
ZB_DEVICE uint32_t e2m1_code(float x) {
  const float a = fabsf(x);
  uint32_t idx = 0;
  idx += a > 0.25f;     // tie 0.25 -> 0   (even mantissa)
  idx += a >= 0.75f;    // tie 0.75 -> 1.0
  idx += a > 1.25f;     // tie 1.25 -> 1.0
  idx += a >= 1.75f;    // tie 1.75 -> 2.0
  idx += a > 2.5f;      // tie 2.5  -> 2.0
  idx += a >= 3.5f;     // tie 3.5  -> 4.0
  idx += a > 5.0f;      // tie 5.0  -> 4.0
  return idx | (signbit(x) ? 8u : 0u);
}

ZB_DEVICE float e2m1_value(uint32_t code) {
  const uint32_t m = code & 7u;
  // 0, .5, 1, 1.5, 2, 3, 4, 6
  const float v = m < 2 ? 0.5f * static_cast<float>(m)
                        : static_cast<float>((2u | (m & 1u)) << ((m >> 1) - 1u)) * 0.5f;
  return (code & 8u) ? -v : v;
}

ZB_DEVICE float fp8_e4m3_to_float(uint8_t b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(b), __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

// 16 values (already rounded to bf16) -> 16 e2m1 codes in two words (value i in nibble i % 8 of word i / 8) and
// the f8e4m3 scale byte of the block: scale = clamp(bf16(amax / 6), 2^-6, 448) rounded to e4m3, code = e2m1(bf16(v / scale)).
ZB_DEVICE uint2 zb_nvfp4_quantize_block(const float (&v)[16], uint8_t& scale_byte) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  float s = bf16_round(amax * (1.0f / 6.0f));
  s = fminf(fmaxf(s, 0.015625f), 448.f);
  scale_byte = static_cast<uint8_t>(__nv_cvt_float_to_fp8(s, __NV_SATFINITE, __NV_E4M3));
  const float div = fmaxf(fp8_e4m3_to_float(scale_byte), 0.015625f);
  uint32_t packed[2] = {0u, 0u};
#pragma unroll
  for (int i = 0; i < 16; ++i) packed[i >> 3] |= e2m1_code(bf16_round(v[i] / div)) << (4 * (i & 7));
  return make_uint2(packed[0], packed[1]);
}
