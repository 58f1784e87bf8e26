// Kernels of the hybrid (linear-attention / short-convolution) decoder layers:
//
//   zb_causal_conv1d      depthwise causal convolution over a flattened varlen batch with a
//                         rolling per-sequence input cache, optional input gate (B * x), output
//                         gate (C * y) and SiLU: the `ShortConv` of LFM2 and the conv stage of
//                         the gated delta net
//   zb_gated_delta_scan   the gated delta rule recurrence with the per-head state held in
//                         registers, fused with the q/k L2 normalisation, the decay / write-gate
//                         transforms and the gated RMSNorm of the output
//   zb_sigmoid_gate_mul   attention output * sigmoid(gate) of the gated full-attention layers
//
// The reference expresses the recurrence as a `stablehlo.while` over tokens (zml/nn.zig:1749-1874)
// and the convolutions as XLA conv1d + scatter on a cache tensor
// (examples/llm/models/qwen3_5/model.zig:882-980, examples/llm/models/lfm2/model.zig:441-500).
// Here a sequence is walked once by one CTA per (sequence, head) or (sequence, channel block);
// prefill chunks and decode steps use the same kernels, the state lives in a slot pool.
#include <cuda_bf16.h>

#include "common.cuh"
#include "host_api.h"

namespace {
constexpr uint32_t kKernelCausalConv = 24;
constexpr uint32_t kKernelGdnScan = 25;

// ------------------------------------------------------------------------------------------
struct ConvParams {
  const __nv_bfloat16* x;      // [T, ldx] conv input columns
  long long ldx;
  const __nv_bfloat16* pre;    // optional [T, ldpre]: input gate, conv input = pre * x
  long long ldpre;
  const __nv_bfloat16* post;   // optional [T, ldpost]: output gate
  long long ldpost;
  const __nv_bfloat16* w;      // [C, K] taps, tap K-1 multiplies the current token
  __nv_bfloat16* out;          // [T, ldo]
  long long ldo;
  __nv_bfloat16* state;        // [slots, K-1, C] last K-1 conv inputs of every sequence
  const int32_t* q_start;      // [S+1] token range of every sequence in this launch
  const int32_t* seq_lens;     // [S] sequence length including this launch's tokens
  const int32_t* slots;        // [S] state slot of every sequence
  int channels;
  int silu;
};

template <int K>
__global__ void __launch_bounds__(128) zb_causal_conv1d_kernel(const ConvParams p) {
  zb_pdl_launch();
  zb_pdl_wait();
  const int c = blockIdx.x * 128 + threadIdx.x;
  const int s = blockIdx.y;
  if (c >= p.channels) return;
  const int t0 = p.q_start[s], t1 = p.q_start[s + 1];
  if (t1 <= t0) return;
  const bool fresh = p.seq_lens[s] - (t1 - t0) <= 0;
  if (!ZB_BC_OK(p.slots[s], ZB_BC_STATE_SLOTS, kKernelCausalConv, 1)) return;
  __nv_bfloat16* st = p.state + static_cast<size_t>(p.slots[s]) * (K - 1) * p.channels + c;
  float w[K], win[K - 1];
#pragma unroll
  for (int j = 0; j < K; ++j) w[j] = __bfloat162float(p.w[static_cast<size_t>(c) * K + j]);
#pragma unroll
  for (int j = 0; j < K - 1; ++j) win[j] = fresh ? 0.f : __bfloat162float(st[static_cast<size_t>(j) * p.channels]);
  for (int t = t0; t < t1; ++t) {
    float xin = __bfloat162float(p.x[t * p.ldx + c]);
    if (p.pre != nullptr) xin = __bfloat162float(__float2bfloat16(xin * __bfloat162float(p.pre[t * p.ldpre + c])));
    float acc = w[K - 1] * xin;
#pragma unroll
    for (int j = 0; j < K - 1; ++j) acc += w[j] * win[j];
#pragma unroll
    for (int j = 0; j + 1 < K - 1; ++j) win[j] = win[j + 1];
    win[K - 2] = xin;
    acc = __bfloat162float(__float2bfloat16(acc));
    if (p.silu) acc = acc / (1.f + __expf(-acc));
    if (p.post != nullptr) acc = __bfloat162float(__float2bfloat16(acc)) * __bfloat162float(p.post[t * p.ldpost + c]);
    p.out[t * p.ldo + c] = __float2bfloat16(acc);
  }
#pragma unroll
  for (int j = 0; j < K - 1; ++j) st[static_cast<size_t>(j) * p.channels] = __float2bfloat16(win[j]);
}

// ------------------------------------------------------------------------------------------
struct GdnParams {
  const __nv_bfloat16* mix;    // [T, ld_mix]: q heads | k heads | v heads (after conv + SiLU)
  long long ld_mix;
  const __nv_bfloat16* z;      // [T, ld_z]: gate of the output norm, hv * dv columns
  long long ld_z;
  const __nv_bfloat16* a;      // [T, ld_ab]: decay projection, hv columns
  const __nv_bfloat16* b;      // [T, ld_ab]: write-gate projection, hv columns
  long long ld_ab;
  const float* a_log;          // [hv]
  const float* dt_bias;        // [hv]
  const __nv_bfloat16* norm_w; // [dv]
  float eps;
  float* state;                // [slots, hv, DK, dv] fp32
  __nv_bfloat16* out;          // [T, ld_out], hv * dv columns
  long long ld_out;
  const int32_t* q_start;
  const int32_t* seq_lens;
  const int32_t* slots;
  int hk, hv, dv;
};

constexpr int kGdnChunk = 16;

// One CTA per (value head, sequence); thread j owns column j of the state S[DK][dv]:
//   v_hat = alpha * (S^T k);  delta = beta * (v - v_hat);  S = alpha * S + k delta^T;  y = S^T q
template <int DK>
__global__ void __launch_bounds__(256) zb_gated_delta_scan_kernel(const GdnParams p) {
  zb_pdl_launch();
  zb_pdl_wait();
  extern __shared__ float gdn_smem[];
  const int h = blockIdx.x, s = blockIdx.y, j = threadIdx.x;
  const int dv = p.dv;
  const int t0 = p.q_start[s], t1 = p.q_start[s + 1];
  const int n = t1 - t0;
  if (n <= 0) return;
  if (!ZB_BC_OK(p.slots[s], ZB_BC_STATE_SLOTS, kKernelGdnScan, 1)) return;      // uniform over the block: no barrier is skipped by a part of it
  float* sq = gdn_smem;                       // [CH][DK]
  float* sk = sq + kGdnChunk * DK;            // [CH][DK]
  float* sv = sk + kGdnChunk * DK;            // [CH][dv]
  float* sy = sv + kGdnChunk * dv;            // [CH][dv]
  float* salpha = sy + kGdnChunk * dv;        // [CH]
  float* sbeta = salpha + kGdnChunk;          // [CH]
  const bool fresh = p.seq_lens[s] - n <= 0;
  const int warp = j >> 5, lane = j & 31, nwarps = blockDim.x >> 5;
  const bool active = j < dv;
  const int jj = active ? j : 0;
  float* st = p.state + (static_cast<size_t>(p.slots[s]) * p.hv + h) * DK * dv + jj;
  float S[DK];
#pragma unroll
  for (int k = 0; k < DK; ++k) S[k] = (fresh || !active) ? 0.f : st[static_cast<size_t>(k) * dv];
  const int kh = h / (p.hv / p.hk);
  const int key_dim = p.hk * DK;
  const float neg_a = -__expf(p.a_log[h]);
  const float dtb = p.dt_bias[h];
  const float q_scale = rsqrtf(static_cast<float>(DK));

  for (int c0 = 0; c0 < n; c0 += kGdnChunk) {
    const int cn = min(kGdnChunk, n - c0);
    for (int idx = j; idx < cn * DK; idx += blockDim.x) {
      const int tt = idx / DK, kk = idx - tt * DK;
      const __nv_bfloat16* row = p.mix + (t0 + c0 + tt) * p.ld_mix + kh * DK + kk;
      sq[idx] = __bfloat162float(row[0]);
      sk[idx] = __bfloat162float(row[key_dim]);
    }
    if (active) {
      for (int tt = 0; tt < cn; ++tt)
        sv[tt * dv + j] = __bfloat162float(p.mix[(t0 + c0 + tt) * p.ld_mix + 2 * key_dim + h * dv + j]);
    }
    if (j < cn) {
      const float av = __bfloat162float(p.a[(t0 + c0 + j) * p.ld_ab + h]) + dtb;
      const float sp = av > 20.f ? av : log1pf(__expf(av));
      salpha[j] = __expf(neg_a * sp);
      const float bv = __bfloat162float(p.b[(t0 + c0 + j) * p.ld_ab + h]);
      sbeta[j] = 1.f / (1.f + __expf(-bv));
    }
    __syncthreads();
    // L2-normalise the chunk's q and k vectors (one warp per vector); q also takes 1/sqrt(DK)
    for (int vec = warp; vec < 2 * cn; vec += nwarps) {
      float* ptr = vec < cn ? sq + vec * DK : sk + (vec - cn) * DK;
      float ss = 0.f;
      for (int k = lane; k < DK; k += 32) ss += ptr[k] * ptr[k];
      ss = zb_warp_sum(ss);
      const float inv = rsqrtf(ss + 1e-6f) * (vec < cn ? q_scale : 1.f);
      for (int k = lane; k < DK; k += 32) ptr[k] *= inv;
    }
    __syncthreads();
    for (int tt = 0; tt < cn; ++tt) {
      const float alpha = salpha[tt], beta = sbeta[tt];
      const float4* k4 = reinterpret_cast<const float4*>(sk + tt * DK);
      const float4* q4 = reinterpret_cast<const float4*>(sq + tt * DK);
      float vh = 0.f;
#pragma unroll
      for (int k = 0; k < DK / 4; ++k) {
        const float4 kv = k4[k];
        vh += S[4 * k] * kv.x + S[4 * k + 1] * kv.y + S[4 * k + 2] * kv.z + S[4 * k + 3] * kv.w;
      }
      const float delta = (sv[tt * dv + jj] - alpha * vh) * beta;
      float y = 0.f;
#pragma unroll
      for (int k = 0; k < DK / 4; ++k) {
        const float4 kv = k4[k];
        const float4 qv = q4[k];
        S[4 * k] = alpha * S[4 * k] + kv.x * delta;
        S[4 * k + 1] = alpha * S[4 * k + 1] + kv.y * delta;
        S[4 * k + 2] = alpha * S[4 * k + 2] + kv.z * delta;
        S[4 * k + 3] = alpha * S[4 * k + 3] + kv.w * delta;
        y += S[4 * k] * qv.x + S[4 * k + 1] * qv.y + S[4 * k + 2] * qv.z + S[4 * k + 3] * qv.w;
      }
      if (active) sy[tt * dv + j] = __bfloat162float(__float2bfloat16(y));
    }
    __syncthreads();
    // gated RMSNorm over the head's dv outputs: weight * y / rms(y) * silu(z); one warp per token
    for (int tt = warp; tt < cn; tt += nwarps) {
      float ss = 0.f;
      for (int e = lane; e < dv; e += 32) ss += sy[tt * dv + e] * sy[tt * dv + e];
      ss = zb_warp_sum(ss);
      const float inv = rsqrtf(ss / static_cast<float>(dv) + p.eps);
      const size_t t = static_cast<size_t>(t0 + c0 + tt);
      for (int e = lane; e < dv; e += 32) {
        const float zg = __bfloat162float(p.z[t * p.ld_z + h * dv + e]);
        const float o = sy[tt * dv + e] * inv * __bfloat162float(p.norm_w[e]) * (zg / (1.f + __expf(-zg)));
        p.out[t * p.ld_out + h * dv + e] = __float2bfloat16(o);
      }
    }
    __syncthreads();
  }
  if (active) {
#pragma unroll
    for (int k = 0; k < DK; ++k) st[static_cast<size_t>(k) * dv] = S[k];
  }
}

// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) zb_sigmoid_gate_mul_kernel(__nv_bfloat16* __restrict__ x, long long ldx,
                                                                  const __nv_bfloat16* __restrict__ gate, long long ldg,
                                                                  int rows, int cols_vec) {
  zb_pdl_launch();
  zb_pdl_wait();
  const long long total = static_cast<long long>(rows) * cols_vec;
  for (long long idx = blockIdx.x * 256ll + threadIdx.x; idx < total; idx += static_cast<long long>(gridDim.x) * 256) {
    const long long r = idx / cols_vec;
    const int cv = static_cast<int>(idx - r * cols_vec);
    uint4 xv = *reinterpret_cast<const uint4*>(x + r * ldx + cv * 8);
    const uint4 gv = *reinterpret_cast<const uint4*>(gate + r * ldg + cv * 8);
    __nv_bfloat162* xp = reinterpret_cast<__nv_bfloat162*>(&xv);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gv);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 xf = __bfloat1622float2(xp[i]);
      const float2 gf = __bfloat1622float2(gp[i]);
      xp[i] = __floats2bfloat162_rn(xf.x / (1.f + __expf(-gf.x)), xf.y / (1.f + __expf(-gf.y)));
    }
    *reinterpret_cast<uint4*>(x + r * ldx + cv * 8) = xv;
  }
}

template <int DK>
int launch_gdn(const GdnParams& p, int num_seqs, cudaStream_t s) {
  const int threads = (p.dv + 31) / 32 * 32;
  const size_t smem = (2 * kGdnChunk * DK + 2 * kGdnChunk * p.dv + 2 * kGdnChunk) * sizeof(float);
  static bool configured[16] = {};
  if (const int rc = zb_config_smem_once(zb_gated_delta_scan_kernel<DK>, (2 * kGdnChunk * DK + 2 * kGdnChunk * 256 + 2 * kGdnChunk) * 4, configured)) return rc;
  zb_launch(zb_gated_delta_scan_kernel<DK>, dim3(p.hv, num_seqs), dim3(threads), smem, s, p);
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

extern "C" {

// Depthwise causal conv over a flattened varlen batch; `kernel_size` taps per channel, 2..5.
int zb_causal_conv1d(const void* x, long long ldx, const void* pre, long long ldpre, const void* post,
                     long long ldpost, const void* w, void* out, long long ldo, void* state,
                     const int32_t* q_start, const int32_t* seq_lens, const int32_t* slots, int num_seqs,
                     int channels, int kernel_size, int silu, void* stream) {
  if (num_seqs <= 0 || channels <= 0) return 0;
  ConvParams p;
  p.x = reinterpret_cast<const __nv_bfloat16*>(x);
  p.ldx = ldx;
  p.pre = reinterpret_cast<const __nv_bfloat16*>(pre);
  p.ldpre = ldpre;
  p.post = reinterpret_cast<const __nv_bfloat16*>(post);
  p.ldpost = ldpost;
  p.w = reinterpret_cast<const __nv_bfloat16*>(w);
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.ldo = ldo;
  p.state = reinterpret_cast<__nv_bfloat16*>(state);
  p.q_start = q_start;
  p.seq_lens = seq_lens;
  p.slots = slots;
  p.channels = channels;
  p.silu = silu;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const dim3 grid((channels + 127) / 128, num_seqs);
  switch (kernel_size) {
    case 2: zb_launch(zb_causal_conv1d_kernel<2>, grid, dim3(128), 0, s, p); break;
    case 3: zb_launch(zb_causal_conv1d_kernel<3>, grid, dim3(128), 0, s, p); break;
    case 4: zb_launch(zb_causal_conv1d_kernel<4>, grid, dim3(128), 0, s, p); break;
    case 5: zb_launch(zb_causal_conv1d_kernel<5>, grid, dim3(128), 0, s, p); break;
    default: return -70;
  }
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

// Gated delta rule over a flattened varlen batch.  dk in {64, 128}; dv a multiple of 32, <= 256.
int zb_gated_delta_scan(const void* mix, long long ld_mix, const void* z, long long ld_z, const void* a,
                        const void* b, long long ld_ab, const float* a_log, const float* dt_bias,
                        const void* norm_w, float eps, float* state, void* out, long long ld_out,
                        const int32_t* q_start, const int32_t* seq_lens, const int32_t* slots, int num_seqs,
                        int hk, int hv, int dk, int dv, void* stream) {
  if (num_seqs <= 0) return 0;
  if (hk <= 0 || hv % hk != 0 || dv % 32 != 0 || dv > 256) return -71;
  GdnParams p;
  p.mix = reinterpret_cast<const __nv_bfloat16*>(mix);
  p.ld_mix = ld_mix;
  p.z = reinterpret_cast<const __nv_bfloat16*>(z);
  p.ld_z = ld_z;
  p.a = reinterpret_cast<const __nv_bfloat16*>(a);
  p.b = reinterpret_cast<const __nv_bfloat16*>(b);
  p.ld_ab = ld_ab;
  p.a_log = a_log;
  p.dt_bias = dt_bias;
  p.norm_w = reinterpret_cast<const __nv_bfloat16*>(norm_w);
  p.eps = eps;
  p.state = state;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.ld_out = ld_out;
  p.q_start = q_start;
  p.seq_lens = seq_lens;
  p.slots = slots;
  p.hk = hk;
  p.hv = hv;
  p.dv = dv;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (dk == 64) return launch_gdn<64>(p, num_seqs, s);
  if (dk == 128) return launch_gdn<128>(p, num_seqs, s);
  return -72;
}

// x[r, c] *= sigmoid(gate[r, c]) in place; cols a multiple of 8, rows 16-byte aligned.
int zb_sigmoid_gate_mul(void* x, long long ldx, const void* gate, long long ldg, int rows, int cols, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (cols % 8 != 0 || ldx % 8 != 0 || ldg % 8 != 0) return -73;
  const long long total = static_cast<long long>(rows) * (cols / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  zb_launch(zb_sigmoid_gate_mul_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0,
            reinterpret_cast<cudaStream_t>(stream), reinterpret_cast<__nv_bfloat16*>(x), ldx,
            reinterpret_cast<const __nv_bfloat16*>(gate), ldg, rows, cols / 8);
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
