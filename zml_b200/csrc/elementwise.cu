// Bandwidth-bound layer glue for sm_100a: RMSNorm(+residual), RoPE fused with the
// paged KV-cache write (and optional per-head q/k RMSNorm), SwiGLU, embedding
// gather, argmax and top-k + Gumbel-max sampling.
//
// These replace XLA's elementwise / reduction fusions of the reference:
// rmsNorm zml/nn.zig:486-493, rope zml/nn.zig:687-716, KvCache.update
// zml/attention/paged_attention.zig:218-254, swiglu
// examples/llm/models/llama/model.zig:491-496, TokenEmbedding zml/nn.zig:432-436,
// sampleTokens zml/nn.zig:1999-2033.
#include "common.cuh"
#include "host_api.h"

namespace {
constexpr uint32_t kKernelRopeKvWrite = 20;
constexpr uint32_t kKernelEmbedding = 21;
constexpr uint32_t kKernelDecodeAdvance = 22;

// ---------------------------------------------------------------- RMSNorm
// y = x_total * rsqrt(mean(x_total^2) + eps) * (w or 1 + w), x_total = x (+ residual).
// When residual_out != null the summed row is written back (pre-norm residual stream).
template <int VEC_PER_THREAD>
__global__ void __launch_bounds__(256) zb_rmsnorm_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
    const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out,
    __nv_bfloat16* __restrict__ residual_out, int rows, int d, long long x_stride,
    long long out_stride, float eps, int unit_offset) {
  zb_pdl_launch();
  zb_pdl_wait();
  const int row = blockIdx.x;
  if (row >= rows) return;
  const int nvec = d >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * x_stride);
  const uint4* rr = residual ? reinterpret_cast<const uint4*>(residual + static_cast<size_t>(row) * d) : nullptr;
  uint4* ro = residual_out ? reinterpret_cast<uint4*>(residual_out + static_cast<size_t>(row) * d) : nullptr;
  float vals[VEC_PER_THREAD][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VEC_PER_THREAD; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v < nvec) {
      uint4 a = xr[v];
      const uint32_t au[4] = {a.x, a.y, a.z, a.w};
      uint32_t bu[4] = {0, 0, 0, 0};
      if (rr) {
        uint4 b = rr[v];
        bu[0] = b.x; bu[1] = b.y; bu[2] = b.z; bu[3] = b.w;
      }
      uint32_t su[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = zb_unpack_bf16x2(au[j]);
        if (rr) {
          float2 g = zb_unpack_bf16x2(bu[j]);
          f.x += g.x;
          f.y += g.y;
          // the residual stream is stored in bf16: normalise what is stored
          su[j] = zb_pack_bf16x2(f.x, f.y);
          f = zb_unpack_bf16x2(su[j]);
        }
        vals[i][2 * j] = f.x;
        vals[i][2 * j + 1] = f.y;
        ss += f.x * f.x + f.y * f.y;
      }
      if (ro) ro[v] = rr ? make_uint4(su[0], su[1], su[2], su[3]) : a;
    }
  }
  __shared__ float red[8];
  ss = zb_warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float inv = rsqrtf(tot / static_cast<float>(d) + eps);
  uint4* orow = reinterpret_cast<uint4*>(out + static_cast<size_t>(row) * out_stride);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
#pragma unroll
  for (int i = 0; i < VEC_PER_THREAD; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v < nvec) {
      uint32_t wu[4] = {0, 0, 0, 0};
      if (w) {
        uint4 ww = wr[v];
        wu[0] = ww.x; wu[1] = ww.y; wu[2] = ww.z; wu[3] = ww.w;
      }
      uint32_t ou[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 g = w ? zb_unpack_bf16x2(wu[j]) : make_float2(1.f, 1.f);
        if (unit_offset) {
          g.x += 1.f;
          g.y += 1.f;
        }
        ou[j] = zb_pack_bf16x2(vals[i][2 * j] * inv * g.x, vals[i][2 * j + 1] * inv * g.y);
      }
      orow[v] = make_uint4(ou[0], ou[1], ou[2], ou[3]);
    }
  }
}

// ---------------------------------------------------------------- RoPE + KV write
// One warp per (token, head) of the fused qkv activation [T, (Hq + 2*Hkv) * hd].
//   q heads : optional RMSNorm over hd, rotate, write to q_out [T, Hq, hd]
//   k heads : optional RMSNorm, rotate, write into the paged K cache at slot_mapping[t]
//   v heads : copy into the paged V cache
// rope layout 0 (real_im_pass, HF rotate_half): pairs (i, i + rot/2), pass-through after rot;
//             1 (interleaved): pairs (2i, 2i + 1);
//             2 (real_pass_im_pass): pairs (i, hd/2 + i) for i < rot/2.
struct RopeParams {
  const __nv_bfloat16* qkv;
  __nv_bfloat16* q_out;
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
  const int32_t* positions;
  const int32_t* slot_mapping;
  const float* inv_freq;        // [rot_dim / 2]
  const __nv_bfloat16* q_norm_w;  // [hd] or null
  const __nv_bfloat16* k_norm_w;
  long long qkv_stride;
  int tokens, hq, hkv, hd, rot_dim, layout, page_size;
  float attn_factor;            // yarn magnitude scaling applied to cos/sin
  float norm_eps;
  int norm_unit_offset;
  long long num_slots;          // bounds for slot_mapping; slots < 0 are skipped (padding)
};

// One warp takes `heads_per_warp` consecutive heads (q, then k, then v) of one token: the rotation angles
// depend on the token only, so sin / cos are computed once per warp and reused for its heads (with one head
// per warp the accurate sincosf on position x frequency dominated prefill: 128 us for 8 192 tokens x 36 heads).
__global__ void __launch_bounds__(128) zb_rope_kvwrite_kernel(const RopeParams p, int heads_per_warp) {
  zb_pdl_launch();
  zb_pdl_wait();
  const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int heads = p.hq + 2 * p.hkv;
  const int groups = (heads + heads_per_warp - 1) / heads_per_warp;
  if (warp_global >= p.tokens * groups) return;
  const int tok = warp_global / groups;
  const int h_begin = (warp_global - tok * groups) * heads_per_warp;
  const int h_end = min(heads, h_begin + heads_per_warp);
  const int half = p.rot_dim >> 1;
  const int hh = p.hd >> 1;
  constexpr int kMaxAngles = 4;                // half <= 128
  float sn_r[kMaxAngles], cs_r[kMaxAngles];
  // Fast path (head_dim 128, whole head rotated, halves layout): a lane holds 4 consecutive elements of the
  // head (one 8-byte load and store per head), its rotation partner sits 16 lanes away.
  const bool fast = p.layout == 0 && p.rot_dim == p.hd && p.hd == 128;
  if (h_begin < p.hq + p.hkv) {
    const float pos = static_cast<float>(p.positions[tok]);
#pragma unroll
    for (int a = 0; a < kMaxAngles; ++a) {
      const int i = fast ? 4 * (lane & 15) + a : lane + 32 * a;
      sn_r[a] = 0.f;
      cs_r[a] = 1.f;
      if (i < half) {
        sincosf(pos * p.inv_freq[i], &sn_r[a], &cs_r[a]);
        sn_r[a] *= p.attn_factor;
        cs_r[a] *= p.attn_factor;
      }
    }
  }
  const long long slot = p.slot_mapping[tok];
  // negative = padding row (no KV write); the checking build reports a slot past the cache instead of dropping it
  if (slot >= p.num_slots) (void)ZB_BC_OK(slot, p.num_slots, kKernelRopeKvWrite, 1);
  const bool slot_ok = slot >= 0 && slot < p.num_slots;
  for (int h = h_begin; h < h_end; ++h) {
    const __nv_bfloat16* __restrict__ src = p.qkv + static_cast<size_t>(tok) * p.qkv_stride + static_cast<size_t>(h) * p.hd;
    const bool is_q = h < p.hq;
    const bool is_k = !is_q && h < p.hq + p.hkv;
    __nv_bfloat16* __restrict__ dst;
    if (is_q) {
      dst = p.q_out + (static_cast<size_t>(tok) * p.hq + h) * p.hd;
    } else {
      if (!slot_ok) continue;
      const int kvh = is_k ? h - p.hq : h - p.hq - p.hkv;
      __nv_bfloat16* cache = is_k ? p.k_cache : p.v_cache;
      dst = cache + (static_cast<size_t>(slot) * p.hkv + kvh) * p.hd;
    }
    if (!is_q && !is_k) {
      // V: plain copy, 16 bytes per lane per step
      const uint4* s4 = reinterpret_cast<const uint4*>(src);
      uint4* d4 = reinterpret_cast<uint4*>(dst);
      for (int i = lane; i < p.hd / 8; i += 32) d4[i] = s4[i];
      continue;
    }
    const __nv_bfloat16* nw = is_q ? p.q_norm_w : p.k_norm_w;
    if (fast) {
      const uint2 raw = reinterpret_cast<const uint2*>(src)[lane];
      const float2 lo = zb_unpack_bf16x2(raw.x), hi = zb_unpack_bf16x2(raw.y);
      float v[4] = {lo.x, lo.y, hi.x, hi.y};
      if (nw) {
        const float ss = zb_warp_sum(v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3]);
        const float inv = rsqrtf(ss / 128.f + p.norm_eps);
        const uint2 graw = reinterpret_cast<const uint2*>(nw)[lane];
        const float2 g0 = zb_unpack_bf16x2(graw.x), g1 = zb_unpack_bf16x2(graw.y);
        const float g[4] = {g0.x, g0.y, g1.x, g1.y};
#pragma unroll
        for (int j = 0; j < 4; ++j)      // normalised in f32, rounded to the activation dtype before rotating (as the reference does)
          v[j] = __bfloat162float(__float2bfloat16(v[j] * inv * (g[j] + (p.norm_unit_offset ? 1.f : 0.f))));
      }
      float o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float partner = __shfl_xor_sync(0xffffffffu, v[j], 16);
        o[j] = lane < 16 ? v[j] * cs_r[j] - partner * sn_r[j] : v[j] * cs_r[j] + partner * sn_r[j];
      }
      reinterpret_cast<uint2*>(dst)[lane] = make_uint2(zb_pack_bf16x2(o[0], o[1]), zb_pack_bf16x2(o[2], o[3]));
      continue;
    }
    float inv_rms = 1.f;
    if (nw) {
      float ss = 0.f;
      for (int i = lane; i < p.hd; i += 32) {
        const float v = __bfloat162float(src[i]);
        ss += v * v;
      }
      ss = zb_warp_sum(ss);
      inv_rms = rsqrtf(ss / static_cast<float>(p.hd) + p.norm_eps);
    }
    auto load = [&](int i) -> float {
      float v = __bfloat162float(src[i]);
      if (nw) {
        float g = __bfloat162float(nw[i]);
        if (p.norm_unit_offset) g += 1.f;
        // the reference normalises in f32 and rounds to the activation dtype before rotating
        v = __bfloat162float(__float2bfloat16(v * inv_rms * g));
      }
      return v;
    };
#pragma unroll
    for (int a = 0; a < kMaxAngles; ++a) {
      const int i = lane + 32 * a;
      if (i >= half) continue;
      const int i0 = p.layout == 1 ? 2 * i : i;
      const int i1 = p.layout == 0 ? i + half : (p.layout == 1 ? 2 * i + 1 : i + hh);
      const float x = load(i0), y = load(i1);
      dst[i0] = __float2bfloat16(x * cs_r[a] - y * sn_r[a]);
      dst[i1] = __float2bfloat16(y * cs_r[a] + x * sn_r[a]);
    }
    if (p.rot_dim < p.hd) {
      for (int i = lane; i < p.hd; i += 32) {
        const bool rotated = p.layout == 2 ? ((i < half) || (i >= hh && i < hh + half)) : (i < p.rot_dim);
        if (!rotated) dst[i] = __float2bfloat16(load(i));
      }
    }
  }
}

// ---------------------------------------------------------------- SwiGLU
// out[t, f] = silu(gu[t, f]) * gu[t, F + f]
__global__ void __launch_bounds__(256) zb_swiglu_kernel(const __nv_bfloat16* __restrict__ gu,
                                                        __nv_bfloat16* __restrict__ out,
                                                        long long total_vec, int f_vec) {
  zb_pdl_launch();
  zb_pdl_wait();
  for (long long idx = blockIdx.x * 256ll + threadIdx.x; idx < total_vec;
       idx += static_cast<long long>(gridDim.x) * 256) {
    const long long t = idx / f_vec;
    const int fv = static_cast<int>(idx % f_vec);
    const uint4* row = reinterpret_cast<const uint4*>(gu) + t * (2ll * f_vec);
    const uint4 g = row[fv];
    const uint4 u = row[f_vec + fv];
    const uint32_t gg[4] = {g.x, g.y, g.z, g.w}, uu[4] = {u.x, u.y, u.z, u.w};
    uint32_t oo[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = zb_unpack_bf16x2(gg[j]);
      const float2 b = zb_unpack_bf16x2(uu[j]);
      const float s0 = a.x / (1.f + __expf(-a.x));
      const float s1 = a.y / (1.f + __expf(-a.y));
      oo[j] = zb_pack_bf16x2(s0 * b.x, s1 * b.y);
    }
    reinterpret_cast<uint4*>(out)[idx] = make_uint4(oo[0], oo[1], oo[2], oo[3]);
  }
}

// ---------------------------------------------------------------- embedding
__global__ void __launch_bounds__(128) zb_embedding_kernel(const int32_t* __restrict__ ids,
                                                           const __nv_bfloat16* __restrict__ table,
                                                           __nv_bfloat16* __restrict__ out, int tokens,
                                                           int d, int vocab) {
  zb_pdl_launch();
  zb_pdl_wait();
  const int t = blockIdx.x;
  if (t >= tokens) return;
  int id = ids[t];
  if (id < 0 || id >= vocab) {
    (void)ZB_BC_OK(id, vocab, kKernelEmbedding, 1);      // the checking build reports the id; both builds read row 0
    id = 0;
  }
  const uint4* src = reinterpret_cast<const uint4*>(table + static_cast<size_t>(id) * d);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * d);
  for (int i = threadIdx.x; i < d / 8; i += 128) dst[i] = src[i];
}

// ---------------------------------------------------------------- argmax
// First index of the row maximum (ties -> lowest index, NaN ignored), f32 logits.
__global__ void __launch_bounds__(1024) zb_argmax_f32_kernel(const float* __restrict__ logits,
                                                             int32_t* __restrict__ out, int vocab,
                                                             long long stride) {
  zb_pdl_launch();
  zb_pdl_wait();
  float best;
  int bi;
  zb_block_argmax_1024(logits + static_cast<size_t>(blockIdx.x) * stride, vocab, best, bi);
  if (threadIdx.x == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
}

// ---------------------------------------------------------------- top-k + Gumbel-max
// Per row: select the k largest logits (k <= 128) with a 4-pass radix select on the
// order-preserving integer image of the floats, then draw one of them with the
// Gumbel-max trick at the given temperature (sampleTokens, zml/nn.zig:2007-2033).
// Also writes the selected (value, index) pairs, sorted descending, when asked.
ZB_DEVICE uint32_t float_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

ZB_DEVICE float uniform01(uint64_t seed, uint64_t idx) {
  // splitmix64 -> 23 mantissa bits -> [1, 2) - 1, as the reference's Rng.uniform does
  uint64_t z = seed + 0x9e3779b97f4a7c15ull * (idx + 1);
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  z ^= z >> 31;
  const uint32_t mant = static_cast<uint32_t>(z >> 41);
  return __uint_as_float(0x3f800000u | mant) - 1.f;
}

constexpr int kMaxTopK = 128;

__global__ void __launch_bounds__(1024) zb_topk_sample_kernel(
    const float* __restrict__ logits, int32_t* __restrict__ out_token, float* __restrict__ topk_vals,
    int32_t* __restrict__ topk_idx, int vocab, long long stride, int k, float temperature,
    uint64_t seed, uint64_t step, const unsigned long long* __restrict__ dev_rng) {
  zb_pdl_launch();
  zb_pdl_wait();
  if (dev_rng != nullptr) {
    // seed and draw counter live on the device: a captured CUDA graph then samples with fresh noise at every
    // replay (the counter is advanced by zb_decode_advance) and with whatever seed was copied in before it
    seed = dev_rng[0];
    step += dev_rng[1];
  }
  const float* row = logits + static_cast<size_t>(blockIdx.x) * stride;
  __shared__ uint32_t hist[256];
  __shared__ uint32_t s_prefix, s_remaining;
  __shared__ float cand_v[kMaxTopK * 2];
  __shared__ int cand_i[kMaxTopK * 2];
  __shared__ uint32_t cand_n;
  if (threadIdx.x == 0) {
    s_prefix = 0;
    s_remaining = k;
    cand_n = 0;
  }
  __syncthreads();
  // radix select: find the key of the k-th largest element
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = threadIdx.x; i < 256; i += 1024) hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const uint32_t mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = threadIdx.x; i < vocab; i += 1024) {
      const uint32_t key = float_key(row[i]);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xff], 1u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t rem = s_remaining;
      int b = 255;
      for (; b > 0; --b) {
        if (hist[b] >= rem) break;
        rem -= hist[b];
      }
      s_prefix = prefix | (static_cast<uint32_t>(b) << shift);
      s_remaining = rem;
    }
    __syncthreads();
  }
  const uint32_t kth = s_prefix;           // key of the k-th largest value
  const uint32_t ties_wanted = s_remaining;  // how many elements equal to it belong to the top-k
  // gather: everything strictly greater than the k-th value, and (separately) the
  // indices of the elements equal to it; the lowest-index ties complete the top-k
  __shared__ int tie_i[256];
  __shared__ uint32_t tie_n;
  if (threadIdx.x == 0) tie_n = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < vocab; i += 1024) {
    const float v = row[i];
    const uint32_t key = float_key(v);
    if (key > kth) {
      const uint32_t slot = atomicAdd(&cand_n, 1u);
      if (slot < kMaxTopK * 2) {
        cand_v[slot] = v;
        cand_i[slot] = i;
      }
    } else if (key == kth) {
      const uint32_t slot = atomicAdd(&tie_n, 1u);
      if (slot < 256) tie_i[slot] = i;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t n = cand_n < static_cast<uint32_t>(k) ? cand_n : static_cast<uint32_t>(k);
    const uint32_t nt = tie_n < 256u ? tie_n : 256u;
    uint32_t need = ties_wanted;
    int last = -1;
    while (need > 0 && n < static_cast<uint32_t>(k)) {
      int best = 0x7fffffff;
      for (uint32_t j = 0; j < nt; ++j)
        if (tie_i[j] > last && tie_i[j] < best) best = tie_i[j];
      if (best == 0x7fffffff) break;
      cand_v[n] = row[best];
      cand_i[n] = best;
      last = best;
      ++n;
      --need;
    }
    cand_n = n;
  }
  __syncthreads();
  const int n = static_cast<int>(cand_n);
  // small sort (descending by value, ascending index on ties): rank by counting
  __shared__ float sort_v[kMaxTopK];
  __shared__ int sort_i[kMaxTopK];
  if (threadIdx.x < n) {
    const float v = cand_v[threadIdx.x];
    const int id = cand_i[threadIdx.x];
    int rank = 0;
    for (int j = 0; j < n; ++j) {
      const float ov = cand_v[j];
      const int oi = cand_i[j];
      if (ov > v || (ov == v && oi < id)) ++rank;
    }
    sort_v[rank] = v;
    sort_i[rank] = id;
  }
  __syncthreads();
  if (topk_vals && threadIdx.x < k) {
    topk_vals[static_cast<size_t>(blockIdx.x) * k + threadIdx.x] = threadIdx.x < n ? sort_v[threadIdx.x] : -INFINITY;
    topk_idx[static_cast<size_t>(blockIdx.x) * k + threadIdx.x] = threadIdx.x < n ? sort_i[threadIdx.x] : 0;
  }
  if (threadIdx.x < 32) {
    float best = -INFINITY;
    int bi = n > 0 ? sort_i[0] : 0;
    for (int j = threadIdx.x; j < n; j += 32) {
      float score = sort_v[j];
      if (temperature > 0.f && k > 1) {
        const float u = fmaxf(uniform01(seed, (step * gridDim.x + blockIdx.x) * kMaxTopK + j), 1e-20f);
        score = score / temperature - __logf(-__logf(u));
      }
      if (score > best) {
        best = score;
        bi = sort_i[j];
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best) {
        best = ov;
        bi = oi;
      }
    }
    if (threadIdx.x == 0) out_token[blockIdx.x] = bi;
  }
}


// ---------------------------------------------------------------- decode bookkeeping
// After sampling: feed the sampled token back as the next input, advance position and
// length, compute the KV slot of the new position from the block table, and append the
// token to the on-device history so that the host can read tokens in batches.
__global__ void zb_decode_advance_kernel(const int32_t* __restrict__ sampled, int32_t* __restrict__ ids,
                                         int32_t* __restrict__ positions, int32_t* __restrict__ seq_lens,
                                         int32_t* __restrict__ slot_mapping,
                                         const int32_t* __restrict__ block_table, int32_t* __restrict__ history,
                                         int32_t* __restrict__ step_counter, int batch, int max_pages,
                                         int page_size, int history_stride, int history_rows) {
  zb_pdl_launch();
  zb_pdl_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  const int step = *step_counter;
  if (b < batch) {
    const int tok = sampled[b];
    ids[b] = tok;
    const int pos = positions[b] + 1;
    positions[b] = pos;
    seq_lens[b] = pos + 1;
    const int pg = pos / page_size;
    int page = pg < max_pages ? block_table[static_cast<size_t>(b) * max_pages + pg] : -1;
    if (page >= 0 && !ZB_BC_OK(page, ZB_BC_PAGES, kKernelDecodeAdvance, 1)) page = -1;
    slot_mapping[b] = page >= 0 ? page * page_size + pos % page_size : -1;
    if (step < history_rows) history[static_cast<size_t>(step) * history_stride + b] = tok;
  }
}

// Runs after the kernel above on the same stream, so every block has read the old value.
__global__ void zb_counter_inc_kernel(int32_t* c, unsigned long long* rng) {
  zb_pdl_launch();
  zb_pdl_wait();
  *c += 1;
  if (rng != nullptr) rng[1] += 1ull;      // one more draw of the sampler (see zb_topk_sample_rng)
}

__global__ void zb_u64_add_kernel(unsigned long long* p, unsigned long long n) {
  zb_pdl_launch();
  zb_pdl_wait();
  *p += n;
}

}  // namespace

extern "C" {

int zb_rmsnorm(const void* x, const void* residual, const void* w, void* out, void* residual_out,
               int rows, int d, long long x_stride, long long out_stride, float eps,
               int unit_offset, void* stream) {
  if (rows <= 0) return 0;
  if (d % 8 != 0 || x_stride % 8 != 0 || out_stride % 8 != 0) return -40;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int nvec = d / 8;
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto R = reinterpret_cast<const __nv_bfloat16*>(residual);
  auto W = reinterpret_cast<const __nv_bfloat16*>(w);
  auto O = reinterpret_cast<__nv_bfloat16*>(out);
  auto RO = reinterpret_cast<__nv_bfloat16*>(residual_out);
  if (nvec <= 256) zb_launch(zb_rmsnorm_kernel<1>, dim3(rows), dim3(256), 0, s, X, R, W, O, RO, rows, d, x_stride, out_stride, eps, unit_offset);
  else if (nvec <= 512) zb_launch(zb_rmsnorm_kernel<2>, dim3(rows), dim3(256), 0, s, X, R, W, O, RO, rows, d, x_stride, out_stride, eps, unit_offset);
  else if (nvec <= 1024) zb_launch(zb_rmsnorm_kernel<4>, dim3(rows), dim3(256), 0, s, X, R, W, O, RO, rows, d, x_stride, out_stride, eps, unit_offset);
  else if (nvec <= 2048) zb_launch(zb_rmsnorm_kernel<8>, dim3(rows), dim3(256), 0, s, X, R, W, O, RO, rows, d, x_stride, out_stride, eps, unit_offset);
  else return -41;
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

int zb_rope_kvwrite(const void* qkv, void* q_out, void* k_cache, void* v_cache,
                    const int32_t* positions, const int32_t* slot_mapping, const float* inv_freq,
                    const void* q_norm_w, const void* k_norm_w, long long qkv_stride, int tokens,
                    int hq, int hkv, int hd, int rot_dim, int layout, int page_size,
                    long long num_slots, float attn_factor, float norm_eps, int norm_unit_offset,
                    void* stream) {
  if (tokens <= 0) return 0;
  if (hd % 8 != 0 || rot_dim % 2 != 0 || rot_dim > hd) return -42;
  RopeParams p;
  p.qkv = reinterpret_cast<const __nv_bfloat16*>(qkv);
  p.q_out = reinterpret_cast<__nv_bfloat16*>(q_out);
  p.k_cache = reinterpret_cast<__nv_bfloat16*>(k_cache);
  p.v_cache = reinterpret_cast<__nv_bfloat16*>(v_cache);
  p.positions = positions;
  p.slot_mapping = slot_mapping;
  p.inv_freq = inv_freq;
  p.q_norm_w = reinterpret_cast<const __nv_bfloat16*>(q_norm_w);
  p.k_norm_w = reinterpret_cast<const __nv_bfloat16*>(k_norm_w);
  p.qkv_stride = qkv_stride;
  p.tokens = tokens;
  p.hq = hq;
  p.hkv = hkv;
  p.hd = hd;
  p.rot_dim = rot_dim;
  p.layout = layout;
  p.page_size = page_size;
  p.attn_factor = attn_factor;
  p.norm_eps = norm_eps;
  p.norm_unit_offset = norm_unit_offset;
  p.num_slots = num_slots;
  if (rot_dim / 2 > 128) return -46;
  // enough warps to fill the SMs a few times; beyond that, more heads per warp (shared sin / cos)
  const int heads = hq + 2 * hkv;
  int heads_per_warp = static_cast<int>(static_cast<long long>(tokens) * heads / 2368);
  heads_per_warp = heads_per_warp < 1 ? 1 : (heads_per_warp > 8 ? 8 : heads_per_warp);      // a warp's heads run one after the other
  const long long warps = static_cast<long long>(tokens) * ((heads + heads_per_warp - 1) / heads_per_warp);
  const int blocks = static_cast<int>((warps + 3) / 4);
  zb_launch(zb_rope_kvwrite_kernel, dim3(blocks), dim3(128), 0, reinterpret_cast<cudaStream_t>(stream), p, heads_per_warp);
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

int zb_swiglu(const void* gate_up, void* out, long long tokens, int f, void* stream) {
  if (tokens <= 0) return 0;
  if (f % 8 != 0) return -43;
  const long long total_vec = tokens * (f / 8);
  long long blocks = (total_vec + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  zb_launch(zb_swiglu_kernel, dim3(static_cast<int>(blocks)), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), 
      reinterpret_cast<const __nv_bfloat16*>(gate_up), reinterpret_cast<__nv_bfloat16*>(out), total_vec,
      f / 8);
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

int zb_embedding(const int32_t* ids, const void* table, void* out, int tokens, int d, int vocab,
                 void* stream) {
  if (tokens <= 0) return 0;
  if (d % 8 != 0) return -44;
  zb_launch(zb_embedding_kernel, dim3(tokens), dim3(128), 0, reinterpret_cast<cudaStream_t>(stream), 
      ids, reinterpret_cast<const __nv_bfloat16*>(table), reinterpret_cast<__nv_bfloat16*>(out), tokens, d,
      vocab);
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

int zb_argmax_f32(const float* logits, int32_t* out, int rows, int vocab, long long stride,
                  void* stream) {
  if (rows <= 0) return 0;
  zb_launch(zb_argmax_f32_kernel, dim3(rows), dim3(1024), 0, reinterpret_cast<cudaStream_t>(stream), logits, out, vocab, stride);
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

// `dev_rng` (may be null): two u64 in device memory, {seed, draws so far}; when given, the seed comes from there
// and the draw counter is added to `step`.
int zb_topk_sample_rng(const float* logits, int32_t* out_token, float* topk_vals, int32_t* topk_idx,
                       int rows, int vocab, long long stride, int k, float temperature,
                       unsigned long long seed, unsigned long long step, const unsigned long long* dev_rng, void* stream) {
  if (rows <= 0) return 0;
  if (k < 1 || k > kMaxTopK) return -45;
  zb_launch(zb_topk_sample_kernel, dim3(rows), dim3(1024), 0, reinterpret_cast<cudaStream_t>(stream),
      logits, out_token, topk_vals, topk_idx, vocab, stride, k, temperature, seed, step, dev_rng);
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

int zb_topk_sample(const float* logits, int32_t* out_token, float* topk_vals, int32_t* topk_idx,
                   int rows, int vocab, long long stride, int k, float temperature,
                   unsigned long long seed, unsigned long long step, void* stream) {
  return zb_topk_sample_rng(logits, out_token, topk_vals, topk_idx, rows, vocab, stride, k, temperature, seed, step, nullptr,
                            stream);
}

// Adds `n` to a u64 in device memory, in stream order (the draw counter of the sampler).
int zb_u64_add(unsigned long long* p, unsigned long long n, void* stream) {
  zb_launch(zb_u64_add_kernel, dim3(1), dim3(1), 0, reinterpret_cast<cudaStream_t>(stream), p, n);
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

// Feeds sampled tokens back for the next decode step (see the kernel's comment).
int zb_decode_advance_rng(const int32_t* sampled, int32_t* ids, int32_t* positions, int32_t* seq_lens,
                          int32_t* slot_mapping, const int32_t* block_table, int32_t* history,
                          int32_t* step_counter, int batch, int max_pages, int page_size,
                          int history_stride, int history_rows, unsigned long long* rng, void* stream);

int zb_decode_advance(const int32_t* sampled, int32_t* ids, int32_t* positions, int32_t* seq_lens,
                      int32_t* slot_mapping, const int32_t* block_table, int32_t* history,
                      int32_t* step_counter, int batch, int max_pages, int page_size,
                      int history_stride, int history_rows, void* stream) {
  return zb_decode_advance_rng(sampled, ids, positions, seq_lens, slot_mapping, block_table, history, step_counter, batch,
                               max_pages, page_size, history_stride, history_rows, nullptr, stream);
}

// The same, and the sampler's draw counter rng[1] (see zb_topk_sample_rng) goes up by one.
int zb_decode_advance_rng(const int32_t* sampled, int32_t* ids, int32_t* positions, int32_t* seq_lens,
                          int32_t* slot_mapping, const int32_t* block_table, int32_t* history,
                          int32_t* step_counter, int batch, int max_pages, int page_size,
                          int history_stride, int history_rows, unsigned long long* rng, void* stream) {
  if (batch <= 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  zb_launch(zb_decode_advance_kernel, dim3((batch + 127) / 128), dim3(128), 0, s, sampled, ids, positions, seq_lens,
                                                             slot_mapping, block_table, history,
                                                             step_counter, batch, max_pages, page_size,
                                                             history_stride, history_rows);
  zb_launch(zb_counter_inc_kernel, dim3(1), dim3(1), 0, s, step_counter, rng);
  zb_count_launch(2);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
