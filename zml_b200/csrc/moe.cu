// Mixture-of-experts kernels for sm_100a: router top-k, token permutation by expert,
// grouped GEMM over the experts (tcgen05 / TMEM, TMA-fed) with a fused SwiGLU epilogue,
// and the finalize step (un-permute x routing weight).
//
// Replaces the fused-MoE back-ends of the reference: the FlashInfer CUTLASS runner
// (zml/moe/cutlass_flashinfer.zig:332-376) and the Triton path
// (zml/moe/triton.zig, zml/moe/triton_kernels/triton_kernels.zig: moe_align_block_size,
// fused_moe_kernel), and the sort-based router (examples/llm/models/qwen3_5_moe/model.zig:727-754).
// Where the reference masks all tokens to the local experts and runs them all, only the
// (token, expert) pairs that are routed to a local expert are gathered and multiplied.
#include <cuda.h>

#include "common.cuh"
#include "host_api.h"
#include "moe_tiles.cuh"
#include "quant.cuh"

int zb_make_tmap_bf16_2d(CUtensorMap* out, const void* base, int rows, int k, int ld, int box_rows);

namespace {

constexpr uint32_t kKernelGrouped = 6;

// ------------------------------------------------------------------ router
// One warp per token: top-k of the logits, then softmax over the selected k
// (top-k then softmax == softmax then top-k then renormalise).
template <int MAX_PER_LANE>
__global__ void __launch_bounds__(128) zb_moe_router_topk_kernel(const float* __restrict__ logits, int32_t* __restrict__ ids,
                                                                 float* __restrict__ weights, int tokens, int experts,
                                                                 int k, long long stride, int renormalize) {
  zb_pdl_launch();
  zb_pdl_wait();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= tokens) return;
  const float* row = logits + static_cast<size_t>(warp) * stride;
  float v[MAX_PER_LANE];
  float rmax = -INFINITY;
#pragma unroll
  for (int i = 0; i < MAX_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < experts ? row[e] : -INFINITY;
    rmax = fmaxf(rmax, v[i]);
  }
  rmax = zb_warp_max(rmax);
  float denom_all = 0.f;
  if (!renormalize) {
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) denom_all += (lane + 32 * i) < experts ? __expf(v[i] - rmax) : 0.f;
    denom_all = zb_warp_sum(denom_all);
  }
  float sel_v = 0.f;
  int sel_i = 0;
  float denom = 0.f;
  for (int j = 0; j < k; ++j) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e < experts && (v[i] > best || (v[i] == best && e < bi))) {
        best = v[i];
        bi = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (bi == 0x7fffffff) bi = 0;
    // remove the winner from its owner's registers
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i)
      if (lane + 32 * i == bi) v[i] = -INFINITY;
    const float p = __expf(best - rmax);
    denom += p;
    if (lane == j) {
      sel_v = p;
      sel_i = bi;
    }
  }
  if (lane < k) {
    ids[static_cast<size_t>(warp) * k + lane] = sel_i;
    weights[static_cast<size_t>(warp) * k + lane] = sel_v / (renormalize ? denom : denom_all);
  }
}

// ------------------------------------------------------------------ permutation by expert
// meta layout (int32): [0, E]      offsets (exclusive prefix of counts, E + 1 entries)
//                      [E+1, 2E]   cursors (scratch)
__global__ void zb_moe_count_kernel(const int32_t* __restrict__ ids, int32_t* __restrict__ meta, int pairs, int e0,
                                    int e_local) {
  zb_pdl_launch();
  zb_pdl_wait();
  int32_t* counts = meta + e_local + 1;      // cursors double as counts in this pass
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < pairs; i += gridDim.x * blockDim.x) {
    const int e = ids[i] - e0;
    if (e >= 0 && e < e_local) atomicAdd(&counts[e], 1);
  }
}

__global__ void zb_moe_offsets_kernel(int32_t* __restrict__ meta, int e_local) {
  zb_pdl_launch();
  zb_pdl_wait();
  // single thread block; E is small (<= 1024)
  __shared__ int32_t s[1025];
  int32_t* counts = meta + e_local + 1;
  for (int i = threadIdx.x; i < e_local; i += blockDim.x) s[i] = counts[i];
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < e_local; ++e) {
      const int c = s[e];
      meta[e] = acc;
      counts[e] = acc;       // cursor starts at the expert's offset
      acc += c;
    }
    meta[e_local] = acc;
  }
}

__global__ void zb_moe_scatter_kernel(const int32_t* __restrict__ ids, int32_t* __restrict__ meta,
                                      int32_t* __restrict__ sorted_pair, int32_t* __restrict__ pair_pos, int pairs,
                                      int e0, int e_local) {
  zb_pdl_launch();
  zb_pdl_wait();
  int32_t* cursors = meta + e_local + 1;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < pairs; i += gridDim.x * blockDim.x) {
    const int e = ids[i] - e0;
    if (e >= 0 && e < e_local) {
      const int pos = atomicAdd(&cursors[e], 1);
      sorted_pair[pos] = i;
      pair_pos[i] = pos;
    } else {
      pair_pos[i] = -1;
    }
  }
}

// Count, prefix and scatter in one launch for the pair counts of a decode step (one CTA; every
// thread keeps its pairs' expert and rank within the expert in registers between the phases).
constexpr int kAlignSmallThreads = 1024;
constexpr int kAlignSmallPerThread = 8;
__global__ void __launch_bounds__(kAlignSmallThreads)
zb_moe_align_small_kernel(const int32_t* __restrict__ ids, int32_t* __restrict__ meta, int32_t* __restrict__ sorted_pair,
                          int32_t* __restrict__ pair_pos, int pairs, int e0, int e_local) {
  zb_pdl_launch();
  zb_pdl_wait();
  __shared__ int32_t hist[1024];
  __shared__ int32_t warp_sum[32];
  const int tid = threadIdx.x;
  hist[tid] = 0;
  __syncthreads();
  int ex[kAlignSmallPerThread], rank[kAlignSmallPerThread];
#pragma unroll
  for (int j = 0; j < kAlignSmallPerThread; ++j) {
    const int i = tid + j * kAlignSmallThreads;
    ex[j] = -1;
    rank[j] = 0;
    if (i < pairs) {
      const int e = ids[i] - e0;
      if (e >= 0 && e < e_local) {
        ex[j] = e;
        rank[j] = atomicAdd(&hist[e], 1);
      }
    }
  }
  __syncthreads();
  // exclusive prefix of hist over 1024 entries: warp scan, scan of the warp totals, add
  const int c = hist[tid];
  int incl = c;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, o);
    if ((tid & 31) >= o) incl += v;
  }
  if ((tid & 31) == 31) warp_sum[tid >> 5] = incl;
  __syncthreads();
  if (tid < 32) {
    const int w = warp_sum[tid];
    int wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, wi, o);
      if (tid >= o) wi += v;
    }
    warp_sum[tid] = wi - w;
  }
  __syncthreads();
  const int excl = incl - c + warp_sum[tid >> 5];
  hist[tid] = excl;
  if (tid < e_local) {
    meta[tid] = excl;
    meta[e_local + 1 + tid] = excl + c;        // cursors as the multi-kernel path leaves them
  }
  if (tid == e_local - 1) meta[e_local] = excl + c;
  __syncthreads();
#pragma unroll
  for (int j = 0; j < kAlignSmallPerThread; ++j) {
    const int i = tid + j * kAlignSmallThreads;
    if (i < pairs) {
      if (ex[j] >= 0) {
        const int pos = hist[ex[j]] + rank[j];
        sorted_pair[pos] = i;
        pair_pos[i] = pos;
      } else {
        pair_pos[i] = -1;
      }
    }
  }
}

// xs[pos, :] = x[sorted_pair[pos] / k, :]
__global__ void __launch_bounds__(128) zb_moe_gather_kernel(const __nv_bfloat16* __restrict__ x,
                                                            const int32_t* __restrict__ sorted_pair,
                                                            const int32_t* __restrict__ meta, __nv_bfloat16* __restrict__ xs,
                                                            int e_local, int k, int d, int cap) {
  zb_pdl_launch();
  zb_pdl_wait();
  const int total = min(meta[e_local], cap);
  for (int pos = blockIdx.x; pos < total; pos += gridDim.x) {
    const int t = sorted_pair[pos] / k;
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * d);
    uint4* dst = reinterpret_cast<uint4*>(xs + static_cast<size_t>(pos) * d);
    for (int i = threadIdx.x; i < d / 8; i += 128) dst[i] = src[i];
  }
}

// The gather with the NVFP4 activation quantiser behind it: xq[pos, :] = e2m1 codes of x[sorted_pair[pos] / k, :],
// xsf[pos, :] = one f8e4m3 scale per 16 values (same numerics as zb_nvfp4_quantize without a per-tensor scale).
// One thread per 16-value block.
__global__ void __launch_bounds__(128) zb_moe_gather_fp4_kernel(const __nv_bfloat16* __restrict__ x,
                                                                const int32_t* __restrict__ sorted_pair,
                                                                const int32_t* __restrict__ meta, uint8_t* __restrict__ xq,
                                                                uint8_t* __restrict__ xsf, int e_local, int k, int d, int cap) {
  zb_pdl_launch();
  zb_pdl_wait();
  const int total = min(meta[e_local], cap);
  const int kblocks = d / 16;
  for (int pos = blockIdx.x; pos < total; pos += gridDim.x) {
    const int t = sorted_pair[pos] / k;
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * d);
    for (int b = threadIdx.x; b < kblocks; b += 128) {
      const uint4 raw[2] = {src[2 * b], src[2 * b + 1]};
      const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(raw);
      float v[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = __bfloat162float(e[i]);
      uint8_t s8;
      const uint2 c = zb_nvfp4_quantize_block(v, s8);
      *reinterpret_cast<uint2*>(xq + (static_cast<size_t>(pos) * kblocks + b) * 8) = c;
      xsf[static_cast<size_t>(pos) * kblocks + b] = s8;
    }
  }
}

// y[t, :] = sum_j weights[t, j] * o[pair_pos[t*k + j], :]   (pairs of remote experts: skipped)
__global__ void __launch_bounds__(128) zb_moe_finalize_kernel(const __nv_bfloat16* __restrict__ o,
                                                              const int32_t* __restrict__ pair_pos,
                                                              const float* __restrict__ weights,
                                                              __nv_bfloat16* __restrict__ y, int tokens, int k, int d) {
  zb_pdl_launch();
  zb_pdl_wait();
  const int t = blockIdx.x;
  if (t >= tokens) return;
  for (int i = threadIdx.x; i < d / 8; i += 128) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < k; ++j) {
      const int pos = pair_pos[static_cast<size_t>(t) * k + j];
      if (pos < 0) continue;
      const float w = weights[static_cast<size_t>(t) * k + j];
      const uint4 v = reinterpret_cast<const uint4*>(o + static_cast<size_t>(pos) * d)[i];
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = zb_unpack_bf16x2(u[q]);
        acc[2 * q] += w * f.x;
        acc[2 * q + 1] += w * f.y;
      }
    }
    reinterpret_cast<uint4*>(y + static_cast<size_t>(t) * d)[i] =
        make_uint4(zb_pack_bf16x2(acc[0], acc[1]), zb_pack_bf16x2(acc[2], acc[3]), zb_pack_bf16x2(acc[4], acc[5]),
                   zb_pack_bf16x2(acc[6], acc[7]));
  }
}

// ------------------------------------------------------------------ combine (+ all-reduce over peer memory)
// y[t, :] = residual[t, :] + sum over ranks r of ( extra_r[t, :] + sum_j weights[t, j] * o_r[pair_pos_r[t*k + j], :] )
//
// One kernel for the un-permute, the routing-weight sum, the expert-parallel all-reduce and the residual
// add.  Every rank rounds its partial row to bf16 and stores it into every peer's slot area as 8-byte
// {two bf16, epoch} words (a word arrives whole, so the tag that says "this is launch `epoch`" needs no
// fence and no flag); then it reads the slots the peers wrote here, waiting on the tags, and sums the
// world's partials in rank order, so all ranks produce the same bits.  Slot areas alternate by epoch
// parity: a rank can start launch n + 1 only after it has read everything of launch n, and it cannot
// finish n + 1 without the peers' n + 1 words, so a peer still reading launch n is never overwritten
// by launch n + 2.  WORLD == 1 is the single-GPU combine (no slots).
//
// Slot area of one parity half: [src rank][token][d / 8 vectors][4 words].
// The reference sums expert-parallel partials with an XLA all-reduce after its MoE custom call
// (zml/moe/moe.zig, zml/nn.zig); here the reduction rides in the combine kernel.
constexpr uint32_t kKernelCombine = 10;

struct CombineAr {
  uint2* slots[8];          // slot area in every rank's heap ([rank] is local)
  size_t half_words;        // 8-byte words of one parity half
  uint32_t* epoch;
  uint32_t* ticket;
  int rank;
  int world;
};

template <bool AR>
__global__ void __launch_bounds__(128)
zb_moe_combine_kernel(const __nv_bfloat16* __restrict__ o, const int32_t* __restrict__ pair_pos,
                      const float* __restrict__ weights, const __nv_bfloat16* __restrict__ extra,
                      const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ y, int tokens, int k, int d,
                      const CombineAr ar, ZbStatus* status) {
  zb_pdl_launch();
  zb_pdl_wait();
  const int t = blockIdx.x;
  const int nvec = d / 8;
  uint32_t epoch = 0;
  if constexpr (AR) epoch = *reinterpret_cast<volatile uint32_t*>(ar.epoch);
  bool timed_out = false;
  for (int i = threadIdx.x; i < nvec; i += 128) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < k; ++j) {
      const int pos = pair_pos[static_cast<size_t>(t) * k + j];
      if (pos < 0) continue;
      const float w = weights[static_cast<size_t>(t) * k + j];
      const uint4 v = reinterpret_cast<const uint4*>(o + static_cast<size_t>(pos) * d)[i];
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = zb_unpack_bf16x2(u[q]);
        acc[2 * q] += w * f.x;
        acc[2 * q + 1] += w * f.y;
      }
    }
    if (extra != nullptr) {
      const uint4 v = reinterpret_cast<const uint4*>(extra + static_cast<size_t>(t) * d)[i];
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = zb_unpack_bf16x2(u[q]);
        acc[2 * q] += f.x;
        acc[2 * q + 1] += f.y;
      }
    }
    uint4 rv = make_uint4(0u, 0u, 0u, 0u);
    if (residual != nullptr) rv = reinterpret_cast<const uint4*>(residual + static_cast<size_t>(t) * d)[i];   // before any store: y may alias it
    if constexpr (AR) {
      const uint32_t mine[4] = {zb_pack_bf16x2(acc[0], acc[1]), zb_pack_bf16x2(acc[2], acc[3]), zb_pack_bf16x2(acc[4], acc[5]),
                                zb_pack_bf16x2(acc[6], acc[7])};
      const size_t word0 = (epoch & 1u) * ar.half_words + ((static_cast<size_t>(ar.rank) * tokens + t) * nvec + i) * 4;
      for (int r = 0; r < ar.world; ++r) {
        if (r == ar.rank) continue;
        uint2* dst = ar.slots[r] + word0;
#pragma unroll
        for (int q = 0; q < 4; ++q) zb_st_ll(dst + q, mine[q], epoch);
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] = 0.f;
      const uint64_t t0 = zb_globaltimer();
      for (int r = 0; r < ar.world; ++r) {
        uint32_t got[4] = {mine[0], mine[1], mine[2], mine[3]};
        if (r != ar.rank) {
          const uint2* src = ar.slots[ar.rank] + (epoch & 1u) * ar.half_words + ((static_cast<size_t>(r) * tokens + t) * nvec + i) * 4;
          uint32_t spins = 0;
          while (true) {
            bool ready = true;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint2 x = zb_ld_ll(src + q);
              got[q] = x.x;
              ready = ready && (x.y == epoch);
            }
            if (ready || timed_out) break;
            if ((++spins & 0x3f) == 0 && zb_globaltimer() - t0 > ZB_WAIT_LIMIT_NS) timed_out = true;
          }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = zb_unpack_bf16x2(got[q]);
          acc[2 * q] += f.x;
          acc[2 * q + 1] += f.y;
        }
      }
    }
    if (residual != nullptr) {
      const uint32_t u[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = zb_unpack_bf16x2(u[q]);
        acc[2 * q] += f.x;
        acc[2 * q + 1] += f.y;
      }
    }
    reinterpret_cast<uint4*>(y + static_cast<size_t>(t) * d)[i] =
        make_uint4(zb_pack_bf16x2(acc[0], acc[1]), zb_pack_bf16x2(acc[2], acc[3]), zb_pack_bf16x2(acc[4], acc[5]),
                   zb_pack_bf16x2(acc[6], acc[7]));
  }
  if constexpr (AR) {
    if (timed_out) zb_record_error(status, ZB_ERR_FLAG_TIMEOUT, kKernelCombine, blockIdx.x, ar.rank);
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      const uint32_t ticket = atomicAdd(ar.ticket, 1u);
      if (ticket == gridDim.x - 1) {
        *ar.ticket = 0u;
        *reinterpret_cast<volatile uint32_t*>(ar.epoch) = epoch + 1u;
      }
    }
  }
}

// ------------------------------------------------------------------ grouped GEMM
// For every local expert e:  out[off_e : off_{e+1}, :] = xs[off_e : off_{e+1}, :K] * W[e][N, K]^T
// with an optional SwiGLU epilogue.  Same pipeline as the dense GEMM (gemm_bf16.cu):
// warp 0 TMA producer, warp 1 tcgen05.mma issuer, warps 2-5 epilogue, two TMEM
// accumulator stages.  Tiles are dealt round-robin to a persistent grid; the tile list
// depends on the per-expert token counts, which live on the device, so every role derives
// it from `offsets` itself.
//
// SwiGLU: the fused gate/up weight of an expert is stored interleaved in blocks of 64
// rows ([64 gate rows | 64 up rows] per 128-row block), so one 128-row weight tile (swap
// mode) or one 256-column tile (token-major mode) holds matching gate and up columns.
constexpr int kBlockP = 128;
constexpr int kBlockK = 64;
constexpr int kUmmaK = 16;
constexpr int kThreads = 192;

struct GroupedParams {
  const int32_t* offsets;   // [e_local + 1]
  int e_local;
  int n;                    // output features per expert (rows of W[e])
  int k;
  int ldo;                  // leading dimension of out
  __nv_bfloat16* out;
  int cap;                  // rows allocated in xs / out
  int act;                  // ZbMoeAct: which gate activation the gated epilogue applies, or relu2 on a plain projection
  ZbStatus* status;
};

__host__ __device__ constexpr int g_stages(int bn) { return bn >= 256 ? 4 : (bn >= 128 ? 5 : 6); }
__host__ __device__ constexpr int g_stage_bytes(int bn) { return (kBlockP + bn) * kBlockK * 2; }

ZB_DEVICE void g_epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int BN, bool SWAP, bool SWIGLU>
__global__ void __launch_bounds__(kThreads, 1)
zb_moe_grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                           const GroupedParams prm) {
  constexpr int kStages = g_stages(BN);
  constexpr int kStageBytes = g_stage_bytes(BN);
  constexpr int kTileABytes = kBlockP * kBlockK * 2;
  constexpr uint32_t kTmemCols = (2 * BN) < 32 ? 32 : (2 * BN);
  constexpr uint32_t kIdesc = zb_make_idesc_bf16(kBlockP, BN);
  constexpr int kXchBytes = (SWAP && SWIGLU) ? BN * 64 * 4 : 0;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  float* xch = reinterpret_cast<float*>(smem + kStages * kStageBytes);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes + kXchBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full = empty_bar + kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile uint32_t* abort_flag = tmem_holder + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb_total = (prm.k + kBlockK - 1) / kBlockK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      zb_mbar_init(&full_bar[s], 1);
      zb_mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      zb_mbar_init(&tmem_full[a], 1);
      zb_mbar_init(&tmem_empty[a], 128);
    }
    *abort_flag = 0u;
    zb_mbar_fence_init();
  }
  if (warp == 1) {
    zb_tmem_alloc(tmem_holder, kTmemCols);
    zb_tmem_relinquish();
  }
  zb_tc_fence_before();
  __syncthreads();
  zb_tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  // The next kernel may start only now that this CTA holds its tensor memory: a dependent CTA
  // that shared the SM and allocated first would block this one for good.  The tile walk reads
  // the expert offsets written by the preceding kernels, so every thread waits for them.
  zb_pdl_launch();
  zb_pdl_wait();

  // tiles of expert e: weight tiles x token tiles
  const int w_tiles = SWAP ? prm.n / kBlockP : prm.n / BN;
  __shared__ int32_t tile_prefix[kZbMaxExperts + 1];
  zb_tile_prefix_build(tile_prefix, prm.offsets, prm.e_local, w_tiles, SWAP ? BN : kBlockP);
  // iterator over this CTA's tiles: global tile index g = blockIdx.x, += gridDim.x
  struct Cursor {
    int e;         // current expert
    int hint;      // where the bisection for the next tile starts
  };
  auto locate = [&](Cursor& c, int g, int& wt, int& tt) -> bool {
    ZbTilePos pos;
    if (!zb_tile_locate(tile_prefix, prm.e_local, w_tiles, g, c.hint, pos)) return false;
    c.e = pos.e;
    wt = pos.wt;
    tt = pos.tt;
    return true;
  };

  if (warp == 0) {
    if (lane == 0) {
      zb_tma_prefetch_desc(&tmap_x);
      zb_tma_prefetch_desc(&tmap_w);
      uint32_t stage = 0, phase = 0;
      Cursor c{0, 0};
      bool ok = true;
      for (int g = blockIdx.x; ok; g += gridDim.x) {
        int wt, tt;
        if (!locate(c, g, wt, tt)) break;
        const int tok0 = prm.offsets[c.e] + tt * (SWAP ? BN : kBlockP);
        const int wrow0 = c.e * prm.n + wt * (SWAP ? kBlockP : BN);
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!zb_mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * kStageBytes;
          uint8_t* sb = sa + kTileABytes;
          zb_mbar_expect_tx(&full_bar[stage], kStageBytes);
          if (SWAP) {
            zb_tma_load_2d(sa, &tmap_w, &full_bar[stage], kb * kBlockK, wrow0);
            zb_tma_load_2d(sb, &tmap_x, &full_bar[stage], kb * kBlockK, tok0);
          } else {
            zb_tma_load_2d(sa, &tmap_x, &full_bar[stage], kb * kBlockK, tok0);
            zb_tma_load_2d(sb, &tmap_w, &full_bar[stage], kb * kBlockK, wrow0);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      Cursor c{0, 0};
      bool ok = true;
      for (int g = blockIdx.x; ok; g += gridDim.x) {
        int wt, tt;
        if (!locate(c, g, wt, tt)) break;
        if (!zb_mbar_wait(&tmem_empty[acc], acc_phase ^ 1u, abort_flag)) break;
        zb_tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!zb_mbar_wait(&full_bar[stage], phase, abort_flag)) {
            ok = false;
            break;
          }
          zb_tc_fence_after();
          const uint32_t sa = zb_smem_u32(smem + stage * kStageBytes);
          const uint64_t da = zb_make_desc_sw128(sa);
          const uint64_t db = zb_make_desc_sw128(sa + kTileABytes);
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k)
            zb_umma_f16(tmem_d, da + 2 * k, db + 2 * k, kIdesc, (kb > 0 || k > 0) ? 1u : 0u);
          zb_umma_commit(&empty_bar[stage]);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        zb_umma_commit(&tmem_full[acc]);
        acc ^= 1u;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    uint32_t acc = 0, acc_phase = 0;
    Cursor c{0, 0};
    for (int g = blockIdx.x;; g += gridDim.x) {
      int wt, tt;
      if (!locate(c, g, wt, tt)) break;
      zb_mbar_wait(&tmem_full[acc], acc_phase, abort_flag);
      g_epi_bar();
      if (*abort_flag != 0u) break;
      zb_tc_fence_after();
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quad * 32) << 16);
      const int off_e = prm.offsets[c.e];
      const int end_e = min(prm.offsets[c.e + 1], prm.cap);
      if constexpr (SWAP) {
        // thread row = weight row (output feature), columns = tokens of this tile
        const int tok0 = off_e + tt * BN;
        if constexpr (!SWIGLU) {
          const int feat = wt * kBlockP + row_in_tile;
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 16) {
            uint32_t r[16];
            zb_tmem_ld16(taddr + c0, r);
            zb_tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int tok = tok0 + c0 + j;
              if (tok < end_e)
                prm.out[static_cast<size_t>(tok) * prm.ldo + feat] = __float2bfloat16(zb_plain_act(__uint_as_float(r[j]), prm.act));
            }
          }
          zb_tc_fence_before();
          zb_mbar_arrive(&tmem_empty[acc]);
        } else {
          // rows 0-63: gate, rows 64-127: up of the same 64 output features
          const bool is_up = row_in_tile >= 64;
          const int feat = wt * 64 + (row_in_tile & 63);
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 16) {
            uint32_t r[16];
            zb_tmem_ld16(taddr + c0, r);
            zb_tmem_ld_wait();
            if (is_up) {
#pragma unroll
              for (int j = 0; j < 16; ++j) xch[(c0 + j) * 64 + (row_in_tile - 64)] = __uint_as_float(r[j]);
            }
            g_epi_bar();
            if (!is_up) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const int tok = tok0 + c0 + j;
                if (tok < end_e) {
                  const float gt = __uint_as_float(r[j]);
                  const float up = xch[(c0 + j) * 64 + row_in_tile];
                  prm.out[static_cast<size_t>(tok) * prm.ldo + feat] = __float2bfloat16(zb_gate_act(gt, prm.act) * up);
                }
              }
            }
            g_epi_bar();
          }
          zb_tc_fence_before();
          zb_mbar_arrive(&tmem_empty[acc]);
        }
      } else {
        // thread row = token, columns = output features
        const int tok = off_e + tt * kBlockP + row_in_tile;
        if constexpr (!SWIGLU) {
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 16) {
            uint32_t r[16];
            zb_tmem_ld16(taddr + c0, r);
            zb_tmem_ld_wait();
            if (prm.act == ZB_ACT_RELU2) {
#pragma unroll
              for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(zb_plain_act(__uint_as_float(r[j]), ZB_ACT_RELU2));
            }
            if (tok < end_e) {
              uint4* op = reinterpret_cast<uint4*>(prm.out + static_cast<size_t>(tok) * prm.ldo + wt * BN + c0);
              op[0] = make_uint4(zb_pack_bf16x2(__uint_as_float(r[0]), __uint_as_float(r[1])),
                                 zb_pack_bf16x2(__uint_as_float(r[2]), __uint_as_float(r[3])),
                                 zb_pack_bf16x2(__uint_as_float(r[4]), __uint_as_float(r[5])),
                                 zb_pack_bf16x2(__uint_as_float(r[6]), __uint_as_float(r[7])));
              op[1] = make_uint4(zb_pack_bf16x2(__uint_as_float(r[8]), __uint_as_float(r[9])),
                                 zb_pack_bf16x2(__uint_as_float(r[10]), __uint_as_float(r[11])),
                                 zb_pack_bf16x2(__uint_as_float(r[12]), __uint_as_float(r[13])),
                                 zb_pack_bf16x2(__uint_as_float(r[14]), __uint_as_float(r[15])));
            }
          }
        } else {
          // columns of the tile: [64 gate | 64 up] blocks; output feature = wt*(BN/2) + blk*64 + i
#pragma unroll 1
          for (int blk = 0; blk < BN / 128; ++blk) {
#pragma unroll 1
            for (int c0 = 0; c0 < 64; c0 += 16) {
              uint32_t gr[16], ur[16];
              zb_tmem_ld16(taddr + blk * 128 + c0, gr);
              zb_tmem_ld16(taddr + blk * 128 + 64 + c0, ur);
              zb_tmem_ld_wait();
              if (tok < end_e) {
                float h[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  const float gt = __uint_as_float(gr[j]);
                  h[j] = zb_gate_act(gt, prm.act) * __uint_as_float(ur[j]);
                }
                uint4* op = reinterpret_cast<uint4*>(prm.out + static_cast<size_t>(tok) * prm.ldo + wt * (BN / 2) +
                                                     blk * 64 + c0);
                op[0] = make_uint4(zb_pack_bf16x2(h[0], h[1]), zb_pack_bf16x2(h[2], h[3]), zb_pack_bf16x2(h[4], h[5]),
                                   zb_pack_bf16x2(h[6], h[7]));
                op[1] = make_uint4(zb_pack_bf16x2(h[8], h[9]), zb_pack_bf16x2(h[10], h[11]),
                                   zb_pack_bf16x2(h[12], h[13]), zb_pack_bf16x2(h[14], h[15]));
              }
            }
          }
        }
        zb_tc_fence_before();
        zb_mbar_arrive(&tmem_empty[acc]);
      }
      acc ^= 1u;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  zb_tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0u) {
    if (threadIdx.x == 0) zb_record_error(prm.status, ZB_ERR_MBAR_TIMEOUT, kKernelGrouped, blockIdx.x, BN);
    const uint64_t t0 = zb_globaltimer();
    while (zb_globaltimer() - t0 < 200000ull) {
    }
    __syncthreads();
  }
  if (warp == 1) {
    zb_tc_fence_after();
    zb_tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int BN, bool SWAP, bool SWIGLU>
int launch_grouped(const CUtensorMap& tx, const CUtensorMap& tw, const GroupedParams& prm, int grid, cudaStream_t s) {
  constexpr int smem = g_stages(BN) * g_stage_bytes(BN) + ((SWAP && SWIGLU) ? BN * 64 * 4 : 0) + 1024 + 256;
  static bool configured[16] = {};
  if (const int rc = zb_config_smem_once(zb_moe_grouped_gemm_kernel<BN, SWAP, SWIGLU>, smem, configured)) return rc;
  zb_launch(zb_moe_grouped_gemm_kernel<BN, SWAP, SWIGLU>, dim3(grid), dim3(kThreads), smem, s, tx, tw, prm);
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

extern "C" {

int zb_moe_router_topk(const float* logits, int32_t* ids, float* weights, int tokens, int experts, int k,
                       long long stride, int renormalize, void* stream) {
  if (tokens <= 0) return 0;
  if (k < 1 || k > 32 || experts < k || experts > 512) return -60;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int blocks = (tokens + 3) / 4;
  if (experts <= 128) zb_launch(zb_moe_router_topk_kernel<4>, dim3(blocks), dim3(128), 0, s, logits, ids, weights, tokens, experts, k, stride, renormalize);
  else if (experts <= 256) zb_launch(zb_moe_router_topk_kernel<8>, dim3(blocks), dim3(128), 0, s, logits, ids, weights, tokens, experts, k, stride, renormalize);
  else zb_launch(zb_moe_router_topk_kernel<16>, dim3(blocks), dim3(128), 0, s, logits, ids, weights, tokens, experts, k, stride, renormalize);
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

// Permutation of the (token, expert) pairs whose expert is in [e0, e0 + e_local): fills
// meta[0..e_local] with the offsets, `sorted_pair` (pair indices grouped by expert) and
// `pair_pos` (position of each pair in that order, -1 for remote experts).
// meta must hold 2 * e_local + 2 int32.
int zb_moe_align(const int32_t* ids, int32_t* meta, int32_t* sorted_pair, int32_t* pair_pos, int pairs, int e0,
                 int e_local, void* stream) {
  if (e_local < 1 || e_local > 1024) return -61;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (pairs > 0 && pairs <= kAlignSmallThreads * kAlignSmallPerThread) {
    zb_launch(zb_moe_align_small_kernel, dim3(1), dim3(kAlignSmallThreads), 0, s, ids, meta, sorted_pair, pair_pos, pairs, e0,
              e_local);
    zb_count_launch(1);
    return static_cast<int>(cudaGetLastError());
  }
  cudaError_t e = cudaMemsetAsync(meta, 0, sizeof(int32_t) * (2 * e_local + 2), s);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (pairs > 0) {
    int blocks = (pairs + 255) / 256;
    if (blocks > 592) blocks = 592;
    zb_launch(zb_moe_count_kernel, dim3(blocks), dim3(256), 0, s, ids, meta, pairs, e0, e_local);
    zb_launch(zb_moe_offsets_kernel, dim3(1), dim3(256), 0, s, meta, e_local);
    zb_launch(zb_moe_scatter_kernel, dim3(blocks), dim3(256), 0, s, ids, meta, sorted_pair, pair_pos, pairs, e0, e_local);
    zb_count_launch(3);
  }
  return static_cast<int>(cudaGetLastError());
}

int zb_moe_gather(const void* x, const int32_t* sorted_pair, const int32_t* meta, void* xs, int e_local, int k, int d,
                  int cap, void* stream) {
  if (cap <= 0) return 0;
  if (d % 8 != 0) return -62;
  int blocks = cap < 2368 ? cap : 2368;
  zb_launch(zb_moe_gather_kernel, dim3(blocks), dim3(128), 0, reinterpret_cast<cudaStream_t>(stream), 
      reinterpret_cast<const __nv_bfloat16*>(x), sorted_pair, meta, reinterpret_cast<__nv_bfloat16*>(xs), e_local, k, d, cap);
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

// xq [cap, d / 2] bytes, xsf [cap, d / 16] bytes; d a multiple of 16.
int zb_moe_gather_fp4(const void* x, const int32_t* sorted_pair, const int32_t* meta, void* xq, void* xsf, int e_local, int k,
                      int d, int cap, void* stream) {
  if (cap <= 0) return 0;
  if (d % 16 != 0) return -62;
  int blocks = cap < 2368 ? cap : 2368;
  zb_launch(zb_moe_gather_fp4_kernel, dim3(blocks), dim3(128), 0, reinterpret_cast<cudaStream_t>(stream),
            reinterpret_cast<const __nv_bfloat16*>(x), sorted_pair, meta, reinterpret_cast<uint8_t*>(xq),
            reinterpret_cast<uint8_t*>(xsf), e_local, k, d, cap);
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

int zb_moe_finalize(const void* o, const int32_t* pair_pos, const float* weights, void* y, int tokens, int k, int d,
                    void* stream) {
  if (tokens <= 0) return 0;
  if (d % 8 != 0) return -62;
  zb_launch(zb_moe_finalize_kernel, dim3(tokens), dim3(128), 0, reinterpret_cast<cudaStream_t>(stream), 
      reinterpret_cast<const __nv_bfloat16*>(o), pair_pos, weights, reinterpret_cast<__nv_bfloat16*>(y), tokens, k, d);
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

// y = residual + all-reduce over the group of (extra + un-permuted, routing-weighted expert outputs); see the kernel.
// `ctx` null: one rank.  `slot_off` / `slot_bytes`: the slot area inside every rank's symmetric heap
// (2 parity halves x world x tokens x d x 4 bytes at least).  extra / residual may be null; y may alias residual.
int zb_moe_combine(const void* o, const int32_t* pair_pos, const float* weights, const void* extra, const void* residual,
                   void* y, int tokens, int k, int d, const ZbArContext* ctx, size_t slot_off, size_t slot_bytes,
                   void* stream) {
  if (tokens <= 0) return 0;
  if (d % 8 != 0) return -62;
  ZbDeviceState* st = zb_device_state();
  if (!st) return -20;
  CombineAr ar = {};
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const auto* o_ = reinterpret_cast<const __nv_bfloat16*>(o);
  const auto* ex_ = reinterpret_cast<const __nv_bfloat16*>(extra);
  const auto* rs_ = reinterpret_cast<const __nv_bfloat16*>(residual);
  auto* y_ = reinterpret_cast<__nv_bfloat16*>(y);
  if (ctx == nullptr || ctx->world == 1) {
    zb_launch(zb_moe_combine_kernel<false>, dim3(tokens), dim3(128), 0, s, o_, pair_pos, weights, ex_, rs_, y_, tokens, k, d, ar,
              st->status);
  } else {
    const size_t half_words = static_cast<size_t>(ctx->world) * tokens * (d / 8) * 4;
    if (slot_off % 16 != 0 || 2 * half_words * sizeof(uint2) > slot_bytes) return -68;
    for (int r = 0; r < ctx->world; ++r) ar.slots[r] = reinterpret_cast<uint2*>(reinterpret_cast<char*>(ctx->heap[r]) + slot_off);
    ar.half_words = half_words;
    ar.epoch = ctx->epoch + 4;
    ar.ticket = ctx->epoch + 5;
    ar.rank = ctx->rank;
    ar.world = ctx->world;
    zb_launch(zb_moe_combine_kernel<true>, dim3(tokens), dim3(128), 0, s, o_, pair_pos, weights, ex_, rs_, y_, tokens, k, d, ar,
              st->status);
  }
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

// out[rows of expert e, :] = xs[rows of expert e, :K] * w[e][N, K]^T for all local experts.
// swiglu = 1 / 2 / 3 (swiglu / geglu / geglu_tanh, see ZbMoeAct): w holds the interleaved gate/up weight (N = 2F, see
// above) and out is [cap, F]; swiglu = 4 (relu2): a plain projection followed by relu(x)^2; 0: a plain projection.
// avg_tokens (expected tokens per expert) picks the tile orientation.
int zb_moe_grouped_gemm(const void* xs, const void* w, void* out, const int32_t* offsets, int e_local, int n, int k,
                        int cap, int ldo, int swiglu, int avg_tokens, void* stream) {
  if (cap <= 0 || e_local <= 0) return 0;
  if (k % 8 != 0 || ldo % 8 != 0) return -63;
  if (e_local > kZbMaxExperts) return -61;

  ZbDeviceState* st = zb_device_state();
  if (!st) return -20;
  const bool swap = avg_tokens <= 48;
  int bn;
  if (swap) {
    bn = 16;
    while (bn < avg_tokens * 2 && bn < 64) bn <<= 1;
    if (n % kBlockP != 0) return -64;
  } else {
    bn = (n % 256 == 0) ? 256 : 128;
    if (n % bn != 0) return -64;
  }
  GroupedParams prm;
  prm.offsets = offsets;
  prm.e_local = e_local;
  prm.n = n;
  prm.k = k;
  prm.ldo = ldo;
  prm.out = reinterpret_cast<__nv_bfloat16*>(out);
  prm.cap = cap;
  prm.act = swiglu;
  prm.status = st->status;
  if (swiglu < 0 || swiglu > ZB_ACT_RELU2) return -67;
  const bool gated = swiglu >= ZB_ACT_SWIGLU && swiglu <= ZB_ACT_GEGLU_TANH;
  CUtensorMap tx, tw;
  int rc = zb_make_tmap_bf16_2d(&tx, xs, cap, k, k, swap ? bn : kBlockP);
  if (rc != 0) return rc;
  rc = zb_make_tmap_bf16_2d(&tw, w, e_local * n, k, k, swap ? kBlockP : bn);
  if (rc != 0) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int grid = st->num_sms;
#define ZB_G(BN_, SW_)                                                                          \
  return gated ? launch_grouped<BN_, SW_, true>(tx, tw, prm, grid, s)                          \
               : launch_grouped<BN_, SW_, false>(tx, tw, prm, grid, s);
  if (swap) {
    switch (bn) {
      case 16: ZB_G(16, true)
      case 32: ZB_G(32, true)
      case 64: ZB_G(64, true)
    }
  } else if (bn == 256) {
    ZB_G(256, false)
  } else {
    ZB_G(128, false)
  }
#undef ZB_G
  return -65;
}

}  // extern "C"
