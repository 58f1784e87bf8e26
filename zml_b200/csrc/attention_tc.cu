// Paged prefill attention on the 5th-generation tensor cores (tcgen05 / TMEM / TMA) for sm_100a.
//
// Replaces the FA2 / Triton unified-attention prefill path of the reference
// (zml/attention/flashattn.zig:764-897, zml/attention/triton_attention.zig:140-494) for the common
// serving shape: head_dim 128, 64-token KV pages, grouped-query attention with an even group size.
// Other shapes keep the mma.sync kernel of attention.cu.
//
// One CTA works on 128 query rows of TWO query heads that share a KV head, so every K / V tile it
// brings in feeds two independent softmax pipelines ("ping-pong": while one head's scores are in the
// softmax warps, the tensor core works for the other head):
//   warps 0-3  : softmax / epilogue of head A (one thread per query row, TMEM lanes 0-127)
//   warps 4-7  : softmax / epilogue of head B
//   warp  8    : TMA producer (Q tiles once, then one K and one V page per step through a 3-stage ring)
//   warp  9    : MMA issuer (one thread)
// Per 64-key page and head:  S = Q K^T  (tcgen05.mma, A = Q and B = K from shared memory, both K-major,
// S in tensor memory) -> the softmax warps read S with tcgen05.ld, scale / mask, update the running
// maximum, rescale the output accumulator in tensor memory only when the maximum moved, and write
// P = exp2(S - m) as bf16 straight back into tensor memory -> O += P V (A = P from tensor memory,
// B = V from shared memory in its natural [key][head_dim] layout, i.e. MN-major).
// Tensor memory columns: S_A 0-63 | S_B 64-127 | P_A 128-159 | P_B 160-191 | O_A 192-319 | O_B 320-447.
// Every wait is bounded; a wait that runs out records a status and the CTA leaves through its normal exit.
#include <cuda.h>

#include "common.cuh"
#include "host_api.h"

int zb_make_tmap_bf16_2d(CUtensorMap* out, const void* base, int rows, int k, int ld, int box_rows);
int zb_make_tmap_kv_cache(CUtensorMap* out, const void* base, long long slots, int kv_heads, int head_dim, int box_rows);

namespace {

constexpr int kHD = 128;
constexpr int kQRows = 128;
constexpr int kKeys = 64;
constexpr int kStages = 3;
constexpr int kQBytes = kQRows * kHD * 2;          // one head's Q tile: two [128][64] sub-tiles
constexpr int kKvBytes = kKeys * kHD * 2;          // one K or V page of one KV head: two [64][64] sub-tiles
constexpr int kThreads = 320;
constexpr uint32_t kKernelId = 13;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0, kColP = 128, kColO = 192;

struct PrefillTcParams {
  __nv_bfloat16* out;           // [tokens, num_q_heads, 128]
  const int32_t* block_table;   // [batch, max_pages]
  const int32_t* seq_lens;      // [batch]
  const int32_t* q_start;       // [batch + 1]
  int batch;
  int num_q_heads;
  int num_kv_heads;
  int max_pages;
  int window;
  float scale_log2;
  uint32_t v_lbo;               // byte offsets of the MN-major descriptor of V (between 64-column groups / 8-key groups)
  uint32_t v_sbo;
  ZbStatus* status;
};

ZB_DEVICE float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Shared-memory descriptor of an MN-major bf16 operand written by TMA with the 128-byte swizzle: rows are K
// (here: keys), 64 contiguous MN elements (128 bytes) per row; `lbo` = bytes between 64-element groups along MN,
// `sbo` = bytes between groups of 8 rows along K.
ZB_DEVICE uint64_t make_desc_sw128_mn(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>((lbo >> 4) & 0x3fffu) << 16;
  d |= static_cast<uint64_t>((sbo >> 4) & 0x3fffu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

ZB_DEVICE void wg_bar_sync(int wg) {
  asm volatile("bar.sync %0, 128;" ::"r"(1 + wg) : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
zb_paged_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                           const __grid_constant__ CUtensorMap tmap_v, const PrefillTcParams p) {
  zb_pdl_launch();
  zb_pdl_wait();                                     // q, the KV cache and the batch description come from preceding work
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* q_s = smem;                               // [2 heads][32 KB]
  uint8_t* k_s = q_s + 2 * kQBytes;                  // [kStages][16 KB]
  uint8_t* v_s = k_s + kStages * kKvBytes;           // [kStages][16 KB]
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + kStages * kKvBytes);
  uint64_t* q_full = bars;                           // 1
  uint64_t* k_full = bars + 1;                       // kStages
  uint64_t* v_full = k_full + kStages;               // kStages
  uint64_t* kv_empty = v_full + kStages;             // kStages
  uint64_t* s_full = kv_empty + kStages;             // 2
  uint64_t* p_full = s_full + 2;                     // 2 (128 arrivals)
  uint64_t* o_ready = p_full + 2;                    // 2
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(o_ready + 2);
  volatile uint32_t* abort_flag = tmem_holder + 1;
  volatile uint32_t* abort_where = tmem_holder + 2;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = p.num_q_heads / p.num_kv_heads;
  const int head0 = blockIdx.y * 2;
  const int kvh = head0 / group;

  // the (sequence, 128-row query block) of this CTA
  int seq = -1, qb = 0;
  {
    // blocks are handed out from the end of the batch backwards, within a sequence from its last (longest) block
    int rem = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
    for (int i = 0; i < p.batch; ++i) {
      const int ql = p.q_start[i + 1] - p.q_start[i];
      const int nb = (ql + kQRows - 1) / kQRows;
      if (rem < nb) {
        seq = i;
        qb = rem;
        break;
      }
      rem -= nb;
    }
  }
  if (seq < 0) return;                               // grid is an upper bound of the number of blocks
  const int q_len = p.q_start[seq + 1] - p.q_start[seq];
  const int len = p.seq_lens[seq];
  const int ctx = len - q_len;
  const int row_base = qb * kQRows;
  const int tok_base = p.q_start[seq] + row_base;
  const int rows_valid = min(kQRows, q_len - row_base);
  const int last_key = min(len, ctx + row_base + kQRows);     // exclusive
  const int n_tiles = (last_key + kKeys - 1) / kKeys;
  int first_tile = 0;
  if (p.window > 0) first_tile = max(0, ctx + row_base - p.window + 1) / kKeys;

  if (threadIdx.x == 0) {
    zb_mbar_init(q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      zb_mbar_init(&k_full[s], 1);
      zb_mbar_init(&v_full[s], 1);
      zb_mbar_init(&kv_empty[s], 1);
    }
    for (int w = 0; w < 2; ++w) {
      zb_mbar_init(&s_full[w], 1);
      zb_mbar_init(&p_full[w], 128);
      zb_mbar_init(&o_ready[w], 1);
    }
    *abort_flag = 0u;
    *abort_where = 0u;
    zb_mbar_fence_init();
    zb_tma_prefetch_desc(&tmap_q);
    zb_tma_prefetch_desc(&tmap_k);
    zb_tma_prefetch_desc(&tmap_v);
  }
  if (warp == 9) {
    zb_tmem_alloc(tmem_holder, kTmemCols);
    zb_tmem_relinquish();
  }
  zb_tc_fence_before();
  __syncthreads();
  zb_tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      zb_mbar_expect_tx(q_full, 2 * kQBytes);
      for (int w = 0; w < 2; ++w)
        for (int c = 0; c < 2; ++c)
          zb_tma_load_2d(q_s + w * kQBytes + c * (kQRows * 128), &tmap_q, q_full, (head0 + w) * kHD + c * 64, tok_base);
      const int32_t* bt = p.block_table + static_cast<size_t>(seq) * p.max_pages;
      uint32_t stage = 0, phase = 0;
      for (int j = first_tile; j < n_tiles; ++j) {
        if (j - first_tile >= kStages) {
          if (!zb_mbar_wait(&kv_empty[stage], phase ^ 1u, abort_flag)) {
            *abort_where = 1u;
            break;
          }
        }
        int page = bt[j];
        if (!ZB_BC_OK(page, ZB_BC_PAGES, kKernelId, 10)) page = 0;
        zb_mbar_expect_tx(&k_full[stage], kKvBytes);
        zb_tma_load_4d(k_s + stage * kKvBytes, &tmap_k, &k_full[stage], 0, page * kKeys, 0, kvh);
        zb_mbar_expect_tx(&v_full[stage], kKvBytes);
        zb_tma_load_4d(v_s + stage * kKvBytes, &tmap_v, &v_full[stage], 0, page * kKeys, 0, kvh);
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t kIdescS = zb_make_idesc_bf16(kQRows, kKeys);
      constexpr uint32_t kIdescO = zb_make_idesc_bf16(kQRows, kHD) | (1u << 16);       // B (= V) is MN-major
      bool ok = zb_mbar_wait(q_full, 0u, abort_flag);
      if (!ok) *abort_where = 2u;
      // S_w = Q_w K^T of one page: 2 sub-tiles of 64 head-dim columns x 4 steps of 16
      auto mma_s = [&](int w, uint32_t st) {
        const uint32_t qa = zb_smem_u32(q_s + w * kQBytes), ka = zb_smem_u32(k_s + st * kKvBytes);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const uint64_t dq = zb_make_desc_sw128(qa + c * (kQRows * 128)), dk = zb_make_desc_sw128(ka + c * (kKeys * 128));
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            zb_umma_f16(tmem_base + kColS + w * kKeys, dq + 2 * kk, dk + 2 * kk, kIdescS, (c > 0 || kk > 0) ? 1u : 0u);
        }
        zb_umma_commit(&s_full[w]);
      };
      uint32_t stage = 0, phase = 0;                 // ring position of tile j
      if (ok && first_tile < n_tiles) {
        ok = zb_mbar_wait(&k_full[0], 0u, abort_flag);
        if (!ok) *abort_where = 3u;
        if (ok) {
          zb_tc_fence_after();
          mma_s(0, 0);
          mma_s(1, 0);
        }
      }
      for (int j = first_tile; ok && j < n_tiles; ++j) {
        const uint32_t jj = static_cast<uint32_t>(j - first_tile);
        uint32_t nstage = stage + 1, nphase = phase;
        if (nstage == kStages) {
          nstage = 0;
          nphase ^= 1u;
        }
        if (!zb_mbar_wait(&v_full[stage], phase, abort_flag)) {
          *abort_where = 4u;
          break;
        }
        for (int w = 0; w < 2 && ok; ++w) {
          if (!zb_mbar_wait(&p_full[w], jj & 1u, abort_flag)) {
            *abort_where = 5u + w;
            ok = false;
            break;
          }
          zb_tc_fence_after();
          // O_w (+)= P_w V: 4 steps of 16 keys; A = P in tensor memory (8 columns per step), B = V, MN-major
          const uint32_t va = zb_smem_u32(v_s + stage * kKvBytes);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t dv = make_desc_sw128_mn(va + k * (16 * 128), p.v_lbo, p.v_sbo);
            zb_umma_f16_ts(tmem_base + kColO + w * kHD, tmem_base + kColP + w * 32 + 8 * k, dv, kIdescO, (jj > 0 || k > 0) ? 1u : 0u);
          }
          zb_umma_commit(&o_ready[w]);
          if (j + 1 < n_tiles) {
            if (w == 0) {
              if (!zb_mbar_wait(&k_full[nstage], nphase, abort_flag)) {
                *abort_where = 7u;
                ok = false;
                break;
              }
              zb_tc_fence_after();
            }
            mma_s(w, nstage);                        // the softmax warps of w have read S_w (they published P_w)
          }
        }
        if (!ok) break;
        zb_umma_commit(&kv_empty[stage]);            // K and V of this stage are consumed once these MMAs retire
        stage = nstage;
        phase = nphase;
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue (one row per thread)
    const int w = warp >> 2;                         // which of the two heads
    const int quad = warp & 3;
    const int r = quad * 32 + lane;                  // query row inside the block
    const int qpos = ctx + row_base + r;             // its position among the keys
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t t_s = tmem_base + kColS + w * kKeys + lane_off;
    const uint32_t t_p = tmem_base + kColP + w * 32 + lane_off;
    const uint32_t t_o = tmem_base + kColO + w * kHD + lane_off;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = first_tile; j < n_tiles; ++j) {
      const uint32_t jj = static_cast<uint32_t>(j - first_tile);
      if (!zb_mbar_wait(&s_full[w], jj & 1u, abort_flag)) {
        *abort_where = 10u + w;
        ok = false;
        break;
      }
      zb_tc_fence_after();
      uint32_t sr[64];
      zb_tmem_ld32(t_s, reinterpret_cast<uint32_t(&)[32]>(sr[0]));
      zb_tmem_ld32(t_s + 32, reinterpret_cast<uint32_t(&)[32]>(sr[32]));
      zb_tmem_ld_wait();
      const int key0 = j * kKeys;
      // pages below the block's first row and inside every row's window need no mask (a branch per page, not a
      // predicate per score: predicated-off instructions still take issue slots, and this loop is issue-bound)
      const bool full = (key0 + kKeys - 1 <= ctx + row_base) && (key0 + kKeys <= len) &&
                        (p.window <= 0 || key0 > ctx + row_base + kQRows - 1 - p.window);
      float mx_raw = -INFINITY;                      // maximum of the raw (unscaled) scores of this page
      if (full) {
#pragma unroll
        for (int i = 0; i < 64; ++i) mx_raw = fmaxf(mx_raw, __uint_as_float(sr[i]));
      } else {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const int kidx = key0 + i;
          bool vis = kidx <= qpos && kidx < len;
          if (p.window > 0) vis = vis && (kidx > qpos - p.window);
          if (!vis) sr[i] = 0xff800000u;             // -inf
          mx_raw = fmaxf(mx_raw, __uint_as_float(sr[i]));
        }
      }
      const float mx = fmaxf(m, mx_raw * p.scale_log2);           // running maximum, in units of log2
      const float m_use = mx == -INFINITY ? 0.f : mx;             // a row without a visible key so far
      if (jj > 0) {
        // the output accumulated so far is relative to the old maximum: rescale it where the maximum moved
        const float alpha = m == -INFINITY ? 1.f : ex2(m - m_use);
        const bool moved = alpha != 1.f;
        if (__any_sync(0xffffffffu, moved)) {
          if (!zb_mbar_wait(&o_ready[w], (jj - 1u) & 1u, abort_flag)) {      // O += P V of the previous page is done
            *abort_where = 12u + w;
            ok = false;
            break;
          }
          zb_tc_fence_after();
#pragma unroll 1
          for (int c0 = 0; c0 < kHD; c0 += 32) {
            uint32_t o[32];
            zb_tmem_ld32(t_o + c0, o);
            zb_tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            zb_tmem_st16(t_o + c0, o);
            zb_tmem_st16(t_o + c0 + 16, o + 16);
          }
          zb_tmem_st_wait();
        }
        l *= alpha;
      }
      m = mx;
      // p = 2^(s * scale - m): one fused multiply-add and one exponential per score
      const float neg_m = -m_use;
      uint32_t pw[32];
      float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float p0 = ex2(fmaf(__uint_as_float(sr[2 * i]), p.scale_log2, neg_m));
        const float p1 = ex2(fmaf(__uint_as_float(sr[2 * i + 1]), p.scale_log2, neg_m));
        pw[i] = zb_pack_bf16x2(p0, p1);
        sum0 += p0;
        sum1 += p1;
      }
      l += sum0 + sum1;
      zb_tmem_st16(t_p, pw);
      zb_tmem_st16(t_p + 16, pw + 16);
      zb_tmem_st_wait();
      zb_tc_fence_before();
      zb_mbar_arrive(&p_full[w]);
    }
    if (ok && first_tile < n_tiles) {
      const uint32_t last = static_cast<uint32_t>(n_tiles - 1 - first_tile);
      if (zb_mbar_wait(&o_ready[w], last & 1u, abort_flag)) {
        zb_tc_fence_after();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* orow = p.out + (static_cast<size_t>(tok_base + r) * p.num_q_heads + head0 + w) * kHD;
#pragma unroll 1
        for (int c0 = 0; c0 < kHD; c0 += 32) {
          uint32_t o[32];
          zb_tmem_ld32(t_o + c0, o);
          zb_tmem_ld_wait();
          if (r < rows_valid) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint32_t wd[4];
#pragma unroll
              for (int q = 0; q < 4; ++q)
                wd[q] = zb_pack_bf16x2(__uint_as_float(o[8 * i + 2 * q]) * inv, __uint_as_float(o[8 * i + 2 * q + 1]) * inv);
              *reinterpret_cast<uint4*>(orow + c0 + 8 * i) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
            }
          }
        }
      } else {
        *abort_where = 14u + w;
      }
    } else if (ok && r < rows_valid) {
      // no key at all (cannot happen for a causal prefill, kept for completeness): zeros
      __nv_bfloat16* orow = p.out + (static_cast<size_t>(tok_base + r) * p.num_q_heads + head0 + w) * kHD;
      for (int c = 0; c < kHD; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0u, 0u, 0u, 0u);
    }
  }

  // ------------------------------------------------------------------ common exit
  zb_tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0u) {
    if (threadIdx.x == 0) zb_record_error(p.status, ZB_ERR_MBAR_TIMEOUT, kKernelId, *abort_where, blockIdx.x);
    const uint64_t t0 = zb_globaltimer();            // copies still in flight must land before the shared memory is reused
    while (zb_globaltimer() - t0 < 200000ull) {
    }
    __syncthreads();
  }
  if (warp == 9) {
    zb_tc_fence_after();
    zb_tmem_dealloc(tmem_base, kTmemCols);
  }
}

constexpr int kSmemBytes = 2 * kQBytes + 2 * kStages * kKvBytes + 1024 + 256;

}  // namespace

extern "C" {

// 1 when the tensor-core prefill kernel takes this shape (head_dim 128, 64-token pages, an even number of query
// heads per KV head), else 0: the caller then uses the mma.sync kernel.
int zb_paged_prefill_tc_supported(int num_q_heads, int num_kv_heads, int head_dim, int page_size) {
  if (head_dim != kHD || page_size != kKeys || num_kv_heads <= 0 || num_q_heads % num_kv_heads != 0) return 0;
  return ((num_q_heads / num_kv_heads) % 2) == 0 ? 1 : 0;
}

// Same contract as zb_paged_prefill.  total_q_blocks128 >= sum over sequences of ceil(q_len / 128).
// `v_lbo` / `v_sbo` = 0 select the defaults of the V descriptor (8192 / 1024 bytes).
int zb_paged_prefill_tc(const void* q, const void* k_cache, const void* v_cache, void* out, const int32_t* block_table,
                        const int32_t* seq_lens, const int32_t* q_start, int batch, int total_q_blocks128, int total_tokens,
                        int num_q_heads, int num_kv_heads, int max_pages, long long q_stride, float scale, int window,
                        unsigned v_lbo, unsigned v_sbo, void* stream) {
  if (batch <= 0 || total_q_blocks128 <= 0) return 0;
  if (!zb_paged_prefill_tc_supported(num_q_heads, num_kv_heads, kHD, kKeys)) return -32;
  ZbDeviceState* st = zb_device_state();
  if (!st) return -20;
  static bool configured[16] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return -21;
  if (!configured[dev]) {
    cudaError_t e = zb_config_smem(zb_paged_prefill_tc_kernel, kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev] = true;
  }
  CUtensorMap tq, tk, tv;
  // q as a [tokens, heads * 128] matrix with leading dimension q_stride: boxes of 128 rows x 64 columns
  int rc = zb_make_tmap_bf16_2d(&tq, q, total_tokens, num_q_heads * kHD, static_cast<int>(q_stride), kQRows);
  if (rc != 0) return rc;
  const long long slots = 1ll << 30;               // bound only: pages are addressed through the block table
  rc = zb_make_tmap_kv_cache(&tk, k_cache, slots, num_kv_heads, kHD, kKeys);
  if (rc != 0) return rc;
  rc = zb_make_tmap_kv_cache(&tv, v_cache, slots, num_kv_heads, kHD, kKeys);
  if (rc != 0) return rc;
  PrefillTcParams p = {};
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.block_table = block_table;
  p.seq_lens = seq_lens;
  p.q_start = q_start;
  p.batch = batch;
  p.num_q_heads = num_q_heads;
  p.num_kv_heads = num_kv_heads;
  p.max_pages = max_pages;
  p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.v_lbo = v_lbo ? v_lbo : 8192u;
  p.v_sbo = v_sbo ? v_sbo : 1024u;
  p.status = st->status;
  const cudaError_t le = zb_launch(zb_paged_prefill_tc_kernel, dim3(total_q_blocks128, num_q_heads / 2), dim3(kThreads), kSmemBytes,
                                   reinterpret_cast<cudaStream_t>(stream), tq, tk, tv, p);
  zb_count_launch(1);
  return static_cast<int>(le != cudaSuccess ? le : cudaGetLastError());
}

}  // extern "C"
