// Paged flash attention for sm_100a: varlen causal prefill and split-KV decode
// with GQA packing, reading K/V straight from a paged cache laid out as
// {page, slot_in_page, kv_head, head_dim} (the reference's KvCache layout,
// zml/attention/paged_attention.zig:218-254).
//
// Replaces the FA2 / Triton "unified attention" paged back-ends of the reference
// (zml/attention/flashattn.zig:532-1136, zml/attention/triton_attention.zig:140-494).
// Semantics follow the pure-tensor oracle (zml/attention/paged_attention.zig:535-777):
// online softmax over pages, causal with the query block placed at the END of
// the sequence (ctx = seq_len - q_len keys precede the first query).
//
// The decode kernel is bandwidth bound (it streams the KV cache once): each warp
// runs its own cp.async pipeline over 16-key blocks, the G query heads that share
// one KV head are packed into the 16 rows of one m16n8k16 tile, and the KV range
// of a sequence is cut into fixed-size chunks, one CTA each, so that all SMs stream
// whatever the mix of sequence lengths.  Partial results (unnormalised O, running
// max m, running sum l) go to scratch and the last chunk of a (sequence, kv head)
// to finish merges them in chunk order, in the same launch.
#include <cuda.h>

#include "common.cuh"
#include "host_api.h"

int zb_make_tmap_kv_cache(CUtensorMap* out, const void* base, long long slots, int kv_heads, int head_dim, int box_rows);

namespace {

constexpr uint32_t kKernelDecode = 2;
constexpr uint32_t kKernelPrefill = 3;

ZB_DEVICE void cp_async16(uint32_t smem_dst, const void* gsrc, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gsrc),
               "r"(src_bytes)
               : "memory");
}
ZB_DEVICE void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
ZB_DEVICE void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

ZB_DEVICE void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
ZB_DEVICE void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
ZB_DEVICE void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// byte offset of 16-byte chunk `chunk` of row `row` in a [rows][HD] bf16 tile whose
// chunks are XOR-swizzled with the row so that ldmatrix is conflict free
template <int HD>
ZB_DEVICE uint32_t tile_off(int row, int chunk) {
  return static_cast<uint32_t>(row * (HD * 2) + ((chunk ^ (row & 7)) << 4));
}

// Same for a tile written by a tensor-map copy with the 128-byte swizzle: HD / 64 sub-tiles of
// [64 rows][64 columns], each row 128 bytes, 16-byte chunks XOR-ed with the row inside its sub-tile.
template <int HD>
ZB_DEVICE uint32_t tile_off_tma(int row, int chunk) {
  return static_cast<uint32_t>((chunk >> 3) * (64 * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}
template <int HD, int LAYOUT>
ZB_DEVICE uint32_t tile_off_l(int row, int chunk) {
  if constexpr (LAYOUT == 0) return tile_off<HD>(row, chunk);
  else return tile_off_tma<HD>(row, chunk);
}

struct AttnParams {
  const __nv_bfloat16* q;       // [tokens, num_q_heads, HD] with token stride q_stride
  const __nv_bfloat16* k_cache; // [pages, page_size, num_kv_heads, HD]
  const __nv_bfloat16* v_cache;
  __nv_bfloat16* out;           // [tokens, num_q_heads, HD], contiguous
  const int32_t* block_table;   // [batch, max_pages]
  const int32_t* seq_lens;      // [batch] keys per sequence, new tokens included
  const int32_t* q_start;       // [batch + 1] prefill only
  float* part_o;                // decode: [batch, num_q_heads, splits, HD]
  float* part_ml;               // decode: [batch, num_q_heads, splits, 2]
  long long q_stride;           // elements between consecutive tokens of q
  int batch;
  int num_q_heads;
  int num_kv_heads;
  int page_size;
  int max_pages;
  int num_splits;               // decode: upper bound of KV chunks per sequence (grid.y)
  int chunk_blocks;             // decode: 16-key blocks per chunk
  uint32_t* counters;           // decode: one per (sequence, kv head), zero between launches
  int window;                   // sliding window (keys), <= 0: none
  float scale_log2;             // softmax scale * log2(e)
  ZbStatus* status;
};

// One 16-key block: S = Q K^T (16 x 16), online softmax update, O += P V.
//   qf     : Q fragments, HD/16 k-steps
//   k_base : shared address of the 16 K rows of this block (tile-relative row0)
//   row0   : first row of the block inside its swizzled tile
//   mask0/mask1 : per-row predicate producers are inlined by the callers via `visible`
template <int HD, int LAYOUT = 0, typename Visible>
ZB_DEVICE void attn_block16(const uint32_t (&qf)[HD / 16][4], uint32_t k_tile, uint32_t v_tile,
                            int row0, float (&o)[HD / 8][4], float (&m)[2], float (&l)[2],
                            float scale_log2, Visible visible) {
  const int lane = threadIdx.x & 31;
  const int mi = lane >> 3;
  const int r8 = lane & 7;
  float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
  for (int kk = 0; kk < HD / 16; ++kk) {
    uint32_t b[4];
    const int krow = row0 + (mi >> 1) * 8 + r8;
    ldmatrix_x4(b, k_tile + tile_off_l<HD, LAYOUT>(krow, 2 * kk + (mi & 1)));
    mma_bf16(s[0], qf[kk], b[0], b[1]);
    mma_bf16(s[1], qf[kk], b[2], b[3]);
  }
  // scale + mask; column of s[nt][j] is nt*8 + 2*(lane%4) + (j&1), row is (lane/4) + 8*(j>>1)
  const int t = lane & 3;
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = nt * 8 + 2 * t + (j & 1);
      const int half = j >> 1;
      float v = s[nt][j] * scale_log2;
      if (!visible(half, col)) v = -INFINITY;
      s[nt][j] = v;
      mx[half] = fmaxf(mx[half], v);
    }
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
  }
  float corr[2], muse[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float mnew = fmaxf(m[h], mx[h]);
    muse[h] = (mnew == -INFINITY) ? 0.f : mnew;
    corr[h] = exp2f(m[h] - muse[h]);   // m = -inf -> 0
    m[h] = mnew;
  }
  float rs[2] = {0.f, 0.f};
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int half = j >> 1;
      const float pv = exp2f(s[nt][j] - muse[half]);
      s[nt][j] = pv;
      rs[half] += pv;
    }
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 1);
    rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 2);
    l[h] = l[h] * corr[h] + rs[h];
  }
  uint32_t pa[4];
  pa[0] = zb_pack_bf16x2(s[0][0], s[0][1]);
  pa[1] = zb_pack_bf16x2(s[0][2], s[0][3]);
  pa[2] = zb_pack_bf16x2(s[1][0], s[1][1]);
  pa[3] = zb_pack_bf16x2(s[1][2], s[1][3]);
#pragma unroll
  for (int c = 0; c < HD / 8; c += 2) {
    uint32_t b[4];
    const int vrow = row0 + (mi & 1) * 8 + r8;
    ldmatrix_x4_trans(b, v_tile + tile_off_l<HD, LAYOUT>(vrow, c + (mi >> 1)));
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      o[c][j] *= corr[j >> 1];
      o[c + 1][j] *= corr[j >> 1];
    }
    mma_bf16(o[c], pa, b[0], b[1]);
    mma_bf16(o[c + 1], pa, b[2], b[3]);
  }
}

// Tail shared by the decode kernels: merges the four consumer warps of the CTA through shared
// memory, writes the chunk's partial (or the final output when the sequence has one chunk), and
// lets the last chunk of a (sequence, kv head) to finish merge all of them.  Every thread of the
// CTA calls it (warps beyond the fourth only take part in the barriers and the element loops).
template <int HD>
ZB_DEVICE void decode_tail(const AttnParams& p, uint8_t* smem, const float (&o)[HD / 8][4], const float (&m)[2],
                           const float (&l)[2], int seq, int kvh, int split, int my_splits, int group) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // merge the four warps through shared memory (pipeline buffers are free now)
  float* sm_o = reinterpret_cast<float*>(smem);                 // [4][16][HD]
  float* sm_ml = sm_o + 4 * 16 * HD;                            // [4][16][2]
  if (warp < 4) {
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt) {
      const int c = nt * 8 + 2 * t;
      float* r0 = sm_o + (warp * 16 + g) * HD + c;
      float* r1 = sm_o + (warp * 16 + g + 8) * HD + c;
      r0[0] = o[nt][0];
      r0[1] = o[nt][1];
      r1[0] = o[nt][2];
      r1[1] = o[nt][3];
    }
    if (t == 0) {
      sm_ml[(warp * 16 + g) * 2 + 0] = m[0];
      sm_ml[(warp * 16 + g) * 2 + 1] = l[0];
      sm_ml[(warp * 16 + g + 8) * 2 + 0] = m[1];
      sm_ml[(warp * 16 + g + 8) * 2 + 1] = l[1];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < group * HD; idx += blockDim.x) {
    const int r = idx / HD, c = idx % HD;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, sm_ml[(w * 16 + r) * 2]);
    const float muse = (mm == -INFINITY) ? 0.f : mm;
    float acc = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = exp2f(sm_ml[(w * 16 + r) * 2] - muse);
      acc += f * sm_o[(w * 16 + r) * HD + c];
      ll += f * sm_ml[(w * 16 + r) * 2 + 1];
    }
    const int head = kvh * group + r;
    if (my_splits == 1) {
      const float inv = ll > 0.f ? 1.f / ll : 0.f;
      p.out[(static_cast<size_t>(seq) * p.num_q_heads + head) * HD + c] = __float2bfloat16(acc * inv);
    } else {
      const size_t pi = (static_cast<size_t>(seq) * p.num_q_heads + head) * p.num_splits + split;
      p.part_o[pi * HD + c] = acc;
      if (c == 0) {
        p.part_ml[pi * 2] = mm;
        p.part_ml[pi * 2 + 1] = ll;
      }
    }
  }
  if (my_splits == 1) return;
  // the last chunk to finish merges all chunks of this (sequence, kv head)
  __shared__ uint32_t s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t prev = atomicAdd(&p.counters[blockIdx.x], 1u);
    s_last = (prev == static_cast<uint32_t>(my_splits - 1)) ? 1u : 0u;
    if (s_last) p.counters[blockIdx.x] = 0u;
  }
  __syncthreads();
  if (s_last == 0u) return;
  __threadfence();
  // Phase 1: (max, sum) of every (row, chunk) -> shared memory, one round trip to L2.
  // Phase 2: every thread combines its output elements with the chunk loads of an element
  // batched eight at a time, so that the merge costs a few round trips, not one per chunk.
  float* s_m = reinterpret_cast<float*>(smem);          // [group][my_splits]
  float* s_l = s_m + 16 * 64;                           // [group][my_splits] (at most 16 rows x 64 chunks)
  const int nsp = min(my_splits, 64);
  for (int i = threadIdx.x; i < group * nsp; i += blockDim.x) {
    const int r = i / nsp, sp = i - r * nsp;
    const size_t base = (static_cast<size_t>(seq) * p.num_q_heads + kvh * group + r) * p.num_splits;
    const float2 ml = __ldcg(reinterpret_cast<const float2*>(&p.part_ml[(base + sp) * 2]));
    s_m[r * 64 + sp] = ml.x;
    s_l[r * 64 + sp] = ml.y;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < group * HD; idx += blockDim.x) {
    const int r = idx / HD, c = idx % HD;
    const int head = kvh * group + r;
    const size_t base = (static_cast<size_t>(seq) * p.num_q_heads + head) * p.num_splits;
    float mm = -INFINITY;
    for (int sp = 0; sp < nsp; ++sp) mm = fmaxf(mm, s_m[r * 64 + sp]);
    const float muse = (mm == -INFINITY) ? 0.f : mm;
    float acc = 0.f, ll = 0.f;
    for (int sp0 = 0; sp0 < nsp; sp0 += 8) {
      float pv[8];
#pragma unroll
      for (int b = 0; b < 8; ++b) pv[b] = __ldcg(&p.part_o[(base + min(sp0 + b, nsp - 1)) * HD + c]);
#pragma unroll
      for (int b = 0; b < 8; ++b) {
        if (sp0 + b < nsp) {
          const float f = exp2f(s_m[r * 64 + sp0 + b] - muse);
          acc += f * pv[b];
          ll += f * s_l[r * 64 + sp0 + b];
        }
      }
    }
    p.out[(static_cast<size_t>(seq) * p.num_q_heads + head) * HD + c] = __float2bfloat16(ll > 0.f ? acc / ll : 0.f);
  }
}

// ---------------------------------------------------------------------- decode
constexpr int kDecStages = 3;

template <int HD>
__global__ void __launch_bounds__(128) zb_paged_decode_kernel(const AttnParams p) {
  zb_pdl_launch();
  zb_pdl_wait();
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int kChunks = HD / 8;
  constexpr int kBlkBytes = 16 * HD * 2;              // one 16-key block of K (or V)
  constexpr int kWarpBytes = kDecStages * 2 * kBlkBytes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = blockIdx.x / p.num_kv_heads;
  const int kvh = blockIdx.x % p.num_kv_heads;
  const int split = blockIdx.y;
  const int group = p.num_q_heads / p.num_kv_heads;
  const int len = p.seq_lens[seq];
  const int nblk = (len + 15) >> 4;
  // the sequence is cut into chunks of `chunk_blocks` 16-key blocks; CTAs beyond the
  // last chunk of a short sequence have nothing to do
  const int per = p.chunk_blocks;
  const int my_splits = max(1, (nblk + per - 1) / per);
  if (split >= my_splits) return;
  const int blk0 = split * per;
  const int blk1 = min(nblk, blk0 + per);
  const int first_visible = p.window > 0 ? max(0, len - p.window) : 0;

  const uint32_t wbase = zb_smem_u32(smem) + warp * kWarpBytes;
  const int32_t* bt = p.block_table + static_cast<size_t>(seq) * p.max_pages;
  const size_t row_elems = static_cast<size_t>(p.num_kv_heads) * HD;

  // Q fragments: row r < group is query head kvh*group + r of this sequence's token
  uint32_t qf[HD / 16][4];
  {
    const int g = lane >> 2, t = lane & 3;
    const __nv_bfloat16* qrow0 = p.q + static_cast<size_t>(seq) * p.q_stride +
                                 static_cast<size_t>(kvh * group + g) * HD;
    const __nv_bfloat16* qrow1 = qrow0 + static_cast<size_t>(8) * HD;
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
      const int c = kk * 16 + 2 * t;
      qf[kk][0] = g < group ? *reinterpret_cast<const uint32_t*>(qrow0 + c) : 0u;
      qf[kk][1] = (g + 8) < group ? *reinterpret_cast<const uint32_t*>(qrow1 + c) : 0u;
      qf[kk][2] = g < group ? *reinterpret_cast<const uint32_t*>(qrow0 + c + 8) : 0u;
      qf[kk][3] = (g + 8) < group ? *reinterpret_cast<const uint32_t*>(qrow1 + c + 8) : 0u;
    }
  }

  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  auto issue = [&](int blk, int stage) {
    if (blk < blk1) {
      const int tok0 = blk << 4;
      int page = bt[tok0 / p.page_size];
      if (!ZB_BC_OK(page, ZB_BC_PAGES, kKernelDecode, 10)) page = 0;      // checking build: reported, page 0 read instead
      const int off0 = tok0 % p.page_size;
      const size_t base = (static_cast<size_t>(page) * p.page_size + off0) * row_elems +
                          static_cast<size_t>(kvh) * HD;
      const uint32_t ks = wbase + stage * 2 * kBlkBytes;
      const uint32_t vs = ks + kBlkBytes;
#pragma unroll
      for (int i = 0; i < (16 * kChunks) / 32; ++i) {
        const int idx = lane + 32 * i;
        const int row = idx / kChunks, chunk = idx % kChunks;
        const uint32_t nbytes = (tok0 + row) < len ? 16u : 0u;
        const size_t goff = base + static_cast<size_t>(row) * row_elems + chunk * 8;
        cp_async16(ks + tile_off<HD>(row, chunk), p.k_cache + goff, nbytes);
        cp_async16(vs + tile_off<HD>(row, chunk), p.v_cache + goff, nbytes);
      }
    }
    cp_async_commit();
  };

  // this warp's blocks: blk0 + warp, blk0 + warp + 4, ...
  int nxt = blk0 + warp;
#pragma unroll
  for (int s = 0; s < kDecStages - 1; ++s) {
    issue(nxt, s);
    nxt += 4;
  }
  int stage = 0;
  for (int blk = blk0 + warp; blk < blk1; blk += 4) {
    cp_async_wait<kDecStages - 2>();
    __syncwarp();
    // refill the stage consumed in the previous iteration BEFORE computing on this one, so that
    // the loads of two blocks are in flight while the tensor cores work (the kernel is bound by
    // memory latency: 8 warps per SM, each waiting on its own copies)
    int fill = stage + kDecStages - 1;
    if (fill >= kDecStages) fill -= kDecStages;
    issue(nxt, fill);
    nxt += 4;
    const uint32_t ks = wbase + stage * 2 * kBlkBytes;
    const int tok0 = blk << 4;
    attn_block16<HD>(qf, ks, ks + kBlkBytes, 0, o, m, l, p.scale_log2,
                     [&](int /*half*/, int col) {
                       const int kidx = tok0 + col;
                       return kidx < len && kidx >= first_visible;
                     });
    __syncwarp();
    if (++stage == kDecStages) stage = 0;
  }
  cp_async_wait<0>();
  __syncthreads();
  decode_tail<HD>(p, smem, o, m, l, seq, kvh, split, my_splits, group);
}

// ------------------------------------------------------- decode, tensor-map fed
// Same math as zb_paged_decode_kernel with the K/V pages brought in by a producer warp through
// tensor-map copies (one 64-key page of one head per copy, 128-byte swizzle) into a ring of
// stages; the four consumer warps each own 16 of the 64 keys of a tile and never wait on their
// own copies.  Needs 64-token pages and KV chunks that are multiples of 64 keys.
template <int HD>
constexpr int dec_tma_stages() { return HD >= 256 ? 2 : 3; }

template <int HD>
__global__ void __launch_bounds__(160) zb_paged_decode_tma_kernel(const __grid_constant__ CUtensorMap tmap_k,
                                                                  const __grid_constant__ CUtensorMap tmap_v,
                                                                  const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  constexpr int kStages = dec_tma_stages<HD>();
  constexpr int kTileBytes = 64 * HD * 2;                 // one page of K (or V) of one head
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * 2 * kTileBytes);
  uint64_t* empty_bar = full_bar + kStages;
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(empty_bar + kStages);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      zb_mbar_init(&full_bar[s], 1);
      zb_mbar_init(&empty_bar[s], 4);
    }
    *abort_flag = 0u;
    zb_mbar_fence_init();
    zb_tma_prefetch_desc(&tmap_k);
    zb_tma_prefetch_desc(&tmap_v);
  }
  __syncthreads();
  zb_pdl_launch();
  zb_pdl_wait();
  const int seq = blockIdx.x / p.num_kv_heads;
  const int kvh = blockIdx.x % p.num_kv_heads;
  const int split = blockIdx.y;
  const int group = p.num_q_heads / p.num_kv_heads;
  const int len = p.seq_lens[seq];
  const int nblk = (len + 15) >> 4;
  const int per = p.chunk_blocks;                          // a multiple of 4 (64 keys)
  const int my_splits = max(1, (nblk + per - 1) / per);
  if (split >= my_splits) return;
  const int blk0 = split * per;
  const int blk1 = min(nblk, blk0 + per);
  const int tile0 = blk0 >> 2, tile1 = (blk1 + 3) >> 2;
  const int first_visible = p.window > 0 ? max(0, len - p.window) : 0;
  const int32_t* bt = p.block_table + static_cast<size_t>(seq) * p.max_pages;

  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  if (warp == 4) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      for (int t = tile0; t < tile1; ++t) {
        if (!zb_mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) break;
        int page = bt[t];
        if (!ZB_BC_OK(page, ZB_BC_PAGES, kKernelDecode, 11)) page = 0;
        uint8_t* ks = smem + stage * 2 * kTileBytes;
        zb_mbar_expect_tx(&full_bar[stage], 2 * kTileBytes);
        zb_tma_load_4d(ks, &tmap_k, &full_bar[stage], 0, page * 64, 0, kvh);
        zb_tma_load_4d(ks + kTileBytes, &tmap_v, &full_bar[stage], 0, page * 64, 0, kvh);
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else {
    // Q fragments: row r < group is query head kvh*group + r of this sequence's token
    uint32_t qf[HD / 16][4];
    {
      const int g = lane >> 2, t = lane & 3;
      const __nv_bfloat16* qrow0 = p.q + static_cast<size_t>(seq) * p.q_stride + static_cast<size_t>(kvh * group + g) * HD;
      const __nv_bfloat16* qrow1 = qrow0 + static_cast<size_t>(8) * HD;
#pragma unroll
      for (int kk = 0; kk < HD / 16; ++kk) {
        const int c = kk * 16 + 2 * t;
        qf[kk][0] = g < group ? *reinterpret_cast<const uint32_t*>(qrow0 + c) : 0u;
        qf[kk][1] = (g + 8) < group ? *reinterpret_cast<const uint32_t*>(qrow1 + c) : 0u;
        qf[kk][2] = g < group ? *reinterpret_cast<const uint32_t*>(qrow0 + c + 8) : 0u;
        qf[kk][3] = (g + 8) < group ? *reinterpret_cast<const uint32_t*>(qrow1 + c + 8) : 0u;
      }
    }
    uint32_t stage = 0, phase = 0;
    for (int t = tile0; t < tile1; ++t) {
      if (!zb_mbar_wait(&full_bar[stage], phase, abort_flag)) break;
      const int tok0 = t * 64 + warp * 16;                 // this warp's 16 keys of the tile
      if (tok0 < len && (tok0 >> 4) >= blk0 && (tok0 >> 4) < blk1) {
        const uint32_t ks = zb_smem_u32(smem + stage * 2 * kTileBytes);
        const uint32_t vs = ks + kTileBytes;
        if (tok0 + 16 > len) {
          // rows past the end of the sequence hold whatever the page held before: their
          // probabilities are zero, but 0 x NaN would still poison the sum - clear those V rows
          for (int idx = lane; idx < 16 * (HD / 8); idx += 32) {
            const int row = warp * 16 + idx / (HD / 8), chunk = idx % (HD / 8);
            if (t * 64 + row >= len)
              *reinterpret_cast<uint4*>(smem + stage * 2 * kTileBytes + kTileBytes + tile_off_tma<HD>(row, chunk)) =
                  make_uint4(0u, 0u, 0u, 0u);
          }
          __syncwarp();
        }
        attn_block16<HD, 1>(qf, ks, vs, warp * 16, o, m, l, p.scale_log2, [&](int /*half*/, int col) {
          const int kidx = tok0 + col;
          return kidx < len && kidx >= first_visible;
        });
      }
      __syncwarp();
      if (lane == 0) zb_mbar_arrive(&empty_bar[stage]);
      if (++stage == kStages) {
        stage = 0;
        phase ^= 1u;
      }
    }
  }
  __syncthreads();
  if (*abort_flag != 0u) {
    if (threadIdx.x == 0) zb_record_error(p.status, ZB_ERR_MBAR_TIMEOUT, 2u, 1u, blockIdx.x);
    // copies that may still be in flight must land before the shared memory is reused
    const uint64_t t0 = zb_globaltimer();
    while (zb_globaltimer() - t0 < 200000ull) {
    }
    __syncthreads();
    return;
  }
  decode_tail<HD>(p, smem, o, m, l, seq, kvh, split, my_splits, group);
}

// --------------------------------------------------------------------- prefill
template <int HD>
__global__ void __launch_bounds__(128) zb_paged_prefill_kernel(const AttnParams p) {
  zb_pdl_launch();
  zb_pdl_wait();
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int kChunks = HD / 8;
  constexpr int kTileBytes = 64 * HD * 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int group = p.num_q_heads / p.num_kv_heads;
  const int kvh = head / group;

  // locate the (sequence, query block) of this CTA
  int seq = -1, qb = 0;
  {
    int rem = blockIdx.x;
    for (int i = 0; i < p.batch; ++i) {
      const int ql = p.q_start[i + 1] - p.q_start[i];
      const int nb = (ql + 63) >> 6;
      if (rem < nb) {
        seq = i;
        qb = rem;
        break;
      }
      rem -= nb;
    }
  }
  if (seq < 0) return;
  const int q_len = p.q_start[seq + 1] - p.q_start[seq];
  const int len = p.seq_lens[seq];
  const int ctx = len - q_len;
  const int row_base = qb * 64;                       // first query row of the block
  const int tok_base = p.q_start[seq] + row_base;     // its token index
  const int rows_valid = min(64, q_len - row_base);
  const int last_key = min(len, ctx + row_base + 64);  // exclusive
  const int n_tiles = (last_key + 63) >> 6;
  int first_tile = 0;
  if (p.window > 0) first_tile = max(0, ctx + row_base - p.window + 1) >> 6;

  const uint32_t q_s = zb_smem_u32(smem);
  const uint32_t kv_s = q_s + kTileBytes;             // 2 stages x (K tile, V tile)
  const int32_t* bt = p.block_table + static_cast<size_t>(seq) * p.max_pages;
  const size_t row_elems = static_cast<size_t>(p.num_kv_heads) * HD;

  // Q tile -> smem
  for (int idx = threadIdx.x; idx < 64 * kChunks; idx += 128) {
    const int row = idx / kChunks, chunk = idx % kChunks;
    const uint32_t nbytes = row < rows_valid ? 16u : 0u;
    const __nv_bfloat16* src = p.q + static_cast<size_t>(tok_base + (row < rows_valid ? row : 0)) * p.q_stride +
                               static_cast<size_t>(head) * HD + chunk * 8;
    cp_async16(q_s + tile_off<HD>(row, chunk), src, nbytes);
  }
  auto issue_kv = [&](int tile, int stage) {
    const uint32_t ks = kv_s + stage * 2 * kTileBytes;
    const uint32_t vs = ks + kTileBytes;
    for (int idx = threadIdx.x; idx < 64 * kChunks; idx += 128) {
      const int row = idx / kChunks, chunk = idx % kChunks;
      const int tok = tile * 64 + row;
      const bool valid = tok < len;
      const int tk = valid ? tok : 0;
      int page = bt[tk / p.page_size];
      if (!ZB_BC_OK(page, ZB_BC_PAGES, kKernelPrefill, 10)) page = 0;
      const size_t goff = (static_cast<size_t>(page) * p.page_size + tk % p.page_size) * row_elems +
                          static_cast<size_t>(kvh) * HD + chunk * 8;
      cp_async16(ks + tile_off<HD>(row, chunk), p.k_cache + goff, valid ? 16u : 0u);
      cp_async16(vs + tile_off<HD>(row, chunk), p.v_cache + goff, valid ? 16u : 0u);
    }
  };
  issue_kv(first_tile, 0);
  cp_async_commit();

  uint32_t qf[HD / 16][4];
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  const int g = lane >> 2;
  const int qpos0 = ctx + row_base + warp * 16 + g;   // key position limit of row g (row g+8: +8)

  for (int tile = first_tile; tile < n_tiles; ++tile) {
    const int stage = (tile - first_tile) & 1;
    cp_async_wait<0>();
    __syncthreads();
    if (tile == first_tile) {
      const int mi = lane >> 3, r8 = lane & 7;
#pragma unroll
      for (int kk = 0; kk < HD / 16; ++kk) {
        const int row = warp * 16 + (mi & 1) * 8 + r8;
        ldmatrix_x4(qf[kk], q_s + tile_off<HD>(row, 2 * kk + (mi >> 1)));
      }
    }
    if (tile + 1 < n_tiles) issue_kv(tile + 1, stage ^ 1);
    cp_async_commit();
    const uint32_t ks = kv_s + stage * 2 * kTileBytes;
    const uint32_t vs = ks + kTileBytes;
    // tiles entirely above the diagonal of this warp's rows contribute nothing
    const int warp_max_q = ctx + row_base + warp * 16 + 15;
#pragma unroll
    for (int sub = 0; sub < 4; ++sub) {
      const int key0 = tile * 64 + sub * 16;
      if (key0 > warp_max_q) break;
      attn_block16<HD>(qf, ks, vs, sub * 16, o, m, l, p.scale_log2, [&](int half, int col) {
        const int kidx = key0 + col;
        const int qp = qpos0 + half * 8;
        bool vis = kidx <= qp && kidx < len;
        if (p.window > 0) vis = vis && (kidx > qp - p.window);
        return vis;
      });
    }
  }
  cp_async_wait<0>();

  // write O / l
  const int t = lane & 3;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = warp * 16 + g + half * 8;
    if (row < rows_valid) {
      const float inv = l[half] > 0.f ? 1.f / l[half] : 0.f;
      __nv_bfloat16* orow = p.out + (static_cast<size_t>(tok_base + row) * p.num_q_heads + head) * HD;
#pragma unroll
      for (int nt = 0; nt < HD / 8; ++nt) {
        const uint32_t v = zb_pack_bf16x2(o[nt][half * 2] * inv, o[nt][half * 2 + 1] * inv);
        *reinterpret_cast<uint32_t*>(orow + nt * 8 + 2 * t) = v;
      }
    }
  }
}

template <int HD>
int launch_decode(const AttnParams& p, cudaStream_t stream) {
  constexpr int pipe = 4 * kDecStages * 2 * 16 * HD * 2;
  constexpr int merge = 4 * 16 * HD * 4 + 4 * 16 * 2 * 4;
  constexpr int smem = pipe > merge ? pipe : merge;
  static bool configured[16] = {};
  if (const int rc = zb_config_smem_once(zb_paged_decode_kernel<HD>, smem, configured)) return rc;
  dim3 grid(p.batch * p.num_kv_heads, p.num_splits);
  zb_launch(zb_paged_decode_kernel<HD>, dim3(grid), dim3(128), smem, stream, p);
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

int g_decode_tma = 1;

template <int HD>
int launch_decode_tma(const AttnParams& p, cudaStream_t stream) {
  constexpr int smem = dec_tma_stages<HD>() * 2 * 64 * HD * 2 + 1024 + 256;
  static bool configured[16] = {};
  if (const int rc = zb_config_smem_once(zb_paged_decode_tma_kernel<HD>, smem, configured)) return rc;
  CUtensorMap tk, tv;
  const long long slots = 1ll << 30;      // bound only: pages are addressed through the block table
  int rc = zb_make_tmap_kv_cache(&tk, p.k_cache, slots, p.num_kv_heads, HD, 64);
  if (rc != 0) return rc;
  rc = zb_make_tmap_kv_cache(&tv, p.v_cache, slots, p.num_kv_heads, HD, 64);
  if (rc != 0) return rc;
  dim3 grid(p.batch * p.num_kv_heads, p.num_splits);
  zb_launch(zb_paged_decode_tma_kernel<HD>, dim3(grid), dim3(160), smem, stream, tk, tv, p);
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

template <int HD>
int launch_prefill(const AttnParams& p, int num_q_blocks, cudaStream_t stream) {
  constexpr int smem = 5 * 64 * HD * 2;
  static bool configured[16] = {};
  if (const int rc = zb_config_smem_once(zb_paged_prefill_kernel<HD>, smem, configured)) return rc;
  dim3 grid(num_q_blocks, p.num_q_heads);
  zb_launch(zb_paged_prefill_kernel<HD>, dim3(grid), dim3(128), smem, stream, p);
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

extern "C" {

// Scratch floats needed by a split decode: partial O plus (m, l) pairs.
size_t zb_decode_scratch_bytes(int batch, int num_q_heads, int head_dim, int num_splits) {
  if (num_splits <= 1) return 0;
  return static_cast<size_t>(batch) * num_q_heads * num_splits * (head_dim + 2) * sizeof(float);
}

// Plans the split of the KV range: returns the chunk length in 16-key blocks that minimises the
// modelled time; *max_chunks receives the chunk count of the longest possible sequence (the grid's
// second dimension).
int zb_decode_plan_chunks(int batch, int num_kv_heads, int max_seq_len, int num_sms, int* max_chunks) {
  // Cost model fitted to measurements on B200 (batch 32 x 8 KV heads x 1 344 keys and 128 x 4 x 1 152, 1 to 7
  // chunks): an SM streams K and V at about 45 GB/s whatever the number of resident CTAs (0.0114 us per key of
  // 128-dim bf16 K + V), one CTA alone at about 32 GB/s (0.016 us per key; 16 x 8 x 1 344: 21.7 us), a CTA of a
  // split sequence pays about 2.5 us more (partial write, fence, ticket) and the merge about 3 us once.
  // Splitting therefore only pays when there are too few (sequence, KV head) pairs to occupy the SMs.
  const long long base = static_cast<long long>(batch) * num_kv_heads;
  const double us_per_key = 0.0114, us_per_key_one_cta = 0.016, cta_fixed_us = 2.5, merge_us = 3.0;
  int best_mc = 1, best_keys = (max_seq_len + 63) / 64 * 64;
  double best_t = 1e30;
  for (int mc = 1; mc <= 64; ++mc) {
    int keys = (max_seq_len + mc - 1) / mc;
    keys = (keys + 63) / 64 * 64;                       // whole 64-key pages per chunk
    if (mc > 1 && keys < 128) break;
    const int real_mc = (max_seq_len + keys - 1) / keys;
    if (real_mc < mc) continue;                         // same plan as a smaller mc
    const long long per_sm = (base * real_mc + num_sms - 1) / num_sms;
    const double stream = per_sm * keys * us_per_key > keys * us_per_key_one_cta ? per_sm * keys * us_per_key : keys * us_per_key_one_cta;
    const double t = stream + (real_mc > 1 ? per_sm * cta_fixed_us + merge_us : 0.0);
    if (t < best_t - 1e-9) {
      best_t = t;
      best_mc = real_mc;
      best_keys = keys;
    }
  }
  if (max_chunks) *max_chunks = best_mc;
  return best_keys / 16;
}

// kept for callers that think in splits: number of chunks the plan uses for max_seq_len
int zb_decode_plan_splits(int batch, int num_kv_heads, int max_seq_len, int num_sms) {
  int mc = 1;
  zb_decode_plan_chunks(batch, num_kv_heads, max_seq_len, num_sms, &mc);
  return mc;
}

// Tensor-map fed decode kernel on (default) / off.
void zb_set_decode_tma(int on) { g_decode_tma = on ? 1 : 0; }

int zb_paged_decode_ex(const void* q, const void* k_cache, const void* v_cache, void* out,
                       const int32_t* block_table, const int32_t* seq_lens, int batch,
                       int num_q_heads, int num_kv_heads, int head_dim, int page_size, int max_pages,
                       long long q_stride, float scale, int window, int num_splits, float* scratch,
                       size_t scratch_bytes, uint32_t* counters, int counters_len, ZbStatus* status,
                       cudaStream_t stream) {
  if (batch <= 0) return 0;
  if (num_q_heads % num_kv_heads != 0 || num_q_heads / num_kv_heads > 16) return -30;
  if (page_size % 16 != 0) return -31;
  if (num_splits < 1) num_splits = 1;
  if (num_splits > 64) num_splits = 64;      // the in-kernel merge keeps per-chunk statistics for 64 chunks
  if (batch * num_kv_heads > counters_len) return -33;
  while (num_splits > 1 &&
         zb_decode_scratch_bytes(batch, num_q_heads, head_dim, num_splits) > scratch_bytes)
    --num_splits;
  // chunk length that lets `num_splits` chunks cover the longest sequence the block table allows
  const int max_blocks = (max_pages * page_size + 15) / 16;
  int chunk_blocks = (max_blocks + num_splits - 1) / num_splits;
  if (page_size == 64) chunk_blocks = (chunk_blocks + 3) / 4 * 4;      // whole pages per chunk (tensor-map fed kernel)
  AttnParams p = {};
  p.q = reinterpret_cast<const __nv_bfloat16*>(q);
  p.k_cache = reinterpret_cast<const __nv_bfloat16*>(k_cache);
  p.v_cache = reinterpret_cast<const __nv_bfloat16*>(v_cache);
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.block_table = block_table;
  p.seq_lens = seq_lens;
  p.q_start = nullptr;
  p.part_o = scratch;
  p.part_ml = scratch ? scratch + static_cast<size_t>(batch) * num_q_heads * num_splits * head_dim
                      : nullptr;
  p.q_stride = q_stride;
  p.batch = batch;
  p.num_q_heads = num_q_heads;
  p.num_kv_heads = num_kv_heads;
  p.page_size = page_size;
  p.max_pages = max_pages;
  p.num_splits = num_splits;
  p.chunk_blocks = chunk_blocks < 1 ? 1 : chunk_blocks;
  p.counters = counters;
  p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  // 64-token pages and chunks of whole pages: the tensor-map fed kernel; otherwise per-warp cp.async
  const bool tma = g_decode_tma != 0 && page_size == 64 && (p.chunk_blocks % 4) == 0 &&
                   (reinterpret_cast<uintptr_t>(k_cache) & 15) == 0 && (reinterpret_cast<uintptr_t>(v_cache) & 15) == 0;
  switch (head_dim) {
    case 64: return tma ? launch_decode_tma<64>(p, stream) : launch_decode<64>(p, stream);
    case 128: return tma ? launch_decode_tma<128>(p, stream) : launch_decode<128>(p, stream);
    case 256: return tma ? launch_decode_tma<256>(p, stream) : launch_decode<256>(p, stream);
  }
  return -32;
}

int zb_paged_decode(const void* q, const void* k_cache, const void* v_cache, void* out,
                    const int32_t* block_table, const int32_t* seq_lens, int batch, int num_q_heads,
                    int num_kv_heads, int head_dim, int page_size, int max_pages,
                    long long q_stride, float scale, int window, int num_splits, void* stream) {
  ZbDeviceState* st = zb_device_state();
  if (!st) return -20;
  return zb_paged_decode_ex(q, k_cache, v_cache, out, block_table, seq_lens, batch, num_q_heads,
                            num_kv_heads, head_dim, page_size, max_pages, q_stride, scale, window,
                            num_splits, st->attn_scratch, st->attn_scratch_bytes, st->attn_counters,
                            st->attn_counters_len, st->status, reinterpret_cast<cudaStream_t>(stream));
}

// total_q_blocks >= sum over sequences of ceil(q_len / 64); a safe bound is
// total_tokens / 64 + batch.
int zb_paged_prefill(const void* q, const void* k_cache, const void* v_cache, void* out,
                     const int32_t* block_table, const int32_t* seq_lens, const int32_t* q_start,
                     int batch, int total_q_blocks, int num_q_heads, int num_kv_heads, int head_dim,
                     int page_size, int max_pages, long long q_stride, float scale, int window,
                     void* stream) {
  if (batch <= 0 || total_q_blocks <= 0) return 0;
  if (num_q_heads % num_kv_heads != 0) return -30;
  ZbDeviceState* st = zb_device_state();
  if (!st) return -20;
  AttnParams p = {};
  p.q = reinterpret_cast<const __nv_bfloat16*>(q);
  p.k_cache = reinterpret_cast<const __nv_bfloat16*>(k_cache);
  p.v_cache = reinterpret_cast<const __nv_bfloat16*>(v_cache);
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.block_table = block_table;
  p.seq_lens = seq_lens;
  p.q_start = q_start;
  p.q_stride = q_stride;
  p.batch = batch;
  p.num_q_heads = num_q_heads;
  p.num_kv_heads = num_kv_heads;
  p.page_size = page_size;
  p.max_pages = max_pages;
  p.num_splits = 1;
  p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = st->status;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (head_dim) {
    case 64: return launch_prefill<64>(p, total_q_blocks, s);
    case 128: return launch_prefill<128>(p, total_q_blocks, s);
    case 256: return launch_prefill<256>(p, total_q_blocks, s);
  }
  return -32;
}

}  // extern "C"
