// bf16 GEMM for sm_100a: out[M,N] = A[M,K] * W[N,K]^T (+ bias[N]) (+ residual[M,N]).
//
// Replaces the `dot_general` -> cuBLASLt / Triton-gemm path of the reference
// (zml/tensor.zig:1388-1459, nn.Linear zml/nn.zig:18-91) with one persistent,
// warp-specialised kernel:
//   warp 0  : TMA producer  (cp.async.bulk.tensor, 128-byte swizzle, no multicast)
//   warp 1  : MMA issuer    (tcgen05.mma kind::f16, fp32 accumulators in TMEM,
//                            two accumulator stages so the epilogue overlaps the
//                            next tile's main loop)
//   warps 2-5: epilogue     (tcgen05.ld -> bias/residual -> bf16/f32 stores)
//
// Both operands are K-major, so either can feed the 128-row "M" side of the MMA.
// For few tokens (decode) the weight rows take the 128-row side and the tokens
// the N side ("swap-AB").
//
// Work is distributed stream-K style: the (output tile, k-block) space is cut into
// one contiguous, equally sized range per CTA, so every SM streams the same number
// of operand bytes whatever the tile count (no wave quantisation).  A CTA whose
// range covers only part of a tile's K extent writes an fp32 partial tile to scratch
// (at most two per CTA); the last CTA to arrive for a tile sums the pieces in CTA
// order (deterministic) and runs the epilogue.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include <type_traits>

#include "common.cuh"
#include "host_api.h"

#include "fused_ar.h"

namespace {

constexpr int kBlockP = 128;   // rows of the MMA-M operand per tile
constexpr int kBlockK = 64;    // 64 bf16 = 128 bytes = one swizzle row
constexpr int kUmmaK = 16;
constexpr int kNumThreads = 192;
constexpr int kEpiThreads = 128;
constexpr uint32_t kKernelId = 1;
constexpr uint32_t kKernelIdFused = 4;

struct GemmParams {
  int rows_p;        // extent of the P operand (MMA M side)
  int rows_q;        // extent of the Q operand (MMA N side)
  int k;
  int ldo;           // leading dimension of out / residual, in elements
  void* out;
  const __nv_bfloat16* residual;   // same layout as out, may be null
  const __nv_bfloat16* bias;       // indexed by output column, may be null
  int out_f32;       // 0: bf16 output, 1: fp32 output
  int units_per_cta; // k-blocks per CTA (stream-K range length)
  int rr_tiles;      // > 0: whole tiles dealt round-robin, this many per CTA (large problems)
  int group_p;       // rasterisation group height (P tiles)
  int flags;         // bit 0: the weight operand is not written by the preceding kernel
  int l2_prefetch;   // weight tiles per CTA to pull into L2 ahead of the shared-memory ring
  int cluster;       // > 1: the CTAs of a cluster split one tile along K and reduce it through shared memory
  unsigned long long* timeline;   // optional [grid][8] globaltimer stamps of this launch's phases (profiling)
  float* workspace;  // [grid][2][BN][128] fp32 partial tiles
  uint32_t* counters;  // one per output tile, zero between launches
  ZbStatus* status;
  ZbGemmEpi epi;       // row scale / SwiGLU / sum-of-squares / next-weight prefetch (host_api.h)
  ZbBandPipe band;     // prefill collectives overlapped band by band (host_api.h)
  ZbFusedAr ar;        // used by the fused GEMM + all-reduce variant only
};

// Pipeline depth: as many stages as fit beside the barriers in one CTA's shared memory.  (Sizing the
// weight-streaming configurations for two CTAs per SM, so that the next GEMM of the stream could
// run under this one's tail, measured slower: 127 vs 121 us per decoder layer on the 8B shapes.)
__host__ __device__ constexpr int stages_for(int bn, bool swap) {
  (void)swap;
  return bn >= 256 ? 4 : (bn >= 128 ? 6 : 8);
}
__host__ __device__ constexpr int stage_bytes(int bn) { return (kBlockP + bn) * kBlockK * 2; }
// Dynamic shared memory of one CTA: the operand ring, 1 KB of alignment slack, 256 bytes of barriers and
// flags, and a table of 256 per-token scales (row scale of the epilogue, swap-AB only).
constexpr int kTailBytes = 256;
constexpr int kScaleTabBytes = 256 * 4;
__host__ __device__ constexpr int smem_bytes_for(int bn, bool swap) {
  return stages_for(bn, swap) * stage_bytes(bn) + 1024 + kTailBytes + kScaleTabBytes;
}

ZB_DEVICE void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
ZB_DEVICE float silu_f(float g) { return g / (1.f + __expf(-g)); }

// MODE 0: the GEMM and its epilogue options; 1: fused with the tensor-parallel all-reduce (fused_ar.h);
// 2: one side of the band pipeline of the prefill collectives (ZbBandPipe; tokens as rows only).  The modes are
// separate instantiations so that the weight-streaming decode kernels do not carry the other modes' code.
// EPI 0 would compile the epilogue options of ZbGemmEpi out, PLAN 0 / 1 only the code of the plans without / with
// cluster split-K.  The library instantiates EPI 1, PLAN 2 (everything) only: with one instantiation per option
// set the four GEMMs of a decoder layer alternate between kernels and a layer measured 9 us slower (157.7 vs
// 148.6 us on Llama-3.1-8B, one GPU) than with one kernel that stays in the instruction cache.
template <int BN, bool SWAP, int MODE, int EPI, int PLAN>
__global__ void __launch_bounds__(kNumThreads, 1)
zb_gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_p,
                    const __grid_constant__ CUtensorMap tmap_q, const GemmParams prm) {
  constexpr bool FUSED = MODE == 1;
  constexpr bool BAND = MODE == 2 && !SWAP;
  constexpr bool kEpi = EPI != 0;
  constexpr bool kCluster = PLAN != 0;      // cluster split-K code present
  constexpr bool kGeneric = PLAN != 1;      // whole-tile / stream-K code present
  const float* const epi_in_sumsq = kEpi ? prm.epi.in_sumsq : nullptr;
  float* const epi_out_sumsq = kEpi ? prm.epi.out_sumsq : nullptr;
  const int epi_swiglu = kEpi ? prm.epi.swiglu : 0;
  const unsigned long long epi_pf_bytes = kEpi ? prm.epi.pf_bytes : 0ull;
  constexpr int kStages = stages_for(BN, SWAP);
  constexpr int kStageBytes = stage_bytes(BN);
  constexpr int kTileABytes = kBlockP * kBlockK * 2;
  constexpr uint32_t kTmemCols = (2 * BN) < 32 ? 32 : (2 * BN);
  constexpr uint32_t kIdesc = zb_make_idesc_bf16(kBlockP, BN);

  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: required by the 128-byte swizzle atoms.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full = empty_bar + kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile uint32_t* abort_flag = tmem_holder + 1;
  volatile uint32_t* is_last_flag = tmem_holder + 2;
  volatile uint32_t* abort_where = tmem_holder + 3;
  float* scale_tab = reinterpret_cast<float*>(smem + kStages * kStageBytes + kTailBytes);   // [256], swap-AB only

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int num_p = (prm.rows_p + kBlockP - 1) / kBlockP;
  const int num_q = (prm.rows_q + BN - 1) / BN;
  const int kb_total = (prm.k + kBlockK - 1) / kBlockK;
  const int num_out_tiles = num_p * num_q;
  // Large problems: whole tiles are dealt round-robin (CTAs running at the same time work on
  // neighbouring tiles and share operands in L2); a CTA's "virtual" tiles are then contiguous
  // and map to actual tile (v % rr_tiles) * grid + cta.  Small problems: stream-K ranges.
  // band pipeline, consumer side: the first comm_ctas CTAs reduce and broadcast, the rest share the tiles
  const int cta_off = (BAND && prm.band.mode == 2) ? prm.band.comm_ctas : 0;
  const int cta_id = static_cast<int>(blockIdx.x) - cta_off;
  const int n_ctas = static_cast<int>(gridDim.x) - cta_off;
  const bool comm_cta = BAND && cta_id < 0;
  const long long total_units =
      comm_cta ? 0 : static_cast<long long>(prm.rr_tiles > 0 ? n_ctas * prm.rr_tiles : num_out_tiles) * kb_total;
  long long u_begin = min(total_units, static_cast<long long>(comm_cta ? 0 : cta_id) * prm.units_per_cta);
  long long u_end = min(total_units, u_begin + prm.units_per_cta);
  if (prm.cluster > 1) {
    // cluster split-K: CTA (tile, rank) takes k-blocks [rank * upc, (rank + 1) * upc) of its tile
    const long long tile = blockIdx.x / prm.cluster;
    const int rank = static_cast<int>(blockIdx.x % prm.cluster);
    u_begin = tile * kb_total + min(kb_total, rank * prm.units_per_cta);
    u_end = tile * kb_total + min(kb_total, (rank + 1) * prm.units_per_cta);
  }

  // output tile -> (p tile, q tile); P tiles are grouped so that CTAs working at the
  // same time share few distinct operand tiles in L2.
  auto decode = [&](int t, int& pt, int& qt) {
    const int per_group = prm.group_p * num_q;
    const int g = t / per_group;
    const int within = t - g * per_group;
    const int p_first = g * prm.group_p;
    const int gp = min(prm.group_p, num_p - p_first);
    pt = p_first + within % gp;
    qt = within / gp;
  };

  unsigned long long* tl = prm.timeline != nullptr ? prm.timeline + static_cast<size_t>(blockIdx.x) * 12 : nullptr;
  int early = 0;     // producer thread: stages whose weight tile was requested ahead of the dependency wait
  if (threadIdx.x == 0) {
    if (tl) tl[0] = zb_globaltimer();
    for (int s = 0; s < kStages; ++s) {
      zb_mbar_init(&full_bar[s], 1);
      zb_mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      zb_mbar_init(&tmem_full[a], 1);
      zb_mbar_init(&tmem_empty[a], kEpiThreads);
    }
    *abort_flag = 0u;
    *is_last_flag = 0u;
    *abort_where = 0u;
    zb_mbar_fence_init();
    zb_tma_prefetch_desc(&tmap_p);
    zb_tma_prefetch_desc(&tmap_q);
    if ((prm.flags & 1) != 0) {
      // The weight operand (P when swapped, Q otherwise) is a parameter, so its first tiles are
      // requested right away - before this CTA's tensor memory is allocated and before the
      // preceding kernel of the stream has finished: a ring of tiles into shared memory, then
      // `l2_prefetch` further tiles into L2.  The activation tiles follow after the dependency wait.
      uint32_t stage = 0;
      int issued = 0;
      const int limit = kStages + prm.l2_prefetch;
      for (long long u = u_begin; issued < limit && u < u_end;) {
        const int v = static_cast<int>(u / kb_total);
        const int kb0 = static_cast<int>(u - static_cast<long long>(v) * kb_total);
        const int kb1 = static_cast<int>(min(static_cast<long long>(kb_total), kb0 + (u_end - u)));
        const int t = prm.rr_tiles > 0 ? (v % prm.rr_tiles) * n_ctas + v / prm.rr_tiles : v;
        u += kb1 - kb0;
        if (t >= num_out_tiles) continue;
        int pt, qt;
        decode(t, pt, qt);
        for (int kb = kb0; kb < kb1 && issued < limit; ++kb, ++issued) {
          const void* wmap = SWAP ? static_cast<const void*>(&tmap_p) : static_cast<const void*>(&tmap_q);
          const int wy = SWAP ? pt * kBlockP : qt * BN;
          if (issued < kStages) {
            uint8_t* dst = smem + stage * kStageBytes + (SWAP ? 0 : kTileABytes);
            zb_mbar_expect_tx(&full_bar[stage], kStageBytes);
            zb_tma_load_2d(dst, wmap, &full_bar[stage], kb * kBlockK, wy);
            ++stage;
            ++early;
          } else {
            zb_tma_prefetch_l2_2d(wmap, kb * kBlockK, wy);
          }
        }
      }
    }
  }
  if (warp == 1) {
    zb_tmem_alloc(tmem_holder, kTmemCols);
    zb_tmem_relinquish();
  }
  zb_tc_fence_before();
  __syncthreads();
  zb_tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  // Everything above touches only parameters and this CTA's shared and tensor memory.  The next
  // kernel may start now that this CTA holds its tensor memory (a dependent CTA sharing the SM
  // that allocated first would block this one for good).  The producer thread waits for the
  // preceding kernel before its first activation load; the epilogue warps, which read the
  // residual and write the output, wait here.
  zb_pdl_launch();
  if (tl && threadIdx.x == 0) tl[1] = zb_globaltimer();
  if (warp >= 2) {
    zb_pdl_wait();
    if constexpr (SWAP) {
      // per-token scale of the accumulators (tokens are the tile's columns; a swap-AB problem has one column
      // tile): computed here, while the main loop runs, from the partial sums the producing kernel left
      if (epi_in_sumsq != nullptr) {
        // kEpiThreads / BN threads share a token (one thread takes 128 / ... tokens when BN > 128); a thread sums
        // every TPT-th part with 8 loads in flight, the TPT sums of a token are added in a fixed order
        constexpr int TPT = BN >= kEpiThreads ? 1 : kEpiThreads / BN;      // threads per token
        float* part_sums = scale_tab + 128;                                 // [TPT][BN] = 128 floats, used when BN < 128
        const int et = threadIdx.x - 64;
        for (int t0 = 0; t0 < BN; t0 += kEpiThreads) {
          const int t = t0 + (et % (BN < kEpiThreads ? BN : kEpiThreads));
          const int sub = BN < kEpiThreads ? et / BN : 0;
          float acc = 0.f;
          if (t < prm.rows_q) {
            const float* src = epi_in_sumsq + t;
            int i = sub;
            for (; i + 7 * TPT < prm.epi.in_parts; i += 8 * TPT) {
              float v[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = __ldcg(src + static_cast<size_t>(i + j * TPT) * prm.epi.in_ld);
#pragma unroll
              for (int j = 0; j < 8; ++j) acc += v[j];
            }
            for (; i < prm.epi.in_parts; i += TPT) acc += __ldcg(src + static_cast<size_t>(i) * prm.epi.in_ld);
          }
          if constexpr (TPT == 1) {
            scale_tab[t] = rsqrtf(acc * prm.epi.in_inv_d + prm.epi.in_eps);
          } else {
            part_sums[sub * BN + t] = acc;
            epi_bar_sync();
            if (et < BN) {
              float tot = 0.f;
#pragma unroll
              for (int j = 0; j < TPT; ++j) tot += part_sums[j * BN + et];
              scale_tab[et] = rsqrtf(tot * prm.epi.in_inv_d + prm.epi.in_eps);
            }
          }
        }
        epi_bar_sync();
      }
    }
  }

  if (comm_cta) {
    // ------------------------------------------ band pipeline: reduce + broadcast CTA (no tensor-core work)
    // Every band this rank owns: wait for the partial sums of all ranks, pull them chunk by chunk from every
    // rank's heap into this CTA's (otherwise idle) operand ring with bulk copies, add them up in rank order with
    // the residual, push the result to every rank with bulk copies and the row statistics with plain stores,
    // then tell every rank that the band is done.  A row of the band belongs to one comm CTA.
    zb_pdl_wait();
    const ZbBandPipe& bp = prm.band;
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(bp.epoch);
    const int W = bp.world;
    const int row_bytes = bp.d * 2;
    const int n_src = W + (bp.residual != nullptr ? 1 : 0);
    // A stage holds n_src source chunks and one output chunk; a chunk is a row or a power-of-two fraction of it.
    // The copies of n_stage - 1 stages are in flight while one is summed: pick the split of the idle operand ring
    // (up to 2 * kStages stages: the ring's full and empty barriers are one array) that keeps most bytes in flight -
    // a peer copy takes microseconds to come back, so bytes in flight are throughput.
    int chunk = row_bytes, n_stage = 0;
    {
      long long best = -1;
      for (int c = row_bytes; c >= 1024 && (c % 16) == 0; c >>= 1) {
        int ns = (kStages * kStageBytes) / ((n_src + 1) * c);
        ns = ns > 2 * kStages ? 2 * kStages : ns;
        const long long inflight = static_cast<long long>(ns - 1) * n_src * c;
        if (ns >= 2 && inflight > best) {
          best = inflight;
          chunk = c;
          n_stage = ns;
        }
        if ((c & 1) != 0) break;
      }
    }
    const int chunks_per_row = row_bytes / chunk;
    const int stage_sz = (n_src + 1) * chunk;
    uint64_t* cbar = full_bar;                       // full_bar[kStages] and empty_bar[kStages] are contiguous (count 1 each)
    float* red = scale_tab;                          // per-warp partial sums of a row
    const int vec_per_chunk = chunk >> 4;
    bool ok = n_stage >= 2;
    if (!ok && threadIdx.x == 0) {
      *abort_flag = 1u;
      *abort_where = 350u;
    }
    uint32_t use = 0;                                // chunks this CTA has pushed through the ring (all bands)
    for (int b = bp.rank; ok && b < bp.num_bands; b += W) {
      if (static_cast<int>(threadIdx.x) < W) {
        if (!zb_wait_flag(bp.ready_peer[bp.rank] + static_cast<size_t>(b) * 8 + threadIdx.x, epoch, abort_flag))
          *abort_where = 300u + threadIdx.x;
      }
      __syncthreads();
      if (*abort_flag != 0u) break;
      const int row0 = b * kBlockP;
      const int rows = min(kBlockP, bp.tokens - row0);
      const int my_rows = rows > static_cast<int>(blockIdx.x) ? (rows - 1 - static_cast<int>(blockIdx.x)) / bp.comm_ctas + 1 : 0;
      const int n_units = my_rows * chunks_per_row;
      auto unit_off = [&](int u) {                   // byte offset of unit u inside the [tokens, d] tensors
        const int r = row0 + static_cast<int>(blockIdx.x) + (u / chunks_per_row) * bp.comm_ctas;
        return static_cast<size_t>(r) * row_bytes + static_cast<size_t>(u % chunks_per_row) * chunk;
      };
      auto issue = [&](int u) {                      // thread 0: the copies of unit u into its stage
        const uint32_t st = (use + u) % n_stage;
        uint8_t* base = smem + st * stage_sz;
        const size_t off = unit_off(u);
        zb_mbar_expect_tx(&cbar[st], static_cast<uint32_t>(n_src * chunk));
        for (int r = 0; r < W; ++r) zb_bulk_load(base + r * chunk, bp.heap[r] + bp.part_off + off, chunk, &cbar[st]);
        if (bp.residual != nullptr)
          zb_bulk_load(base + W * chunk, reinterpret_cast<const char*>(bp.residual) + off, chunk, &cbar[st]);
      };
      if (threadIdx.x == 0) {
        for (int u = 0; u < n_stage - 1 && u < n_units; ++u) issue(u);
      }
      float ss = 0.f;
      for (int u = 0; u < n_units && ok; ++u) {
        const uint32_t g = use + u;
        const uint32_t st = g % n_stage;
        uint8_t* base = smem + st * stage_sz;
        if (threadIdx.x == 0) {
          // the stage refilled now was computed on one iteration ago (everybody passed that iteration's barrier); the
          // output chunk written below was last pushed n_stage iterations ago: that push must have read it
          if (u + n_stage - 1 < n_units) issue(u + n_stage - 1);
          // at most n_stage - 1 pushes may still be reading their output chunk
          switch (n_stage) {
            case 2: zb_bulk_wait_read<1>(); break;
            case 3: zb_bulk_wait_read<2>(); break;
            case 4: zb_bulk_wait_read<3>(); break;
            case 5: zb_bulk_wait_read<4>(); break;
            case 6: zb_bulk_wait_read<5>(); break;
            case 7: zb_bulk_wait_read<6>(); break;
            default: zb_bulk_wait_read<7>(); break;
          }
        }
        if (!zb_mbar_wait(&cbar[st], (g / n_stage) & 1u, abort_flag)) {
          *abort_where = 360u;
          ok = false;
        }
        __syncthreads();                             // stage complete for everybody; thread 0's wait_read done
        if (*abort_flag != 0u) {
          ok = false;
          break;
        }
        uint4* outc = reinterpret_cast<uint4*>(base + n_src * chunk);
        for (int v = threadIdx.x; v < vec_per_chunk; v += kNumThreads) {
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          for (int r = 0; r < n_src; ++r) {          // ranks in ascending order, then the residual
            const uint4 x = reinterpret_cast<const uint4*>(base + r * chunk)[v];
            const uint32_t w4[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float2 f = zb_unpack_bf16x2(w4[q]);
              acc[2 * q] += f.x;
              acc[2 * q + 1] += f.y;
            }
          }
          uint32_t o[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            o[q] = zb_pack_bf16x2(acc[2 * q], acc[2 * q + 1]);
            const float2 fo = zb_unpack_bf16x2(o[q]);           // statistics of what is stored
            ss += fo.x * fo.x + fo.y * fo.y;
          }
          outc[v] = make_uint4(o[0], o[1], o[2], o[3]);
        }
        zb_fence_proxy_async_smem();
        const bool row_end = (u % chunks_per_row) == chunks_per_row - 1;
        if (row_end) {
          const float ws = zb_warp_sum(ss);
          if (lane == 0) red[warp] = ws;
          ss = 0.f;
        }
        __syncthreads();                             // output chunk (and the row's partial sums) written
        if (threadIdx.x == 0) {
          const size_t off = unit_off(u);
          for (int r = 0; r < W; ++r) zb_bulk_store(bp.heap[r] + bp.x_off + off, outc, chunk);
          zb_bulk_commit();
        }
        if (row_end && static_cast<int>(threadIdx.x) < W) {
          float tot = 0.f;
#pragma unroll
          for (int i = 0; i < kNumThreads / 32; ++i) tot += red[i];
          const int r = row0 + static_cast<int>(blockIdx.x) + (u / chunks_per_row) * bp.comm_ctas;
          bp.sumsq_peer[threadIdx.x][r] = tot;
        }
      }
      use += static_cast<uint32_t>(n_units);
      if (threadIdx.x == 0) zb_bulk_wait<0>();       // every push of this band is in the peers' memory
      __syncthreads();
      if (threadIdx.x == 0) {
        __threadfence_system();
        const uint32_t prev = atomicAdd(&bp.count_c[b], 1u);
        if (prev == static_cast<uint32_t>(bp.comm_ctas - 1)) {
          bp.count_c[b] = 0u;
          __threadfence_system();
          for (int r = 0; r < W; ++r) zb_st_release_sys(bp.done_peer[r] + b, epoch);
        }
      }
    }
    if (threadIdx.x == 0) zb_bulk_wait<0>();
  } else if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      zb_tma_prefetch_desc(&tmap_p);
      zb_tma_prefetch_desc(&tmap_q);
      zb_pdl_wait();
      if (tl) tl[2] = zb_globaltimer();
      const uint32_t band_epoch = (BAND && prm.band.mode == 2) ? *reinterpret_cast<volatile uint32_t*>(prm.band.epoch) : 0u;
      int band_seen = -1;                     // band pipeline: last band whose done flag this producer has seen
      uint32_t stage = 0, phase = 0;
      int issued = 0;
      bool ok = true;
      for (long long u = u_begin; ok && u < u_end;) {
        const int v = static_cast<int>(u / kb_total);
        const int kb0 = static_cast<int>(u - static_cast<long long>(v) * kb_total);
        const int kb1 = static_cast<int>(min(static_cast<long long>(kb_total), kb0 + (u_end - u)));
        const int t = prm.rr_tiles > 0 ? (v % prm.rr_tiles) * n_ctas + v / prm.rr_tiles : v;
        if (t >= num_out_tiles) {
          u += kb1 - kb0;
          continue;
        }
        int pt, qt;
        decode(t, pt, qt);
        if constexpr (BAND) {
          if (prm.band.mode == 2 && pt != band_seen) {
            // the rows of this tile are band `pt` of the reduced activation: wait until its owner has written it here
            if (!zb_wait_flag(prm.band.done_peer[prm.band.rank] + pt, band_epoch, abort_flag)) {
              *abort_where = 400u;
              ok = false;
              break;
            }
            asm volatile("fence.proxy.async;" ::: "memory");      // the copies below go through the async proxy
            band_seen = pt;
          }
        }
        for (int kb = kb0; kb < kb1; ++kb, ++issued) {
          uint8_t* sa = smem + stage * kStageBytes;
          uint8_t* sb = sa + kTileABytes;
          if (issued < early) {
            // the weight tile of this stage is already in flight: add the activation tile
            if constexpr (SWAP) zb_tma_load_2d(sb, &tmap_q, &full_bar[stage], kb * kBlockK, qt * BN);
            else zb_tma_load_2d(sa, &tmap_p, &full_bar[stage], kb * kBlockK, pt * kBlockP);
          } else {
            if (!zb_mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) {
              ok = false;
              break;
            }
            zb_mbar_expect_tx(&full_bar[stage], kStageBytes);
            zb_tma_load_2d(sa, &tmap_p, &full_bar[stage], kb * kBlockK, pt * kBlockP);
            zb_tma_load_2d(sb, &tmap_q, &full_bar[stage], kb * kBlockK, qt * BN);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        u += kb1 - kb0;
      }
      if (epi_pf_bytes != 0ull) {
        // this CTA's share of the next GEMM's weights goes to L2 while the epilogue (and, in the tensor-parallel
        // variant, the exchange with the peers) runs: HBM is otherwise idle from here on
        constexpr unsigned long long kChunk = 16384ull;
        const unsigned long long nchunks = (epi_pf_bytes + kChunk - 1) / kChunk;
        for (unsigned long long c = blockIdx.x; c < nchunks; c += gridDim.x) {
          const unsigned long long off = c * kChunk;
          const uint32_t sz = static_cast<uint32_t>(min(kChunk, epi_pf_bytes - off)) & ~15u;
          if (sz != 0u)
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(static_cast<const char*>(prm.epi.pf_ptr) + off), "r"(sz)
                         : "memory");
        }
      }
    }
    if (prm.cluster > 1) {
      // the cluster barriers of the epilogue count every thread of every CTA
      __syncwarp();
      zb_cluster_arrive();
      zb_cluster_wait();
      zb_cluster_arrive();
      zb_cluster_wait();
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      uint32_t acc = 0, acc_phase = 0;
      bool ok = true;
      for (long long u = u_begin; ok && u < u_end;) {
        const int v = static_cast<int>(u / kb_total);
        const int kb0 = static_cast<int>(u - static_cast<long long>(v) * kb_total);
        const int kb1 = static_cast<int>(min(static_cast<long long>(kb_total), kb0 + (u_end - u)));
        u += kb1 - kb0;
        if (prm.rr_tiles > 0 && (v % prm.rr_tiles) * n_ctas + v / prm.rr_tiles >= num_out_tiles) continue;
        if (!zb_mbar_wait(&tmem_empty[acc], acc_phase ^ 1u, abort_flag)) break;
        zb_tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!zb_mbar_wait(&full_bar[stage], phase, abort_flag)) {
            ok = false;
            break;
          }
          if (tl && tl[3] == 0ull) tl[3] = zb_globaltimer();
          zb_tc_fence_after();
          const uint32_t sa = zb_smem_u32(smem + stage * kStageBytes);
          const uint32_t sb = sa + kTileABytes;
          const uint64_t da = zb_make_desc_sw128(sa);
          const uint64_t db = zb_make_desc_sw128(sb);
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            // advance 32 bytes (16 bf16) along K inside the swizzle row: +2 in 16-byte units
            zb_umma_f16(tmem_d, da + 2 * k, db + 2 * k, kIdesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          zb_umma_commit(&empty_bar[stage]);   // frees the smem stage when the MMAs retire
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        zb_umma_commit(&tmem_full[acc]);       // accumulator complete
        if (tl) tl[4] = zb_globaltimer();
        acc ^= 1u;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
    if (prm.cluster > 1) {
      // the cluster barriers of the epilogue count every thread of every CTA
      __syncwarp();
      zb_cluster_arrive();
      zb_cluster_wait();
      zb_cluster_arrive();
      zb_cluster_wait();
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int epi_tid = threadIdx.x - 64;          // 0..127
    const int quad = warp & 3;                     // TMEM lane quadrant of this warp
    const int row_in_tile = quad * 32 + lane;      // MMA-M row held by this thread
    uint32_t acc = 0, acc_phase = 0;
    bool did_cluster_sync = false;
    uint32_t epoch = 0;
    if constexpr (FUSED) epoch = *reinterpret_cast<volatile uint32_t*>(prm.ar.epoch);
    for (long long u = u_begin; u < u_end;) {
      const int v = static_cast<int>(u / kb_total);
      const int kb0 = static_cast<int>(u - static_cast<long long>(v) * kb_total);
      const int kb1 = static_cast<int>(min(static_cast<long long>(kb_total), kb0 + (u_end - u)));
      const bool partial = !(kb0 == 0 && kb1 == kb_total);
      const int my_slot = (u == u_begin) ? 0 : 1;
      u += kb1 - kb0;
      const int t = prm.rr_tiles > 0 ? (v % prm.rr_tiles) * n_ctas + v / prm.rr_tiles : v;
      if (t >= num_out_tiles) continue;
      int pt, qt;
      decode(t, pt, qt);
      // CTAs that hold a piece of this tile: [first_cta, last_cta]
      const long long t_begin = static_cast<long long>(t) * kb_total;
      const int first_cta = static_cast<int>(t_begin / prm.units_per_cta);
      const int last_cta = static_cast<int>((t_begin + kb_total - 1) / prm.units_per_cta);
      float row_scale = 1.f;       // !SWAP: tokens are the tile's rows, this thread owns one
      auto load_row_scale = [&]() {
        const int pr = min(pt * kBlockP + row_in_tile, prm.rows_p - 1);
        float ssum = 0.f;
        for (int i = 0; i < prm.epi.in_parts; ++i) ssum += __ldcg(epi_in_sumsq + static_cast<size_t>(i) * prm.epi.in_ld + pr);
        row_scale = rsqrtf(ssum * prm.epi.in_inv_d + prm.epi.in_eps);
      };
      if constexpr (!SWAP) {
        // ahead of the wait for the accumulator, unless the statistics arrive with the band (band pipeline)
        if (epi_in_sumsq != nullptr && !(BAND && prm.band.mode == 2)) load_row_scale();
      }
      zb_mbar_wait(&tmem_full[acc], acc_phase, abort_flag);
      if constexpr (BAND) {
        if (epi_in_sumsq != nullptr && prm.band.mode == 2) {
          // the band's rows were loaded, so its done flag is set: acquire it, then read the statistics its owner wrote
          (void)zb_ld_acquire_sys(prm.band.done_peer[prm.band.rank] + pt);
          load_row_scale();
        }
      }
      if (tl && epi_tid == 0 && tl[5] == 0ull) tl[5] = zb_globaltimer();
      epi_bar_sync();
      if (*abort_flag != 0u) break;
      zb_tc_fence_after();
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quad * 32) << 16);
      const int p = pt * kBlockP + row_in_tile;
      const int q0 = qt * BN;
      const int out_tile = pt * num_q + qt;

      if constexpr (kCluster && SWAP && (BN <= 64 || (!FUSED && BN <= 128))) {
        if (prm.cluster > 1) {
          // Cluster split-K: every CTA of the cluster holds a partial of the same tile.  Partials go
          // to the CTA's own shared memory (the operand ring is idle: this CTA has no other tile),
          // and after a cluster barrier every CTA sums a band of rows over all peers through
          // distributed shared memory - no trip through L2, no last-arriver tail.
          float* part = reinterpret_cast<float*>(smem);          // [BN][128]
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 16) {
            uint32_t r[16];
            zb_tmem_ld16(taddr + c0, r);
            zb_tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) part[(c0 + j) * kBlockP + row_in_tile] = __uint_as_float(r[j]);
          }
          zb_tc_fence_before();
          zb_mbar_arrive(&tmem_empty[acc]);
          zb_cluster_arrive();
          zb_cluster_wait();
          did_cluster_sync = true;
          if (tl && epi_tid == 0) tl[8] = zb_globaltimer();
          const int S = prm.cluster;
          const int rank = static_cast<int>(zb_cluster_ctarank());
          // bands begin on even rows: with interleaved gate / up rows (SwiGLU epilogue) a pair never straddles two CTAs
          const int rb0 = (rank * (kBlockP / 2) / S) * 2, rb1 = ((rank + 1) * (kBlockP / 2) / S) * 2;
          const int nrows = rb1 - rb0;
          const int total = BN * nrows;
          const uint32_t part_u32 = zb_smem_u32(part);
          uint32_t peer_base[8];
#pragma unroll
          for (int c = 0; c < 8; ++c) peer_base[c] = zb_mapa(part_u32, static_cast<uint32_t>(c < S ? c : 0));
          // squares of this band's finished outputs, [BN][nrows | 1] fp32 in the idle operand ring (behind the
          // partial tile), summed per token in a fixed order once the band is done
          float* sq = reinterpret_cast<float*>(smem + 96 * 1024);
          const int sq_ld = nrows | 1;
          const bool has_scale = epi_in_sumsq != nullptr;
          auto emit_sumsq = [&]() {
            epi_bar_sync();
            for (int c = epi_tid; c < BN; c += kEpiThreads) {
              if (q0 + c < prm.rows_q) {
                float acc = 0.f;
                for (int j = 0; j < nrows; ++j) acc += sq[c * sq_ld + j];
                epi_out_sumsq[(static_cast<size_t>(out_tile) * S + rank) * prm.epi.out_ld + q0 + c] = acc;
              }
            }
          };
          // all loads of a batch (peer partials, residual, bias) are issued before its first store:
          // `out` may alias `residual`, so the compiler would otherwise serialise them
          auto reduce_batch = [&](auto kb_tag, auto kc_tag, int e0) {
            constexpr int KB = decltype(kb_tag)::value, KC = decltype(kc_tag)::value;
            float tv[KB][KC], rsd[KB], bs[KB], sc[KB];
            int off[KB];
#pragma unroll
            for (int i = 0; i < KB; ++i) {
              const int e = min(e0 + i * kEpiThreads, total - 1);
              const int col = e / nrows, row = rb0 + (e - col * nrows);
              off[i] = col * kBlockP + row;
#pragma unroll
              for (int c = 0; c < KC; ++c) tv[i][c] = c < S ? zb_ld_dsmem_f32(peer_base[c] + off[i] * 4) : 0.f;
              const int pp = min(pt * kBlockP + row, prm.rows_p - 1), qq = min(q0 + col, prm.rows_q - 1);
              rsd[i] = prm.residual ? __bfloat162float(prm.residual[static_cast<size_t>(qq) * prm.ldo + pp]) : 0.f;
              bs[i] = prm.bias ? __bfloat162float(prm.bias[pp]) : 0.f;
              sc[i] = has_scale ? scale_tab[col] : 1.f;
            }
#pragma unroll
            for (int i = 0; i < KB; ++i) {
              const int e = e0 + i * kEpiThreads;
              float v = 0.f;
#pragma unroll
              for (int c = 0; c < KC; ++c) v += tv[i][c];            // ascending rank: deterministic
              v = v * sc[i] + bs[i] + rsd[i];
              const int col = off[i] / kBlockP, row = off[i] - col * kBlockP;
              const int pp = pt * kBlockP + row, qq = q0 + col;
              if (epi_swiglu) {
                // even lanes hold gate_i, their neighbours up_i (element and row parity agree: bands and their
                // heights are even); every lane of the warp takes part in the exchange
                const float up = __shfl_xor_sync(0xffffffffu, v, 1);
                if (e < total && (e & 1) == 0 && pp < prm.rows_p && qq < prm.rows_q)
                  reinterpret_cast<__nv_bfloat16*>(prm.out)[static_cast<size_t>(qq) * prm.ldo + (pp >> 1)] =
                      __float2bfloat16(silu_f(v) * up);
                continue;
              }
              if (e >= total) continue;
              float stored = 0.f;
              if (pp < prm.rows_p && qq < prm.rows_q) {
                const size_t o = static_cast<size_t>(qq) * prm.ldo + pp;
                if (prm.out_f32) {
                  reinterpret_cast<float*>(prm.out)[o] = v;
                  stored = v;
                } else {
                  const __nv_bfloat16 b = __float2bfloat16(v);
                  reinterpret_cast<__nv_bfloat16*>(prm.out)[o] = b;
                  stored = __bfloat162float(b);
                }
              }
              if (epi_out_sumsq != nullptr) sq[col * sq_ld + (row - rb0)] = stored * stored;
            }
          };
          if constexpr (!FUSED) {
            // every thread runs every batch (the SwiGLU exchange is warp-wide); elements past the band are masked
            if (S <= 4) {
              for (int base = 0; base < total; base += 8 * kEpiThreads)
                reduce_batch(std::integral_constant<int, 8>{}, std::integral_constant<int, 4>{}, base + epi_tid);
            } else {
              for (int base = 0; base < total; base += 4 * kEpiThreads)
                reduce_batch(std::integral_constant<int, 4>{}, std::integral_constant<int, 8>{}, base + epi_tid);
            }
            if (epi_out_sumsq != nullptr) emit_sumsq();
            if (tl && epi_tid == 0) tl[10] = zb_globaltimer();
            // nobody may leave (and release its shared memory) while a peer still reads it
            zb_cluster_arrive();
            zb_cluster_wait();
          } else {
            // Tensor-parallel variant: the band this CTA reduced over the cluster is this rank's
            // partial; it goes to every rank in one hop, in 8-byte {two bf16 values, epoch} slots
            // indexed by thread on both sides (the peer's thread with this index holds the same
            // elements) - no fence, no flags - and the band is finished from the copies of all ranks
            // (fused_ar.h, one_shot).  A thread holds up to 32 elements, handled as two halves of 16.
            const ZbFusedAr& ar = prm.ar;
            constexpr int kE = 16, kHalves = 2;
            const int n_el = (total - epi_tid + kEpiThreads - 1) / kEpiThreads;      // this thread's elements
            const size_t per_band = static_cast<size_t>(kHalves) * (kE / 2) * kEpiThreads;   // uint2 slots per (src, tile, band)
            const size_t band_idx = static_cast<size_t>(out_tile) * S + rank;
            const size_t src_stride = static_cast<size_t>(num_out_tiles) * S * per_band;
            const size_t half_sz = static_cast<size_t>(ar.world) * src_stride;
            const size_t my_slot = (epoch & 1u) * half_sz + band_idx * per_band + epi_tid;
            auto elem_off = [&](int i) {                  // element i of this thread -> offset in a [BN][128] tile
              const int e = min(epi_tid + i * kEpiThreads, total - 1);
              const int col = e / nrows;
              return col * kBlockP + rb0 + (e - col * nrows);
            };
            uint32_t mine_w[kHalves][kE / 2];
#pragma unroll
            for (int hf = 0; hf < kHalves; ++hf) {
              const int i0 = hf * kE;
              if (i0 >= n_el) {
#pragma unroll
                for (int j = 0; j < kE / 2; ++j) mine_w[hf][j] = 0u;
                continue;
              }
              float val[kE];
#pragma unroll
              for (int b4 = 0; b4 < kE; b4 += 4) {
                if (i0 + b4 >= n_el) {
#pragma unroll
                  for (int i = 0; i < 4; ++i) val[b4 + i] = 0.f;
                  continue;
                }
                float tv[4][8];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const int o_t = elem_off(i0 + b4 + i);
#pragma unroll
                  for (int c = 0; c < 8; ++c) tv[i][c] = c < S ? zb_ld_dsmem_f32(peer_base[c] + o_t * 4) : 0.f;
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  float v = 0.f;
#pragma unroll
                  for (int c = 0; c < 8; ++c) v += tv[i][c];
                  val[b4 + i] = (i0 + b4 + i) < n_el ? v : 0.f;
                }
              }
#pragma unroll
              for (int j = 0; j < kE / 2; ++j) mine_w[hf][j] = zb_pack_bf16x2(val[2 * j], val[2 * j + 1]);
              const int n_pair = (min(n_el - i0, kE) + 1) / 2;
              for (int d = 0; d < ar.world; ++d) {
                if (d == ar.rank) continue;
                uint2* dst = reinterpret_cast<uint2*>(ar.recv_peer[d]) + my_slot + static_cast<size_t>(ar.rank) * src_stride +
                             static_cast<size_t>(hf) * (kE / 2) * kEpiThreads;
#pragma unroll
                for (int j = 0; j < kE / 2; ++j)
                  if (j < n_pair) zb_st_ll(dst + static_cast<size_t>(j) * kEpiThreads, mine_w[hf][j], epoch);
              }
            }
            zb_cluster_arrive();                 // peers' shared memory is no longer needed; waited for below
            if (tl && epi_tid == 0) tl[9] = zb_globaltimer();
            const uint2* slots = reinterpret_cast<const uint2*>(ar.recv_peer[ar.rank]) + my_slot;
            const uint64_t t_wait0 = zb_globaltimer();
#pragma unroll
            for (int hf = 0; hf < kHalves; ++hf) {
              const int i0 = hf * kE;
              if (i0 >= n_el || *abort_flag != 0u) continue;
              const int n_here = min(n_el - i0, kE);
              const int n_pair = (n_here + 1) / 2;
              // bias / residual loads go out while the peers' slots are in flight
              float add[kE];
#pragma unroll
              for (int i = 0; i < kE; ++i) {
                add[i] = 0.f;
                if (i < n_here) {
                  const int o_t = elem_off(i0 + i);
                  const int col = o_t / kBlockP, row = o_t - col * kBlockP;
                  const int pp = min(pt * kBlockP + row, prm.rows_p - 1), qq = min(q0 + col, prm.rows_q - 1);
                  if (prm.residual) add[i] = __bfloat162float(prm.residual[static_cast<size_t>(qq) * prm.ldo + pp]);
                  if (prm.bias) add[i] += __bfloat162float(prm.bias[pp]);
                }
              }
              float sum[kE];
#pragma unroll
              for (int i = 0; i < kE; ++i) sum[i] = 0.f;
              for (int src = 0; src < ar.world; ++src) {              // ascending rank: the same bits everywhere
                uint32_t w[kE / 2];
                if (src == ar.rank) {
#pragma unroll
                  for (int j = 0; j < kE / 2; ++j) w[j] = mine_w[hf][j];
                } else {
                  const uint2* sp = slots + static_cast<size_t>(src) * src_stride + static_cast<size_t>(hf) * (kE / 2) * kEpiThreads;
                  bool ready = false;
                  uint32_t spins = 0;
                  while (!ready) {
                    ready = true;
#pragma unroll
                    for (int j = 0; j < kE / 2; ++j) {
                      w[j] = 0u;
                      if (j < n_pair) {
                        const uint2 x = zb_ld_ll(sp + static_cast<size_t>(j) * kEpiThreads);
                        w[j] = x.x;
                        ready = ready && (x.y == epoch);
                      }
                    }
                    if (!ready && (++spins & 0x3f) == 0) {
                      if (*abort_flag != 0u || zb_globaltimer() - t_wait0 > ZB_WAIT_LIMIT_NS) {
                        *abort_flag = 1u;
                        *abort_where = 100u + src;
                        break;
                      }
                    }
                  }
                }
#pragma unroll
                for (int j = 0; j < kE / 2; ++j) {
                  const float2 f2 = zb_unpack_bf16x2(w[j]);
                  sum[2 * j] += f2.x;
                  sum[2 * j + 1] += f2.y;
                }
              }
              if (*abort_flag == 0u) {
#pragma unroll
                for (int i = 0; i < kE; ++i) {
                  if (i < n_here) {
                    const int o_t = elem_off(i0 + i);
                    const int col = o_t / kBlockP, row = o_t - col * kBlockP;
                    const int pp = pt * kBlockP + row, qq = q0 + col;
                    float stored = 0.f;
                    if (pp < prm.rows_p && qq < prm.rows_q) {
                      const __nv_bfloat16 b = __float2bfloat16(sum[i] + add[i]);
                      ar.out_peer[ar.rank][static_cast<size_t>(qq) * prm.ldo + pp] = b;
                      stored = __bfloat162float(b);
                    }
                    if (epi_out_sumsq != nullptr) sq[col * sq_ld + (row - rb0)] = stored * stored;
                  }
                }
              }
            }
            if (epi_out_sumsq != nullptr) emit_sumsq();
            if (tl && epi_tid == 0) tl[10] = zb_globaltimer();
            if (tl && epi_tid == 0) tl[11] = zb_globaltimer();
            zb_cluster_wait();
            if (*abort_flag != 0u) break;
          }
          acc ^= 1u;
          if (acc == 0) acc_phase ^= 1u;
          continue;
        }
      }
      if constexpr (kGeneric) {
      bool do_store = true;
      if (partial) {
        // write this CTA's piece: ws[((cta*2 + slot)*BN + c)*128 + row]
        float* ws = prm.workspace + (static_cast<size_t>(blockIdx.x) * 2 + my_slot) * (BN * kBlockP);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          uint32_t r[16];
          zb_tmem_ld16(taddr + c0, r);
          zb_tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) ws[(c0 + j) * kBlockP + row_in_tile] = __uint_as_float(r[j]);
        }
        __threadfence();
        epi_bar_sync();
        if (epi_tid == 0) {
          const uint32_t prev = atomicAdd(&prm.counters[out_tile], 1u);
          const uint32_t last = (prev == static_cast<uint32_t>(last_cta - first_cta)) ? 1u : 0u;
          if (last) prm.counters[out_tile] = 0u;   // ready for the next launch
          *is_last_flag = last;
        }
        epi_bar_sync();
        do_store = (*is_last_flag != 0u);
        if (do_store) __threadfence();
      }
      // the accumulator stage can be reused as soon as it has been read
      if (partial) {
        zb_tc_fence_before();
        zb_mbar_arrive(&tmem_empty[acc]);
      }

      // chunk of 16 accumulator columns of this thread's row (summed over the pieces if any)
      auto load_chunk = [&](int c0, float (&v)[16]) {
        if (partial) {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0.f;
          // four pieces per round trip to L2: the loads of a batch are all in flight before the
          // first add (summation order stays ascending in c, so the result does not depend on it)
          for (int c = first_cta; c <= last_cta; c += 4) {
            float t4[4][16];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              const int cc = min(c + b, last_cta);
              const long long c_begin = static_cast<long long>(cc) * prm.units_per_cta;
              const int slot = (max(t_begin, c_begin) == c_begin) ? 0 : 1;
              const float* ws = prm.workspace + (static_cast<size_t>(cc) * 2 + slot) * (BN * kBlockP);
#pragma unroll
              for (int j = 0; j < 16; ++j) t4[b][j] = __ldcg(&ws[(c0 + j) * kBlockP + row_in_tile]);
            }
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              if (c + b <= last_cta) {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] += t4[b][j];
              }
            }
          }
        } else {
          uint32_t r[16];
          zb_tmem_ld16(taddr + c0, r);
          zb_tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
        }
      };
      // bias / residual (read from this rank's memory) then store into `outp`
      auto finish_chunk = [&](int c0, float (&v)[16]) {
        if constexpr (SWAP) {
          const float b = (prm.bias && p < prm.rows_p) ? __bfloat162float(prm.bias[p]) : 0.f;
          const bool has_scale = epi_in_sumsq != nullptr;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int q = q0 + c0 + j;
            if (has_scale) v[j] *= scale_tab[c0 + j];
            v[j] += b;
            if (prm.residual && q < prm.rows_q)
              v[j] += __bfloat162float(prm.residual[static_cast<size_t>(q) * prm.ldo + p]);
          }
        } else {
          const int q = q0 + c0;
          const size_t o = static_cast<size_t>(p) * prm.ldo + q;
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] *= row_scale;
          if (q + 16 <= prm.rows_q) {
            if (prm.bias) {
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] += __bfloat162float(prm.bias[q + j]);
            }
            if (prm.residual) {
              const uint4* rp = reinterpret_cast<const uint4*>(prm.residual + o);
              uint4 r0 = rp[0], r1 = rp[1];
              const uint32_t rr[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float2 f = zb_unpack_bf16x2(rr[j]);
                v[2 * j] += f.x;
                v[2 * j + 1] += f.y;
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (q + j < prm.rows_q) {
                if (prm.bias) v[j] += __bfloat162float(prm.bias[q + j]);
                if (prm.residual) v[j] += __bfloat162float(prm.residual[o + j]);
              }
            }
          }
        }
      };
      auto store_chunk = [&](int c0, const float (&v)[16], void* outp) {
        if constexpr (SWAP) {
          // p = output column n, q = output row m
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int q = q0 + c0 + j;
            if (q < prm.rows_q) {
              const size_t o = static_cast<size_t>(q) * prm.ldo + p;
              if (prm.out_f32) reinterpret_cast<float*>(outp)[o] = v[j];
              else reinterpret_cast<__nv_bfloat16*>(outp)[o] = __float2bfloat16(v[j]);
            }
          }
        } else {
          // p = output row m, q = output column n (16 consecutive columns per step)
          const int q = q0 + c0;
          const size_t o = static_cast<size_t>(p) * prm.ldo + q;
          if (q + 16 <= prm.rows_q) {
            if (prm.out_f32) {
              float4* op = reinterpret_cast<float4*>(reinterpret_cast<float*>(outp) + o);
#pragma unroll
              for (int j = 0; j < 4; ++j)
                op[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            } else {
              uint4* op = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(outp) + o);
              op[0] = make_uint4(zb_pack_bf16x2(v[0], v[1]), zb_pack_bf16x2(v[2], v[3]),
                                 zb_pack_bf16x2(v[4], v[5]), zb_pack_bf16x2(v[6], v[7]));
              op[1] = make_uint4(zb_pack_bf16x2(v[8], v[9]), zb_pack_bf16x2(v[10], v[11]),
                                 zb_pack_bf16x2(v[12], v[13]), zb_pack_bf16x2(v[14], v[15]));
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (q + j < prm.rows_q) {
                if (prm.out_f32) reinterpret_cast<float*>(outp)[o + j] = v[j];
                else reinterpret_cast<__nv_bfloat16*>(outp)[o + j] = __float2bfloat16(v[j]);
              }
            }
          }
        }
      };

      // SwiGLU epilogue: rows of the weight interleave gate and up, the output has half as many columns.
      // Swap-AB: this thread holds one weight row, its neighbour lane the partner (all lanes take part).
      auto swiglu_store_chunk = [&](int c0, const float (&v)[16]) {
        __nv_bfloat16* outp = reinterpret_cast<__nv_bfloat16*>(prm.out);
        if constexpr (SWAP) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float up = __shfl_xor_sync(0xffffffffu, v[j], 1);
            const int q = q0 + c0 + j;
            if ((row_in_tile & 1) == 0 && p < prm.rows_p && q < prm.rows_q)
              outp[static_cast<size_t>(q) * prm.ldo + (p >> 1)] = __float2bfloat16(silu_f(v[j]) * up);
          }
        } else {
          const int q = q0 + c0;
          if (p < prm.rows_p) {
            const size_t o = static_cast<size_t>(p) * prm.ldo + (q >> 1);
            if (q + 16 <= prm.rows_q) {
              uint32_t w[4];
#pragma unroll
              for (int j = 0; j < 4; ++j)
                w[j] = zb_pack_bf16x2(silu_f(v[4 * j]) * v[4 * j + 1], silu_f(v[4 * j + 2]) * v[4 * j + 3]);
              *reinterpret_cast<uint4*>(outp + o) = make_uint4(w[0], w[1], w[2], w[3]);
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if (q + 2 * j + 1 < prm.rows_q) outp[o + j] = __float2bfloat16(silu_f(v[2 * j]) * v[2 * j + 1]);
            }
          }
        }
      };
      // one chunk through the generic epilogue
      auto epilogue_chunk = [&](int c0) {
        float v[16];
        load_chunk(c0, v);
        if (epi_swiglu) {
          finish_chunk(c0, v);
          swiglu_store_chunk(c0, v);
        } else if (p < prm.rows_p) {
          finish_chunk(c0, v);
          store_chunk(c0, v, prm.out);
        }
      };

      if constexpr (!FUSED && SWAP && BN <= 64) {
        if (partial && do_store) {
          // Fix-up of a split tile, few tokens: the pieces are summed straight from the workspace by
          // all 128 epilogue threads with 16-byte loads - thread (lane, g) owns rows 4*lane..4*lane+3
          // and columns g, g+4, ... - several pieces per round trip to L2 (this serial tail is what a
          // weight-streaming GEMM of a few tens of megabytes spends most of its time on otherwise).
          constexpr int kCols = BN / 4;                        // columns per thread
          constexpr int kBatch = BN <= 16 ? 6 : (BN <= 32 ? 3 : 1);
          const int r4 = (epi_tid & 31) * 4;
          const int cg = epi_tid >> 5;
          float4 accv[kCols];
#pragma unroll
          for (int i = 0; i < kCols; ++i) accv[i] = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int c = first_cta; c <= last_cta; c += kBatch) {
            float4 tv[kBatch][kCols];
#pragma unroll
            for (int b = 0; b < kBatch; ++b) {
              const int cc = min(c + b, last_cta);
              const long long c_begin = static_cast<long long>(cc) * prm.units_per_cta;
              const int slot = (max(t_begin, c_begin) == c_begin) ? 0 : 1;
              const float4* w4 = reinterpret_cast<const float4*>(
                  prm.workspace + (static_cast<size_t>(cc) * 2 + slot) * (BN * kBlockP));
#pragma unroll
              for (int i = 0; i < kCols; ++i) tv[b][i] = __ldcg(&w4[(cg + 4 * i) * (kBlockP / 4) + (epi_tid & 31)]);
            }
#pragma unroll
            for (int b = 0; b < kBatch; ++b) {
              if (c + b <= last_cta) {
#pragma unroll
                for (int i = 0; i < kCols; ++i) {
                  accv[i].x += tv[b][i].x;
                  accv[i].y += tv[b][i].y;
                  accv[i].z += tv[b][i].z;
                  accv[i].w += tv[b][i].w;
                }
              }
            }
          }
          const int pb = pt * kBlockP + r4;                     // first of this thread's 4 output columns
          float bz[4] = {0.f, 0.f, 0.f, 0.f};
          if (prm.bias) {
#pragma unroll
            for (int e = 0; e < 4; ++e) bz[e] = (pb + e) < prm.rows_p ? __bfloat162float(prm.bias[pb + e]) : 0.f;
          }
          const bool vec = (pb + 3) < prm.rows_p && (prm.ldo % 4) == 0;
          // residual loads first, all of them: `out` may alias `residual`, which would otherwise
          // order every load behind the previous column's store
          uint2 rres[kCols];
          if (vec && prm.residual) {
#pragma unroll
            for (int i = 0; i < kCols; ++i) {
              const int q = min(q0 + cg + 4 * i, prm.rows_q - 1);
              rres[i] = *reinterpret_cast<const uint2*>(prm.residual + static_cast<size_t>(q) * prm.ldo + pb);
            }
          }
#pragma unroll
          for (int i = 0; i < kCols; ++i) {
            const int q = q0 + cg + 4 * i;
            if (q >= prm.rows_q) continue;
            const float sc = epi_in_sumsq != nullptr ? scale_tab[cg + 4 * i] : 1.f;
            float v4[4] = {accv[i].x * sc + bz[0], accv[i].y * sc + bz[1], accv[i].z * sc + bz[2], accv[i].w * sc + bz[3]};
            if (epi_swiglu) {
              // rows pb .. pb + 3 are (gate, up, gate, up): two outputs at columns pb / 2, pb / 2 + 1
              __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(prm.out) + static_cast<size_t>(q) * prm.ldo + (pb >> 1);
              if (pb + 3 < prm.rows_p) {
                *reinterpret_cast<uint32_t*>(op) = zb_pack_bf16x2(silu_f(v4[0]) * v4[1], silu_f(v4[2]) * v4[3]);
              } else if (pb + 1 < prm.rows_p) {
                op[0] = __float2bfloat16(silu_f(v4[0]) * v4[1]);
              }
              continue;
            }
            const size_t o = static_cast<size_t>(q) * prm.ldo + pb;
            if (vec) {
              if (prm.residual) {
                const uint2 rr = rres[i];
                const float2 f0 = zb_unpack_bf16x2(rr.x), f1 = zb_unpack_bf16x2(rr.y);
                v4[0] += f0.x;
                v4[1] += f0.y;
                v4[2] += f1.x;
                v4[3] += f1.y;
              }
              if (prm.out_f32) {
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(prm.out) + o) = make_float4(v4[0], v4[1], v4[2], v4[3]);
              } else {
                *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(prm.out) + o) =
                    make_uint2(zb_pack_bf16x2(v4[0], v4[1]), zb_pack_bf16x2(v4[2], v4[3]));
              }
            } else {
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                if (pb + e < prm.rows_p) {
                  float x = v4[e];
                  if (prm.residual) x += __bfloat162float(prm.residual[o + e]);
                  if (prm.out_f32) reinterpret_cast<float*>(prm.out)[o + e] = x;
                  else reinterpret_cast<__nv_bfloat16*>(prm.out)[o + e] = __float2bfloat16(x);
                }
              }
            }
          }
        } else if (do_store) {
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 16) epilogue_chunk(c0);
        }
      } else if constexpr (!FUSED) {
        if (do_store) {
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 16) epilogue_chunk(c0);
        }
        if constexpr (BAND) {
          if (prm.band.mode == 1) {
            // band pipeline, producer side: count the stored tiles of the band; the CTA that stores the last
            // one tells the band's owner that this rank's partial sums of the band are complete
            __threadfence_system();
            epi_bar_sync();
            if (epi_tid == 0) {
              const uint32_t prev = atomicAdd(&prm.band.count_p[pt], 1u);
              if (prev == static_cast<uint32_t>(prm.band.tiles_per_band - 1)) {
                prm.band.count_p[pt] = 0u;
                __threadfence_system();
                const uint32_t ep = *reinterpret_cast<volatile uint32_t*>(prm.band.epoch);
                zb_st_release_sys(prm.band.ready_peer[pt % prm.band.world] + static_cast<size_t>(pt) * 8 + prm.band.rank, ep);
              }
            }
          }
        }
      } else if (SWAP && BN <= 64 && prm.ar.one_shot != 0) {
        if (do_store) {
          // single-hop all-reduce of a tile (few tokens)
          const ZbFusedAr& ar = prm.ar;
          const size_t tile_elems = static_cast<size_t>(kBlockP) * BN;
          const size_t half = static_cast<size_t>(ar.world) * num_out_tiles * tile_elems;
          const size_t my_off = (epoch & 1u) * half + (static_cast<size_t>(ar.rank) * num_out_tiles + out_tile) * tile_elems +
                                static_cast<size_t>(row_in_tile) * BN;
          // 1. this rank's partial -> every rank's staging slot [parity][src = rank][tile][row][BN]
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 16) {
            float v[16];
            load_chunk(c0, v);
            const uint4 lo = make_uint4(zb_pack_bf16x2(v[0], v[1]), zb_pack_bf16x2(v[2], v[3]),
                                        zb_pack_bf16x2(v[4], v[5]), zb_pack_bf16x2(v[6], v[7]));
            const uint4 hi = make_uint4(zb_pack_bf16x2(v[8], v[9]), zb_pack_bf16x2(v[10], v[11]),
                                        zb_pack_bf16x2(v[12], v[13]), zb_pack_bf16x2(v[14], v[15]));
            for (int d = 0; d < ar.world; ++d) {
              uint4* d4 = reinterpret_cast<uint4*>(ar.recv_peer[d] + my_off + c0);
              d4[0] = lo;
              d4[1] = hi;
            }
          }
          if (!partial) {
            zb_tc_fence_before();
            zb_mbar_arrive(&tmem_empty[acc]);
          }
          __threadfence_system();
          epi_bar_sync();
          const size_t fidx = static_cast<size_t>(out_tile) * ar.world;
          if (epi_tid < ar.world) zb_st_release_sys(ar.push_flag_peer[epi_tid] + fidx + ar.rank, epoch);
          // 2. wait for the copies of all ranks, sum in rank order, finish, store locally
          if (epi_tid < ar.world) {
            if (!zb_wait_flag(ar.push_flag_peer[ar.rank] + fidx + epi_tid, epoch, abort_flag)) *abort_where = 100u + epi_tid;
          }
          epi_bar_sync();
          if (*abort_flag != 0u) break;
          const __nv_bfloat16* mine = ar.recv_peer[ar.rank] + (epoch & 1u) * half +
                                      static_cast<size_t>(out_tile) * tile_elems + static_cast<size_t>(row_in_tile) * BN;
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 16) {
            uint4 x[kZbMaxRanks][2];
#pragma unroll
            for (int src = 0; src < kZbMaxRanks; ++src) {
              const int ss = src < ar.world ? src : 0;
              const uint4* s4 = reinterpret_cast<const uint4*>(mine + static_cast<size_t>(ss) * num_out_tiles * tile_elems + c0);
              x[src][0] = __ldcg(s4);
              x[src][1] = __ldcg(s4 + 1);
            }
            float v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0.f;
#pragma unroll
            for (int src = 0; src < kZbMaxRanks; ++src) {
              if (src < ar.world) {
                const uint32_t xx[8] = {x[src][0].x, x[src][0].y, x[src][0].z, x[src][0].w,
                                        x[src][1].x, x[src][1].y, x[src][1].z, x[src][1].w};
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const float2 f2 = zb_unpack_bf16x2(xx[j]);
                  v[2 * j] += f2.x;
                  v[2 * j + 1] += f2.y;
                }
              }
            }
            if (p < prm.rows_p) {
              finish_chunk(c0, v);
              store_chunk(c0, v, ar.out_peer[ar.rank]);
            }
          }
        }
      } else {
        if (do_store) {
          const ZbFusedAr& ar = prm.ar;
          const int owner = out_tile % ar.world;
          const int slot = out_tile / ar.world;
          // 1. partial tile -> owner's staging slot [src = rank][slot][row][BN]
          __nv_bfloat16* dst = ar.recv_peer[owner] +
                               ((static_cast<size_t>(ar.rank) * ar.slots_per_src + slot) * kBlockP + row_in_tile) * BN;
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 16) {
            float v[16];
            load_chunk(c0, v);
            uint4* d4 = reinterpret_cast<uint4*>(dst + c0);
            d4[0] = make_uint4(zb_pack_bf16x2(v[0], v[1]), zb_pack_bf16x2(v[2], v[3]),
                               zb_pack_bf16x2(v[4], v[5]), zb_pack_bf16x2(v[6], v[7]));
            d4[1] = make_uint4(zb_pack_bf16x2(v[8], v[9]), zb_pack_bf16x2(v[10], v[11]),
                               zb_pack_bf16x2(v[12], v[13]), zb_pack_bf16x2(v[14], v[15]));
          }
          if (!partial) {
            zb_tc_fence_before();
            zb_mbar_arrive(&tmem_empty[acc]);
          }
          __threadfence_system();
          epi_bar_sync();
          if (epi_tid == 0)
            zb_st_release_sys(ar.push_flag_peer[owner] + static_cast<size_t>(slot) * ar.world + ar.rank, epoch);
          if (owner == ar.rank) {
            // 2. reduce the partials of all ranks and broadcast the result
            if (epi_tid < ar.world) {
              const uint32_t* f = ar.push_flag_peer[ar.rank] + static_cast<size_t>(slot) * ar.world + epi_tid;
              if (!zb_wait_flag(f, epoch, abort_flag)) *abort_where = 100u + epi_tid;
            }
            epi_bar_sync();
            if (*abort_flag != 0u) break;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
              float v[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] = 0.f;
              for (int src = 0; src < ar.world; ++src) {
                const uint4* s4 = reinterpret_cast<const uint4*>(
                    ar.recv_peer[ar.rank] +
                    ((static_cast<size_t>(src) * ar.slots_per_src + slot) * kBlockP + row_in_tile) * BN + c0);
                const uint4 x0 = __ldcg(s4), x1 = __ldcg(s4 + 1);
                const uint32_t xx[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const float2 f2 = zb_unpack_bf16x2(xx[j]);
                  v[2 * j] += f2.x;
                  v[2 * j + 1] += f2.y;
                }
              }
              if (p < prm.rows_p) {
                finish_chunk(c0, v);
                for (int d = 0; d < ar.world; ++d) store_chunk(c0, v, ar.out_peer[d]);
              }
            }
            __threadfence_system();
            epi_bar_sync();
            if (epi_tid < ar.world) zb_st_release_sys(ar.done_flag_peer[epi_tid] + out_tile, epoch);
          }
        }
      }
      if (!FUSED && !partial) {
        zb_tc_fence_before();
        zb_mbar_arrive(&tmem_empty[acc]);
      }
      }  // kGeneric
      acc ^= 1u;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (prm.cluster > 1 && !did_cluster_sync) {
      // gave up before the exchange (a bounded wait ran out): still meet the peers at both barriers
      __syncwarp();
      zb_cluster_arrive();
      zb_cluster_wait();
      zb_cluster_arrive();
      zb_cluster_wait();
    }
    if (tl && epi_tid == 0) tl[6] = zb_globaltimer();
    if constexpr (FUSED) {
      // 3. the all-reduced output is complete on this rank once every tile is marked done
      if (*abort_flag == 0u && !(SWAP && BN <= 64 && prm.ar.one_shot != 0)) {
        for (int t = blockIdx.x * kEpiThreads + epi_tid; t < num_out_tiles; t += gridDim.x * kEpiThreads) {
          if (!zb_wait_flag(prm.ar.done_flag_peer[prm.ar.rank] + t, epoch, abort_flag)) {
            *abort_where = 200u;
            break;
          }
        }
      }
      epi_bar_sync();
      if (epi_tid == 0) {
        __threadfence();
        const uint32_t ticket = atomicAdd(prm.ar.exit_ticket, 1u);
        if (ticket == gridDim.x - 1) {
          *prm.ar.exit_ticket = 0u;
          *reinterpret_cast<volatile uint32_t*>(prm.ar.epoch) = epoch + 1u;
        }
      }
    }
  }

  // ------------------------------------------------------------ common exit
  zb_tc_fence_before();
  __syncthreads();
  if (BAND && prm.band.mode == 2 && threadIdx.x == 0) {
    // band pipeline: every wait of this launch is over once all CTAs are here; the last one opens the next epoch
    __threadfence();
    const uint32_t ticket = atomicAdd(prm.band.epoch + 1, 1u);
    if (ticket == gridDim.x - 1) {
      prm.band.epoch[1] = 0u;
      const uint32_t e = *reinterpret_cast<volatile uint32_t*>(prm.band.epoch);
      *reinterpret_cast<volatile uint32_t*>(prm.band.epoch) = e + 1u;
    }
  }
  if (*abort_flag != 0u) {
    if (threadIdx.x == 0)
      zb_record_error(prm.status, *abort_where >= 100u ? ZB_ERR_FLAG_TIMEOUT : ZB_ERR_MBAR_TIMEOUT,
                      FUSED ? kKernelIdFused : kKernelId, *abort_where, blockIdx.x);
    // give copies that may still be in flight time to land before the CTA's
    // shared memory is handed to another CTA
    const uint64_t t0 = zb_globaltimer();
    while (zb_globaltimer() - t0 < 200000ull) {
    }
    __syncthreads();
  }
  if (warp == 1) {
    zb_tc_fence_after();
    zb_tmem_dealloc(tmem_base, kTmemCols);
  }
  if (tl && threadIdx.x == 64) tl[7] = zb_globaltimer();
}

// Sum of squares of every row of a bf16 matrix: out[row] = sum_c x[row][c]^2 (fp32, fixed summation order).
// The one-part form of the partial sums the GEMM epilogue emits, for producers that do not emit them.
__global__ void __launch_bounds__(256) zb_row_sumsq_kernel(const __nv_bfloat16* __restrict__ x, long long ld, int d,
                                                           float* __restrict__ out) {
  zb_pdl_launch();
  zb_pdl_wait();
  const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(blockIdx.x) * ld);
  float ss = 0.f;
  for (int v = threadIdx.x; v < (d >> 3); v += 256) {
    const uint4 a = xr[v];
    const uint32_t au[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = zb_unpack_bf16x2(au[j]);
      ss += f.x * f.x + f.y * f.y;
    }
  }
  __shared__ float red[8];
  ss = zb_warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    out[blockIdx.x] = tot;
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  });
  return fn;
}

}  // namespace

// K-major bf16 matrix [rows, k] with leading dimension ld -> tensor map with a
// (64 x box_rows) box and the 128-byte swizzle.  Returns 0 on success.
int zb_make_tmap_bf16_2d(CUtensorMap* out, const void* base, int rows, int k, int ld,
                         int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (ld % 8) != 0) return -2;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

// Byte matrix [rows, row_bytes] -> tensor map with a (box_bytes x box_rows) box, no swizzle (packed
// sub-byte data such as NVFP4 codes).  row_bytes and box_bytes multiples of 16.
// `swizzle128`: rows of the box are 128 bytes and land with the 128-byte swizzle (16-byte chunk j of row r at j ^ (r % 8)).
int zb_make_tmap_u8_2d_ex(CUtensorMap* out, const void* base, long long rows, long long row_bytes, int box_bytes, int box_rows,
                          int swizzle128) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (row_bytes % 16) != 0 || (box_bytes % 16) != 0 || box_rows > 256) return -2;
  if (swizzle128 && box_bytes != 128) return -2;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(row_bytes), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_bytes)};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_bytes), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

int zb_make_tmap_u8_2d(CUtensorMap* out, const void* base, long long rows, long long row_bytes, int box_bytes, int box_rows) {
  return zb_make_tmap_u8_2d_ex(out, base, rows, row_bytes, box_bytes, box_rows, 0);
}

// Paged K or V cache [slots, kv_heads, head_dim] bf16 -> 4-D tensor map (64 columns, slots, head_dim / 64
// column groups, kv heads) with box (64, box_rows, head_dim / 64, 1) and the 128-byte swizzle: one copy
// brings `box_rows` consecutive slots of one head into shared memory as head_dim / 64 tiles of
// [box_rows][64], each with 128-byte rows.  Returns 0 on success.
int zb_make_tmap_kv_cache(CUtensorMap* out, const void* base, long long slots, int kv_heads, int head_dim,
                          int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || head_dim % 64 != 0 || box_rows < 1 || box_rows > 256) return -2;
  const cuuint64_t row_bytes = static_cast<cuuint64_t>(kv_heads) * head_dim * 2;
  cuuint64_t dims[4] = {64, static_cast<cuuint64_t>(slots), static_cast<cuuint64_t>(head_dim / 64),
                        static_cast<cuuint64_t>(kv_heads)};
  cuuint64_t strides[3] = {row_bytes, 128, static_cast<cuuint64_t>(head_dim) * 2};
  cuuint32_t box[4] = {64, static_cast<cuuint32_t>(box_rows), static_cast<cuuint32_t>(head_dim / 64), 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

namespace {

template <int BN, bool SWAP, int MODE, int EPI, int PLAN>
int launch_k(const CUtensorMap& tp, const CUtensorMap& tq, const GemmParams& prm, int grid, cudaStream_t stream) {
  constexpr int smem = smem_bytes_for(BN, SWAP);
  // the shared-memory attribute of a kernel is per device: one flag per device for every instantiation
  static bool configured[16] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return -21;
  if (!configured[dev]) {
    cudaError_t e = zb_config_smem(zb_gemm_bf16_kernel<BN, SWAP, MODE, EPI, PLAN>, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev] = true;
  }
  const cudaError_t le = zb_launch_cluster(zb_gemm_bf16_kernel<BN, SWAP, MODE, EPI, PLAN>, dim3(grid), dim3(kNumThreads), smem,
                                           stream, prm.cluster, tp, tq, prm);
  zb_count_launch(1);
  return static_cast<int>(le != cudaSuccess ? le : cudaGetLastError());
}

template <int BN, bool SWAP, int MODE = 0>
int launch(const CUtensorMap& tp, const CUtensorMap& tq, const GemmParams& prm, int grid, cudaStream_t stream) {
  constexpr bool can_cluster = SWAP && (BN <= 64 || (MODE != 1 && BN <= 128));
  if (prm.cluster > 1 && !can_cluster) return -12;
  return launch_k<BN, SWAP, MODE, 1, 2>(tp, tq, prm, grid, stream);
}

// CTAs of the swap-AB kernel that can be resident at once when launched in clusters of `s`.
template <int BN>
int max_cluster_ctas(int s) {
  static int cache[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
  if (s < 2 || s > 8) return 0;
  if (cache[s] != 0) return cache[s] < 0 ? 0 : cache[s];
  constexpr int smem = smem_bytes_for(BN, true);
  if (zb_config_smem(zb_gemm_bf16_kernel<BN, true, 0, 1, 2>, smem) != cudaSuccess) {
    (void)cudaGetLastError();
    cache[s] = -1;
    return 0;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(s) * 64);
  cfg.blockDim = dim3(kNumThreads);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(s);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, zb_gemm_bf16_kernel<BN, true, 0, 1, 2>, &cfg) != cudaSuccess) {
    (void)cudaGetLastError();
    n = 0;
  }
  cache[s] = n > 0 ? n * s : -1;
  return n * s;
}

int g_cluster_splitk = 1;

// Cluster split-K plan for a weight-streaming GEMM with fewer tiles than SMs: every tile is cut
// along K over the CTAs of one cluster, which reduce it through distributed shared memory.
// Returns the cluster size (1: keep the stream-K plan) and updates grid / units per CTA.
int zb_gemm_cluster_capacity_of(int bn, int s);
int plan_cluster(int bn, int tiles, int kb_total, int num_sms, int* grid, int* upc, bool allow_tiny = true) {
  if (!g_cluster_splitk || bn > 128 || tiles >= num_sms) return 1;
  int best = 1, best_ctas = 0;
  const int sizes[5] = {8, 6, 4, 3, 2};
  for (int i = 0; i < 5; ++i) {
    const int s = sizes[i];
    const int per_rank = (kb_total + s - 1) / s;
    if (per_rank < 2 || (s - 1) * per_rank >= kb_total) continue;      // every CTA of the cluster gets k-blocks
    const int cap = zb_gemm_cluster_capacity_of(bn, s);
    const int ctas = tiles * s;
    if (ctas > cap || ctas > num_sms) continue;
    if (ctas > best_ctas) {
      best = s;
      best_ctas = ctas;
    }
  }
  // Under half of the SMs busy: stream-K (all SMs stream) does better - unless the whole problem is a few
  // k-blocks (a router or a small head: 1 - 2 tiles), or a handful of tiles would each be cut into many pieces:
  // the stream-K fix-up then costs more than the whole GEMM (measured inside a decoder layer: 12 us for 16
  // pieces of a 32-token tile, against 2.5 us for the cluster reduction through shared memory).
  const bool tiny = allow_tiny && static_cast<long long>(tiles) * kb_total <= 64;
  const int pieces = (kb_total + *upc - 1) / *upc;
  const bool shredded = allow_tiny && tiles <= 8 && pieces >= 8;
  if (best == 1 || (best_ctas * 2 < num_sms && !tiny && !shredded)) return 1;
  *grid = best_ctas;
  *upc = (kb_total + best - 1) / best;
  return best;
}

int zb_gemm_cluster_capacity_of(int bn, int s) {
  return bn <= 16 ? max_cluster_ctas<16>(s) : (bn <= 32 ? max_cluster_ctas<32>(s) : (bn <= 64 ? max_cluster_ctas<64>(s) : max_cluster_ctas<128>(s)));
}

// Weight tiles per CTA to pull into L2 ahead of the shared-memory ring while the preceding
// kernel drains: only for the weight-streaming (few tokens) regime, and at most ~40 MB in all,
// a third of the L2.
int g_l2_prefetch_mb = 40;
unsigned long long* g_timeline = nullptr;
int g_timeline_slots = 0;
int g_timeline_next = 0;
unsigned long long* next_timeline(int grid) {
  if (g_timeline == nullptr || g_timeline_slots <= 0 || grid > 160) return nullptr;
  unsigned long long* p = g_timeline + static_cast<size_t>(g_timeline_next % g_timeline_slots) * 160 * 12;
  ++g_timeline_next;
  return p;
}
int l2_prefetch_tiles(int swap, int bn, int grid, int rr_tiles) {
  if (!swap || rr_tiles > 0 || grid <= 0 || g_l2_prefetch_mb <= 0) return 0;
  const long long tile_bytes = static_cast<long long>(kBlockP) * kBlockK * 2;
  (void)bn;
  const long long per_cta = (static_cast<long long>(g_l2_prefetch_mb) << 20) / grid / tile_bytes;
  return static_cast<int>(per_cta > 64 ? 64 : per_cta);
}

}  // namespace

extern "C" {

// Profiling aid: when set, every CTA of the following GEMM launches writes globaltimer stamps to
// buf[cta][12] = {entry, prologue done, producer past the dependency wait, first tile landed,
// last accumulator committed, first accumulator seen by the epilogue, epilogue done, exit,
// partial tiles of the cluster visible, partial pushed to the peers, band finished (peers' copies seen,
// output and statistics stored), unused}.
// `buf` holds `slots` records of 160 * 12 zeroed u64; consecutive launches take consecutive records
// (wrapping around).  Null turns it off.
void zb_gemm_set_timeline(unsigned long long* buf, int slots) {
  g_timeline = buf;
  g_timeline_slots = slots;
  g_timeline_next = 0;
}

// Cluster split-K (see plan_cluster) on / off.
void zb_set_cluster_splitk(int on) { g_cluster_splitk = on ? 1 : 0; }

// Megabytes of weight tiles (over the whole grid) that a weight-streaming GEMM pulls into L2
// ahead of its shared-memory ring; 0 turns the prefetch off.
void zb_set_l2_prefetch_mb(int mb) { g_l2_prefetch_mb = mb < 0 ? 0 : (mb > 96 ? 96 : mb); }

// Tile shape and grid for a problem: swap-AB for few tokens, and a stream-K grid in
// which every CTA owns at least `min_units` k-blocks.  `split_hint` > 0 asks for about
// that many CTAs per output tile (used by tests).  Returns the number of output tiles.
int zb_gemm_plan(int m, int n, int k, int num_sms, int split_hint, int* swap, int* bn, int* grid,
                 int* units_per_cta, int* rr_tiles) {
  const int kb_total = (k + kBlockK - 1) / kBlockK;
  const int sw = m <= 256 ? 1 : 0;
  int b;
  if (sw) {
    b = 16;
    while (b < m) b <<= 1;
  } else {
    b = n >= 256 ? 256 : 128;
  }
  const int rows_p = sw ? n : m;
  const int rows_q = sw ? m : n;
  const int tiles = ((rows_p + kBlockP - 1) / kBlockP) * ((rows_q + b - 1) / b);
  *swap = sw;
  *bn = b;
  if (tiles >= 4 * num_sms && split_hint <= 0) {
    // many tiles: whole tiles, round-robin; wave quantisation is below 1/4 of a wave in 4+
    const int per = (tiles + num_sms - 1) / num_sms;
    *grid = num_sms;
    *rr_tiles = per;
    *units_per_cta = per * kb_total;
    return tiles;
  }
  *rr_tiles = 0;
  const long long total = static_cast<long long>(tiles) * kb_total;
  const int min_units = 4;
  long long g = total / min_units;
  if (g < 1) g = 1;
  if (g > num_sms) g = num_sms;
  if (split_hint > 0) {
    g = static_cast<long long>(tiles) * split_hint;
    if (g > num_sms) g = num_sms;
    if (g > total) g = total;
  }
  int upc = static_cast<int>((total + g - 1) / g);
  g = (total + upc - 1) / upc;            // drop CTAs that would get nothing
  *grid = static_cast<int>(g);
  *units_per_cta = upc;
  return tiles;
}

size_t zb_gemm_workspace_bytes(int m, int n, int k, int num_sms) {
  int sw, bn, grid, upc, rr;
  zb_gemm_plan(m, n, k, num_sms, 0, &sw, &bn, &grid, &upc, &rr);
  return static_cast<size_t>(grid) * 2 * bn * kBlockP * sizeof(float);
}

}  // extern "C"

int zb_gemm_2cta_wants(int m, int n, int k);
int zb_gemm_2cta_launch(const void* a, const void* w, void* out, const void* residual, const void* bias, int m, int n, int k, int lda,
                        int ldw, int ldo, int out_f32, const ZbGemmEpi* epi, ZbStatus* status, int num_sms, cudaStream_t stream);

namespace {

int launch_row_sumsq(const void* x, int rows, int d, long long ld, float* out, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((d % 8) != 0 || (ld % 8) != 0) return -10;
  const cudaError_t e = zb_launch(zb_row_sumsq_kernel, dim3(static_cast<unsigned>(rows)), dim3(256), 0, stream,
                                  reinterpret_cast<const __nv_bfloat16*>(x), ld, d, out);
  zb_count_launch(1);
  return static_cast<int>(e != cudaSuccess ? e : cudaGetLastError());
}

// Checks the epilogue options against the problem; returns 0 when they can be honoured.
int check_epi(const ZbGemmEpi* epi, int m, int n, int ldo, int out_f32, const void* residual, const void* bias) {
  if (epi == nullptr) return 0;
  if (epi->in_sumsq != nullptr && (epi->in_parts < 1 || epi->in_ld < m)) return -15;
  if (epi->swiglu) {
    // gate / up pairs: an even number of weight rows, bf16 output of n / 2 columns, no bias or residual
    if ((n % 2) != 0 || out_f32 || residual != nullptr || bias != nullptr || (ldo % 8) != 0 || epi->out_sumsq != nullptr) return -16;
  }
  if (epi->out_sumsq != nullptr && (out_f32 || epi->out_ld < m)) return -17;
  if (epi->pf_bytes != 0ull && (epi->pf_ptr == nullptr || (reinterpret_cast<uintptr_t>(epi->pf_ptr) & 15) != 0)) return -18;
  return 0;
}

// The GEMM proper.  `epi` may be null.  `out_parts` (may be null) receives the number of sum-of-squares
// parts written to epi->out_sumsq: tiles x cluster size when the cluster epilogue emits them, else 1 (a
// follow-up kernel over the finished output).
int gemm_impl(const void* a, const void* w, void* out, const void* residual, const void* bias,
              int m, int n, int k, int lda, int ldw, int ldo, int out_f32, int split_hint,
              float* scratch, size_t scratch_bytes, uint32_t* counters, int counters_len,
              ZbStatus* status, int num_sms, const ZbGemmEpi* epi, int* out_parts, cudaStream_t stream,
              const ZbBandPipe* band = nullptr) {
  if (out_parts) *out_parts = 0;
  if (m <= 0 || n <= 0 || k <= 0) return 0;
  if ((k % 8) != 0 || (lda % 8) != 0 || (ldw % 8) != 0) return -10;
  const int static_w = (out_f32 >> 1) & 1;
  out_f32 &= 1;
  if (!out_f32 && (ldo % 8) != 0) return -11;
  int rc = check_epi(epi, m, n, ldo, out_f32, residual, bias);
  if (rc != 0) return rc;
  if ((band == nullptr || band->mode == 0) && split_hint <= 0 && zb_gemm_2cta_wants(m, n, k)) {
    // prefill-sized: 256 x 256 tiles on pairs of SMs (gemm_2cta.cu); the row statistics of the output, when asked
    // for, come from the follow-up kernel as on every plan without an emitting epilogue
    rc = zb_gemm_2cta_launch(a, w, out, residual, bias, m, n, k, lda, ldw, ldo, out_f32, epi, status, num_sms, stream);
    if (rc == 0 && epi != nullptr && epi->out_sumsq != nullptr) {
      if (out_parts) *out_parts = 1;
      rc = launch_row_sumsq(out, m, n, ldo, epi->out_sumsq, stream);
    }
    return rc;
  }
  int sw, bn, grid, upc, rr;
  const int tiles = zb_gemm_plan(m, n, k, num_sms, split_hint, &sw, &bn, &grid, &upc, &rr);
  int cluster = 1;
  if (sw && rr == 0 && split_hint <= 0) cluster = plan_cluster(bn, tiles, (k + kBlockK - 1) / kBlockK, num_sms, &grid, &upc);
  if (band != nullptr && band->mode != 0) {
    // band pipeline: whole tiles only (a band is complete when its column tiles are), tokens as rows, and on the
    // consumer side the first comm_ctas CTAs of the grid do the reduction instead of tiles
    if (sw || cluster > 1) return -70;
    const int workers = num_sms - (band->mode == 2 ? band->comm_ctas : 0);
    if (workers < 1) return -70;
    rr = (tiles + workers - 1) / workers;
    grid = num_sms;
    upc = rr * ((k + kBlockK - 1) / kBlockK);
  }
  if (cluster == 1 && rr == 0 && static_cast<size_t>(grid) * 2 * bn * kBlockP * sizeof(float) > scratch_bytes) return -13;
  if (tiles > counters_len) return -14;
  GemmParams prm;
  prm.band = ZbBandPipe{};
  if (band != nullptr) {
    prm.band = *band;
    prm.band.tiles_per_band = (n + bn - 1) / bn;
  }
  prm.cluster = cluster;
  prm.rows_p = sw ? n : m;
  prm.rows_q = sw ? m : n;
  prm.k = k;
  prm.ldo = ldo;
  prm.out = out;
  prm.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  prm.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  prm.out_f32 = out_f32;
  prm.flags = static_w;
  prm.l2_prefetch = l2_prefetch_tiles(sw, bn, grid, rr);
  prm.timeline = next_timeline(grid);
  prm.group_p = (band != nullptr && band->mode != 0) ? 8 : 16;     // band pipeline: bands finish (and start) in groups of 8
  prm.units_per_cta = upc;
  prm.rr_tiles = rr;
  prm.workspace = scratch;
  prm.counters = counters;
  prm.status = status;
  prm.epi = ZbGemmEpi{};
  bool sumsq_after = false;
  if (epi != nullptr) {
    prm.epi = *epi;
    if (epi->out_sumsq != nullptr) {
      if (cluster > 1) {
        if (out_parts) *out_parts = tiles * cluster;
      } else {
        prm.epi.out_sumsq = nullptr;      // no emitting epilogue on this plan: one part from a follow-up kernel
        sumsq_after = true;
        if (out_parts) *out_parts = 1;
      }
    }
  }
  CUtensorMap tp, tq;
  rc = zb_make_tmap_bf16_2d(&tp, sw ? w : a, prm.rows_p, k, sw ? ldw : lda, kBlockP);
  if (rc != 0) return rc;
  rc = zb_make_tmap_bf16_2d(&tq, sw ? a : w, prm.rows_q, k, sw ? lda : ldw, bn);
  if (rc != 0) return rc;
  rc = -12;
#define ZB_GEMM_CASE(BN_)                                                           \
  case BN_:                                                                         \
    rc = launch<BN_, true>(tp, tq, prm, grid, stream);                              \
    break;
  if (band != nullptr && band->mode != 0) {
    if (bn == 256) rc = launch<256, false, 2>(tp, tq, prm, grid, stream);
    else if (bn == 128) rc = launch<128, false, 2>(tp, tq, prm, grid, stream);
  } else if (!sw) {
    if (bn == 256) rc = launch<256, false>(tp, tq, prm, grid, stream);
    else if (bn == 128) rc = launch<128, false>(tp, tq, prm, grid, stream);
  } else {
    switch (bn) {
      ZB_GEMM_CASE(16)
      ZB_GEMM_CASE(32)
      ZB_GEMM_CASE(64)
      ZB_GEMM_CASE(128)
      ZB_GEMM_CASE(256)
    }
  }
#undef ZB_GEMM_CASE
  if (rc == 0 && sumsq_after) rc = launch_row_sumsq(out, m, n, ldo, epi->out_sumsq, stream);
  return rc;
}

}  // namespace

extern "C" {

// out[M,N] = a[M,K] * w[N,K]^T (+bias) (+residual).  `out_f32` is a bit set: bit 0 selects an
// fp32 output, bit 1 states that `w` is a parameter (not written by the kernel that precedes
// this one on the stream), which lets the kernel request weight tiles while that kernel is
// still finishing.  `scratch` receives the partial
// tiles of CTAs whose k-range does not cover a whole tile (2 per CTA); `counters`
// holds one zeroed u32 per output tile (kept zero by the kernel).
int zb_gemm_bf16_ex(const void* a, const void* w, void* out, const void* residual, const void* bias,
                    int m, int n, int k, int lda, int ldw, int ldo, int out_f32, int split_hint,
                    float* scratch, size_t scratch_bytes, uint32_t* counters, int counters_len,
                    ZbStatus* status, int num_sms, cudaStream_t stream) {
  return gemm_impl(a, w, out, residual, bias, m, n, k, lda, ldw, ldo, out_f32, split_hint, scratch, scratch_bytes,
                   counters, counters_len, status, num_sms, nullptr, nullptr, stream);
}

// Scratch bytes the launch of [m, n, k] needs (the plan `zb_gemm_bf16_ex` will run, cluster plans included:
// those reduce through shared memory and need none).
size_t zb_gemm_scratch_needed(int m, int n, int k, int num_sms) {
  int sw, bn, grid, upc, rr;
  const int tiles = zb_gemm_plan(m, n, k, num_sms, 0, &sw, &bn, &grid, &upc, &rr);
  if (sw && rr == 0 && plan_cluster(bn, tiles, (k + kBlockK - 1) / kBlockK, num_sms, &grid, &upc) > 1) return 0;
  return static_cast<size_t>(grid) * 2 * bn * kBlockP * sizeof(float);
}

// Sum of squares of the rows of a bf16 matrix [rows, d] (leading dimension ld) -> out[rows] fp32.
int zb_row_sumsq(const void* x, int rows, int d, long long ld, float* out, void* stream) {
  return launch_row_sumsq(x, rows, d, ld, out, reinterpret_cast<cudaStream_t>(stream));
}

// zb_gemm_bf16 with the epilogue options of ZbGemmEpi (host_api.h) passed as scalars:
//   in_sumsq [in_parts][in_ld], inv_d, eps  -> accumulators of token t scaled by rsqrt(sum * inv_d + eps)
//   swiglu                                  -> interleaved gate / up rows, n / 2 output columns
//   out_sumsq [..][out_ld], *out_parts      -> partial sums of squares of the output rows and how many parts
//   pf_ptr, pf_bytes                        -> bytes to pull into L2 behind this kernel's own loads
int zb_gemm_bf16_epi(const void* a, const void* w, void* out, const void* residual, const void* bias, int m, int n, int k,
                     int lda, int ldw, int ldo, int out_f32, int split_hint, const float* in_sumsq, int in_parts, int in_ld,
                     float in_inv_d, float in_eps, int swiglu, float* out_sumsq, int out_ld, int* out_parts,
                     const void* pf_ptr, unsigned long long pf_bytes, void* stream) {
  ZbDeviceState* st = zb_device_state();
  if (st == nullptr) return -20;
  ZbGemmEpi epi = {};
  epi.in_sumsq = in_sumsq;
  epi.in_parts = in_parts;
  epi.in_ld = in_ld;
  epi.in_inv_d = in_inv_d;
  epi.in_eps = in_eps;
  epi.swiglu = swiglu ? 1 : 0;
  epi.out_sumsq = out_sumsq;
  epi.out_ld = out_ld;
  epi.pf_ptr = pf_bytes ? pf_ptr : nullptr;
  epi.pf_bytes = pf_ptr ? pf_bytes : 0ull;
  return gemm_impl(a, w, out, residual, bias, m, n, k, lda, ldw, ldo, out_f32, split_hint, st->gemm_scratch,
                   st->gemm_scratch_bytes, st->gemm_counters, st->gemm_counters_len, st->status, st->num_sms, &epi,
                   out_parts, reinterpret_cast<cudaStream_t>(stream));
}

// The decomposition zb_gemm_bf16 would use for [m, n, k]: out[0..5] = swap-AB, tile columns, grid, k-blocks per
// CTA, cluster size (1: none), resident-CTA capacity of that cluster size (0 without a cluster).
int zb_gemm_describe_plan(int m, int n, int k, int* out6) {
  ZbDeviceState* st = zb_device_state();
  if (st == nullptr) return -20;
  int sw, bn, grid, upc, rr;
  const int tiles = zb_gemm_plan(m, n, k, st->num_sms, 0, &sw, &bn, &grid, &upc, &rr);
  int cluster = 1;
  if (sw && rr == 0) cluster = plan_cluster(bn, tiles, (k + kBlockK - 1) / kBlockK, st->num_sms, &grid, &upc);
  int cap = 0;
  if (cluster > 1) cap = zb_gemm_cluster_capacity_of(bn, cluster);
  out6[0] = sw, out6[1] = bn, out6[2] = grid, out6[3] = upc, out6[4] = cluster, out6[5] = cap;
  return 0;
}

// Resident-CTA capacity of the swap-AB kernel (tile of `bn` tokens) launched in clusters of `s`.
int zb_gemm_cluster_capacity(int bn, int s) { return zb_gemm_cluster_capacity_of(bn, s); }

// Convenience entry point using the library's per-device scratch (see runtime.cu).
int zb_gemm_bf16(const void* a, const void* w, void* out, const void* residual, const void* bias,
                 int m, int n, int k, int lda, int ldw, int ldo, int out_f32, int split_hint,
                 void* stream) {
  ZbDeviceState* st = zb_device_state();
  if (st == nullptr) return -20;
  return zb_gemm_bf16_ex(a, w, out, residual, bias, m, n, k, lda, ldw, ldo, out_f32, split_hint,
                         st->gemm_scratch, st->gemm_scratch_bytes, st->gemm_counters,
                         st->gemm_counters_len, st->status, st->num_sms,
                         reinterpret_cast<cudaStream_t>(stream));
}

// Prefill collectives overlapped band by band (ZbBandPipe in host_api.h).  All ranks call both modes with the same
// shapes, in the same order, producer first.
//   mode 1: part[tokens, d] (at part_off of this rank's heap) = a[tokens, k] * w[d, k]^T; bands of 128 tokens are
//           announced to their owners as their last column tile is stored.
//   mode 2: out[tokens, n] = f(x[tokens, d]) * w[n, d]^T (+ bias) where x (at x_off of every heap) = residual +
//           sum over ranks of part, pulled from and pushed to the peers' heaps with bulk copies by the first `comm_ctas`
//           CTAs of this launch while the other CTAs multiply the bands that are already there; f is the RMSNorm
//           scale of the row (statistics travel with the band; eps < 0: none); `swiglu` as in zb_gemm_bf16_epi.
// `flag_off` addresses the pipeline's flag region in every heap, laid out for `nb_cap` bands:
// ready [nb_cap][8] u32 | done [nb_cap] | producer counts [nb_cap] | consumer counts [nb_cap] | row statistics
// [nb_cap * 128] fp32 (256-byte aligned).  Needs tokens > 256 and a hidden size whose rows are a multiple of 16 bytes.
size_t zb_band_flag_bytes(int nb_cap) {
  return ((static_cast<size_t>(nb_cap) * 44 + 255) / 256) * 256 + static_cast<size_t>(nb_cap) * 128 * 4;
}

int zb_gemm_band(const ZbArContext* ctx, int mode, const void* a, const void* w, void* out, const void* bias,
                 const void* residual, int tokens, int n, int k, int lda, int ldw, int ldo, size_t part_off, size_t x_off,
                 size_t flag_off, int nb_cap, int comm_ctas, int swiglu, float eps, void* stream) {
  ZbDeviceState* st = zb_device_state();
  if (st == nullptr || ctx == nullptr) return -20;
  if (mode != 1 && mode != 2) return -10;
  const int nb = (tokens + kBlockP - 1) / kBlockP;
  if (tokens <= 256 || nb > nb_cap || (part_off % 16) != 0 || (x_off % 16) != 0 || (flag_off % 256) != 0) return -70;
  if (mode == 2 && (comm_ctas < 1 || comm_ctas >= st->num_sms)) return -70;
  ZbBandPipe bp = {};
  bp.mode = mode;
  bp.num_bands = nb;
  bp.comm_ctas = comm_ctas;
  bp.world = ctx->world;
  bp.rank = ctx->rank;
  bp.tokens = tokens;
  bp.d = mode == 1 ? n : k;
  bp.epoch = ctx->epoch + 10;
  const size_t stats_off = ((static_cast<size_t>(nb_cap) * 44 + 255) / 256) * 256;
  for (int r = 0; r < ctx->world; ++r) {
    char* base = reinterpret_cast<char*>(ctx->heap[r]) + flag_off;
    bp.ready_peer[r] = reinterpret_cast<uint32_t*>(base);
    bp.done_peer[r] = reinterpret_cast<uint32_t*>(base + static_cast<size_t>(nb_cap) * 32);
    bp.sumsq_peer[r] = reinterpret_cast<float*>(base + stats_off);
  }
  char* mine = reinterpret_cast<char*>(ctx->heap[ctx->rank]);
  bp.count_p = reinterpret_cast<uint32_t*>(mine + flag_off + static_cast<size_t>(nb_cap) * 36);
  bp.count_c = reinterpret_cast<uint32_t*>(mine + flag_off + static_cast<size_t>(nb_cap) * 40);
  for (int r = 0; r < ctx->world; ++r) bp.heap[r] = reinterpret_cast<char*>(ctx->heap[r]);
  bp.part_off = part_off;
  bp.x_off = x_off;
  bp.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (mode == 1) {
    // `w` is a parameter (flag bit 1): its tiles may be requested before the preceding kernel has finished
    return gemm_impl(a, w, mine + part_off, nullptr, nullptr, tokens, n, k, lda, ldw, n, 2, 0, st->gemm_scratch,
                     st->gemm_scratch_bytes, st->gemm_counters, st->gemm_counters_len, st->status, st->num_sms, nullptr, nullptr,
                     s, &bp);
  }
  ZbGemmEpi epi = {};
  if (eps >= 0.f) {
    epi.in_sumsq = bp.sumsq_peer[ctx->rank];
    epi.in_parts = 1;
    epi.in_ld = tokens;
    epi.in_inv_d = 1.0f / static_cast<float>(k);
    epi.in_eps = eps;
  }
  epi.swiglu = swiglu ? 1 : 0;
  return gemm_impl(mine + x_off, w, out, nullptr, bias, tokens, n, k, k, ldw, ldo, 2, 0, st->gemm_scratch, st->gemm_scratch_bytes,
                   st->gemm_counters, st->gemm_counters_len, st->status, st->num_sms, &epi, nullptr, s, &bp);
}

// Row-parallel GEMM fused with the tensor-parallel all-reduce (and bias / residual):
//   out_r = sum over ranks r' of a_r'[M,K_r'] * w_r'[N,K_r']^T (+ bias) (+ residual), on every rank.
// `out_off` is the byte offset of the output inside every rank's symmetric heap.  All ranks
// must call this with the same shapes, in the same order.  See fused_ar.h for the protocol.
// `out_sumsq` (may be null) receives partial sums of squares of the finished output rows, [*out_parts][out_ld];
// `pf_ptr` / `pf_bytes` name the next GEMM's weights, pulled into L2 while the exchange with the peers runs.
int zb_gemm_ar_fused_epi(const ZbArContext* ctx, const void* a, const void* w, size_t out_off,
                         const void* residual, const void* bias, int m, int n, int k, int lda, int ldw,
                         int ldo, int split_hint, float* out_sumsq, int out_ld, int* out_parts, const void* pf_ptr,
                         unsigned long long pf_bytes, void* stream) {
  if (out_parts) *out_parts = 0;
  if (ctx == nullptr || ctx->world < 1 || ctx->world > kZbMaxRanks) return -50;
  if (m <= 0 || n <= 0 || k <= 0) return 0;
  if (out_sumsq != nullptr && out_ld < m) return -17;
  if (pf_bytes != 0ull && (pf_ptr == nullptr || (reinterpret_cast<uintptr_t>(pf_ptr) & 15) != 0)) return -18;
  if ((k % 8) != 0 || (lda % 8) != 0 || (ldw % 8) != 0 || (ldo % 8) != 0 || (out_off % 16) != 0) return -10;
  ZbDeviceState* st = zb_device_state();
  if (st == nullptr) return -20;
  int sw, bn, grid, upc, rr;
  const int tiles = zb_gemm_plan(m, n, k, st->num_sms, split_hint, &sw, &bn, &grid, &upc, &rr);
  if (static_cast<size_t>(grid) * 2 * bn * kBlockP * sizeof(float) > st->gemm_scratch_bytes) return -13;
  if (tiles > st->gemm_counters_len) return -14;
  int cluster = 1;
  const bool one_shot_fits = sw && bn <= 64 && static_cast<long long>(tiles) * ctx->world <= ctx->max_tiles &&
                             2 * static_cast<size_t>(ctx->world) * tiles * kBlockP * bn * 2 <= ctx->recv_bytes;
  if (one_shot_fits && rr == 0 && split_hint <= 0) {
    int cg = grid, cu = upc;
    const int cs = plan_cluster(bn, tiles, (k + kBlockK - 1) / kBlockK, st->num_sms, &cg, &cu, /*allow_tiny=*/false);
    // the tensor-parallel epilogue keeps at most 32 elements per thread (two halves of 16); bands have even heights
    if (cs > 1 && bn * (2 * ((kBlockP / 2 + cs - 1) / cs)) <= 32 * kEpiThreads &&
        2 * static_cast<size_t>(ctx->world) * tiles * cs * 16 * kEpiThreads * sizeof(uint2) <= ctx->recv_bytes) {
      cluster = cs;
      grid = cg;
      upc = cu;
    }
  }
  GemmParams prm;
  prm.band = ZbBandPipe{};
  prm.cluster = cluster;
  prm.rows_p = sw ? n : m;
  prm.rows_q = sw ? m : n;
  prm.k = k;
  prm.ldo = ldo;
  prm.out = nullptr;
  prm.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  prm.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  prm.out_f32 = 0;
  prm.flags = 1;     // `w` is a model parameter in every use of the fused kernel
  prm.l2_prefetch = l2_prefetch_tiles(sw, bn, grid, rr);
  prm.timeline = next_timeline(grid);
  prm.group_p = 16;
  prm.units_per_cta = upc;
  prm.rr_tiles = rr;
  prm.workspace = st->gemm_scratch;
  prm.counters = st->gemm_counters;
  prm.status = st->status;
  prm.epi = ZbGemmEpi{};
  prm.epi.pf_ptr = pf_bytes ? pf_ptr : nullptr;
  prm.epi.pf_bytes = pf_ptr ? pf_bytes : 0ull;
  bool sumsq_after = false;
  if (out_sumsq != nullptr) {
    if (cluster > 1) {
      prm.epi.out_sumsq = out_sumsq;
      prm.epi.out_ld = out_ld;
      if (out_parts) *out_parts = tiles * cluster;
    } else {
      sumsq_after = true;
      if (out_parts) *out_parts = 1;
    }
  }
  ZbFusedAr& ar = prm.ar;
  ar.rank = ctx->rank;
  ar.world = ctx->world;
  ar.slots_per_src = (tiles + ctx->world - 1) / ctx->world;
  ar.one_shot = (sw && bn <= 64) ? 1 : 0;
  size_t need = static_cast<size_t>(ctx->world) * ar.slots_per_src * kBlockP * bn * 2;
  if (ar.one_shot) {
    need = 2 * static_cast<size_t>(ctx->world) * tiles * kBlockP * bn * 2;          // two halves, every source, every tile
    if (static_cast<long long>(tiles) * ctx->world > ctx->max_tiles) ar.one_shot = 0;
    if (need > ctx->recv_bytes) ar.one_shot = 0;
    if (!ar.one_shot) need = static_cast<size_t>(ctx->world) * ar.slots_per_src * kBlockP * bn * 2;
  }
  if (need > ctx->recv_bytes || tiles > ctx->max_tiles) return -51;
  for (int r = 0; r < ctx->world; ++r) {
    char* base = reinterpret_cast<char*>(ctx->heap[r]);
    ar.recv_peer[r] = reinterpret_cast<__nv_bfloat16*>(base + ctx->recv_off);
    ar.out_peer[r] = reinterpret_cast<__nv_bfloat16*>(base + out_off);
    ar.push_flag_peer[r] = reinterpret_cast<uint32_t*>(base + ctx->push_flag_off);
    ar.done_flag_peer[r] = reinterpret_cast<uint32_t*>(base + ctx->done_flag_off);
  }
  ar.epoch = ctx->epoch;
  ar.exit_ticket = ctx->exit_ticket;
  CUtensorMap tp, tq;
  int rc = zb_make_tmap_bf16_2d(&tp, sw ? w : a, prm.rows_p, k, sw ? ldw : lda, kBlockP);
  if (rc != 0) return rc;
  rc = zb_make_tmap_bf16_2d(&tq, sw ? a : w, prm.rows_q, k, sw ? lda : ldw, bn);
  if (rc != 0) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  rc = -12;
#define ZB_GEMM_CASE(BN_)                                                     \
  case BN_:                                                                   \
    rc = launch<BN_, true, 1>(tp, tq, prm, grid, s);                          \
    break;
  if (!sw) {
    if (bn == 256) rc = launch<256, false, 1>(tp, tq, prm, grid, s);
    else if (bn == 128) rc = launch<128, false, 1>(tp, tq, prm, grid, s);
  } else {
    switch (bn) {
      ZB_GEMM_CASE(16)
      ZB_GEMM_CASE(32)
      ZB_GEMM_CASE(64)
      ZB_GEMM_CASE(128)
      ZB_GEMM_CASE(256)
    }
  }
#undef ZB_GEMM_CASE
  if (rc == 0 && sumsq_after)
    rc = launch_row_sumsq(reinterpret_cast<const char*>(ctx->heap[ctx->rank]) + out_off, m, n, ldo, out_sumsq, s);
  return rc;
}

int zb_gemm_ar_fused(const ZbArContext* ctx, const void* a, const void* w, size_t out_off,
                     const void* residual, const void* bias, int m, int n, int k, int lda, int ldw,
                     int ldo, int split_hint, void* stream) {
  return zb_gemm_ar_fused_epi(ctx, a, w, out_off, residual, bias, m, n, k, lda, ldw, ldo, split_hint, nullptr, 0, nullptr,
                              nullptr, 0ull, stream);
}

}  // extern "C"
