// bf16 GEMM for prefill-sized problems on PAIRS of SMs: out[M,N] = A[M,K] * W[N,K]^T with the epilogue
// options of the one-SM kernel (bias, residual, fp32 output, RMSNorm row scale, SwiGLU).
//
// The reference leaves dense contractions to cuBLASLt / XLA (zml/tensor.zig:1388-1459).  The one-SM kernel
// of gemm_bf16.cu is bound by shared-memory bandwidth on 128 x 256 tiles: every k-block of a tile moves
// 48 KB of operands through one SM's shared memory.  Here two CTAs of a cluster own one 256 x 256 tile
// (`tcgen05.mma.cta_group::2`): each CTA loads 128 rows of A and 128 rows of W per k-block (32 KB), the
// tensor cores of both SMs read both halves of W, and each SM accumulates its own 128 rows of the tile in
// its tensor memory - a third less shared-memory traffic per FLOP.  No load carries a multicast qualifier:
// each CTA fetches its own halves.
//
// Roles per CTA (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer (leader CTA only), warps 2-5 =
// epilogue of this CTA's 128 rows.  Synchronisation of the pair:
//   full[s]      (leader's)  the loads of BOTH CTAs complete their bytes on the leader's barrier
//   empty[s]     (each CTA)  the leader's commit is multicast to both CTAs when the MMAs of a stage retire
//   tmem_full[a] (each CTA)  multicast commit after the last k-block of a tile
//   tmem_empty[a](leader's)  one arrival per CTA once its epilogue has read accumulator stage a
// Tiles are dealt round-robin to the clusters (persistent kernel, two accumulator stages so that the
// epilogue of a tile overlaps the main loop of the next one).  Every wait is bounded.
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"
#include "host_api.h"

int zb_make_tmap_bf16_2d(CUtensorMap* out, const void* base, int rows, int k, int ld, int box_rows);

namespace {

constexpr int kBM = 128;          // rows of A per CTA (256 per pair)
constexpr int kBNH = 128;         // rows of W per CTA (the pair's tile is 256 columns wide)
constexpr int kBN = 2 * kBNH;
constexpr int kBK = 64;
constexpr int kStages = 6;
constexpr int kStageBytes = (kBM + kBNH) * kBK * 2;          // 32 KB
constexpr int kTileABytes = kBM * kBK * 2;
constexpr int kThreads = 192;
constexpr int kEpiThreads = 128;
constexpr uint32_t kKernelId = 14;
constexpr uint32_t kTmemCols = 512;                           // two accumulator stages of 256 fp32 columns
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;               // clears the CTA-rank bit of a shared::cluster address

struct Gemm2Params {
  int m, n, k;
  int ldo;
  void* out;
  const __nv_bfloat16* residual;
  const __nv_bfloat16* bias;
  int out_f32;
  int num_m, num_n;             // tiles of 256 x 256
  int group_m;                  // rasterisation: tiles of `group_m` consecutive row blocks share their W tiles in L2
  ZbGemmEpi epi;                // row scale (in_sumsq, in_parts, in_ld, in_inv_d, in_eps) and swiglu are honoured
  ZbStatus* status;
};

ZB_DEVICE void tma_load_2d_pair(void* smem_dst, const void* tmap, uint32_t leader_bar, int32_t x, int32_t y) {
  // the bytes of this copy are counted on the LEADER CTA's barrier (`leader_bar` has the rank bit cleared)
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(zb_smem_u32(smem_dst)), "l"(tmap), "r"(leader_bar), "r"(x), "r"(y)
      : "memory");
}

ZB_DEVICE void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  const uint32_t z = 0u;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(z)
      : "memory");
}

// Arrives on the barrier at the same shared-memory offset in both CTAs of the pair once every tcgen05
// operation issued so far by this thread has completed.
ZB_DEVICE void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   zb_smem_u32(bar)),
               "h"(mask)
               : "memory");
}

ZB_DEVICE void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

ZB_DEVICE void epi_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
ZB_DEVICE float silu2(float g) { return g / (1.f + __expf(-g)); }

__global__ void __launch_bounds__(kThreads, 1)
zb_gemm_2cta_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w, const Gemm2Params prm) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full = empty_bar + kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile uint32_t* abort_flag = tmem_holder + 1;
  volatile uint32_t* abort_where = tmem_holder + 2;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta_rank = zb_cluster_ctarank();              // 0: leader
  const int cluster_id = static_cast<int>(blockIdx.x >> 1);
  const int n_clusters = static_cast<int>(gridDim.x >> 1);
  const int kb_total = (prm.k + kBK - 1) / kBK;
  const int num_tiles = prm.num_m * prm.num_n;

  auto decode = [&](int t, int& mt, int& nt) {
    const int per_group = prm.group_m * prm.num_n;
    const int g = t / per_group;
    const int within = t - g * per_group;
    const int m_first = g * prm.group_m;
    const int gm = min(prm.group_m, prm.num_m - m_first);
    mt = m_first + within % gm;
    nt = within / gm;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      zb_mbar_init(&full_bar[s], 1);
      zb_mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      zb_mbar_init(&tmem_full[a], 1);
      zb_mbar_init(&tmem_empty[a], 2);               // one arrival per CTA of the pair
    }
    *abort_flag = 0u;
    *abort_where = 0u;
    zb_mbar_fence_init();
    zb_tma_prefetch_desc(&tmap_a);
    zb_tma_prefetch_desc(&tmap_w);
  }
  if (warp == 1) {
    // the same warp of both CTAs allocates: the columns are reserved in both SMs' tensor memory
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(zb_smem_u32(tmem_holder)), "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  zb_tc_fence_before();
  __syncthreads();
  zb_tc_fence_after();
  // both CTAs' barriers must exist before either side signals the other
  zb_cluster_arrive();
  zb_cluster_wait();
  const uint32_t tmem_base = *tmem_holder;
  zb_pdl_launch();
  zb_pdl_wait();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int t = cluster_id; ok && t < num_tiles; t += n_clusters) {
        int mt, nt;
        decode(t, mt, nt);
        const int row_a = mt * (2 * kBM) + static_cast<int>(cta_rank) * kBM;
        const int row_w = nt * kBN + static_cast<int>(cta_rank) * kBNH;
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!zb_mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) {
            *abort_where = 1u;
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * kStageBytes;
          const uint32_t lbar = zb_smem_u32(&full_bar[stage]) & kPeerBitMask;
          if (cta_rank == 0) zb_mbar_expect_tx(&full_bar[stage], 2 * kStageBytes);       // both CTAs' bytes
          tma_load_2d_pair(sa, &tmap_a, lbar, kb * kBK, row_a);
          tma_load_2d_pair(sa + kTileABytes, &tmap_w, lbar, kb * kBK, row_w);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (cta_rank == 0 && lane == 0) {
      constexpr uint32_t kIdesc = zb_make_idesc_bf16(2 * kBM, kBN);
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int t = cluster_id; ok && t < num_tiles; t += n_clusters) {
        if (!zb_mbar_wait(&tmem_empty[acc], acc_phase ^ 1u, abort_flag)) {
          *abort_where = 2u;
          break;
        }
        zb_tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * kBN;
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!zb_mbar_wait(&full_bar[stage], phase, abort_flag)) {
            *abort_where = 3u;
            ok = false;
            break;
          }
          zb_tc_fence_after();
          const uint32_t sa = zb_smem_u32(smem + stage * kStageBytes);
          const uint64_t da = zb_make_desc_sw128(sa), db = zb_make_desc_sw128(sa + kTileABytes);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) umma_f16_pair(tmem_d, da + 2 * k, db + 2 * k, kIdesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit_pair(&empty_bar[stage]);       // both CTAs may refill this stage once the MMAs retire
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit_pair(&tmem_full[acc]);           // the accumulators of both CTAs are complete
        acc ^= 1u;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue: this CTA's 128 rows of the tile
    const int epi_tid = threadIdx.x - 64;
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    const uint32_t leader_empty0 = zb_mapa(zb_smem_u32(&tmem_empty[0]), 0u);
    uint32_t acc = 0, acc_phase = 0;
    for (int t = cluster_id; t < num_tiles; t += n_clusters) {
      int mt, nt;
      decode(t, mt, nt);
      const int p = mt * (2 * kBM) + static_cast<int>(cta_rank) * kBM + row_in_tile;      // output row (token)
      const int q0 = nt * kBN;
      float row_scale = 1.f;
      if (prm.epi.in_sumsq != nullptr) {
        const int pr = min(p, prm.m - 1);
        float ssum = 0.f;
        for (int i = 0; i < prm.epi.in_parts; ++i) ssum += __ldcg(prm.epi.in_sumsq + static_cast<size_t>(i) * prm.epi.in_ld + pr);
        row_scale = rsqrtf(ssum * prm.epi.in_inv_d + prm.epi.in_eps);
      }
      if (!zb_mbar_wait(&tmem_full[acc], acc_phase, abort_flag)) *abort_where = 4u;
      epi_sync();
      if (*abort_flag != 0u) break;
      zb_tc_fence_after();
      const uint32_t taddr = tmem_base + acc * kBN + (static_cast<uint32_t>(quad * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < kBN; c0 += 32) {
        uint32_t r[32];
        zb_tmem_ld32(taddr + c0, r);
        zb_tmem_ld_wait();
        if (p >= prm.m) continue;
        const int q = q0 + c0;
        if (q >= prm.n) continue;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * row_scale;
        const bool whole = q + 32 <= prm.n;
        if (prm.bias != nullptr) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (whole || q + j < prm.n) v[j] += __bfloat162float(prm.bias[q + j]);
        }
        if (prm.epi.swiglu) {
          // columns interleave gate and up: 16 outputs at columns q / 2 ..
          __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(prm.out) + static_cast<size_t>(p) * prm.ldo + (q >> 1);
          if (whole) {
            uint32_t w[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) w[j] = zb_pack_bf16x2(silu2(v[4 * j]) * v[4 * j + 1], silu2(v[4 * j + 2]) * v[4 * j + 3]);
            reinterpret_cast<uint4*>(op)[0] = make_uint4(w[0], w[1], w[2], w[3]);
            reinterpret_cast<uint4*>(op)[1] = make_uint4(w[4], w[5], w[6], w[7]);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (q + 2 * j + 1 < prm.n) op[j] = __float2bfloat16(silu2(v[2 * j]) * v[2 * j + 1]);
          }
          continue;
        }
        const size_t o = static_cast<size_t>(p) * prm.ldo + q;
        if (prm.residual != nullptr) {
          if (whole) {
            const uint4* rp = reinterpret_cast<const uint4*>(prm.residual + o);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint4 rr = rp[i];
              const uint32_t ru[4] = {rr.x, rr.y, rr.z, rr.w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 f = zb_unpack_bf16x2(ru[j]);
                v[8 * i + 2 * j] += f.x;
                v[8 * i + 2 * j + 1] += f.y;
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (q + j < prm.n) v[j] += __bfloat162float(prm.residual[o + j]);
          }
        }
        if (prm.out_f32) {
          float* op = reinterpret_cast<float*>(prm.out) + o;
          if (whole) {
#pragma unroll
            for (int j = 0; j < 8; ++j) reinterpret_cast<float4*>(op)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (q + j < prm.n) op[j] = v[j];
          }
        } else {
          __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(prm.out) + o;
          if (whole) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              reinterpret_cast<uint4*>(op)[i] = make_uint4(zb_pack_bf16x2(v[8 * i], v[8 * i + 1]), zb_pack_bf16x2(v[8 * i + 2], v[8 * i + 3]),
                                                           zb_pack_bf16x2(v[8 * i + 4], v[8 * i + 5]), zb_pack_bf16x2(v[8 * i + 6], v[8 * i + 7]));
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (q + j < prm.n) op[j] = __float2bfloat16(v[j]);
          }
        }
      }
      // this CTA has read accumulator stage `acc`: one arrival on the leader's barrier
      zb_tc_fence_before();
      epi_sync();
      if (epi_tid == 0) mbar_arrive_remote(leader_empty0 + acc * 8u);
      acc ^= 1u;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  // ------------------------------------------------------------ common exit
  zb_tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0u) {
    if (threadIdx.x == 0) zb_record_error(prm.status, ZB_ERR_MBAR_TIMEOUT, kKernelId, *abort_where, blockIdx.x);
    const uint64_t t0 = zb_globaltimer();            // copies still in flight must land before the shared memory is reused
    while (zb_globaltimer() - t0 < 200000ull) {
    }
    __syncthreads();
  }
  // neither CTA may leave (and free its shared / tensor memory) while the other can still touch it
  zb_cluster_arrive();
  zb_cluster_wait();
  if (warp == 1) {
    zb_tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;

}  // namespace

// 1 when the two-SM kernel takes the problem: tokens as rows (more than 256 of them) and at least one full tile of
// columns.  ZB_GEMM_2CTA=0 in the environment turns the kernel off.
int zb_gemm_2cta_wants(int m, int n, int k) {
  static int enabled = -1;
  if (enabled < 0) {
    const char* e = getenv("ZB_GEMM_2CTA");
    enabled = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return enabled && m >= 512 && n >= 256 && k >= 64;
}

// out[M,N] = a[M,K] * w[N,K]^T (* row scale) (+ bias) (+ residual) or its SwiGLU: same contract as the one-SM
// kernel's launch for the options it supports (epi->out_sumsq and epi->pf_* are ignored here; the caller
// handles them).  Returns 0 on success.
int zb_gemm_2cta_launch(const void* a, const void* w, void* out, const void* residual, const void* bias, int m, int n, int k, int lda,
                        int ldw, int ldo, int out_f32, const ZbGemmEpi* epi, ZbStatus* status, int num_sms, cudaStream_t stream) {
  static bool configured[16] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return -21;
  if (!configured[dev]) {
    cudaError_t e = zb_config_smem(zb_gemm_2cta_kernel, kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev] = true;
  }
  Gemm2Params prm = {};
  prm.m = m;
  prm.n = n;
  prm.k = k;
  prm.ldo = ldo;
  prm.out = out;
  prm.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  prm.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  prm.out_f32 = out_f32 & 1;
  prm.num_m = (m + 2 * kBM - 1) / (2 * kBM);
  prm.num_n = (n + kBN - 1) / kBN;
  prm.group_m = 8;
  if (epi != nullptr) prm.epi = *epi;
  prm.status = status;
  CUtensorMap ta, tw;
  int rc = zb_make_tmap_bf16_2d(&ta, a, m, k, lda, kBM);
  if (rc != 0) return rc;
  rc = zb_make_tmap_bf16_2d(&tw, w, n, k, ldw, kBNH);
  if (rc != 0) return rc;
  const int tiles = prm.num_m * prm.num_n;
  int clusters = num_sms / 2;
  if (clusters > tiles) clusters = tiles;
  const cudaError_t le = zb_launch_cluster(zb_gemm_2cta_kernel, dim3(2 * clusters), dim3(kThreads), kSmemBytes, stream, 2, ta, tw, prm);
  zb_count_launch(1);
  return static_cast<int>(le != cudaSuccess ? le : cudaGetLastError());
}
