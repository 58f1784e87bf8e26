// Grouped GEMM over experts whose weights are NVFP4 (e2m1 codes, two per byte, one f8e4m3fn
// scale per 16 values along K, one fp32 scale per expert matrix) with bf16 activations:
//
//   out[token, :] = xs[token, :] . dequant(W[expert(token)])^T       (+ SwiGLU for the gate|up GEMM)
//
// for the few-tokens-per-expert (decode) regime, where the expert weights are what the step
// reads from HBM: 4.5 bits per weight instead of 16.  Same warp-specialised structure as the bf16
// grouped kernel (moe.cu) with one more stage: a producer thread brings packed code tiles
// (128 weight rows x 32 bytes) and activation tiles in with TMA, four de-quantising warps turn a
// code tile into the bf16, 128-byte-swizzled operand tile that tcgen05.mma reads, one thread
// issues the MMAs into TMEM, four warps run the epilogue.
//
// The reference reaches this through the FlashInfer CUTLASS NVFP4 runner
// (zml/moe/cutlass_flashinfer.zig:275-330) or XLA's scaled-dot composite (zml/nn.zig:294-398).
#include <cuda.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "common.cuh"
#include "host_api.h"

int zb_make_tmap_bf16_2d(CUtensorMap* out, const void* base, int rows, int k, int ld, int box_rows);
int zb_make_tmap_u8_2d(CUtensorMap* out, const void* base, long long rows, long long row_bytes, int box_bytes, int box_rows);

namespace {

constexpr uint32_t kKernelGroupedW4 = 9;
constexpr int kBlockP = 128;
constexpr int kBlockK = 64;
constexpr int kUmmaK = 16;
constexpr int kThreads = 320;        // producer, MMA, 4 epilogue warps, 4 de-quantising warps
constexpr int kRawBytes = kBlockP * kBlockK / 2;      // packed codes of one weight tile

struct W4Params {
  const int32_t* offsets;   // [e_local + 1]
  int e_local;
  int n;                    // output features per expert
  int k;
  int ldo;
  __nv_bfloat16* out;
  int cap;
  const uint8_t* scales;    // [e_local * n, k / 16] f8e4m3fn
  const float* gscale;      // [e_local] per-matrix scale
  ZbStatus* status;
};

__host__ __device__ constexpr int w4_stages(int bn) { return bn >= 64 ? 5 : 6; }
__host__ __device__ constexpr int w4_stage_bytes(int bn) { return (kBlockP + bn) * kBlockK * 2 + kRawBytes; }

ZB_DEVICE void w4_epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
ZB_DEVICE void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

ZB_DEVICE float fp8_e4m3_to_float(uint32_t b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(b & 0xffu), __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

// 8 codes (one u32) x scale -> 8 bf16 (one 16-byte chunk)
ZB_DEVICE uint4 dequant8(uint32_t codes, float s) {
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2_raw hr = __nv_cvt_fp4x2_to_halfraw2(static_cast<__nv_fp4x2_storage_t>((codes >> (8 * i)) & 0xffu), __NV_E2M1);
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hr));
    o[i] = zb_pack_bf16x2(f.x * s, f.y * s);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

template <int BN, bool SWIGLU>
__global__ void __launch_bounds__(kThreads, 1)
zb_moe_grouped_gemm_w4_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                              const W4Params prm) {
  constexpr int kStages = w4_stages(BN);
  constexpr int kStageBytes = w4_stage_bytes(BN);
  constexpr int kTileABytes = kBlockP * kBlockK * 2;
  constexpr int kTileBBytes = BN * kBlockK * 2;
  constexpr uint32_t kTmemCols = (2 * BN) < 32 ? 32 : (2 * BN);
  constexpr uint32_t kIdesc = zb_make_idesc_bf16(kBlockP, BN);
  constexpr int kXchBytes = SWIGLU ? BN * 64 * 4 : 0;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  // stage s: [A bf16 tile 16 KB | B tile | raw codes 4 KB]; the raw tiles come after all operand tiles
  uint8_t* raw_base = smem + kStages * (kTileABytes + kTileBBytes);
  float* xch = reinterpret_cast<float*>(raw_base + kStages * kRawBytes);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(xch) + kXchBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* raw_full = empty_bar + kStages;
  uint64_t* raw_empty = raw_full + kStages;
  uint64_t* tmem_full = raw_empty + kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile uint32_t* abort_flag = tmem_holder + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb_total = prm.k / kBlockK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      zb_mbar_init(&full_bar[s], 1 + 4);     // producer (activation tile, with bytes) + one lane per de-quantising warp
      zb_mbar_init(&empty_bar[s], 1);        // MMA commit
      zb_mbar_init(&raw_full[s], 1);         // producer (code tile, with bytes)
      zb_mbar_init(&raw_empty[s], 4);        // one lane per de-quantising warp
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
  zb_pdl_launch();
  zb_pdl_wait();

  const int w_tiles = prm.n / kBlockP;
  auto token_tiles = [&](int e) { return (prm.offsets[e + 1] - prm.offsets[e] + BN - 1) / BN; };
  struct Cursor {
    int e, base;
  };
  auto locate = [&](Cursor& c, int g, int& wt, int& tt) -> bool {
    while (c.e < prm.e_local) {
      const int n_e = w_tiles * token_tiles(c.e);
      if (g < c.base + n_e) {
        const int local = g - c.base;
        tt = local / w_tiles;
        wt = local - tt * w_tiles;
        return true;
      }
      c.base += n_e;
      ++c.e;
    }
    return false;
  };
  auto a_tile = [&](uint32_t stage) { return smem + stage * (kTileABytes + kTileBBytes); };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      zb_tma_prefetch_desc(&tmap_x);
      zb_tma_prefetch_desc(&tmap_w);
      uint32_t stage = 0, phase = 0;
      Cursor c{0, 0};
      bool ok = true;
      for (int g = blockIdx.x; ok; g += gridDim.x) {
        int wt, tt;
        if (!locate(c, g, wt, tt)) break;
        const int tok0 = prm.offsets[c.e] + tt * BN;
        const int wrow0 = c.e * prm.n + wt * kBlockP;
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!zb_mbar_wait(&raw_empty[stage], phase ^ 1u, abort_flag) ||
              !zb_mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          zb_mbar_expect_tx(&raw_full[stage], kRawBytes);
          zb_tma_load_2d(raw_base + stage * kRawBytes, &tmap_w, &raw_full[stage], kb * (kBlockK / 2), wrow0);
          zb_mbar_expect_tx(&full_bar[stage], kTileBBytes);
          zb_tma_load_2d(a_tile(stage) + kTileABytes, &tmap_x, &full_bar[stage], kb * kBlockK, tok0);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
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
          const uint32_t sa = zb_smem_u32(a_tile(stage));
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
  } else if (warp >= 6) {
    // ------------------------------------------------------------------ de-quantisers: thread = weight row
    const int r = threadIdx.x - 192;                        // 0..127
    uint32_t stage = 0, phase = 0;
    Cursor c{0, 0};
    bool ok = true;
    for (int g = blockIdx.x; ok; g += gridDim.x) {
      int wt, tt;
      if (!locate(c, g, wt, tt)) break;
      const int wrow = c.e * prm.n + wt * kBlockP + r;
      const float gs = prm.gscale != nullptr ? prm.gscale[c.e] : 1.f;
      const uint32_t* srow = reinterpret_cast<const uint32_t*>(prm.scales + static_cast<size_t>(wrow) * (prm.k / 16));
      uint32_t s_next = __ldg(srow);                        // the 4 block scales of k-block 0
      for (int kb = 0; kb < kb_total; ++kb) {
        const uint32_t s4 = s_next;
        if (kb + 1 < kb_total) s_next = __ldg(srow + kb + 1);
        if (!zb_mbar_wait(&raw_full[stage], phase, abort_flag) || !zb_mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        const uint4* raw = reinterpret_cast<const uint4*>(raw_base + stage * kRawBytes + r * 32);
        const uint4 c0 = raw[0], c1 = raw[1];
        const uint32_t cw[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        // operand tile: 8-row atoms of 1 KB, 128-byte rows, 16-byte chunk j at (j ^ (row % 8))
        uint8_t* arow = a_tile(stage) + (r >> 3) * 1024 + (r & 7) * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float s = fp8_e4m3_to_float(s4 >> (8 * (j >> 1))) * gs;
          *reinterpret_cast<uint4*>(arow + ((j ^ (r & 7)) << 4)) = dequant8(cw[j], s);
        }
        fence_proxy_async();                                 // generic-proxy writes -> visible to the tensor core's reads
        __syncwarp();
        if (lane == 0) {
          zb_mbar_arrive(&full_bar[stage]);
          zb_mbar_arrive(&raw_empty[stage]);
        }
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue: thread row = output feature
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    uint32_t acc = 0, acc_phase = 0;
    Cursor c{0, 0};
    for (int g = blockIdx.x;; g += gridDim.x) {
      int wt, tt;
      if (!locate(c, g, wt, tt)) break;
      zb_mbar_wait(&tmem_full[acc], acc_phase, abort_flag);
      w4_epi_bar();
      if (*abort_flag != 0u) break;
      zb_tc_fence_after();
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quad * 32) << 16);
      const int off_e = prm.offsets[c.e];
      const int end_e = min(prm.offsets[c.e + 1], prm.cap);
      const int tok0 = off_e + tt * BN;
      if constexpr (!SWIGLU) {
        const int feat = wt * kBlockP + row_in_tile;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          uint32_t rr[16];
          zb_tmem_ld16(taddr + c0, rr);
          zb_tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int tok = tok0 + c0 + j;
            if (tok < end_e) prm.out[static_cast<size_t>(tok) * prm.ldo + feat] = __float2bfloat16(__uint_as_float(rr[j]));
          }
        }
      } else {
        // rows 0-63: gate, rows 64-127: up of the same 64 output features
        const bool is_up = row_in_tile >= 64;
        const int feat = wt * 64 + (row_in_tile & 63);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          uint32_t rr[16];
          zb_tmem_ld16(taddr + c0, rr);
          zb_tmem_ld_wait();
          if (is_up) {
#pragma unroll
            for (int j = 0; j < 16; ++j) xch[(c0 + j) * 64 + (row_in_tile - 64)] = __uint_as_float(rr[j]);
          }
          w4_epi_bar();
          if (!is_up) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int tok = tok0 + c0 + j;
              if (tok < end_e) {
                const float gt = __uint_as_float(rr[j]);
                const float up = xch[(c0 + j) * 64 + row_in_tile];
                prm.out[static_cast<size_t>(tok) * prm.ldo + feat] = __float2bfloat16(gt / (1.f + __expf(-gt)) * up);
              }
            }
          }
          w4_epi_bar();
        }
      }
      zb_tc_fence_before();
      zb_mbar_arrive(&tmem_empty[acc]);
      acc ^= 1u;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  zb_tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0u) {
    if (threadIdx.x == 0) zb_record_error(prm.status, ZB_ERR_MBAR_TIMEOUT, kKernelGroupedW4, blockIdx.x, BN);
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

template <int BN, bool SWIGLU>
int launch_w4(const CUtensorMap& tx, const CUtensorMap& tw, const W4Params& prm, int grid, cudaStream_t s) {
  constexpr int smem = w4_stages(BN) * w4_stage_bytes(BN) + (SWIGLU ? BN * 64 * 4 : 0) + 1024 + 256;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = zb_config_smem(zb_moe_grouped_gemm_w4_kernel<BN, SWIGLU>, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  zb_launch(zb_moe_grouped_gemm_w4_kernel<BN, SWIGLU>, dim3(grid), dim3(kThreads), smem, s, tx, tw, prm);
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

extern "C" {

// xs [cap, k] bf16 rows grouped by expert (offsets [e_local + 1]); codes [e_local * n, k / 2] packed e2m1
// (low nibble first); scales [e_local * n, k / 16] f8e4m3fn; gscale [e_local] fp32 or null.
// out [cap, ldo] bf16; with `swiglu` the weight rows are interleaved [64 gate | 64 up] per 128 and the
// output has n / 2 features.  k a multiple of 64, n a multiple of 128.  Few tokens per expert only
// (tiles of 16 / 32 / 64 tokens).
int zb_moe_grouped_gemm_w4(const void* xs, const void* codes, const void* scales, const float* gscale, void* out,
                           const int32_t* offsets, int e_local, int n, int k, int cap, int ldo, int swiglu,
                           int avg_tokens, void* stream) {
  if (cap <= 0 || e_local <= 0) return 0;
  if (k % 64 != 0 || n % kBlockP != 0 || ldo % 8 != 0) return -66;
  ZbDeviceState* st = zb_device_state();
  if (!st) return -20;
  int bn = 16;
  while (bn < avg_tokens * 2 && bn < 64) bn <<= 1;
  W4Params prm;
  prm.offsets = offsets;
  prm.e_local = e_local;
  prm.n = n;
  prm.k = k;
  prm.ldo = ldo;
  prm.out = reinterpret_cast<__nv_bfloat16*>(out);
  prm.cap = cap;
  prm.scales = reinterpret_cast<const uint8_t*>(scales);
  prm.gscale = gscale;
  prm.status = st->status;
  CUtensorMap tx, tw;
  int rc = zb_make_tmap_bf16_2d(&tx, xs, cap, k, k, bn);
  if (rc != 0) return rc;
  rc = zb_make_tmap_u8_2d(&tw, codes, static_cast<long long>(e_local) * n, k / 2, kBlockK / 2, kBlockP);
  if (rc != 0) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int grid = st->num_sms;
#define ZB_W4(BN_) return swiglu ? launch_w4<BN_, true>(tx, tw, prm, grid, s) : launch_w4<BN_, false>(tx, tw, prm, grid, s);
  switch (bn) {
    case 16: ZB_W4(16)
    case 32: ZB_W4(32)
    case 64: ZB_W4(64)
  }
#undef ZB_W4
  return -65;
}

}  // extern "C"
