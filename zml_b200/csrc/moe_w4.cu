// Grouped GEMM over experts whose weights are NVFP4 (e2m1 codes, two per byte, one f8e4m3fn
// scale per 16 values along K, one fp32 scale per expert matrix) with bf16 activations:
//
//   out[token, :] = xs[token, :] . dequant(W[expert(token)])^T       (+ SwiGLU for the gate|up GEMM)
//
// for the few-tokens-per-expert (decode) regime, where the expert weights are what the step
// reads from HBM: 4.5 bits per weight instead of 16.  Same warp-specialised structure as the bf16
// grouped kernel (moe.cu) with one more stage: a producer thread brings a block of packed codes
// and block scales (one bulk copy) and the activation tiles (TMA) of four k-blocks per stage, eight
// de-quantising warps turn the codes into bf16 and write them with tcgen05.st straight into tensor
// memory, where tcgen05.mma reads its A operand (a de-quantised tile never passes through shared
// memory: at 4.5 bits per weight the shared-memory traffic of a bf16 staging tile would be four
// times the HBM traffic), one thread issues the MMAs, four warps run the epilogue.
//
// The weights arrive in a tile-major layout made at load time (Nvfp4Experts, moe/ops.py): for every
// expert, 128-row tile and 256-wide K chunk one contiguous 18 KB block
//     [8 chunks of 16 bytes][128 rows] codes (chunk c of row r = bytes 16c .. 16c+15 of the row's 128)
//     [128 rows][16] f8e4m3 block scales
// which is exactly the shared-memory image the de-quantising threads read without bank conflicts, so
// the weights of a load stage are ONE untiled bulk copy of sequential memory.
//
// Measured on B200, 128 experts x [1536, 2048], 8 tokens per expert: 84 us against 129 us for the bf16
// kernel (down projection 48 against 67).  What set the pace at each step of the way: conversion
// instructions (140 us), the shared-memory traffic of a bf16 staging tile (140), one commit per k-block
// (135), walking the expert offsets in global memory at every tile change (110 -> 106), and one thread
// issuing the 16 small-N MMAs of a stage (770 ns per stage; two issuing threads: 106 -> 84).  Now the bit
// placement (about 600 ns per stage on the ALU pipe) and the tensor pipe (about 30 ns per 128 x 16 x 16
// MMA) are level; four groups of de-quantising warps instead of two measured slower (94 us).
//
// De-quantisation is integer bit placement plus one packed bf16 multiply per two weights (no
// conversion instructions, which issue at a fraction of the ALU rate):
//   * the codes arrive re-ordered (Nvfp4Experts, moe/ops.py): in each 32-bit word of 8 weights,
//     nibble i holds weight 2i and nibble i + 4 holds weight 2i + 1, so one shift and one mask put
//     the exponent / mantissa bits of a PAIR at bits 8..6 of both halves of a bf16x2, and a second
//     shift and mask put the two signs at bits 15 and 31;
//   * those bits read as bf16 are the e2m1 value x 2^-126 (the code's sub-normal 0.5 included);
//   * the f8e4m3 block scale shifted left by 4 reads as bf16 scale x 2^-120; two multiplies by
//     powers of two turn it into scale x 2^117;
//   * value bits x scale = e2m1 x scale x 2^-9, exact in bf16 (2 + 4 significant bits);
//   * the epilogue multiplies the fp32 accumulator by (matrix scale x 2^9).
//
// The reference reaches this through the FlashInfer CUTLASS NVFP4 runner
// (zml/moe/cutlass_flashinfer.zig:275-330) or XLA's scaled-dot composite (zml/nn.zig:294-398).
#include <cuda.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "common.cuh"
#include "host_api.h"
#include "moe_tiles.cuh"

int zb_make_tmap_bf16_2d(CUtensorMap* out, const void* base, int rows, int k, int ld, int box_rows);

namespace {

constexpr uint32_t kKernelGroupedW4 = 9;
constexpr int kBlockP = 128;
constexpr int kBlockK = 64;
constexpr int kUmmaK = 16;
constexpr int kDqGroups = 2;          // groups of 4 de-quantising warps; group g takes k-block g of every stage
constexpr int kIssuerBWarp = 6 + 4 * kDqGroups;          // second MMA-issuing warp, after the de-quantising warps
constexpr int kThreads = (kIssuerBWarp + 1) * 32;   // producer, MMA, 4 epilogue warps, the de-quantising warps, MMA
// Two threads issue the MMAs of a stage (two k-blocks each, into accumulators of their own that the epilogue
// adds) when tensor memory has room for four accumulators: one thread needs about 770 ns for the 16 small-N
// MMAs of a stage, which was the period of the whole pipeline.
__host__ __device__ constexpr int w4_issuers(int bn) { return bn <= 32 ? 2 : 1; }
constexpr int kSub = 4;              // k-blocks per load stage: 128 bytes of codes and 16 bytes of scales per weight row
constexpr int kCodeBytes = kBlockP * kSub * kBlockK / 2;      // 16 KB of packed codes per load stage
constexpr int kScaleBytes = kBlockP * kSub * kBlockK / 16;    // 2 KB of block scales per load stage

struct W4Params {
  const int32_t* offsets;   // [e_local + 1]
  int e_local;
  int n;                    // output features per expert
  int k;
  int ldo;
  __nv_bfloat16* out;
  int cap;
  const uint8_t* blocks;    // [e_local, n / 128, k / 256] blocks of 18 KB (codes, then scales)
  const float* gscale;      // [e_local, gs_per] per-matrix scale (gs_per = 2: gate rows, up rows)
  int gs_per;
  int act;                  // ZbMoeAct
  ZbStatus* status;
  unsigned long long* timeline;   // null, or [kTimelineStages][8] time stamps of CTA 0 (see zb_moe_w4_set_timeline)
};

constexpr int kTimelineStages = 64;

// Two rings.  The LOAD ring is what hides the latency of HBM: a stage holds everything the copy engine
// brings for 4 k-blocks of one tile (codes, block scales, the activation tiles), and the ring is as deep
// as shared memory allows, because at 4.5 bits per weight a k-block is only 4.6 KB of HBM traffic and tens
// of KB must be in flight per SM to reach the memory bandwidth.  The OPERAND ring holds de-quantised bf16
// weight tiles (32 columns of tensor memory each) between the de-quantising warps and the MMA thread.
__host__ __device__ constexpr int w4_load_stage_bytes(int bn) { return kCodeBytes + kScaleBytes + kSub * bn * kBlockK * 2; }
__host__ __device__ constexpr int w4_load_stages(int bn) { return bn >= 64 ? 4 : (bn >= 32 ? 6 : 8); }
constexpr int kAStages = 3;                  // operand stages; one holds the 4 k-blocks of a load stage
constexpr int kACols = kBlockK / 2;          // 32-bit tensor-memory columns of one k-block of the operand (two bf16 per column)
constexpr int kAStageCols = kSub * kACols;   // 128
constexpr uint32_t kTmemACol = 128;          // accumulators in columns [0, 2 BN), operand stages in [128, 512)
constexpr uint32_t kTmemCols = 512;          // one CTA per SM: the whole tensor memory
__host__ __device__ constexpr int w4_smem_bytes(int bn, bool swiglu) {
  return w4_load_stages(bn) * w4_load_stage_bytes(bn) + (swiglu ? bn * 64 * 4 : 0) + 1024 + 512;   // alignment slack + barriers
}

ZB_DEVICE void w4_epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

ZB_DEVICE uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// byte j of s4 (an f8e4m3 block scale) -> bf16x2 with scale x 2^117 in both halves
ZB_DEVICE uint32_t scale_pair(uint32_t s4, int j) {
  const uint32_t b = (s4 >> (8 * j)) & 0x7fu;
  const uint32_t bits = (b << 4) | (b << 20);                  // bf16 bits: scale x 2^-120
  return mul_bf16x2(mul_bf16x2(bits, 0x7B807B80u), 0x7A007A00u);   // x 2^120, x 2^117
}

// 8 re-ordered codes (one u32) x scale pair -> 8 bf16 in K order (one 16-byte chunk)
ZB_DEVICE uint4 dequant8(uint32_t c, uint32_t m2) {
  constexpr uint32_t kMag = 0x01C001C0u, kSgn = 0x80008000u;
  const uint32_t x0 = ((c << 6) & kMag) | ((c << 12) & kSgn);
  const uint32_t x1 = ((c << 2) & kMag) | ((c << 8) & kSgn);
  const uint32_t x2 = ((c >> 2) & kMag) | ((c << 4) & kSgn);
  const uint32_t x3 = ((c >> 6) & kMag) | (c & kSgn);
  return make_uint4(mul_bf16x2(x0, m2), mul_bf16x2(x1, m2), mul_bf16x2(x2, m2), mul_bf16x2(x3, m2));
}

template <int BN, bool SWIGLU>
__global__ void __launch_bounds__(kThreads, 1)
zb_moe_grouped_gemm_w4_kernel(const __grid_constant__ CUtensorMap tmap_x, const W4Params prm) {
  constexpr int kLoadStages = w4_load_stages(BN);
  constexpr int kLoadBytes = w4_load_stage_bytes(BN);
  constexpr int kTileBBytes = BN * kBlockK * 2;
  constexpr int kIssuers = w4_issuers(BN);
  static_assert(2 * kIssuers * BN <= static_cast<int>(kTmemACol), "accumulators below the operand tiles");
  constexpr uint32_t kIdesc = zb_make_idesc_bf16(kBlockP, BN);
  constexpr int kXchBytes = SWIGLU ? BN * 64 * 4 : 0;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  // load stage: [codes 16 KB | scales 2 KB | 4 activation tiles]; the activation tiles start on 1 KB
  uint8_t* load_base = smem;
  float* xch = reinterpret_cast<float*>(smem + kLoadStages * kLoadBytes);
  uint64_t* load_full = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(xch) + kXchBytes);
  uint64_t* load_empty = load_full + kLoadStages;
  uint64_t* a_full = load_empty + kLoadStages;
  uint64_t* a_empty = a_full + kAStages;
  uint64_t* tmem_full = a_empty + kAStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile uint32_t* abort_flag = tmem_holder + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int lb_total = prm.k / (kBlockK * kSub);          // load stages per tile

  if (threadIdx.x == 0) {
    for (int s = 0; s < kLoadStages; ++s) {
      zb_mbar_init(&load_full[s], 1);        // producer, with the bytes of the three copies
      zb_mbar_init(&load_empty[s], 4 * kDqGroups + kIssuers);   // one lane per de-quantising warp + the MMA commits (activation tiles)
    }
    for (int s = 0; s < kAStages; ++s) {
      zb_mbar_init(&a_full[s], 4 * kDqGroups);   // one lane per de-quantising warp (each wrote its k-blocks of its 32 rows)
      zb_mbar_init(&a_empty[s], kIssuers);   // MMA commits
    }
    for (int a = 0; a < 2; ++a) {
      zb_mbar_init(&tmem_full[a], kIssuers);
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

  unsigned long long* tl = blockIdx.x == 0 ? prm.timeline : nullptr;
  const int w_tiles = prm.n / kBlockP;
  __shared__ int32_t tile_prefix[kZbMaxExperts + 1];
  zb_tile_prefix_build(tile_prefix, prm.offsets, prm.e_local, w_tiles, BN);
  struct Cursor {
    int e, hint;
  };
  auto locate = [&](Cursor& c, int g, int& wt, int& tt) -> bool {
    ZbTilePos pos;
    if (!zb_tile_locate(tile_prefix, prm.e_local, w_tiles, g, c.hint, pos)) return false;
    c.e = pos.e;
    wt = pos.wt;
    tt = pos.tt;
    return true;
  };
  auto codes_of = [&](uint32_t ls) { return load_base + ls * kLoadBytes; };
  auto scales_of = [&](uint32_t ls) { return load_base + ls * kLoadBytes + kCodeBytes; };
  auto btile_of = [&](uint32_t ls, int sub) { return load_base + ls * kLoadBytes + kCodeBytes + kScaleBytes + sub * kTileBBytes; };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      zb_tma_prefetch_desc(&tmap_x);
      uint32_t ls = 0, lphase = 0;
      int q = 0;
      Cursor c{0, 0};
      bool ok = true;
      for (int g = blockIdx.x; ok; g += gridDim.x) {
        int wt, tt;
        if (!locate(c, g, wt, tt)) break;
        const int tok0 = prm.offsets[c.e] + tt * BN;
        const uint8_t* wblock = prm.blocks + (static_cast<size_t>(c.e) * w_tiles + wt) * lb_total * (kCodeBytes + kScaleBytes);
        for (int lb = 0; lb < lb_total; ++lb) {
          if (!zb_mbar_wait(&load_empty[ls], lphase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          if (tl != nullptr && q < kTimelineStages) tl[q * 8 + 0] = zb_globaltimer();
          ++q;
          zb_mbar_expect_tx(&load_full[ls], kCodeBytes + kScaleBytes + kSub * kTileBBytes);
          zb_bulk_load(codes_of(ls), wblock + static_cast<size_t>(lb) * (kCodeBytes + kScaleBytes), kCodeBytes + kScaleBytes,
                       &load_full[ls]);
#pragma unroll
          for (int sub = 0; sub < kSub; ++sub)
            zb_tma_load_2d(btile_of(ls, sub), &tmap_x, &load_full[ls], (lb * kSub + sub) * kBlockK, tok0);
          if (++ls == kLoadStages) {
            ls = 0;
            lphase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1 || warp == kIssuerBWarp) {
    // ------------------------------------------------------------------ MMA issuers
    const int issuer = warp == 1 ? 0 : 1;
    constexpr int kSubsPer = kSub / kIssuers;
    if (lane == 0 && issuer < kIssuers) {
      if (issuer != 0) tl = nullptr;
      uint32_t ls = 0, lphase = 0, as = 0, aphase = 0, acc = 0, acc_phase = 0;
      int q = 0;
      Cursor c{0, 0};
      bool ok = true;
      for (int g = blockIdx.x; ok; g += gridDim.x) {
        int wt, tt;
        if (!locate(c, g, wt, tt)) break;
        if (!zb_mbar_wait(&tmem_empty[acc], acc_phase ^ 1u, abort_flag)) break;
        zb_tc_fence_after();
        const uint32_t tmem_d = tmem_base + (acc * kIssuers + issuer) * BN;
        for (int lb = 0; lb < lb_total && ok; ++lb) {
          if (!zb_mbar_wait(&load_full[ls], lphase, abort_flag)) {      // the activation tiles of 4 k-blocks
            ok = false;
            break;
          }
          if (!zb_mbar_wait(&a_full[as], aphase, abort_flag)) {          // the de-quantised weights of the same 4 k-blocks
            ok = false;
            break;
          }
          zb_tc_fence_after();
          if (tl != nullptr && q < kTimelineStages) tl[q * 8 + 5] = zb_globaltimer();
          {
#pragma unroll
            for (int s2 = 0; s2 < kSubsPer; ++s2) {
              const int sub = issuer * kSubsPer + s2;
              const uint32_t ta = tmem_base + kTmemACol + as * kAStageCols + sub * kACols;
              const uint64_t db = zb_make_desc_sw128(zb_smem_u32(btile_of(ls, sub)));
#pragma unroll
              for (int k = 0; k < kBlockK / kUmmaK; ++k)
                zb_umma_f16_ts(tmem_d, ta + 8 * k, db + 2 * k, kIdesc, (lb > 0 || s2 > 0 || k > 0) ? 1u : 0u);
            }
          }
          zb_umma_commit(&a_empty[as]);
          if (++as == kAStages) {
            as = 0;
            aphase ^= 1u;
          }
          if (!ok) break;
          zb_umma_commit(&load_empty[ls]);
          if (tl != nullptr && q < kTimelineStages) tl[q * 8 + 6] = zb_globaltimer();
          ++q;
          if (++ls == kLoadStages) {
            ls = 0;
            lphase ^= 1u;
          }
        }
        if (!ok) break;
        zb_umma_commit(&tmem_full[acc]);
        acc ^= 1u;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else if (warp >= 6 && warp < kIssuerBWarp) {
    // ------------------------------------------------------------------ de-quantisers: thread = weight row
    // every group of four warps de-quantises its share of the four k-blocks of a stage
    const int group = (warp - 6) >> 2;
    const int r = (warp & 3) * 32 + lane;                  // a warp reaches the 32 tensor-memory lanes of its quarter
    const uint32_t ta_row = tmem_base + kTmemACol + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    uint32_t ls = 0, lphase = 0, as = 0, aphase = 0;
    int q = 0;
    unsigned long long* tlw = (lane == 0 && (warp & 3) == 2) ? tl : nullptr;      // one warp of each group stamps
    Cursor c{0, 0};
    bool ok = true;
    for (int g = blockIdx.x; ok; g += gridDim.x) {
      int wt, tt;
      if (!locate(c, g, wt, tt)) break;
      for (int lb = 0; lb < lb_total && ok; ++lb, ++q) {
        if (!zb_mbar_wait(&load_full[ls], lphase, abort_flag)) {
          ok = false;
          break;
        }
        if (tlw != nullptr && group == 0 && q < kTimelineStages) tlw[q * 8 + 1] = zb_globaltimer();
        const uint4* crow = reinterpret_cast<const uint4*>(codes_of(ls)) + r;      // chunk c of this row at crow[c * 128]
        const uint4 sc = *reinterpret_cast<const uint4*>(scales_of(ls) + r * 16);
        const uint32_t s4s[kSub] = {sc.x, sc.y, sc.z, sc.w};
        if (!zb_mbar_wait(&a_empty[as], aphase ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        zb_tc_fence_after();
        if (tlw != nullptr && group == 0 && q < kTimelineStages) tlw[q * 8 + 2] = zb_globaltimer();
        {
#pragma unroll
          for (int sub = 0; sub < kSub; ++sub) {
            if ((sub % kDqGroups) != group) continue;
            const uint4 c0 = crow[(2 * sub) * kBlockP];
            const uint4 c1 = crow[(2 * sub + 1) * kBlockP];
            const uint32_t cw[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
            uint32_t v[32];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint4 d = dequant8(cw[j], scale_pair(s4s[sub], j >> 1));
              v[4 * j] = d.x, v[4 * j + 1] = d.y, v[4 * j + 2] = d.z, v[4 * j + 3] = d.w;
            }
            zb_tmem_st16(ta_row + as * kAStageCols + sub * kACols, v);
            zb_tmem_st16(ta_row + as * kAStageCols + sub * kACols + 16, v + 16);
          }
        }
        zb_tmem_st_wait();
        if (tlw != nullptr && q < kTimelineStages) tlw[q * 8 + 3 + (group != 0 ? 1 : 0)] = zb_globaltimer();
        zb_tc_fence_before();
        __syncwarp();
        if (lane == 0) zb_mbar_arrive(&a_full[as]);
        if (++as == kAStages) {
          as = 0;
          aphase ^= 1u;
        }
        __syncwarp();
        if (lane == 0) zb_mbar_arrive(&load_empty[ls]);      // this warp has read its codes and scales of the stage
        if (++ls == kLoadStages) {
          ls = 0;
          lphase ^= 1u;
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
      const uint32_t taddr = tmem_base + acc * kIssuers * BN + (static_cast<uint32_t>(quad * 32) << 16);
      const int off_e = prm.offsets[c.e];
      const int end_e = min(prm.offsets[c.e + 1], prm.cap);
      const int tok0 = off_e + tt * BN;
      // matrix scale x 2^9; with two scales per expert the up rows (64..127 of the tile) take the second
      const float oscale = (prm.gscale != nullptr ? prm.gscale[c.e * prm.gs_per + ((SWIGLU && row_in_tile >= 64) ? prm.gs_per - 1 : 0)]
                                                  : 1.f) * 512.f;
      if constexpr (!SWIGLU) {
        const int feat = wt * kBlockP + row_in_tile;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          uint32_t rr[16];
          zb_tmem_ld16(taddr + c0, rr);
          if constexpr (kIssuers == 2) {
            uint32_t r2[16];
            zb_tmem_ld16(taddr + BN + c0, r2);
            zb_tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) rr[j] = __float_as_uint(__uint_as_float(rr[j]) + __uint_as_float(r2[j]));
          }
          zb_tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int tok = tok0 + c0 + j;
            if (tok < end_e)
              prm.out[static_cast<size_t>(tok) * prm.ldo + feat] = __float2bfloat16(zb_plain_act(__uint_as_float(rr[j]) * oscale, prm.act));
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
          if constexpr (kIssuers == 2) {
            uint32_t r2[16];
            zb_tmem_ld16(taddr + BN + c0, r2);
            zb_tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) rr[j] = __float_as_uint(__uint_as_float(rr[j]) + __uint_as_float(r2[j]));
          }
          zb_tmem_ld_wait();
          if (is_up) {
#pragma unroll
            for (int j = 0; j < 16; ++j) xch[(c0 + j) * 64 + (row_in_tile - 64)] = __uint_as_float(rr[j]) * oscale;
          }
          w4_epi_bar();
          if (!is_up) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int tok = tok0 + c0 + j;
              if (tok < end_e) {
                const float gt = __uint_as_float(rr[j]) * oscale;
                const float up = xch[(c0 + j) * 64 + row_in_tile];
                prm.out[static_cast<size_t>(tok) * prm.ldo + feat] = __float2bfloat16(zb_gate_act(gt, prm.act) * up);
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
int launch_w4(const CUtensorMap& tx, const W4Params& prm, int grid, cudaStream_t s) {
  constexpr int smem = w4_smem_bytes(BN, SWIGLU);
  static_assert(smem <= 232448, "shared memory of one CTA");
  static bool configured[16] = {};
  if (const int rc = zb_config_smem_once(zb_moe_grouped_gemm_w4_kernel<BN, SWIGLU>, smem, configured)) return rc;
  zb_launch(zb_moe_grouped_gemm_w4_kernel<BN, SWIGLU>, dim3(grid), dim3(kThreads), smem, s, tx, prm);
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

unsigned long long* g_w4_timeline = nullptr;

}  // namespace

extern "C" {

// Phase time stamps of the next launches' CTA 0: `buf` holds 64 x 8 u64 (device memory), or null to switch off.
// Per load stage q: [0] producer issues the copies, [1] a de-quantising warp sees them, [2] it has an operand
// stage, [3] / [4] the two groups' tensor-memory stores are done, [5] the MMA thread has both operands, [6] it
// has issued the MMAs and commits.  %globaltimer nanoseconds.
void zb_moe_w4_set_timeline(void* buf) { g_w4_timeline = reinterpret_cast<unsigned long long*>(buf); }

// xs [cap, k] bf16 rows grouped by expert (offsets [e_local + 1]); blocks [e_local, n / 128, k / 256, 18432]
// bytes: the tile-major packed e2m1 codes and f8e4m3fn block scales (see the head of this file); gscale
// [e_local, gs_per] fp32 or null (gs_per = 2 with `swiglu`: one scale for the gate rows, one for the up rows).
// out [cap, ldo] bf16; with `swiglu` the weight rows are interleaved [64 gate | 64 up] per 128 and the
// output has n / 2 features.  k a multiple of 256, n a multiple of 128.  Few tokens per expert only
// (tiles of 16 / 32 / 64 tokens).
int zb_moe_grouped_gemm_w4(const void* xs, const void* blocks, const float* gscale, int gs_per,
                           void* out, const int32_t* offsets, int e_local, int n, int k, int cap, int ldo, int swiglu,
                           int avg_tokens, void* stream) {
  if (cap <= 0 || e_local <= 0) return 0;
  if (e_local > kZbMaxExperts) return -61;
  if (k % (kBlockK * kSub) != 0 || n % kBlockP != 0 || ldo % 8 != 0) return -66;
  if (swiglu < 0 || swiglu > ZB_ACT_RELU2) return -67;
  const bool gated = swiglu >= ZB_ACT_SWIGLU && swiglu <= ZB_ACT_GEGLU_TANH;
  if (gs_per != 1 && !(gs_per == 2 && gated)) return -67;
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
  prm.gscale = gscale;
  prm.gs_per = gs_per;
  prm.act = swiglu;
  prm.status = st->status;
  prm.timeline = g_w4_timeline;
  if ((reinterpret_cast<uintptr_t>(blocks) & 15) != 0) return -66;
  prm.blocks = reinterpret_cast<const uint8_t*>(blocks);
  CUtensorMap tx;
  int rc = zb_make_tmap_bf16_2d(&tx, xs, cap, k, k, bn);
  if (rc != 0) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int grid = st->num_sms;
#define ZB_W4(BN_) return gated ? launch_w4<BN_, true>(tx, prm, grid, s) : launch_w4<BN_, false>(tx, prm, grid, s);
  switch (bn) {
    case 16: ZB_W4(16)
    case 32: ZB_W4(32)
    case 64: ZB_W4(64)
  }
#undef ZB_W4
  return -65;
}

}  // extern "C"
