// Grouped GEMM over experts with NVFP4 weights AND NVFP4 activations on the block-scaled tensor-core path:
//
//   out[token, :] = (x_q[token, :] . W_q[expert(token)]^T) * x_scale * w_scale[expert]      (+ SwiGLU for gate|up)
//
// `tcgen05.mma.kind::mxf4nvf4.block_scale.block16` multiplies packed e2m1 codes straight from shared memory and
// applies one f8e4m3 (ue4m3) scale per 16 values along K to both operands inside the tensor core, so nothing is
// de-quantised by threads: the weight tile goes HBM -> shared memory -> tensor core as 4.5 bits per weight, and
// the MMA of a 128 x 64 code tile costs one instruction per K = 64.  (The W4A16 kernel in moe_w4.cu de-quantises
// the weights to bf16 with eight warps and is bound by their bit placement and by K = 16 MMAs.)
//
// Operands of one MMA (M = 128 weight rows, N = BN tokens, K = 64 values = 32 bytes of codes per row):
//   A  weight codes, K-major in shared memory with the 128-byte swizzle (a row of 128 bytes = K = 256: one load
//      stage holds four MMAs' worth), described by a shared-memory matrix descriptor;
//   B  activation codes, same layout, brought by TMA from the row-major [cap, K / 2] byte matrix;
//   SFA / SFB  the block scales, in TENSOR MEMORY: for rows r = 0..127 and the 4 scales s of this K = 64, lane
//      (r % 32) + 32 p (replicated over the four 32-lane quarters p) and byte 4 (r / 32) + s of four consecutive
//      32-bit columns.  `tcgen05.cp.32x128b.warpx4` fills them from a 512-byte shared-memory image
//      [32 rows][16 bytes] (row r % 32, bytes 4 (r / 32) + s).
//
// The weights arrive in a tile-major layout made at load time (`nvfp4_pack_blocks_mma`, moe/ops.py): for every
// expert, 128-row tile and 256-wide K chunk one contiguous 18 KB block - the swizzled 16 KB code image followed by
// four 512-byte scale images - so the weights of a load stage are ONE untiled bulk copy of sequential memory.
// The activation scales stay row-major [cap, K / 16] as the quantiser writes them (token tiles start at arbitrary
// rows, so their image cannot be made in advance); one warp reads the 16 bytes of each token row of a stage and
// writes them into the four images.
//
// Roles: warp 0 producer (bulk copy + TMA), warp 1 MMA issuer (scale copies + MMAs, one thread), warps 2-5
// epilogue (thread = output feature, like moe_w4.cu), warp 6 activation-scale loader.
//
// Measured on B200, 128 experts x [1536, 2048], 8 tokens per expert: 65.5 us (W4A16 kernel: 88 - 90; the down
// projection 41 against 51 - 53); 64 tokens per expert 123 us against 163 for the bf16 grouped GEMM; at 512 tokens per
// expert the bf16 kernel wins (65 against 92 us: 128 x 128 tiles of 4-bit operands are bound by operand traffic into
// shared memory), so the caller uses this kernel up to 128 tokens per expert.  With the tensor-core work switched
// off the pipeline streams the same weights in 56 us (a bare ring of 18 KB bulk copies reads 226 MB in 42 us); scale
// copies and MMAs add 10 us on the issuing thread.  What did not help: an L2 prefetch of the next tile's weights
// (73.7 us), the weight block as four copies, batching more activation-scale loads, issuing the scale copies from
// the scale warp (71.7 us).
//
// The reference reaches this shape of kernel through the FlashInfer CUTLASS NVFP4 runner
// (zml/moe/cutlass_flashinfer.zig:275-330, 573-630).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "common.cuh"
#include "host_api.h"
#include "moe_tiles.cuh"
#include "quant.cuh"

int zb_make_tmap_u8_2d_ex(CUtensorMap* out, const void* base, long long rows, long long row_bytes, int box_bytes, int box_rows,
                          int swizzle128);

namespace {

constexpr uint32_t kKernelGroupedFp4 = 15;
constexpr int kBlockP = 128;                 // weight rows per tile (the MMA's M)
constexpr int kStageK = 256;                 // values along K per load stage (128 bytes of codes per row)
constexpr int kMmaK = 64;                    // values along K per MMA
constexpr int kSub = kStageK / kMmaK;        // MMAs per stage
constexpr int kCodeBytes = kBlockP * kStageK / 2;       // 16 KB
constexpr int kSfImage = 512;                // one scale image: [32][16] bytes
constexpr int kSfBytes = kSub * kSfImage;    // 2 KB per operand and stage
constexpr int kThreads = 7 * 32;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kSfColsPerStage = 32;     // 4 MMAs x (4 columns SFA + 4 columns SFB)

struct Fp4Params {
  const int32_t* offsets;   // [e_local + 1]
  int e_local;
  int n;                    // output rows of the weight matrix per expert
  int k;
  int ldo;
  __nv_bfloat16* out;
  int cap;
  const uint8_t* blocks;    // [e_local, n / 128, k / 256] blocks of 18 KB (code image, then 4 scale images)
  const uint8_t* x_sf;      // [cap, k / 16] f8e4m3 activation block scales, row-major
  const float* w_gscale;    // [e_local, gs_per] per-matrix weight scale, or null
  int gs_per;
  const float* x_gscale;    // one fp32: the activations' per-tensor scale, or null (1)
  uint8_t* out_q;           // QOUT: [cap, ldo / 2] e2m1 codes of the (SwiGLU) output instead of `out`
  uint8_t* out_sf;          // QOUT: [cap, ldo / 16] f8e4m3 block scales
  int act;                  // ZbMoeAct
  ZbStatus* status;
};

__host__ __device__ constexpr int fp4_stage_bytes(int bn) { return kCodeBytes + kSfBytes + bn * (kStageK / 2) + kSfBytes; }
__host__ __device__ constexpr int fp4_stages(int bn) {
  return bn <= 32 ? 8 : (bn <= 64 ? 7 : 5);
}
__host__ __device__ constexpr int fp4_smem_bytes(int bn, bool swiglu) {
  return fp4_stages(bn) * fp4_stage_bytes(bn) + (swiglu ? bn * 64 * 4 : 0) + 1024 + 512;
}

ZB_DEVICE void fp4_epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Shared-memory matrix descriptor of a [32 rows][16 bytes] scale image: K-major, no swizzle, rows 16 bytes apart,
// groups of 8 rows 128 bytes apart.
ZB_DEVICE uint64_t make_desc_sf(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(16 >> 4) << 16;       // leading byte offset (one 16-byte column only: not used)
  d |= static_cast<uint64_t>(128 >> 4) << 32;      // stride byte offset between 8-row groups
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}

// 32 rows x 128 bits of shared memory -> 4 columns of tensor memory, the same data in all four 32-lane quarters.
ZB_DEVICE void tmem_cp_sf(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}

// Instruction descriptor of kind::mxf4nvf4: bits 7-9 / 10-12 A / B format (1 = e2m1), 15 / 16 majors (0 = K),
// 17-22 N >> 3, 23 scale format (0 = ue4m3), 24-28 M >> 4, 4-5 / 29-30 byte offset of SFB / SFA inside their
// column (0: all four bytes are used with one scale per 16 values).
__host__ __device__ constexpr uint32_t make_idesc_fp4(uint32_t m, uint32_t n) {
  return (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

ZB_DEVICE void umma_fp4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t tmem_sfa,
                        uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}

// QOUT (with SWIGLU): the output leaves as NVFP4 (codes + one f8e4m3 scale per 16 features), ready to be the
// activation operand of the down projection: no bf16 round trip through memory and no quantiser launch.
template <int BN, bool SWIGLU, bool QOUT>
__global__ void __launch_bounds__(kThreads, 1)
zb_moe_grouped_gemm_fp4_kernel(const __grid_constant__ CUtensorMap tmap_x, const Fp4Params prm) {
  constexpr int kStages = fp4_stages(BN);
  constexpr int kStageBytes = fp4_stage_bytes(BN);
  constexpr int kXBytes = BN * (kStageK / 2);
  static_assert(kXBytes % 1024 == 0, "activation tiles start on 1 KB");
  constexpr uint32_t kIdesc = make_idesc_fp4(kBlockP, BN);
  constexpr int kXchBytes = SWIGLU ? BN * 64 * 4 : 0;
  constexpr uint32_t kTmemSf = 2 * BN;                // accumulators in columns [0, 2 BN), scales behind them
  static_assert(2 * BN + kStages * kSfColsPerStage <= kTmemCols, "tensor memory");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  // stage: [weight codes 16 KB | weight scale images 2 KB | activation codes BN x 128 | activation scale images 2 KB]
  float* xch = reinterpret_cast<float*>(smem + kStages * kStageBytes);
  uint64_t* full = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(xch) + kXchBytes);
  uint64_t* empty = full + kStages;
  uint64_t* tmem_full = empty + kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile uint32_t* abort_flag = tmem_holder + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int lb_total = prm.k / kStageK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      zb_mbar_init(&full[s], 2);         // the producer (with the bytes of its copies) and the scale loader
      zb_mbar_init(&empty[s], 1);        // the MMA thread's commit
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
  __shared__ int32_t tile_prefix[kZbMaxExperts + 1];
  __shared__ int32_t offs_s[kZbMaxExperts + 1];      // the expert offsets: every role reads them at every tile change
  for (int i = threadIdx.x; i <= prm.e_local; i += kThreads) offs_s[i] = prm.offsets[i];
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
  auto wcodes_of = [&](uint32_t s) { return smem + s * kStageBytes; };
  auto wsf_of = [&](uint32_t s) { return smem + s * kStageBytes + kCodeBytes; };
  auto xcodes_of = [&](uint32_t s) { return smem + s * kStageBytes + kCodeBytes + kSfBytes; };
  auto xsf_of = [&](uint32_t s) { return smem + s * kStageBytes + kCodeBytes + kSfBytes + kXBytes; };

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      zb_tma_prefetch_desc(&tmap_x);
      uint32_t s = 0, phase = 0;
      Cursor c{0, 0};
      bool ok = true;
      for (int g = blockIdx.x; ok; g += gridDim.x) {
        int wt, tt;
        if (!locate(c, g, wt, tt)) break;
        const int tok0 = offs_s[c.e] + tt * BN;
        const uint8_t* wblock = prm.blocks + (static_cast<size_t>(c.e) * w_tiles + wt) * lb_total * (kCodeBytes + kSfBytes);
        for (int lb = 0; lb < lb_total; ++lb) {
          if (!zb_mbar_wait(&empty[s], phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          zb_mbar_expect_tx(&full[s], kCodeBytes + kSfBytes + kXBytes);
          zb_bulk_load(wcodes_of(s), wblock + static_cast<size_t>(lb) * (kCodeBytes + kSfBytes), kCodeBytes + kSfBytes, &full[s]);
          zb_tma_load_2d(xcodes_of(s), &tmap_x, &full[s], lb * (kStageK / 2), tok0);
          if (++s == kStages) {
            s = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 6) {
    // ------------------------------------------------------------------ activation scales: row-major -> images
    // A lane owns the token rows lane, lane + 32, ... of the tile.  The 16 scale bytes of a row and stage are one
    // 16-byte load; the loads of kBatch stages are issued together (one global-memory latency per batch, not
    // per stage: with one load per stage the whole pipeline ran at that latency, 790 ns per stage).
    constexpr int kRowsPerLane = (BN + 31) / 32;
    constexpr int kBatch = 8 / kRowsPerLane;
    uint32_t s = 0, phase = 0;
    Cursor c{0, 0};
    const int sf_ld = prm.k / 16;
    // the loads of batch i + 1 are in flight while the images of batch i are written: a flat list of
    // (tile, first stage of the batch) pairs, walked one ahead
    struct Batch {
      int tok0, lb0;
      bool valid;
    };
    int g_next = blockIdx.x, lb_next = 0, tok0_next = 0;
    bool have_tile = false;
    auto next_batch = [&]() -> Batch {
      if (!have_tile || lb_next >= lb_total) {
        int wt, tt;
        if (!locate(c, g_next, wt, tt)) return Batch{0, 0, false};
        tok0_next = offs_s[c.e] + tt * BN;
        g_next += gridDim.x;
        lb_next = 0;
        have_tile = true;
      }
      Batch b{tok0_next, lb_next, true};
      lb_next += kBatch;
      return b;
    };
    auto load_batch = [&](const Batch& bt, uint4 (&v)[kBatch][kRowsPerLane]) {
#pragma unroll
      for (int b = 0; b < kBatch; ++b) {
#pragma unroll
        for (int i = 0; i < kRowsPerLane; ++i) {
          const int r = lane + 32 * i;
          const int tok = bt.tok0 + r;
          v[b][i] = make_uint4(0u, 0u, 0u, 0u);
          if (bt.valid && r < BN && tok < prm.cap && bt.lb0 + b < lb_total)
            v[b][i] = __ldg(reinterpret_cast<const uint4*>(prm.x_sf + static_cast<size_t>(tok) * sf_ld + (bt.lb0 + b) * 16));
        }
      }
    };
    uint4 va[kBatch][kRowsPerLane], vb[kBatch][kRowsPerLane];
    Batch cur = next_batch();
    load_batch(cur, va);
    bool ok = true;
    while (cur.valid && ok) {
      const Batch nxt = next_batch();
      load_batch(nxt, vb);
#pragma unroll
      for (int b = 0; b < kBatch; ++b) {
        if (cur.lb0 + b >= lb_total) break;
        if (!zb_mbar_wait(&empty[s], phase ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        uint32_t* img = reinterpret_cast<uint32_t*>(xsf_of(s));
#pragma unroll
        for (int i = 0; i < kRowsPerLane; ++i) {
          const int r = lane + 32 * i;
          if (r < BN) {
            // image j (the j-th K = 64 of the stage): row r % 32, word r / 32
            const int w = lane * 4 + i;
            img[w] = va[b][i].x;
            img[kSfImage / 4 + w] = va[b][i].y;
            img[2 * (kSfImage / 4) + w] = va[b][i].z;
            img[3 * (kSfImage / 4) + w] = va[b][i].w;
          }
        }
        zb_fence_proxy_async_smem();          // tcgen05.cp reads the images through the async proxy
        __syncwarp();
        if (lane == 0) zb_mbar_arrive(&full[s]);
        if (++s == kStages) {
          s = 0;
          phase ^= 1u;
        }
      }
#pragma unroll
      for (int b = 0; b < kBatch; ++b) {
#pragma unroll
        for (int i = 0; i < kRowsPerLane; ++i) va[b][i] = vb[b][i];
      }
      cur = nxt;
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t s = 0, phase = 0, acc = 0, acc_phase = 0;
      Cursor c{0, 0};
      bool ok = true;
      for (int g = blockIdx.x; ok; g += gridDim.x) {
        int wt, tt;
        if (!locate(c, g, wt, tt)) break;
        if (!zb_mbar_wait(&tmem_empty[acc], acc_phase ^ 1u, abort_flag)) break;
        zb_tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int lb = 0; lb < lb_total; ++lb) {
          if (!zb_mbar_wait(&full[s], phase, abort_flag)) {
            ok = false;
            break;
          }
          zb_tc_fence_after();
          // (moving these copies to the scale warp's first lane, with a barrier of its own, was slower: 71.7 against
          // 65.5 us on 128 experts x [1536, 2048], 8 tokens each)
          const uint32_t sf_col = tmem_base + kTmemSf + s * kSfColsPerStage;
          const uint32_t wsf = zb_smem_u32(wsf_of(s)), xsf = zb_smem_u32(xsf_of(s));
#pragma unroll
          for (int j = 0; j < kSub; ++j) {
            tmem_cp_sf(sf_col + 4 * j, make_desc_sf(wsf + j * kSfImage));
            tmem_cp_sf(sf_col + 16 + 4 * j, make_desc_sf(xsf + j * kSfImage));
          }
          const uint64_t da = zb_make_desc_sw128(zb_smem_u32(wcodes_of(s)));
          const uint64_t db = zb_make_desc_sw128(zb_smem_u32(xcodes_of(s)));
#pragma unroll
          for (int j = 0; j < kSub; ++j)
            umma_fp4(tmem_d, da + 2 * j, db + 2 * j, kIdesc, sf_col + 4 * j, sf_col + 16 + 4 * j, (lb > 0 || j > 0) ? 1u : 0u);
          zb_umma_commit(&empty[s]);
          if (++s == kStages) {
            s = 0;
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
    // ------------------------------------------------------------------ epilogue: thread row = output feature
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    const float xg = prm.x_gscale != nullptr ? *prm.x_gscale : 1.f;
    uint32_t acc = 0, acc_phase = 0;
    Cursor c{0, 0};
    for (int g = blockIdx.x;; g += gridDim.x) {
      int wt, tt;
      if (!locate(c, g, wt, tt)) break;
      zb_mbar_wait(&tmem_full[acc], acc_phase, abort_flag);
      fp4_epi_bar();
      if (*abort_flag != 0u) break;
      zb_tc_fence_after();
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quad * 32) << 16);
      const int off_e = offs_s[c.e];
      const int end_e = min(offs_s[c.e + 1], prm.cap);
      const int tok0 = off_e + tt * BN;
      // with two scales per expert the up rows (64..127 of the tile) take the second
      const float oscale = xg * (prm.w_gscale != nullptr
                                     ? prm.w_gscale[c.e * prm.gs_per + ((SWIGLU && row_in_tile >= 64) ? prm.gs_per - 1 : 0)]
                                     : 1.f);
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
          zb_tmem_ld_wait();
          if (is_up) {
#pragma unroll
            for (int j = 0; j < 16; ++j) xch[(c0 + j) * 64 + (row_in_tile - 64)] = __uint_as_float(rr[j]) * oscale;
          }
          fp4_epi_bar();
          if constexpr (!QOUT) {
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
            fp4_epi_bar();
          } else {
            // gate threads put h (rounded to bf16, as the two-kernel path would store it) where the up values
            // were; then every thread quantises one (token, 16-feature block) of the 16 x 64 chunk
            if (!is_up) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float gt = __uint_as_float(rr[j]) * oscale;
                const float up = xch[(c0 + j) * 64 + row_in_tile];
                xch[(c0 + j) * 64 + row_in_tile] = bf16_round(zb_gate_act(gt, prm.act) * up);
              }
            }
            fp4_epi_bar();
            const int item = threadIdx.x - 64;                 // epilogue threads are 64 .. 191
            if (item >= 0 && item < 64) {
              const int j = item >> 2, blk = item & 3;
              const int tok = tok0 + c0 + j;
              if (tok < end_e) {
                float vv[16];
                const float4* src4 = reinterpret_cast<const float4*>(xch + (c0 + j) * 64 + blk * 16);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float4 q4 = src4[i];
                  vv[4 * i] = q4.x, vv[4 * i + 1] = q4.y, vv[4 * i + 2] = q4.z, vv[4 * i + 3] = q4.w;
                }
                uint8_t s8;
                const uint2 cw = zb_nvfp4_quantize_block(vv, s8);
                const int fblk = wt * 4 + blk;                 // 16-feature block of the output row
                *reinterpret_cast<uint2*>(prm.out_q + static_cast<size_t>(tok) * (prm.ldo / 2) + fblk * 8) = cw;
                prm.out_sf[static_cast<size_t>(tok) * (prm.ldo / 16) + fblk] = s8;
              }
            }
            fp4_epi_bar();
          }
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
    if (threadIdx.x == 0) zb_record_error(prm.status, ZB_ERR_MBAR_TIMEOUT, kKernelGroupedFp4, blockIdx.x, BN);
    // copies in flight may still land in this CTA's shared memory: give them time before the CTA exits
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

template <int BN, bool SWIGLU, bool QOUT>
int launch_fp4(const CUtensorMap& tx, const Fp4Params& prm, int grid, cudaStream_t s) {
  constexpr int smem = fp4_smem_bytes(BN, SWIGLU);
  static_assert(smem <= 232448, "shared memory of one CTA");
  static bool configured[16] = {};
  if (const int rc = zb_config_smem_once(zb_moe_grouped_gemm_fp4_kernel<BN, SWIGLU, QOUT>, smem, configured)) return rc;
  zb_launch(zb_moe_grouped_gemm_fp4_kernel<BN, SWIGLU, QOUT>, dim3(grid), dim3(kThreads), smem, s, tx, prm);
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

extern "C" {

// xq [cap, k / 2] packed e2m1 activation codes (rows grouped by expert: offsets [e_local + 1]), x_sf [cap, k / 16]
// their f8e4m3 block scales, x_gscale one fp32 on the device or null; blocks [e_local, n / 128, k / 256, 18432]
// the weights as packed by nvfp4_pack_blocks_mma; w_gscale [e_local, gs_per] fp32 or null (gs_per = 2 with
// `swiglu`: gate rows, up rows).  out [cap, ldo] bf16; with `swiglu` the weight rows are interleaved
// [64 gate | 64 up] per 128 and the output has n / 2 features.  k a multiple of 256, n a multiple of 128.
// Token tiles of 16 .. 128 chosen from `avg_tokens` per expert.  With `out_q` / `out_sf` (and `swiglu`) the output
// is written as NVFP4 instead: codes [cap, ldo / 2], scales [cap, ldo / 16] (`out` may be null; ldo a multiple of 64).
int zb_moe_grouped_gemm_fp4(const void* xq, const void* x_sf, const float* x_gscale, const void* blocks,
                            const float* w_gscale, int gs_per, void* out, void* out_q, void* out_sf, const int32_t* offsets,
                            int e_local, int n, int k, int cap, int ldo, int swiglu, int avg_tokens, void* stream) {
  if (cap <= 0 || e_local <= 0) return 0;
  if (e_local > kZbMaxExperts) return -61;
  if (k % kStageK != 0 || n % kBlockP != 0 || ldo % 8 != 0) return -66;
  if (swiglu < 0 || swiglu > ZB_ACT_RELU2) return -67;
  const bool gated = swiglu >= ZB_ACT_SWIGLU && swiglu <= ZB_ACT_GEGLU_TANH;
  if (gs_per != 1 && !(gs_per == 2 && gated)) return -67;
  const bool qout = out_q != nullptr;
  if (qout && (!gated || out_sf == nullptr || ldo % 64 != 0 || (reinterpret_cast<uintptr_t>(out_q) & 7) != 0)) return -68;
  if ((reinterpret_cast<uintptr_t>(blocks) & 15) != 0 || (reinterpret_cast<uintptr_t>(x_sf) & 15) != 0) return -66;
  ZbDeviceState* st = zb_device_state();
  if (!st) return -20;
  int bn = 16;
  while (bn < avg_tokens * 2 && bn < 128) bn <<= 1;
  Fp4Params prm;
  prm.offsets = offsets;
  prm.e_local = e_local;
  prm.n = n;
  prm.k = k;
  prm.ldo = ldo;
  prm.out = reinterpret_cast<__nv_bfloat16*>(out);
  prm.cap = cap;
  prm.blocks = reinterpret_cast<const uint8_t*>(blocks);
  prm.x_sf = reinterpret_cast<const uint8_t*>(x_sf);
  prm.w_gscale = w_gscale;
  prm.gs_per = gs_per;
  prm.x_gscale = x_gscale;
  prm.out_q = reinterpret_cast<uint8_t*>(out_q);
  prm.out_sf = reinterpret_cast<uint8_t*>(out_sf);
  prm.act = swiglu;
  prm.status = st->status;
  CUtensorMap tx;
  int rc = zb_make_tmap_u8_2d_ex(&tx, xq, cap, k / 2, kStageK / 2, bn, 1);
  if (rc != 0) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int grid = st->num_sms;
#define ZB_FP4(BN_)                                                                  \
  return qout ? launch_fp4<BN_, true, true>(tx, prm, grid, s)                         \
              : (gated ? launch_fp4<BN_, true, false>(tx, prm, grid, s) : launch_fp4<BN_, false, false>(tx, prm, grid, s));
  switch (bn) {
    case 16: ZB_FP4(16)
    case 32: ZB_FP4(32)
    case 64: ZB_FP4(64)
    case 128: ZB_FP4(128)
  }
#undef ZB_FP4
  return -65;
}

}  // extern "C"
