// Description of the peer memory used by the fused GEMM + all-reduce kernel
// (row-parallel o_proj / down_proj followed by the tensor-parallel all-reduce).
//
// Protocol, per output tile t of the GEMM (owner(t) = t % world):
//   1. every rank writes its partial tile (bf16) into the owner's `recv` slot
//      [src = rank][t / world] with plain peer stores over NVLink, then publishes
//      push_flag[owner][(t / world) * world + rank] = epoch (st.release.sys);
//   2. the CTA that produced tile t on the owner waits for the `world` flags, sums the
//      partials in rank order in fp32 (deterministic), adds bias / residual, and stores
//      the bf16 result into the output buffer of EVERY rank, then publishes
//      done_flag[dst][t] = epoch on every rank;
//   3. before the kernel ends each rank waits until done_flag[t] == epoch for all t,
//      so kernel completion means the all-reduced output is complete locally.
// Few tokens (one_shot): latency matters more than bytes, so the exchange is a single hop.
//   1. every rank stores its partial tile (bf16) into the staging area of EVERY rank, slot
//      [epoch parity][src = rank][tile], then publishes push_flag[dst][tile * world + rank] = epoch;
//   2. on every rank the CTA that produced tile t waits for the `world` flags of t, sums the
//      partials in rank order in fp32 (the same bits on every rank), adds bias / residual and
//      stores the tile into its own output.  No done flags: a rank's kernel ends when it has
//      finished all its tiles.  Two staging halves alternate by epoch parity: a rank cannot
//      finish launch n+1 before every peer has published launch n+1, i.e. has finished launch
//      n, so writes of launch n+2 never meet reads of launch n.
// `epoch` is a device-side launch counter (same sequence on every rank), so flags are
// never reset and CUDA-graph replays need no host-side change.  Every wait is bounded.
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

constexpr int kZbMaxRanks = 8;

struct ZbFusedAr {
  int rank;
  int world;
  int slots_per_src;                       // ceil(num_out_tiles / world)
  int one_shot;                            // 1: single-hop exchange (few tokens), see above
  __nv_bfloat16* recv_peer[kZbMaxRanks];   // staging area of each rank
  __nv_bfloat16* out_peer[kZbMaxRanks];    // output buffer of each rank (same layout as `out`)
  uint32_t* push_flag_peer[kZbMaxRanks];
  uint32_t* done_flag_peer[kZbMaxRanks];
  uint32_t* epoch;                         // local: current launch number (starts at 1)
  uint32_t* exit_ticket;                   // local: CTAs that finished this launch
};
