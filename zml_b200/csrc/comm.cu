// Communication runtime: symmetric heap over CUDA IPC, peer pointer tables, a
// device-side barrier with bounded waits, and a stand-alone in-kernel all-reduce.
//
// One process drives one GPU.  Every rank allocates the same-sized heap with
// cudaMalloc, exports it with cudaIpcGetMemHandle, and opens the handles of its
// peers, which gives plain device pointers into the peers' HBM; loads and stores
// through them travel over NVLink 5 / NVSwitch.  The host-side exchange of the
// 64-byte handles goes through torch.distributed (see parallel/symm.py).
//
// This replaces what NCCL (through XLA) does for the reference
// (zml/ops.zig:24-173; platforms/cuda/cuda.bzl:229-238): the collectives of the hot
// path are issued by the compute kernels themselves (see fused_ar.h), and this
// file provides the memory they talk through.
#include <cstring>

#include "host_api.h"

namespace {

constexpr uint32_t kKernelBarrier = 5;

// Barrier over all ranks: rank r writes `epoch` into slot [r] of every peer's flag
// array, then waits until its own array holds `epoch` in every slot.
__global__ void zb_barrier_kernel(ZbArContext ctx, size_t flag_off, ZbStatus* status,
                                  uint32_t* epoch_ptr) {
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) abort_flag = 0u;
  __syncthreads();
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(epoch_ptr);
  const int r = threadIdx.x;
  if (r < ctx.world) {
    uint32_t* peer = reinterpret_cast<uint32_t*>(reinterpret_cast<char*>(ctx.heap[r]) + flag_off);
    __threadfence_system();
    zb_st_release_sys(peer + ctx.rank, epoch);
    const uint32_t* mine =
        reinterpret_cast<const uint32_t*>(reinterpret_cast<char*>(ctx.heap[ctx.rank]) + flag_off);
    if (!zb_wait_flag(mine + r, epoch, &abort_flag))
      zb_record_error(status, ZB_ERR_FLAG_TIMEOUT, kKernelBarrier, static_cast<uint32_t>(r), epoch);
  }
  __syncthreads();
  if (threadIdx.x == 0) *reinterpret_cast<volatile uint32_t*>(epoch_ptr) = epoch + 1u;
}

// One-shot all-reduce (sum) of a bf16 buffer that lives at the same offset of every
// rank's heap: every rank reads all peers' copies and writes the sum to `out` locally.
// Used for small messages and as the in-kernel counterpart of the NCCL baseline in tests.
__global__ void zb_allreduce_oneshot_kernel(ZbArContext ctx, size_t in_off, __nv_bfloat16* out,
                                            size_t n_vec) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n_vec;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < ctx.world; ++r) {
      const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<char*>(ctx.heap[r]) + in_off);
      const uint4 v = __ldcg(src + i);
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = zb_unpack_bf16x2(u[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    reinterpret_cast<uint4*>(out)[i] =
        make_uint4(zb_pack_bf16x2(acc[0], acc[1]), zb_pack_bf16x2(acc[2], acc[3]),
                   zb_pack_bf16x2(acc[4], acc[5]), zb_pack_bf16x2(acc[6], acc[7]));
  }
}

// ------------------------------------------------------------------ two-shot all-reduce in tagged slots
// out = residual + sum over ranks of `in` (bf16 [tokens, d]) for decode-sized tensors (tens of KB to a few MB),
// where a bandwidth-optimal ring pays its latency many times over.  The tensor is cut into `world` shards of
// `vs` 16-byte vectors.  Every thread owns vector g of every shard:
//   1. it stores its partial of every foreign shard into the owner's slot area (8-byte {two bf16, epoch}
//      words: a word arrives whole, so the tag needs no fence and no flag);
//   2. for its own shard it waits for the peers' words, sums all ranks in rank order, adds the residual and
//      rounds to bf16 - one rank computes every element, so all ranks end with the same bits;
//   3. it stores the result into every peer's second slot area and collects the other shards from its own.
// Each rank sends 2 x (world - 1) / world of the tensor (twice that in slot bytes) and waits two NVLink
// latencies.  Slot areas alternate by epoch parity (see fused_ar.h for why one alternation is enough).
// The reference leaves this reduction to NCCL through XLA (zml/ops.zig:24-173).
constexpr uint32_t kKernelAllReduceLl = 11;

struct LlAllReduce {
  uint2* slots[8];          // slot area in every rank's heap ([rank] is local)
  size_t region_words;      // 8-byte words of one (phase, parity) region: world * vs * 4
  uint32_t* epoch;
  uint32_t* ticket;
  int rank;
  int world;
};

__global__ void __launch_bounds__(128)
zb_allreduce_ll_kernel(const uint4* __restrict__ in, const uint4* __restrict__ residual, uint4* __restrict__ out, long long vs,
                       const LlAllReduce ar, ZbStatus* status) {
  zb_pdl_launch();
  zb_pdl_wait();
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(ar.epoch);
  const size_t par = epoch & 1u;
  const int W = ar.world, rank = ar.rank;
  bool timed_out = false;
  const uint64_t t0 = zb_globaltimer();
  auto wait4 = [&](const uint2* src, uint32_t (&w)[4]) {
    uint32_t spins = 0;
    while (true) {
      bool ready = true;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint2 x = zb_ld_ll(src + q);
        w[q] = x.x;
        ready = ready && (x.y == epoch);
      }
      if (ready || timed_out) return;
      if ((++spins & 0x3f) == 0 && zb_globaltimer() - t0 > ZB_WAIT_LIMIT_NS) timed_out = true;
    }
  };
  for (long long g = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; g < vs;
       g += static_cast<long long>(gridDim.x) * blockDim.x) {
    // 1. partials of the foreign shards go to their owners
    for (int s = 0; s < W; ++s) {
      if (s == rank) continue;
      const uint4 v = in[s * vs + g];
      uint2* dst = ar.slots[s] + ((0 * 2 + par) * W + rank) * static_cast<size_t>(vs) * 4 + g * 4;
      zb_st_ll(dst + 0, v.x, epoch);
      zb_st_ll(dst + 1, v.y, epoch);
      zb_st_ll(dst + 2, v.z, epoch);
      zb_st_ll(dst + 3, v.w, epoch);
    }
    // 2. own shard: sum of all ranks in rank order
    const uint4 mine = in[rank * vs + g];
    uint4 rv = make_uint4(0u, 0u, 0u, 0u);
    if (residual != nullptr) rv = residual[rank * vs + g];
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < W; ++r) {
      uint32_t w[4] = {mine.x, mine.y, mine.z, mine.w};
      if (r != rank) wait4(ar.slots[rank] + ((0 * 2 + par) * W + r) * static_cast<size_t>(vs) * 4 + g * 4, w);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = zb_unpack_bf16x2(w[q]);
        acc[2 * q] += f.x;
        acc[2 * q + 1] += f.y;
      }
    }
    {
      const uint32_t w[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = zb_unpack_bf16x2(w[q]);
        acc[2 * q] += f.x;
        acc[2 * q + 1] += f.y;
      }
    }
    const uint4 res = make_uint4(zb_pack_bf16x2(acc[0], acc[1]), zb_pack_bf16x2(acc[2], acc[3]), zb_pack_bf16x2(acc[4], acc[5]),
                                 zb_pack_bf16x2(acc[6], acc[7]));
    // 3. the finished shard goes to every peer; the other shards come from theirs
    for (int p = 0; p < W; ++p) {
      if (p == rank) continue;
      uint2* dst = ar.slots[p] + ((1 * 2 + par) * W + rank) * static_cast<size_t>(vs) * 4 + g * 4;
      zb_st_ll(dst + 0, res.x, epoch);
      zb_st_ll(dst + 1, res.y, epoch);
      zb_st_ll(dst + 2, res.z, epoch);
      zb_st_ll(dst + 3, res.w, epoch);
    }
    out[rank * vs + g] = res;
    for (int s = 0; s < W; ++s) {
      if (s == rank) continue;
      uint32_t w[4];
      wait4(ar.slots[rank] + ((1 * 2 + par) * W + s) * static_cast<size_t>(vs) * 4 + g * 4, w);
      out[s * vs + g] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
  if (timed_out) zb_record_error(status, ZB_ERR_FLAG_TIMEOUT, kKernelAllReduceLl, blockIdx.x, rank);
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

// ------------------------------------------------------------------ arg-max over a vocabulary split across ranks
// Greedy sampling under a vocab-parallel lm_head: every rank holds the logits of its own columns.  One block per
// row finds the local maximum and its first index, writes {value, tag} and {global index, tag} into its slot of
// every peer's heap, then the first `world` lanes of warp 0 collect the peers' pairs and pick the winner (highest
// value; equal values -> lowest global index, which is what an arg-max over the gathered row would return).  Every
// rank ends with the same token, and nothing but 16 bytes per row and peer crosses NVLink - the reference (and the
// fallback here) all-gathers the candidates with two NCCL calls and reduces them with tensor ops
// (examples/llm/models/llama/model.zig: sampling after the lm_head).  Slots alternate by epoch parity, as in the
// two-shot all-reduce above; waits are bounded and end in the status word, the row then keeps the local candidate.
constexpr uint32_t kKernelArgmaxTp = 15;
constexpr int kArgmaxTpMaxRows = 1024;

struct TpArgmax {
  uint2* slots[8];          // [2 parities][world sources][kArgmaxTpMaxRows][2] in every rank's heap ([rank] is local)
  uint32_t* epoch;
  uint32_t* ticket;
  int rank;
  int world;
};

__global__ void __launch_bounds__(1024)
zb_argmax_tp_kernel(const float* __restrict__ logits, int32_t* __restrict__ out, int rows, int vocab, long long stride,
                    int col_offset, const TpArgmax ar, ZbStatus* status) {
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(ar.epoch);
  const size_t par = epoch & 1u;
  const int W = ar.world, rank = ar.rank;
  bool timed_out = false;
  const uint64_t t0 = zb_globaltimer();
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    float best;
    int bi;
    zb_block_argmax_1024(logits + static_cast<size_t>(row) * stride, vocab, best, bi);
    if (threadIdx.x < 32) {
      const int gi = bi == 0x7fffffff ? bi : bi + col_offset;
      const int lane = threadIdx.x;
      if (lane < W && lane != rank) {          // lane p publishes to peer p ...
        uint2* dst = ar.slots[lane] + ((par * W + rank) * kArgmaxTpMaxRows + row) * 2;
        zb_st_ll(dst, __float_as_uint(best), epoch);
        zb_st_ll(dst + 1, static_cast<uint32_t>(gi), epoch);
      }
      float cv = best;
      int ci = gi;
      if (lane < W && lane != rank) {          // ... and collects peer p's candidate
        const uint2* src = ar.slots[rank] + ((par * W + lane) * kArgmaxTpMaxRows + row) * 2;
        uint32_t spins = 0;
        while (true) {
          const uint2 a = zb_ld_ll(src), b = zb_ld_ll(src + 1);
          if (a.y == epoch && b.y == epoch) {
            cv = __uint_as_float(a.x);
            ci = static_cast<int>(b.x);
            break;
          }
          if ((++spins & 0x3f) == 0 && zb_globaltimer() - t0 > ZB_WAIT_LIMIT_NS) {
            timed_out = true;
            break;
          }
        }
      }
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) {         // lanes >= world hold copies of the local candidate
        const float ov = __shfl_xor_sync(0xffffffffu, cv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, ci, o);
        zb_argmax_merge(cv, ci, ov, oi);
      }
      if (lane == 0) out[row] = ci == 0x7fffffff ? 0 : ci;
    }
    __syncthreads();                            // the reduction's shared memory is reused by the next row
  }
  if (timed_out) zb_record_error(status, ZB_ERR_FLAG_TIMEOUT, kKernelArgmaxTp, blockIdx.x, rank);
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

// ------------------------------------------------------------------ all-reduce through NVSwitch (multimem)
// out = residual + sum over ranks of `in`, bf16, any size that is a multiple of 16 bytes; `in` and `out` live at
// the same offsets of every rank's heap, and the heap is bound to a multicast address.  Every rank owns a
// contiguous shard of the tensor: it loads the shard with multimem.ld_reduce (NVSwitch fetches the W copies
// and returns their sum, accumulated in fp32 - one rank computes every element, so all ranks end with the
// same bits), adds the residual, and writes the result into every rank's `out` with one multimem.st.  Per
// rank about one tensor's worth of bytes crosses NVLink in each direction, against 2 (W - 1) / W through a
// ring or peer stores.  A cross-rank barrier per block brackets the pass: before it, every rank's partial
// sums are complete (the kernel that wrote them precedes this one on the stream); after it, every shard has
// been written everywhere.  `in` == `out` is allowed: an element is read and written by its owner only.
// The reference gets this sum from NCCL through XLA (zml/ops.zig:24-173).
constexpr uint32_t kKernelAllReduceMm = 12;
constexpr int kMmMaxBlocks = 128;

struct MmAllReduce {
  char* mc;                 // multicast base of the heaps
  uint32_t* flags[8];       // [2 phases][kMmMaxBlocks][8] u32 in every rank's heap ([rank] is local)
  uint32_t* epoch;
  uint32_t* ticket;
  int rank;
  int world;
};

__global__ void __launch_bounds__(512)
zb_allreduce_mm_kernel(size_t in_off, size_t out_off, const uint4* __restrict__ residual, long long n_vec, const MmAllReduce ar,
                       ZbStatus* status) {
  // No programmatic dependent launch around this kernel (it is launched without the attribute and never triggers
  // its dependents early): its blocks wait for another GPU, and with the two-SM GEMMs of a large model's prefill
  // started early on every SM behind it, one rank's GPU stopped making progress (Llama-3.1-70B shapes, 64 x 2048
  // tokens, 2 and 4 ranks; any one of: no early launch, the one-SM GEMM, NCCL instead of this kernel - and the
  // run completes).  The kernel before it has finished when it starts, the kernel after it starts when it is done.
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) abort_flag = 0u;
  __syncthreads();
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(ar.epoch);
  const int W = ar.world, rank = ar.rank;
  auto block_barrier = [&](int phase) {
    // rank r's block b tells block b of every rank that it got here, and waits for all of them
    if (static_cast<int>(threadIdx.x) < W) {
      const size_t slot = (static_cast<size_t>(phase) * kMmMaxBlocks + blockIdx.x) * 8;
      __threadfence_system();
      zb_st_release_sys(ar.flags[threadIdx.x] + slot + rank, epoch);
      if (!zb_wait_flag(ar.flags[rank] + slot + threadIdx.x, epoch, &abort_flag))
        zb_record_error(status, ZB_ERR_FLAG_TIMEOUT, kKernelAllReduceMm, static_cast<uint32_t>(phase * 8 + threadIdx.x), epoch);
    }
    __syncthreads();
  };
  block_barrier(0);
  if (abort_flag == 0u) {
    const long long vs = (n_vec + W - 1) / W;                       // vectors per shard
    const long long v0 = static_cast<long long>(rank) * vs;
    const long long mine = max(0ll, min(vs, n_vec - v0));
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    constexpr int kUnroll = 4;                                      // loads in flight per thread
    for (long long base = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; base < mine; base += stride * kUnroll) {
      uint4 v[kUnroll], r[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const long long i = base + u * stride;
        if (i < mine) {
          v[u] = zb_multimem_ld_reduce_bf16x8(ar.mc + in_off + static_cast<size_t>(v0 + i) * 16);
          r[u] = residual != nullptr ? residual[v0 + i] : make_uint4(0u, 0u, 0u, 0u);
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const long long i = base + u * stride;
        if (i < mine) {
          if (residual != nullptr) {
            const uint32_t a[4] = {v[u].x, v[u].y, v[u].z, v[u].w}, b[4] = {r[u].x, r[u].y, r[u].z, r[u].w};
            uint32_t o[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float2 fa = zb_unpack_bf16x2(a[q]), fb = zb_unpack_bf16x2(b[q]);
              o[q] = zb_pack_bf16x2(fa.x + fb.x, fa.y + fb.y);
            }
            v[u] = make_uint4(o[0], o[1], o[2], o[3]);
          }
          zb_multimem_st_16(ar.mc + out_off + static_cast<size_t>(v0 + i) * 16, v[u]);
        }
      }
    }
  }
  __syncthreads();
  block_barrier(1);
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t ticket = atomicAdd(ar.ticket, 1u);
    if (ticket == gridDim.x - 1) {
      *ar.ticket = 0u;
      *reinterpret_cast<volatile uint32_t*>(ar.epoch) = epoch + 1u;
    }
  }
}

}  // namespace

// A wait with a caller-chosen limit on a flag the caller owns: the building block of every
// in-kernel collective, exposed so that the timeout path (status word, clean return, context
// still usable) can be exercised without a peer.
constexpr uint32_t kKernelWaitProbe = 8;
__global__ void zb_wait_probe_kernel(const uint32_t* flag, uint32_t expected, unsigned long long limit_ns,
                                     ZbStatus* status, uint32_t phase, uint32_t* reached) {
  __shared__ uint32_t abort_flag;
  abort_flag = 0u;
  const bool ok = zb_wait_flag_limit(flag, expected, &abort_flag, limit_ns);
  if (!ok) zb_record_error(status, ZB_ERR_FLAG_TIMEOUT, kKernelWaitProbe, phase, expected);
  if (reached != nullptr) *reached = ok ? 1u : 0u;
}

extern "C" {

// Launches one thread that waits until *flag >= expected or `limit_ns` passed.  On a timeout the
// device status records {flag timeout, wait_probe, phase, expected} and *reached is 0.
int zb_wait_probe(const void* flag, unsigned expected, unsigned long long limit_ns, unsigned phase,
                  void* reached, void* stream) {
  ZbDeviceState* st = zb_device_state();
  if (st == nullptr) return -20;
  if (limit_ns > 5000000000ull) return -21;      // a probe never waits longer than 5 s
  zb_wait_probe_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint32_t*>(flag), expected, limit_ns, st->status, phase,
      reinterpret_cast<uint32_t*>(reached));
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

int zb_symm_alloc(size_t bytes, void** ptr) {
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaMemset(*ptr, 0, bytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaDeviceSynchronize());
}

int zb_symm_free(void* ptr) { return static_cast<int>(cudaFree(ptr)); }

int zb_symm_ipc_handle(void* ptr, unsigned char* out64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return static_cast<int>(e);
  static_assert(sizeof(h) == 64, "IPC handle size");
  std::memcpy(out64, &h, 64);
  return 0;
}

int zb_symm_ipc_open(const unsigned char* in64, void** ptr) {
  cudaIpcMemHandle_t h;
  std::memcpy(&h, in64, 64);
  return static_cast<int>(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
}

int zb_symm_ipc_close(void* ptr) { return static_cast<int>(cudaIpcCloseMemHandle(ptr)); }

// heap[r] for r != rank are the opened peer pointers; heap[rank] is the local allocation.
ZbArContext* zb_ar_ctx_create(int rank, int world, void* const* heap, size_t recv_off,
                              size_t recv_bytes, size_t push_flag_off, size_t done_flag_off,
                              int max_tiles) {
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return nullptr;
  ZbArContext* c = new ZbArContext();
  c->rank = rank;
  c->world = world;
  for (int r = 0; r < 8; ++r) c->heap[r] = r < world ? heap[r] : nullptr;
  c->recv_off = recv_off;
  c->recv_bytes = recv_bytes;
  c->push_flag_off = push_flag_off;
  c->done_flag_off = done_flag_off;
  c->max_tiles = max_tiles;
  uint32_t* ctr = nullptr;
  if (cudaMalloc(&ctr, 16 * sizeof(uint32_t)) != cudaSuccess) {
    delete c;
    return nullptr;
  }
  // {gemm epoch, exit ticket, barrier epoch, unused, combine epoch, combine exit ticket, tagged-slot all-reduce epoch,
  //  its exit ticket, multimem all-reduce epoch, its exit ticket, band-pipeline epoch, its ticket, vocab-parallel arg-max
  //  epoch, its exit ticket, unused ...}
  const uint32_t init[16] = {1u, 0u, 1u, 0u, 1u, 0u, 1u, 0u, 1u, 0u, 1u, 0u, 1u, 0u, 1u, 0u};
  cudaMemcpy(ctr, init, sizeof(init), cudaMemcpyHostToDevice);
  c->epoch = ctr;
  c->exit_ticket = ctr + 1;
  c->mc_heap = nullptr;
  return c;
}

// Tells the context the NVLink multicast address that aliases every rank's heap (null: none).
void zb_ar_ctx_set_multicast(ZbArContext* c, void* mc_heap) {
  if (c != nullptr) c->mc_heap = mc_heap;
}

void zb_ar_ctx_destroy(ZbArContext* c) {
  if (c == nullptr) return;
  cudaFree(c->epoch);
  delete c;
}

// Device-side barrier across the group on `stream`; flag_off addresses 8 u32 slots in the heap.
int zb_comm_barrier(const ZbArContext* c, size_t flag_off, void* stream) {
  ZbDeviceState* st = zb_device_state();
  if (!st || !c) return -20;
  zb_barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(*c, flag_off, st->status,
                                                                         c->epoch + 2);
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

// Sum of the bf16 buffers at `in_off` of every heap -> local `out`.  The caller brackets it
// with zb_comm_barrier (inputs written before, inputs reusable after).
int zb_allreduce_oneshot(const ZbArContext* c, size_t in_off, void* out, size_t n_elems, void* stream) {
  if (!c) return -20;
  if (n_elems % 8 != 0 || in_off % 16 != 0) return -10;
  const size_t n_vec = n_elems / 8;
  size_t blocks = (n_vec + 255) / 256;
  if (blocks > 296) blocks = 296;
  zb_allreduce_oneshot_kernel<<<static_cast<int>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      *c, in_off, reinterpret_cast<__nv_bfloat16*>(out), n_vec);
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

// out = residual + sum over the group of `in`, bf16 [tokens, d], by the two-shot tagged-slot kernel.  `in`,
// `residual` (may be null) and `out` are local; the exchange goes through the slot area at `slot_off` of every
// rank's heap (at least 16 bytes per element of the tensor).  tokens * d / 8 must be a multiple of the group size.
int zb_allreduce_ll(const ZbArContext* c, const void* in, const void* residual, void* out, long long elems, size_t slot_off,
                    size_t slot_bytes, void* stream) {
  ZbDeviceState* st = zb_device_state();
  if (!st || !c) return -20;
  if (elems <= 0) return 0;
  if (elems % (8ll * c->world) != 0 || slot_off % 16 != 0) return -10;
  const long long vs = elems / 8 / c->world;
  LlAllReduce ar = {};
  ar.region_words = static_cast<size_t>(c->world) * vs * 4;
  if (4 * ar.region_words * sizeof(uint2) > slot_bytes) return -68;
  for (int r = 0; r < c->world; ++r) ar.slots[r] = reinterpret_cast<uint2*>(reinterpret_cast<char*>(c->heap[r]) + slot_off);
  ar.epoch = c->epoch + 6;
  ar.ticket = c->epoch + 7;
  ar.rank = c->rank;
  ar.world = c->world;
  long long blocks = (vs + 127) / 128;
  // Threads of one rank wait for the same threads of its peers, so every block of the grid must be resident at once
  // on every rank: the grid never exceeds what the occupancy calculator says fits (the grid-stride loop covers the rest).
  static int resident_per_sm = 0;
  if (resident_per_sm == 0) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, zb_allreduce_ll_kernel, 128, 0) != cudaSuccess || n < 1) n = 1;
    resident_per_sm = n > 8 ? 8 : n;
  }
  const long long cap = static_cast<long long>(st->num_sms) * resident_per_sm;
  if (blocks > cap) blocks = cap;
  zb_launch(zb_allreduce_ll_kernel, dim3(static_cast<unsigned>(blocks)), dim3(128), 0, reinterpret_cast<cudaStream_t>(stream),
            reinterpret_cast<const uint4*>(in), reinterpret_cast<const uint4*>(residual), reinterpret_cast<uint4*>(out), vs, ar,
            st->status);
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

// out[r] = arg-max over the whole vocabulary of row r; every rank passes the f32 logits of its own `vocab` columns
// (global column of local column j: col_offset + j; padding columns hold -inf).  `slot_off` addresses
// zb_argmax_tp_slot_bytes(world) bytes of every rank's heap.  rows <= 1024.
size_t zb_argmax_tp_slot_bytes(int world) { return static_cast<size_t>(2) * world * kArgmaxTpMaxRows * 2 * sizeof(uint2); }

int zb_argmax_tp(const ZbArContext* c, const float* logits, int32_t* out, int rows, int vocab, long long stride, int col_offset,
                 size_t slot_off, void* stream) {
  ZbDeviceState* st = zb_device_state();
  if (!st || !c) return -20;
  if (rows <= 0) return 0;
  if (rows > kArgmaxTpMaxRows || slot_off % 16 != 0 || vocab < 0) return -10;
  TpArgmax ar = {};
  for (int r = 0; r < c->world; ++r) ar.slots[r] = reinterpret_cast<uint2*>(reinterpret_cast<char*>(c->heap[r]) + slot_off);
  ar.epoch = c->epoch + 12;
  ar.ticket = c->epoch + 13;
  ar.rank = c->rank;
  ar.world = c->world;
  // A block waits for the same block of every peer, so all blocks must be resident at once on every rank: at most one
  // per SM, the loop over rows covers the rest (every rank visits the rows in the same order, publishing before it waits).
  const int blocks = rows < st->num_sms ? rows : st->num_sms;
  // Launched without programmatic dependent launch, like the all-reduce inside NVSwitch below: a kernel that waits for
  // its peers starts only after the kernel in front of it (the lm_head GEMM) has left the SMs.
  zb_argmax_tp_kernel<<<dim3(static_cast<unsigned>(blocks)), dim3(1024), 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      logits, out, rows, vocab, stride, col_offset, ar, st->status);
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

// out = residual + sum over the group of `in` by multimem load-reduce and store (see zb_allreduce_mm_kernel).  `in_off` and
// `out_off` are byte offsets into every rank's heap (16-byte aligned, may be equal); `flag_off` addresses
// 2 * 128 * 8 u32 of flags; `residual` (may be null) is local.  Needs a context with a multicast address.
int zb_allreduce_mm(const ZbArContext* c, size_t in_off, size_t out_off, const void* residual, long long elems, size_t flag_off,
                    void* stream) {
  ZbDeviceState* st = zb_device_state();
  if (!st || !c) return -20;
  if (c->mc_heap == nullptr) return -69;
  if (elems <= 0) return 0;
  if (elems % 8 != 0 || in_off % 16 != 0 || out_off % 16 != 0 || flag_off % 16 != 0) return -10;
  const long long n_vec = elems / 8;
  MmAllReduce ar = {};
  ar.mc = reinterpret_cast<char*>(c->mc_heap);
  for (int r = 0; r < c->world; ++r) ar.flags[r] = reinterpret_cast<uint32_t*>(reinterpret_cast<char*>(c->heap[r]) + flag_off);
  ar.epoch = c->epoch + 8;
  ar.ticket = c->epoch + 9;
  ar.rank = c->rank;
  ar.world = c->world;
  const long long vs = (n_vec + c->world - 1) / c->world;
  long long blocks = (vs + 512 * 4 - 1) / (512 * 4);
  if (blocks < 1) blocks = 1;
  if (blocks > kMmMaxBlocks) blocks = kMmMaxBlocks;
  zb_allreduce_mm_kernel<<<dim3(static_cast<unsigned>(blocks)), dim3(512), 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      in_off, out_off, reinterpret_cast<const uint4*>(residual), n_vec, ar, st->status);
  zb_count_launch(1);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
