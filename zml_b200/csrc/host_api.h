// Host-side declarations shared by the .cu files of libzb_cuda.so.
// Every exported symbol is `extern "C"` and takes raw device pointers plus a
// `cudaStream_t` passed as `void*`, so the library can be driven from Python
// (ctypes) or from C/C++ without any framework headers.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "common.cuh"

// Per-device state owned by the library (created by zb_init on that device).
struct ZbDeviceState {
  int device;
  int num_sms;
  ZbStatus* status;            // device memory, zeroed by zb_status_reset
  float* gemm_scratch;         // split-K partial tiles
  size_t gemm_scratch_bytes;
  uint32_t* gemm_counters;     // one per output tile, zero between launches
  int gemm_counters_len;
  float* attn_scratch;         // split-KV partial outputs + (m, l) pairs
  size_t attn_scratch_bytes;
  uint32_t* attn_counters;     // one per (sequence, kv head), zero between launches
  int attn_counters_len;
};

// Peer-memory description of one tensor-parallel group, built by zb_ar_ctx_create (comm.cu).
struct ZbArContext {
  int rank;
  int world;
  void* heap[8];          // base of every rank's symmetric heap (peer pointers; [rank] is local)
  size_t recv_off;        // staging area for partial tiles
  size_t recv_bytes;
  size_t push_flag_off;   // u32 flags [max_tiles / world + 1][world]
  size_t done_flag_off;   // u32 flags [max_tiles]
  int max_tiles;
  uint32_t* epoch;        // local device counter, starts at 1
  uint32_t* exit_ticket;  // local device counter
  void* mc_heap;          // NVLink multicast address of the heaps (one address, every rank's copy), or null
};

// Optional epilogue work of the bf16 GEMM (gemm_bf16.cu).  All pointers are local device memory.
//   in_sumsq : partial sums of squares of the activation rows, [in_parts][in_ld] fp32; the accumulator of
//              token t is multiplied by rsqrt(sum_i in_sumsq[i][t] * in_inv_d + in_eps) before bias and
//              residual.  With the RMSNorm weight folded into the columns of `w` this makes the GEMM
//              compute rmsnorm(a) * w^T without a normalisation kernel (zml/nn.zig:486-493).
//   swiglu   : the rows of `w` interleave gate and up (row 2 i = gate_i, row 2 i + 1 = up_i); the output has
//              n / 2 columns, out[t][i] = silu(gate_i) * up_i (examples/llm/models/llama/model.zig:491-496).
//   out_sumsq: the kernel writes partial sums of squares of its (bf16-rounded) output rows, [parts][out_ld];
//              `parts` is reported by the entry point.
//   pf_ptr   : contiguous bytes (the next GEMM's weights) that the kernel pulls into L2 once its own operand
//              loads have been issued.
struct ZbGemmEpi {
  const float* in_sumsq;
  float* out_sumsq;
  const void* pf_ptr;
  unsigned long long pf_bytes;
  int in_parts;
  int in_ld;
  int out_ld;
  float in_inv_d;
  float in_eps;
  int swiglu;
};

// Band pipeline of the prefill collectives (gemm_bf16.cu): the tensor-parallel all-reduce of a row-parallel
// GEMM's output, cut into bands of 128 tokens and overlapped with the GEMM that consumes the sum.
//   mode 1 (producer, the row-parallel GEMM): partial sums go to `part` in this rank's heap; when the last
//     column tile of a band is stored the band's owner (band % world) is told: ready[owner][band][rank] = epoch.
//   mode 2 (consumer, the column-parallel GEMM that follows): the first `comm_ctas` CTAs of the grid do not
//     multiply.  For every band this rank owns they wait for the `world` ready flags, pull the band's partial
//     sums from every rank's heap with bulk copies (cp.async.bulk, peer memory over NVLink, no multicast) into
//     shared memory, add them up in rank order in fp32 together with the residual, and push the new residual
//     stream with bulk copies - and its row statistics with plain stores - into every rank's heap, then publish
//     done[rank'][band] = epoch on every rank.  The other CTAs run the GEMM; their TMA producer waits for
//     done[band] before it loads the band's rows.
// Flags carry a device-side launch counter, so nothing is reset and CUDA-graph replays need no host change.
struct ZbBandPipe {
  int mode;                    // 0: off
  int num_bands;
  int tiles_per_band;          // producer: column tiles per band
  int comm_ctas;               // consumer
  int world;
  int rank;
  int d;                       // row length of the reduced tensor (hidden size)
  int tokens;
  uint32_t* epoch;             // local device counter {epoch, exit ticket}
  uint32_t* count_p;           // local [num_bands]: tiles of the band stored (producer), zero between launches
  uint32_t* count_c;           // local [num_bands]: comm CTAs done with the band (consumer), zero between launches
  uint32_t* ready_peer[8];     // [num_bands][8] in every rank's heap
  uint32_t* done_peer[8];      // [num_bands] in every rank's heap
  float* sumsq_peer[8];        // [tokens] in every rank's heap: sum of squares of the rows of the new residual stream
  char* heap[8];               // base of every rank's heap ([rank] is local)
  size_t part_off;             // heap offset of the partial sums [tokens, d] bf16
  size_t x_off;                // heap offset of the reduced tensor [tokens, d] bf16
  const __nv_bfloat16* residual;   // local [tokens, d] or null
};

ZbDeviceState* zb_device_state();       // state of the current device, or nullptr before zb_init
void zb_count_launch(int n);            // adds to the process-wide kernel-launch counter

bool zb_pdl_enabled();                  // programmatic dependent launch on (default) or off

// Launches `kernel` so that it may start while the preceding kernel of the stream is still
// running (programmatic stream serialisation).  Only for kernels that execute `zb_pdl_wait()`
// before their first access to memory another kernel writes or reads.
template <typename... KArgs, typename... Args>
inline cudaError_t zb_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     int cluster_x, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (zb_pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = static_cast<unsigned>(cluster_x);
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
inline cudaError_t zb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args&&... args) {
  return zb_launch_cluster(kernel, grid, block, smem, stream, 1, static_cast<Args&&>(args)...);
}

// Opts a kernel into `smem` bytes of dynamic shared memory and asks for the largest shared-memory
// carve-out, so that as many CTAs as the byte count allows are resident per SM (the default
// carve-out is only as large as one CTA needs).
template <typename K>
inline cudaError_t zb_config_smem(K kernel, int smem) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

// The same, once per device and kernel: `done` is the caller's static flag array (a function attribute belongs to
// the device that was current when it was set, and one process may drive several GPUs).  Returns 0 or a CUDA error.
template <typename K>
inline int zb_config_smem_once(K kernel, int smem, bool (&done)[16]) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return -21;
  if (!done[dev]) {
    cudaError_t e = zb_config_smem(kernel, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    done[dev] = true;
  }
  return 0;
}

extern "C" {
void zb_set_pdl(int on);
int zb_init(int device);
int zb_num_sms();
int zb_status_read(uint32_t* out4);     // copies {code, kernel, where, detail}; synchronises the device
int zb_status_reset();
ZbStatus* zb_status_ptr();
unsigned long long zb_launch_count();
void zb_launch_count_reset();
void zb_launch_count_add(unsigned long long n);  // e.g. nodes of a replayed CUDA graph
}
