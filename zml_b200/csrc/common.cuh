// Shared device-side building blocks for the sm_100a kernels of this library:
// mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (MMA / TMEM) wrappers in inline
// PTX, bounded waits that fail soft, and the per-device status word.
//
// Every wait in this library is bounded.  A wait that runs out records a code in
// the status word (see ZbStatus) and makes the kernel leave through its normal
// exit (TMEM freed, no trap), so the CUDA context stays usable and the host can
// turn the code into an exception.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#ifndef ZB_WAIT_LIMIT_NS
// Upper bound of any single device-side wait (mbarrier, flag, peer): 2 s.
#define ZB_WAIT_LIMIT_NS 2000000000ull
#endif

#define ZB_DEVICE __device__ __forceinline__

// ----------------------------------------------------------------------------
// Status word: one per device, in global memory, read by the host after a step.
// ----------------------------------------------------------------------------
enum ZbStatusCode : uint32_t {
  ZB_OK = 0,
  ZB_ERR_MBAR_TIMEOUT = 1,     // an mbarrier wait ran out
  ZB_ERR_FLAG_TIMEOUT = 2,     // a wait on a peer/global flag ran out
  ZB_ERR_BOUNDS = 3,           // bounds-check build: index outside the extents
  ZB_ERR_BAD_ARG = 4,
};

struct ZbStatus {
  uint32_t code;      // first error code seen (0 = ok)
  uint32_t kernel;    // id of the kernel that recorded it
  uint32_t where;     // kernel-specific location (role / phase / stage)
  uint32_t detail;    // kernel-specific payload (tile, rank, index ...)
};

ZB_DEVICE void zb_record_error(ZbStatus* st, uint32_t code, uint32_t kernel,
                               uint32_t where, uint32_t detail) {
  if (st == nullptr) return;
  if (atomicCAS(&st->code, 0u, code) == 0u) {
    st->kernel = kernel;
    st->where = where;
    st->detail = detail;
    __threadfence_system();
  }
}

// ----------------------------------------------------------------------------
// Bounds-checking build (-DZB_BOUNDS_CHECK -rdc=true, built beside the normal library as libzb_cuda_bc.so): every
// index that a kernel reads from memory (token ids, KV slots, page numbers, expert ids, state slots) is checked
// against its extent before it is used; a bad one is RECORDED in the status word as ZB_ERR_BOUNDS with the kernel
// id, the site and the index, and the access is skipped.  The normal build masks the same indices silently (or
// trusts them where it has no extent).  Extents a kernel's arguments do not carry (the number of KV pages) are
// declared once by the host with zb_bc_set_extents.  Stands in for compute-sanitizer's memcheck.
// ----------------------------------------------------------------------------
#ifdef ZB_BOUNDS_CHECK
struct ZbBcExtents {
  long long num_pages;        // pages of the paged KV cache (0 = not declared: page numbers are not checked)
  long long num_state_slots;  // rows of the recurrent-state pools (0 = not declared)
};
extern __device__ ZbStatus* zb_bc_status;
extern __device__ ZbBcExtents zb_bc_ext;
// true when idx is inside [0, extent); records the first offender otherwise.  extent <= 0: unchecked.
ZB_DEVICE bool zb_bc_ok(long long idx, long long extent, uint32_t kernel, uint32_t site) {
  if (extent <= 0 || (idx >= 0 && idx < extent)) return true;
  zb_record_error(zb_bc_status, ZB_ERR_BOUNDS, kernel, site, static_cast<uint32_t>(idx));
  return false;
}
#define ZB_BC_OK(idx, extent, kernel, site) zb_bc_ok((idx), (extent), (kernel), (site))
#define ZB_BC_PAGES (zb_bc_ext.num_pages)
#define ZB_BC_STATE_SLOTS (zb_bc_ext.num_state_slots)
#else
#define ZB_BC_OK(idx, extent, kernel, site) true
#define ZB_BC_PAGES 0
#define ZB_BC_STATE_SLOTS 0
#endif

ZB_DEVICE uint64_t zb_globaltimer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

ZB_DEVICE uint32_t zb_smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

ZB_DEVICE bool zb_elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred P1;\n\t"
      "elect.sync _|P1, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P1;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ----------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------
ZB_DEVICE void zb_mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(zb_smem_u32(bar)), "r"(count));
}

ZB_DEVICE void zb_mbar_fence_init() {
  // Makes the initialised barriers visible to the async proxy (TMA, tcgen05.commit).
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

ZB_DEVICE void zb_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(zb_smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

ZB_DEVICE void zb_mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(zb_smem_u32(bar)) : "memory");
}

ZB_DEVICE uint32_t zb_mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(zb_smem_u32(bar)), "r"(parity)
      : "memory");
  return ok;
}

// Bounded wait.  `abort_flag` is a CTA-shared word: once any role of the CTA gave
// up, every other wait of the CTA returns false at its next poll, so that all
// roles reach the common exit.  Returns true when the phase completed.
ZB_DEVICE bool zb_mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag) {
  if (zb_mbar_test(bar, parity)) return true;
  const uint64_t t0 = zb_globaltimer();
  uint32_t spins = 0;
  while (true) {
    if (zb_mbar_test(bar, parity)) return true;
    if ((++spins & 0x3f) == 0) {
      if (*abort_flag != 0u) return false;
      if (zb_globaltimer() - t0 > ZB_WAIT_LIMIT_NS) {
        *abort_flag = 1u;
        return false;
      }
    }
  }
}

// ----------------------------------------------------------------------------
// TMA: tiled 2-D / 3-D loads into shared memory, completion on an mbarrier.
// No load in this library carries a cluster-multicast qualifier.
// The innermost coordinate times the element size must be a multiple of 16 B.
// ----------------------------------------------------------------------------
// Untiled bulk copy global -> shared of `bytes` contiguous bytes (both addresses 16-byte aligned,
// size a multiple of 16), completion counted on an mbarrier.
ZB_DEVICE void zb_bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      :
      : "r"(zb_smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(zb_smem_u32(bar))
      : "memory");
}

// Untiled bulk copy shared -> global (both addresses 16-byte aligned, size a multiple of 16), tracked by the issuing
// thread's bulk async-group: commit the group, then wait until its copies have read their source (the shared
// memory may be overwritten) or are complete (the data is in global memory).
ZB_DEVICE void zb_bulk_store(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst), "r"(zb_smem_u32(smem_src)), "r"(bytes)
               : "memory");
}
ZB_DEVICE void zb_bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
ZB_DEVICE void zb_bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
ZB_DEVICE void zb_bulk_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// Orders this thread's earlier generic-proxy writes to shared memory before later async-proxy (bulk copy) reads of it.
ZB_DEVICE void zb_fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

ZB_DEVICE void zb_tma_load_2d(void* smem_dst, const void* tmap, uint64_t* bar, int32_t x,
                              int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(zb_smem_u32(smem_dst)), "l"(tmap), "r"(zb_smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// Brings a tile into L2 only (no shared-memory destination, no barrier).
ZB_DEVICE void zb_tma_prefetch_l2_2d(const void* tmap, int32_t x, int32_t y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(tmap), "r"(x), "r"(y)
               : "memory");
}

ZB_DEVICE void zb_tma_load_2d_hint(void* smem_dst, const void* tmap, uint64_t* bar, int32_t x,
                                   int32_t y, uint64_t cache_policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4}], [%2], %5;"
      :
      : "r"(zb_smem_u32(smem_dst)), "l"(tmap), "r"(zb_smem_u32(bar)), "r"(x), "r"(y),
        "l"(cache_policy)
      : "memory");
}

ZB_DEVICE void zb_tma_load_3d(void* smem_dst, const void* tmap, uint64_t* bar, int32_t x,
                              int32_t y, int32_t z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(zb_smem_u32(smem_dst)), "l"(tmap), "r"(zb_smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

ZB_DEVICE void zb_tma_load_4d(void* smem_dst, const void* tmap, uint64_t* bar, int32_t x, int32_t y,
                              int32_t z, int32_t w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      :
      : "r"(zb_smem_u32(smem_dst)), "l"(tmap), "r"(zb_smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}

// Thread-block clusters: rank, cluster-wide barrier (every thread of every CTA of the cluster
// takes part), and loads from a peer CTA's shared memory (distributed shared memory).
ZB_DEVICE uint32_t zb_cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
ZB_DEVICE void zb_cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
ZB_DEVICE void zb_cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
ZB_DEVICE uint32_t zb_mapa(uint32_t smem_addr, uint32_t cta_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta_rank));
  return r;
}
ZB_DEVICE float zb_ld_dsmem_f32(uint32_t cluster_addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
  return v;
}

// 8-byte "data + tag" slots for latency-bound exchanges over NVLink: an aligned 8-byte store
// arrives whole, so a receiver that sees the expected tag also has the data - no fence, no
// separate flag.
ZB_DEVICE void zb_st_ll(uint2* p, uint32_t data, uint32_t tag) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(data), "r"(tag) : "memory");
}
ZB_DEVICE uint2 zb_ld_ll(const uint2* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}

// Row maximum and its first index over `n` floats by a block of 1024 threads: ties go to the lowest index, NaN
// never wins, an empty row gives (-inf, 0x7fffffff).  The result is valid in warp 0 (every lane).  Uses 256 bytes
// of static shared memory; callers that loop over rows must __syncthreads() between calls.
ZB_DEVICE void zb_argmax_merge(float& best, int& bi, float ov, int oi) {
  if (ov > best || (ov == best && oi < bi)) {
    best = ov;
    bi = oi;
  }
}
ZB_DEVICE void zb_block_argmax_1024(const float* __restrict__ row, int n, float& best, int& bi) {
  __shared__ float sv[32];
  __shared__ int si[32];
  best = -INFINITY;
  bi = 0x7fffffff;
  for (int i = threadIdx.x; i < n; i += 1024) zb_argmax_merge(best, bi, row[i], i);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    zb_argmax_merge(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
  if ((threadIdx.x & 31) == 0) {
    sv[threadIdx.x >> 5] = best;
    si[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    best = sv[threadIdx.x];
    bi = si[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      zb_argmax_merge(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
  }
}

// Programmatic dependent launch.  `zb_pdl_wait` blocks until every grid this one depends on has
// finished and its writes are visible; nothing produced or still read by a preceding kernel may
// be touched before it.  `zb_pdl_launch` lets the next kernel in the stream begin its own
// prologue while this one is still running.  Both are no-ops for a kernel launched without the
// programmatic-serialisation attribute.
ZB_DEVICE void zb_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
ZB_DEVICE void zb_pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

ZB_DEVICE void zb_tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// L2 eviction policies for streamed (read-once) and reused operands.
ZB_DEVICE uint64_t zb_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
ZB_DEVICE uint64_t zb_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// ----------------------------------------------------------------------------
// tcgen05: tensor memory management, MMA issue, commit, TMEM loads.
// ----------------------------------------------------------------------------
// Allocation is a warp-wide (.sync.aligned) instruction; ncols is a power of two
// in [32, 512].  The TMEM base address is written to *smem_holder.
ZB_DEVICE void zb_tmem_alloc(uint32_t* smem_holder, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   zb_smem_u32(smem_holder)),
               "r"(ncols)
               : "memory");
}
ZB_DEVICE void zb_tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
ZB_DEVICE void zb_tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}

ZB_DEVICE void zb_tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
ZB_DEVICE void zb_tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]; issued by ONE thread.
ZB_DEVICE void zb_umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                           uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The same MMA with the A operand in tensor memory: lane = row of A (0..127), each 32-bit column holds two
// consecutive K elements (lower K in the low half), so one K = 16 step reads 8 columns from `tmem_a`.
ZB_DEVICE void zb_umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                              uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrives on `bar` once every tcgen05 operation issued so far by this thread is done.
ZB_DEVICE void zb_umma_commit(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
          zb_smem_u32(bar))
      : "memory");
}

// 32 lanes x 32 columns of 32-bit: thread i of the warp gets lane (base_lane + i),
// columns [col, col+32).  A warp may only touch lanes 32*(warp_id % 4) .. +31.
ZB_DEVICE void zb_tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
ZB_DEVICE void zb_tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
ZB_DEVICE void zb_tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Registers -> tensor memory: lane i of the warp writes 16 consecutive 32-bit columns of TMEM lane
// (32 * (warp % 4) + i) starting at column `taddr`.
ZB_DEVICE void zb_tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 "
      "[%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
ZB_DEVICE void zb_tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major bf16 tile written by TMA with the
// 128-byte swizzle: rows of 64 elements (128 B), 8-row groups 1024 B apart.
//   bits  0-13 start address >> 4       bits 16-29 leading byte offset >> 4 (unused: 1)
//   bits 32-45 stride byte offset >> 4  bits 46-47 version (1 on sm_100)
//   bits 61-63 layout type (2 = 128-byte swizzle)
ZB_DEVICE uint64_t zb_make_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Instruction descriptor for kind::f16 with bf16 inputs, fp32 accumulate, A and B K-major.
//   bits 4-5 D format (1 = f32), 7-9 A format (1 = bf16), 10-12 B format,
//   15 A major, 16 B major (0 = K), 17-22 N >> 3, 24-28 M >> 4.
__host__ __device__ constexpr uint32_t zb_make_idesc_bf16(uint32_t m, uint32_t n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// ----------------------------------------------------------------------------
// small numeric helpers
// ----------------------------------------------------------------------------
// Activations of the expert MLPs (the reference's zml/moe/cutlass_flashinfer.zig:24-28).  The grouped GEMMs take
// the code in their `swiglu` argument: 0 none, 1 swiglu (silu(gate) * up), 2 geglu (erf GELU), 3 geglu_tanh,
// 4 relu2 (not gated: relu(x)^2 on a plain projection).
enum ZbMoeAct : int { ZB_ACT_NONE = 0, ZB_ACT_SWIGLU = 1, ZB_ACT_GEGLU = 2, ZB_ACT_GEGLU_TANH = 3, ZB_ACT_RELU2 = 4 };
ZB_DEVICE bool zb_act_is_gated(int act) { return act >= ZB_ACT_SWIGLU && act <= ZB_ACT_GEGLU_TANH; }
ZB_DEVICE float zb_gate_act(float g, int act) {
  if (act == ZB_ACT_GEGLU) return 0.5f * g * (1.f + erff(g * 0.70710678118654752f));
  if (act == ZB_ACT_GEGLU_TANH) {
    const float u = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    return 0.5f * g * (1.f + tanhf(u));
  }
  return g / (1.f + __expf(-g));
}
ZB_DEVICE float zb_plain_act(float x, int act) {
  if (act == ZB_ACT_RELU2) {
    const float r = fmaxf(x, 0.f);
    return r * r;
  }
  return x;
}
ZB_DEVICE uint32_t zb_pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
ZB_DEVICE float2 zb_unpack_bf16x2(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}

ZB_DEVICE float zb_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
ZB_DEVICE float zb_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ----------------------------------------------------------------------------
// cross-GPU flags (peer memory over NVLink): release stores, bounded acquire waits
// ----------------------------------------------------------------------------
ZB_DEVICE void zb_st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
ZB_DEVICE uint32_t zb_ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Waits until *p has reached `epoch` (flags only grow).  Gives up after `limit_ns` or as soon
// as another role of the CTA gave up; returns false and raises `abort_flag`.
ZB_DEVICE bool zb_wait_flag_limit(const uint32_t* p, uint32_t epoch, volatile uint32_t* abort_flag,
                                  unsigned long long limit_ns) {
  if (static_cast<int32_t>(zb_ld_acquire_sys(p) - epoch) >= 0) return true;
  const uint64_t t0 = zb_globaltimer();
  uint32_t spins = 0;
  while (true) {
    if (static_cast<int32_t>(zb_ld_acquire_sys(p) - epoch) >= 0) return true;
    if ((++spins & 0x3f) == 0) {
      if (*abort_flag != 0u) return false;
      if (zb_globaltimer() - t0 > limit_ns) {
        *abort_flag = 1u;
        return false;
      }
    }
  }
}

ZB_DEVICE bool zb_wait_flag(const uint32_t* p, uint32_t epoch, volatile uint32_t* abort_flag) {
  return zb_wait_flag_limit(p, epoch, abort_flag, ZB_WAIT_LIMIT_NS);
}

// ----------------------------------------------------------------------------
// multimem: loads and stores on an NVLink multicast address (one virtual address bound to the same buffer of
// every GPU of the group).  A load-reduce returns the sum over all GPUs' copies, added up inside NVSwitch
// (fp32 accumulation of the bf16 pairs); a store writes every GPU's copy.  16 bytes per instruction.
// ----------------------------------------------------------------------------
ZB_DEVICE uint4 zb_multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
ZB_DEVICE void zb_multimem_st_16(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}
