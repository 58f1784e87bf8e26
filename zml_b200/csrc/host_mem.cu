// Host memory for DMA: page-locked allocations, registration of existing ranges, and two
// block pools used by the weight loader (a fixed pool carved from one slab, and a pool that
// grows on demand up to a cap on blocks in flight).  A taker blocks, with a timeout, until a
// block is returned.  When no CUDA device is usable the allocators fall back to page-aligned
// pageable memory, so the same code paths run on a CPU-only machine.
//
// Plays the role of zml/mem.zig of the reference (DmaAllocator = host alloc + PJRT dmaMap,
// FixedBufferPool, DynamicBufferPool with max in-flight blocks).
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <chrono>
#include <condition_variable>
#include <mutex>
#include <vector>

namespace {

bool cuda_usable() {
  static int state = -1;
  if (state < 0) {
    int n = 0;
    state = (cudaGetDeviceCount(&n) == cudaSuccess && n > 0) ? 1 : 0;
    if (state == 0) (void)cudaGetLastError();
  }
  return state == 1;
}

struct Pool {
  size_t block_bytes = 0;
  int max_blocks = 0;
  bool pinned = false;
  bool fixed = false;
  char* slab = nullptr;                 // fixed pools: one allocation
  std::vector<void*> owned;             // dynamic pools: every block ever allocated
  std::vector<void*> free_list;
  int in_flight = 0;
  int pinned_blocks = 0;
  std::mutex mu;
  std::condition_variable cv;
};

void* alloc_block(size_t bytes, bool want_pinned, bool* got_pinned) {
  void* p = nullptr;
  *got_pinned = false;
  if (want_pinned && cuda_usable()) {
    if (cudaHostAlloc(&p, bytes, cudaHostAllocPortable) == cudaSuccess) {
      *got_pinned = true;
      return p;
    }
    (void)cudaGetLastError();
  }
  if (posix_memalign(&p, 4096, bytes) != 0) return nullptr;
  return p;
}

void free_block(void* p, bool pinned) {
  if (p == nullptr) return;
  if (pinned) cudaFreeHost(p);
  else free(p);
}

}  // namespace

extern "C" {

// Page-locked host allocation (pageable fallback).  *pinned_out tells which one was obtained.
int zb_host_alloc(size_t bytes, void** out, int* pinned_out) {
  bool pinned = false;
  void* p = alloc_block(bytes, true, &pinned);
  if (p == nullptr) return -1;
  *out = p;
  if (pinned_out != nullptr) *pinned_out = pinned ? 1 : 0;
  return 0;
}

void zb_host_free(void* p, int pinned) { free_block(p, pinned != 0); }

// Page-locks an existing range for DMA (the "dmaMap" of a buffer the caller owns).
int zb_host_register(void* p, size_t bytes) {
  if (!cuda_usable()) return 1;      // nothing to do: reported as "not pinned", not as an error
  cudaError_t e = cudaHostRegister(p, bytes, cudaHostRegisterPortable);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return -static_cast<int>(e);
  }
  return 0;
}

int zb_host_unregister(void* p) {
  if (!cuda_usable()) return 1;
  cudaError_t e = cudaHostUnregister(p);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return -static_cast<int>(e);
  }
  return 0;
}

// fixed != 0: `blocks` blocks carved from one slab allocated now.
// fixed == 0: blocks are allocated on first use, at most `blocks` in flight at any time.
void* zb_pool_create(size_t block_bytes, int blocks, int pinned, int fixed) {
  if (block_bytes == 0 || blocks <= 0) return nullptr;
  Pool* p = new Pool();
  p->block_bytes = block_bytes;
  p->max_blocks = blocks;
  p->fixed = fixed != 0;
  if (p->fixed) {
    bool got = false;
    p->slab = static_cast<char*>(alloc_block(block_bytes * blocks, pinned != 0, &got));
    if (p->slab == nullptr) {
      delete p;
      return nullptr;
    }
    p->pinned = got;
    p->pinned_blocks = got ? blocks : 0;
    for (int i = blocks - 1; i >= 0; --i) p->free_list.push_back(p->slab + static_cast<size_t>(i) * block_bytes);
  } else {
    p->pinned = pinned != 0;
  }
  return p;
}

// Takes a block; waits up to timeout_ms (< 0: for ever) while `blocks` are in flight.
// Returns null on timeout or allocation failure.
void* zb_pool_get(void* pool, int timeout_ms) {
  Pool* p = static_cast<Pool*>(pool);
  std::unique_lock<std::mutex> lk(p->mu);
  auto ready = [&] { return !p->free_list.empty() || (!p->fixed && p->in_flight < p->max_blocks); };
  if (timeout_ms < 0) {
    p->cv.wait(lk, ready);
  } else if (!p->cv.wait_for(lk, std::chrono::milliseconds(timeout_ms), ready)) {
    return nullptr;
  }
  void* b = nullptr;
  if (!p->free_list.empty()) {
    b = p->free_list.back();
    p->free_list.pop_back();
  } else {
    bool got = false;
    b = alloc_block(p->block_bytes, p->pinned, &got);
    if (b == nullptr) return nullptr;
    if (got) ++p->pinned_blocks;
    else p->pinned = false;            // stay consistent: one kind of memory per pool from here on
    p->owned.push_back(b);
  }
  ++p->in_flight;
  return b;
}

int zb_pool_put(void* pool, void* block) {
  Pool* p = static_cast<Pool*>(pool);
  {
    std::lock_guard<std::mutex> lk(p->mu);
    if (p->fixed) {
      const char* c = static_cast<const char*>(block);
      if (c < p->slab || c >= p->slab + p->block_bytes * p->max_blocks ||
          static_cast<size_t>(c - p->slab) % p->block_bytes != 0)
        return -1;
    }
    if (p->in_flight <= 0) return -2;
    p->free_list.push_back(block);
    --p->in_flight;
  }
  p->cv.notify_one();
  return 0;
}

// out4 = {in flight, allocated blocks, pinned blocks, max blocks}
void zb_pool_stats(void* pool, int* out4) {
  Pool* p = static_cast<Pool*>(pool);
  std::lock_guard<std::mutex> lk(p->mu);
  out4[0] = p->in_flight;
  out4[1] = p->fixed ? p->max_blocks : static_cast<int>(p->owned.size());
  out4[2] = p->pinned_blocks;
  out4[3] = p->max_blocks;
}

void zb_pool_destroy(void* pool) {
  Pool* p = static_cast<Pool*>(pool);
  if (p == nullptr) return;
  if (p->fixed) {
    free_block(p->slab, p->pinned);
  } else {
    // dynamic pools: blocks pinned so far are the first `pinned_blocks` ones allocated
    for (size_t i = 0; i < p->owned.size(); ++i) free_block(p->owned[i], static_cast<int>(i) < p->pinned_blocks);
  }
  delete p;
}

}  // extern "C"
