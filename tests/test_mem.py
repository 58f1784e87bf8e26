"""Host allocators and block pools (native, CPU fallback when no GPU is present)."""
import threading
import time

import numpy as np
import pytest

from zml_b200 import mem


def test_dma_allocator_and_register():
    a = mem.DmaAllocator()
    with a.alloc(1 << 16) as b:
        v = b.numpy()
        v[:] = 7
        assert b.torch().sum().item() == 7 * (1 << 16) and b.ptr % 4096 == 0 or b.pinned
    x = np.zeros(8192, dtype=np.uint8)
    pinned = a.register(x)
    if pinned:
        a.unregister(x)


def test_fixed_pool_blocks_until_put():
    pool = mem.FixedBufferPool(4096, 2, pinned=False)
    b1, b2 = pool.get(), pool.get()
    assert {b1.ptr, b2.ptr} == {min(b1.ptr, b2.ptr), min(b1.ptr, b2.ptr) + 4096}
    assert pool.stats()["in_flight"] == 2
    with pytest.raises(mem.PoolTimeout):
        pool.get(timeout_s=0.05)
    got = []
    t = threading.Thread(target=lambda: got.append(pool.get(timeout_s=5.0)))
    t.start()
    time.sleep(0.05)
    b1.free()
    t.join(5)
    assert got and got[0].ptr == b1.ptr
    with pytest.raises(ValueError):
        pool.put(mem.HostBlock(b2.ptr + 8, 4096, False))
    got[0].free(); b2.free()
    assert pool.stats()["in_flight"] == 0
    pool.close()


def test_dynamic_pool_grows_to_cap_and_recycles():
    pool = mem.DynamicBufferPool(3, 1 << 12, pinned=False)
    assert pool.stats()["allocated"] == 0
    blocks = [pool.get() for _ in range(3)]
    assert pool.stats() == {"in_flight": 3, "allocated": 3, "pinned": 0, "max_blocks": 3}
    with pytest.raises(mem.PoolTimeout):
        pool.get(timeout_s=0.02)
    p0 = blocks[0].ptr
    blocks[0].free()
    again = pool.get(timeout_s=1.0)
    assert again.ptr == p0 and pool.stats()["allocated"] == 3
    for b in blocks[1:] + [again]:
        b.free()
    pool.close()
