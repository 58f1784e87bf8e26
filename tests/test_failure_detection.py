"""Failure detection without faulting a GPU: the flag protocol's state machine on CPU threads
with host-injected faults, heartbeats over a store, a process group whose peer left (gloo),
and - on a GPU - a bounded wait on a flag that nothing sets."""
import os
import subprocess
import sys
import time

import numpy as np
import pytest
import torch

from zml_b200.parallel import health
from zml_b200.parallel import protocol_sim as sim


def _partials(world, tiles, elems, seed=0):
    rng = np.random.default_rng(seed)
    return [rng.standard_normal((tiles, elems)).astype(np.float32) for _ in range(world)]


@pytest.mark.parametrize("world,tiles", [(2, 5), (4, 8), (8, 3)])
def test_protocol_all_ranks_agree_over_several_epochs(world, tiles):
    heap = sim.SharedHeap(world, tiles, 16)
    for epoch in (1, 2, 3):
        parts = _partials(world, tiles, 16, epoch)
        res = sim.run_step(heap, epoch, parts, limit_s=2.0)
        assert all(v is None for v in res.values())
        want = sum(parts)
        for r in range(world):
            np.testing.assert_allclose(heap.out[r], want, rtol=1e-6)


def test_protocol_dead_rank_is_reported_not_deadlocked():
    heap = sim.SharedHeap(4, 8, 4)
    t0 = time.monotonic()
    res = sim.run_step(heap, 1, _partials(4, 8, 4), limit_s=0.2, faults=sim.Faults(dead_ranks={2}))
    assert time.monotonic() - t0 < 5.0
    assert set(res) == {0, 1, 3}
    for r, to in res.items():
        assert isinstance(to, sim.Timeout) and to.epoch == 1
        # owners miss rank 2's partial; a rank that owns nothing pending waits on a tile rank 2 owns
        assert (to.phase == sim.PHASE_PUSH_WAIT and to.awaited == 2) or (to.phase == sim.PHASE_DONE_WAIT)


def test_protocol_lost_flag_writes_name_phase_and_rank():
    heap = sim.SharedHeap(2, 4, 4)
    res = sim.run_step(heap, 1, _partials(2, 4, 4), limit_s=0.2, faults=sim.Faults(drop_push={(1, 2)}))
    assert res[0] == sim.Timeout(0, sim.PHASE_PUSH_WAIT, 2, 1, 1)          # owner of tile 2 misses rank 1
    assert res[1].phase == sim.PHASE_DONE_WAIT and res[1].tile == 2
    heap = sim.SharedHeap(2, 4, 4)
    res = sim.run_step(heap, 1, _partials(2, 4, 4), limit_s=0.2, faults=sim.Faults(drop_done={(1, 0, 3)}))
    assert res[1] is None and res[0] == sim.Timeout(0, sim.PHASE_DONE_WAIT, 3, 1, 1)


def test_protocol_slow_rank_within_limit_is_fine_and_stale_epoch_does_not_satisfy():
    heap = sim.SharedHeap(2, 3, 4)
    assert all(v is None for v in sim.run_step(heap, 1, _partials(2, 3, 4), limit_s=2.0,
                                               faults=sim.Faults(delay_s={1: 0.1})).values())
    # flags left at epoch 1 must not satisfy the waits of epoch 2 when a rank is missing
    res = sim.run_step(heap, 2, _partials(2, 3, 4), limit_s=0.15, faults=sim.Faults(dead_ranks={1}))
    assert isinstance(res[0], sim.Timeout) and res[0].epoch == 2


@pytest.mark.parametrize("world,vs", [(2, 16), (4, 5), (8, 3)])
def test_two_shot_allreduce_protocol_over_several_epochs(world, vs):
    """Same slot indexing and parity halves as the device kernel: every rank ends with the same, correct sum, launch
    after launch, although the slots of older launches are never cleared."""
    heap = sim.SlotHeap(world, vs)
    rng = np.random.default_rng(world * 100 + vs)
    for epoch in range(1, 6):
        xs = [rng.standard_normal(world * vs).astype(np.float32) for _ in range(world)]
        res = sim.run_two_shot(heap, epoch, xs)
        assert not res["timeouts"]
        want = np.zeros(world * vs, dtype=np.float32)
        for shard in range(world):                      # the owner sums its shard in rank order
            acc = np.zeros(vs, dtype=np.float32)
            for r in range(world):
                acc += xs[r][shard * vs:(shard + 1) * vs]
            want[shard * vs:(shard + 1) * vs] = acc
        for r in range(world):
            assert np.array_equal(res["out"][r], want), (epoch, r)


def test_two_shot_allreduce_dead_rank_and_lost_words_are_reported():
    heap = sim.SlotHeap(4, 8)
    xs = [np.full(32, float(r + 1), dtype=np.float32) for r in range(4)]
    res = sim.run_two_shot(heap, 1, xs, limit_s=0.1, faults=sim.Faults(dead_ranks={2}))
    assert set(res["timeouts"]) == {0, 1, 3}
    for r, t in res["timeouts"].items():
        assert t.phase == sim.PHASE_SHARD_WAIT and t.awaited == 2 and t.epoch == 1
    # rank 1's partial for shard 3 never arrives: the owner (3) names rank 1, everybody else misses shard 3
    heap = sim.SlotHeap(4, 8)
    res = sim.run_two_shot(heap, 1, xs, limit_s=0.1, faults=sim.Faults(drop_push={(1, 3)}))
    assert res["timeouts"][3].phase == sim.PHASE_SHARD_WAIT and res["timeouts"][3].awaited == 1
    for r in (0, 1, 2):
        assert res["timeouts"][r].phase == sim.PHASE_GATHER_WAIT and res["timeouts"][r].awaited == 3
    # a stale half (two launches old, same parity) does not satisfy a wait
    heap = sim.SlotHeap(2, 4)
    ys = [np.ones(8, dtype=np.float32), np.ones(8, dtype=np.float32)]
    assert not sim.run_two_shot(heap, 1, ys)["timeouts"]
    assert not sim.run_two_shot(heap, 2, ys)["timeouts"]
    res = sim.run_two_shot(heap, 3, ys, limit_s=0.1, faults=sim.Faults(dead_ranks={1}))
    assert res["timeouts"][0].phase == sim.PHASE_SHARD_WAIT and res["timeouts"][0].epoch == 3


def test_heartbeat_detects_silent_and_departed_ranks():
    store = torch.distributed.HashStore()
    hb = [health.Heartbeat(store, r, 3, timeout_s=5.0) for r in range(3)]
    hb[0].check(now=100.0)
    hb[1].beat(); hb[2].beat()
    hb[0].check(now=104.0)
    hb[1].beat()
    with pytest.raises(health.RankFailure) as e:
        hb[0].check(now=110.0)                                   # rank 2 silent since t=104
    assert e.value.ranks == [2]
    hb[2].leave()
    with pytest.raises(health.RankFailure) as e:
        hb[0].check(now=111.0)
    assert e.value.ranks == [2] and "left" in e.value.reason


_WORKER = r"""
import os, sys, time, datetime, torch
import torch.distributed as dist
sys.path.insert(0, os.environ["ZB_ROOT"])
from zml_b200.parallel import health
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]) + 1, world, rank == 0, timeout=datetime.timedelta(seconds=30))
dist.init_process_group("gloo", store=dist.PrefixStore("pg", store), rank=rank, world_size=world,
                        timeout=datetime.timedelta(seconds=5))
hb = health.Heartbeat(store, rank, world, timeout_s=2.0)
x = torch.ones(4)
dist.all_reduce(x)                         # step 1: everybody is here
assert x[0].item() == world
hb.beat()
if rank == world - 1:
    hb.leave()                             # leaves between steps, nothing in flight
    print("LEFT", rank, flush=True)
    os._exit(0)
deadline = time.time() + 20
while True:                                # the others learn of it on the host, before the next collective
    try:
        hb.check()
    except health.RankFailure as e:
        print("DETECTED", rank, e.ranks, flush=True)
        break
    assert time.time() < deadline
    time.sleep(0.05)
store.set(f"seen/{rank}", b"1")
if rank == 0:                              # rank 0 hosts the store: it goes last
    store.wait([f"seen/{r}" for r in range(world - 1)], datetime.timedelta(seconds=20))
    time.sleep(0.2)
os._exit(0)
"""


def test_rank_leaving_between_steps_is_seen_before_the_next_collective(tmp_path):
    script = tmp_path / "w.py"
    script.write_text(_WORKER)
    env = dict(os.environ, ZB_ROOT=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3",
                        "--master-addr", "127.0.0.1", "--master-port", "29641", str(script)],
                       capture_output=True, text=True, env=env, timeout=180)
    assert r.stdout.count("DETECTED") == 2 and "LEFT 2" in r.stdout, r.stdout[-1500:] + r.stderr[-1500:]
    assert "[2]" in r.stdout


_ENGINE_WORKER = r"""
import os, sys, time, torch
sys.path.insert(0, os.environ["ZB_ROOT"])
from zml_b200.models import registry
from zml_b200.parallel import health
from zml_b200.parallel.comm import Comm
from zml_b200.serving import Engine
c = Comm.from_env(backend="gloo", timeout_s=20)
c.enable_heartbeat(timeout_s=3.0)
model = registry.build_model("tiny-llama-test", c, device="cpu", seed=3, dtype=torch.float32)
eng = Engine(model, num_pages=16, page_size=16, max_batch=2, max_seq_len=64)
prompts = [[5, 6, 7, 8], [9, 10, 11]]
out, _ = eng.serve(prompts, 4, sync_interval=2)              # every rank is here
assert all(len(o) == 4 for o in out)
if c.rank == c.world - 1:
    c.leave()                                                # between requests, nothing in flight
    print("LEFT", c.rank, flush=True)
    os._exit(0)
time.sleep(0.3)
try:
    eng.serve(prompts, 4, sync_interval=2)                   # must not reach a collective the departed rank never joins
    print("NOT DETECTED", c.rank, flush=True)
except health.RankFailure as e:
    print("DETECTED", c.rank, e.ranks, flush=True)
assert eng.pool.num_free == 15                               # nothing was admitted
os._exit(0)
"""


def test_serving_loop_notices_a_departed_rank_before_launching(tmp_path):
    script = tmp_path / "w.py"
    script.write_text(_ENGINE_WORKER)
    env = dict(os.environ, ZB_ROOT=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29645", str(script)],
                       capture_output=True, text=True, env=env, timeout=240)
    assert "DETECTED 0 [1]" in r.stdout and "LEFT 1" in r.stdout and "NOT DETECTED" not in r.stdout, \
        r.stdout[-1500:] + r.stderr[-1500:]


@pytest.mark.gpu
def test_bounded_wait_times_out_cleanly_on_the_gpu():
    from zml_b200 import ops
    from zml_b200.ops import _lib
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    reached = torch.full((1,), 7, dtype=torch.int32, device="cuda")
    l = _lib.lib()
    t0 = time.time()
    _lib.check(l.zb_wait_probe(flag.data_ptr(), 1, 50_000_000, 3, reached.data_ptr(), _lib.stream_ptr()), "probe")
    with pytest.raises(ops.CollectiveTimeout) as e:
        ops.raise_on_status()
    assert time.time() - t0 < 2.0
    assert e.value.kernel == "wait_probe" and e.value.phase == 3 and e.value.detail == 1
    assert int(reached.item()) == 0
    # the context is still usable and a satisfied wait returns at once
    flag.fill_(5)
    _lib.check(l.zb_wait_probe(flag.data_ptr(), 5, 50_000_000, 4, reached.data_ptr(), _lib.stream_ptr()), "probe")
    ops.raise_on_status()
    assert int(reached.item()) == 1
    assert torch.ones(4, device="cuda").sum().item() == 4.0
    assert l.zb_wait_probe(flag.data_ptr(), 9, 6_000_000_000, 0, None, _lib.stream_ptr()) == -21


@pytest.mark.parametrize("world", [2, 4, 8])
def test_vocab_parallel_argmax_protocol(world):
    """The exchange of the in-kernel arg-max over a split vocabulary: every rank ends with the arg-max of the gathered
    row, ties across ranks go to the lowest global index, launch after launch on slots that are never cleared."""
    rows, v_per = 6, 11
    heap = sim.ArgmaxHeap(world, max_rows=8)
    rng = np.random.default_rng(world)
    for epoch in range(1, 6):
        lg = [rng.standard_normal((rows, v_per)).astype(np.float32) for _ in range(world)]
        if epoch % 2 == 0:
            for r in range(world):
                lg[r][:, 3] = 7.0                      # the same maximum on every rank
        if epoch == 3:
            for r in range(world):
                lg[r][0, :] = -np.inf                  # nothing to choose in row 0: token 0
        res = sim.run_argmax(heap, epoch, lg, v_per)
        assert not res["timeouts"]
        full = np.concatenate(lg, axis=1)
        want = full.argmax(1)
        if epoch == 3:
            want[0] = 0
        for r in range(world):
            assert np.array_equal(res["out"][r], want), (epoch, r)
        if epoch % 2 == 0:
            assert (want == 3).all()


def test_vocab_parallel_argmax_dead_rank_is_reported_and_local_candidate_kept():
    heap = sim.ArgmaxHeap(2, max_rows=4)
    lg = [np.array([[0.0, 1.0, 0.5]], dtype=np.float32), np.array([[2.0, 0.0, 0.0]], dtype=np.float32)]
    assert not sim.run_argmax(heap, 1, lg, 3)["timeouts"]
    assert not sim.run_argmax(heap, 2, lg, 3)["timeouts"]
    res = sim.run_argmax(heap, 3, lg, 3, limit_s=0.1, faults=sim.Faults(dead_ranks={1}))      # stale parity-1 slots hold epoch 1
    t = res["timeouts"][0]
    assert (t.phase, t.awaited, t.epoch) == (sim.PHASE_ARGMAX_WAIT, 1, 3)
    assert res["out"][0][0] == 1                       # rank 0's own candidate
