"""Host simulation of the peer-memory protocol of the fused GEMM + all-reduce kernel, rank per
thread, with the same state machine as the device code (csrc/fused_ar.h):

  per tile t (owner = t % world):
    1. every rank stores its partial tile into the owner's receive slot [src][t // world],
       then sets push_flag[owner][(t // world) * world + src] = epoch;
    2. the owner waits for its `world` push flags, sums the partials in rank order, writes the
       result into every rank's output and sets done_flag[dst][t] = epoch on every rank;
    3. every rank waits for done_flag[t] == epoch for all t before it leaves the step.
  Flags are never reset: `epoch` counts launches.  Every wait is bounded; a wait that runs out
  records (phase, tile, awaited rank) and the rank returns instead of hanging.

It exists to test the protocol logic and its failure behaviour without a GPU: ranks can be
dropped, delayed, or have single flag writes suppressed, and the survivors must report a
`Timeout` naming the phase and the missing rank rather than deadlock.
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Optional

import numpy as np

PHASE_PUSH_WAIT = 1      # owner waiting for a partial tile
PHASE_DONE_WAIT = 2      # rank waiting for a finished tile


@dataclass
class Timeout:
    rank: int
    phase: int
    tile: int
    awaited: int          # rank whose flag did not arrive (push wait) or the tile's owner (done wait)
    epoch: int


class SharedHeap:
    """What the symmetric heaps hold, for all ranks."""

    def __init__(self, world: int, tiles: int, tile_elems: int):
        self.world, self.tiles = world, tiles
        slots = (tiles + world - 1) // world
        self.recv = np.zeros((world, world, slots, tile_elems), dtype=np.float32)     # [owner][src][slot]
        self.push = np.zeros((world, slots * world), dtype=np.int64)                   # [owner][slot * world + src]
        self.done = np.zeros((world, tiles), dtype=np.int64)                           # [rank][tile]
        self.out = np.zeros((world, tiles, tile_elems), dtype=np.float32)


@dataclass
class Faults:
    """Host-side fault injection."""
    dead_ranks: set = field(default_factory=set)                 # never run the step
    drop_push: set = field(default_factory=set)                  # {(src, tile)}: partial stored, flag write lost
    drop_done: set = field(default_factory=set)                  # {(owner, dst, tile)}
    delay_s: dict = field(default_factory=dict)                  # rank -> seconds before it starts


def _wait(read: Callable[[], int], epoch: int, limit_s: float) -> bool:
    t0 = time.monotonic()
    while read() < epoch:
        if time.monotonic() - t0 > limit_s:
            return False
        time.sleep(0.0002)
    return True


def run_rank(heap: SharedHeap, rank: int, epoch: int, partial: np.ndarray, limit_s: float, faults: Faults) -> Optional[Timeout]:
    """One launch of the kernel on `rank`; partial is [tiles, tile_elems]."""
    w = heap.world
    if rank in faults.delay_s:
        time.sleep(faults.delay_s[rank])
    # 1. push every partial tile to its owner
    for t in range(heap.tiles):
        owner, slot = t % w, t // w
        heap.recv[owner, rank, slot] = partial[t]
        if (rank, t) not in faults.drop_push:
            heap.push[owner, slot * w + rank] = epoch
    # 2. reduce the tiles this rank owns
    for t in range(rank, heap.tiles, w):
        slot = t // w
        for src in range(w):
            if not _wait(lambda s=src: heap.push[rank, slot * w + s], epoch, limit_s):
                return Timeout(rank, PHASE_PUSH_WAIT, t, src, epoch)
        acc = np.zeros_like(partial[t])
        for src in range(w):
            acc = acc + heap.recv[rank, src, slot]
        for dst in range(w):
            heap.out[dst, t] = acc
            if (rank, dst, t) not in faults.drop_done:
                heap.done[dst, t] = epoch
    # 3. leave only when every tile is complete locally
    for t in range(heap.tiles):
        if not _wait(lambda tt=t: heap.done[rank, tt], epoch, limit_s):
            return Timeout(rank, PHASE_DONE_WAIT, t, t % w, epoch)
    return None


def run_step(heap: SharedHeap, epoch: int, partials: list, limit_s: float = 0.3, faults: Optional[Faults] = None) -> dict:
    """Runs one launch on every live rank concurrently; returns {rank: Timeout or None}."""
    faults = faults or Faults()
    results: dict = {}

    def body(r):
        results[r] = run_rank(heap, r, epoch, partials[r], limit_s, faults)
    threads = [threading.Thread(target=body, args=(r,)) for r in range(heap.world) if r not in faults.dead_ranks]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    return results


# ---------------------------------------------------------------------------------------------
# Two-shot all-reduce in tagged slots (csrc/comm.cu: zb_allreduce_ll), rank per thread.
#
# A slot word carries (value, epoch); a reader accepts a word only when its tag equals the launch's
# epoch, so there are no flags.  Slot areas: [phase 0 / 1][epoch parity][source rank][vector].  Every
# launch uses the half of its parity; the simulation keeps the words of older launches in place, as
# the device does, so a protocol that read a stale half would be caught by the tags or by the sums.
PHASE_SHARD_WAIT = 3     # owner waiting for a peer's partial of its shard
PHASE_GATHER_WAIT = 4    # rank waiting for a finished shard


class SlotHeap:
    def __init__(self, world: int, vs: int):
        self.world, self.vs = world, vs
        self.value = np.zeros((world, 2, 2, world, vs), dtype=np.float32)     # [rank][phase][parity][src][g]
        self.tag = np.zeros((world, 2, 2, world, vs), dtype=np.int64)


def run_two_shot_rank(heap: SlotHeap, rank: int, epoch: int, x: np.ndarray, limit_s: float, faults: Faults,
                      out: np.ndarray) -> Optional[Timeout]:
    """x: this rank's input [world * vs]; out: [world * vs] receives the sum over ranks."""
    w, vs, par = heap.world, heap.vs, epoch & 1
    if rank in faults.delay_s:
        time.sleep(faults.delay_s[rank])
    for s in range(w):                       # 1. partials of foreign shards go to their owners
        if s == rank or (rank, s) in faults.drop_push:
            continue
        heap.value[s, 0, par, rank] = x[s * vs:(s + 1) * vs]
        heap.tag[s, 0, par, rank] = epoch
    acc = np.zeros(vs, dtype=np.float32)     # 2. own shard, summed in rank order
    for r in range(w):
        if r == rank:
            acc += x[rank * vs:(rank + 1) * vs]
            continue
        if not _wait(lambda: int(heap.tag[rank, 0, par, r].min()), epoch, limit_s):
            return Timeout(rank, PHASE_SHARD_WAIT, rank, r, epoch)
        acc += heap.value[rank, 0, par, r]
    for p in range(w):                       # 3. the finished shard goes to every peer
        if p == rank or (rank, p, rank) in faults.drop_done:
            continue
        heap.value[p, 1, par, rank] = acc
        heap.tag[p, 1, par, rank] = epoch
    out[rank * vs:(rank + 1) * vs] = acc
    for s in range(w):
        if s == rank:
            continue
        if not _wait(lambda: int(heap.tag[rank, 1, par, s].min()), epoch, limit_s):
            return Timeout(rank, PHASE_GATHER_WAIT, s, s, epoch)
        out[s * vs:(s + 1) * vs] = heap.value[rank, 1, par, s]
    return None


def run_two_shot(heap: SlotHeap, epoch: int, inputs: list, limit_s: float = 0.3, faults: Optional[Faults] = None) -> dict:
    """One launch on every live rank; returns {"out": [world][world * vs], "timeouts": {rank: Timeout}}."""
    faults = faults or Faults()
    w = heap.world
    outs = [np.zeros(w * heap.vs, dtype=np.float32) for _ in range(w)]
    timeouts: dict = {}

    def body(r):
        t = run_two_shot_rank(heap, r, epoch, inputs[r], limit_s, faults, outs[r])
        if t is not None:
            timeouts[r] = t

    threads = [threading.Thread(target=body, args=(r,)) for r in range(w) if r not in faults.dead_ranks]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    return {"out": outs, "timeouts": timeouts}


# ---- arg-max over a vocabulary split across the ranks (csrc/comm.cu: zb_argmax_tp_kernel) -----------------
# Per row every rank writes {value, tag} and {global index, tag} into its slot of every peer
# ([parity][source][row][2]), then collects the peers' pairs and keeps the highest value, equal
# values going to the lowest global index.  A wait that runs out leaves the local candidate in
# place and is reported.
PHASE_ARGMAX_WAIT = 5    # rank waiting for a peer's candidate


class ArgmaxHeap:
    def __init__(self, world: int, max_rows: int):
        self.world, self.max_rows = world, max_rows
        self.word = np.zeros((world, 2, world, max_rows, 2), dtype=np.float64)     # [rank][parity][src][row][value | index]
        self.tag = np.zeros((world, 2, world, max_rows, 2), dtype=np.int64)


def run_argmax_rank(heap: ArgmaxHeap, rank: int, epoch: int, logits: np.ndarray, col_offset: int, limit_s: float,
                    faults: Faults, out: np.ndarray) -> Optional[Timeout]:
    """logits: this rank's columns [rows, v_local]; out: int64 [rows] receives the global arg-max."""
    w, par = heap.world, epoch & 1
    if rank in faults.delay_s:
        time.sleep(faults.delay_s[rank])
    first: Optional[Timeout] = None
    for row in range(logits.shape[0]):
        r = logits[row]
        finite = ~np.isnan(r)
        if r.size and finite.any() and np.max(r[finite]) > -np.inf:
            best = float(np.max(r[finite]))
            gi = int(np.flatnonzero(finite & (r == best))[0]) + col_offset
        else:
            best, gi = -np.inf, 0x7FFFFFFF
        for p in range(w):
            if p == rank or (rank, p) in faults.drop_push:
                continue
            heap.word[p, par, rank, row] = (best, gi)
            heap.tag[p, par, rank, row] = epoch
        cv, ci = best, gi
        for p in range(w):
            if p == rank:
                continue
            if not _wait(lambda: int(heap.tag[rank, par, p, row].min()), epoch, limit_s):
                first = first or Timeout(rank, PHASE_ARGMAX_WAIT, row, p, epoch)
                continue
            ov, oi = float(heap.word[rank, par, p, row, 0]), int(heap.word[rank, par, p, row, 1])
            if ov > cv or (ov == cv and oi < ci):
                cv, ci = ov, oi
        out[row] = 0 if ci == 0x7FFFFFFF else ci
    return first


def run_argmax(heap: ArgmaxHeap, epoch: int, logits: list, v_per: int, limit_s: float = 0.3,
               faults: Optional[Faults] = None) -> dict:
    """One launch on every live rank; returns {"out": [world][rows], "timeouts": {rank: Timeout}}."""
    faults = faults or Faults()
    w = heap.world
    outs = [np.full(logits[r].shape[0], -1, dtype=np.int64) for r in range(w)]
    timeouts: dict = {}

    def body(r):
        t = run_argmax_rank(heap, r, epoch, logits[r], r * v_per, limit_s, faults, outs[r])
        if t is not None:
            timeouts[r] = t

    threads = [threading.Thread(target=body, args=(r,)) for r in range(w) if r not in faults.dead_ranks]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    return {"out": outs, "timeouts": timeouts}
