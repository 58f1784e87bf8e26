"""Process-group plumbing: one process per GPU, `torch.distributed` for bring-up.

`Comm` is the small interface the models use for tensor / expert parallelism.
With world size 1 every collective is the identity.  On CUDA the group is NCCL
(over NVLink 5 / NVSwitch), on CPU it is gloo, which is how the multi-rank logic
is tested without GPUs.  The fused GEMM+collective kernels plug in through
`zml_b200.parallel.symm` and replace the NCCL calls on the hot path; the NCCL
calls stay as the baseline and the oracle.

The reference has a single process that addresses every device through PJRT and
lets XLA insert NCCL collectives (zml/ops.zig:24-173, zml/module.zig:629-746).
"""
from __future__ import annotations

import datetime
import os
from typing import Optional

import torch
import torch.distributed as dist


class Comm:
    def __init__(self, rank: int = 0, world: int = 1, group=None, device: Optional[torch.device] = None):
        self.rank = rank
        self.world = world
        self.group = group
        self.device = device
        self.fused = None       # zml_b200.parallel.symm.SymmetricContext when fused kernels are on

    # ----------------------------------------------------------------- construction
    @staticmethod
    def single(device=None) -> "Comm":
        return Comm(0, 1, None, device)

    @staticmethod
    def from_env(backend: Optional[str] = None, timeout_s: float = 600.0) -> "Comm":
        """Joins the job described by RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT."""
        world = int(os.environ.get("WORLD_SIZE", "1"))
        rank = int(os.environ.get("RANK", "0"))
        local = int(os.environ.get("LOCAL_RANK", str(rank)))
        use_cuda = torch.cuda.is_available()
        device = torch.device("cuda", local) if use_cuda else torch.device("cpu")
        if use_cuda:
            torch.cuda.set_device(device)
        if world == 1:
            return Comm(0, 1, None, device)
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if not dist.is_initialized():
            kw = {}
            if use_cuda:
                kw["device_id"] = device
            dist.init_process_group(backend or ("nccl" if use_cuda else "gloo"), rank=rank,
                                    world_size=world,
                                    timeout=datetime.timedelta(seconds=timeout_s), **kw)
        return Comm(rank, world, dist.group.WORLD, device)

    # ----------------------------------------------------------------- liveness
    def enable_heartbeat(self, timeout_s: float = 30.0, store=None) -> None:
        """Starts host-side failure detection (`zml_b200.parallel.health`): every `check_peers()` bumps this rank's
        counter in the job's rendezvous store and raises `RankFailure` if a peer announced its exit or has not
        bumped its own for `timeout_s`."""
        if self.world == 1:
            return
        from .health import Heartbeat
        if store is None:
            store = dist.distributed_c10d._get_default_store()
        self.heartbeat = Heartbeat(store, self.rank, self.world, timeout_s)

    def check_peers(self) -> None:
        """Call between steps, with none of this rank's kernels or collectives waiting on a peer: the serving loop
        does before every decode block.  A no-op until `enable_heartbeat`."""
        hb = getattr(self, "heartbeat", None)
        if hb is not None:
            hb.beat()
            hb.check()

    def leave(self) -> None:
        """Announces an orderly exit to the other ranks (they see it at their next `check_peers`)."""
        hb = getattr(self, "heartbeat", None)
        if hb is not None:
            hb.leave()

    # ----------------------------------------------------------------- collectives
    def all_reduce_(self, t: torch.Tensor, op: str = "sum") -> torch.Tensor:
        if self.world > 1:
            ops = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN,
                   "prod": dist.ReduceOp.PRODUCT}
            dist.all_reduce(t, op=ops[op], group=self.group)
        return t

    def all_reduce_max_(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return t

    def all_gather(self, t: torch.Tensor, dim: int = 0) -> torch.Tensor:
        if self.world == 1:
            return t
        t = t.contiguous()
        if t.dim() == 0:
            t = t[None]
        # the flat [world * n, ...] form is the one every back-end accepts (gloo rejects [world, n, ...])
        out = torch.empty((self.world * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t, group=self.group)
        if dim == 0:
            return out
        return torch.cat(list(out.reshape(self.world, *t.shape).unbind(0)), dim=dim)

    def reduce_scatter(self, t: torch.Tensor) -> torch.Tensor:
        """Sums over ranks and leaves rank r with rows [r*n/P, (r+1)*n/P)."""
        if self.world == 1:
            return t
        t = t.contiguous()
        out = torch.empty((t.shape[0] // self.world,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.reduce_scatter_tensor(out, t, group=self.group)
        return out

    def all_to_all(self, t: torch.Tensor) -> torch.Tensor:
        """Equal-split all-to-all along dim 0."""
        if self.world == 1:
            return t
        out = torch.empty_like(t)
        dist.all_to_all_single(out, t.contiguous(), group=self.group)
        return out

    def broadcast_(self, t: torch.Tensor, src: int = 0) -> torch.Tensor:
        if self.world > 1:
            dist.broadcast(t, src=src, group=self.group)
        return t

    def broadcast_object(self, obj, src: int = 0):
        """Any picklable host value from `src` to every rank (the chat loop's input line)."""
        if self.world == 1:
            return obj
        box = [obj]
        dist.broadcast_object_list(box, src=src, group=self.group)
        return box[0]

    def all_gather_object(self, obj):
        if self.world == 1:
            return [obj]
        out = [None] * self.world
        dist.all_gather_object(out, obj, group=self.group)
        return out

    def barrier(self) -> None:
        if self.world > 1:
            if self.device is not None and self.device.type == "cuda":
                dist.barrier(group=self.group, device_ids=[self.device.index])
            else:
                dist.barrier(group=self.group)

    def max_over_ranks(self, value: float) -> float:
        """Host scalar -> max over ranks (used for device-timed multi-GPU numbers)."""
        if self.world == 1:
            return float(value)
        t = torch.tensor([value], dtype=torch.float64, device=self.device if self.device is not None else "cpu")
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return float(t.item())

    def close(self) -> None:
        """Leaves the group.  The NCCL communicator is not destroyed explicitly: with collectives
        captured in CUDA graphs the teardown can wait forever on the graph's pending work, so the
        process group is left to process exit (see `finish`)."""
        if self.world > 1 and dist.is_initialized():
            if self.device is not None and self.device.type == "cuda":
                torch.cuda.synchronize()
            self.barrier()

    def finish(self, code: int = 0) -> None:
        """Barrier, flush, and end the process without running NCCL / CUDA destructors.  Every
        rank calls it as its last statement."""
        import os
        import sys
        self.close()
        sys.stdout.flush()
        sys.stderr.flush()
        if self.world > 1:
            os._exit(code)
