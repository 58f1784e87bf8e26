"""Buffer: a (possibly sharded) array living on the devices of a Platform.

Matches zml/buffer.zig: one shard per device in canonical mesh order, created by slicing
host data with the `Placement` of (shape, sharding), gathered back with `to_tensor` /
`to_slice`.  A process holds the shards of its local devices: all devices when one process
drives the machine (CPU tests with virtual devices, single-process multi-GPU), one shard in
SPMD mode (one process per GPU), where gathering goes through the process group.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from .dtype import DataType
from .shape import Shape
from .sharding import Sharding
from .slice import Slice


class Buffer:
    def __init__(self, shape: Shape, sharding: Sharding, shards: dict, platform=None):
        self._shape = shape
        self.sharding = sharding
        self.shards = shards                   # mesh device id -> torch.Tensor (local shards only)
        self.platform = platform
        self.placement = sharding.placement(shape)

    # ------------------------------------------------------------------ constructors
    @staticmethod
    def from_tensor(platform, host: torch.Tensor, shape: Optional[Shape] = None, sharding: Optional[Sharding] = None,
                    wait: bool = True, memory: str = "default") -> "Buffer":
        """`wait` / `memory` are the reference's `FromOptions` (zml/buffer.zig:69): with wait=False the copies are
        left in flight on the devices' streams (`await_` joins them); `memory` places the shards in device memory
        (device | default) or keeps them on the host (host_pinned | host_unpinned)."""
        if memory not in ("default", "device", "host_pinned", "host_unpinned"):
            raise ValueError(f"unknown memory kind {memory!r}")
        shape = shape or Shape(tuple(host.shape), DataType.from_torch(host.dtype))
        sharding = sharding or platform.pick_sharding(shape)
        pl = sharding.placement(shape)
        shards = {}
        for dev in platform.local_devices():
            piece = host[pl.shard_index(dev.mesh_device)]
            if memory in ("host_pinned", "host_unpinned"):
                piece = piece.cpu().contiguous().clone()
                if memory == "host_pinned" and torch.cuda.is_available():
                    piece = piece.pin_memory()
                shards[dev.id] = piece
            else:
                shards[dev.id] = piece.to(dev.torch_device, non_blocking=True).contiguous()
        buf = Buffer(shape, sharding, shards, platform)
        return buf.await_() if wait else buf

    @staticmethod
    def from_slice(platform, s: Slice, sharding: Optional[Sharding] = None, **opts) -> "Buffer":
        return Buffer.from_tensor(platform, s.to_torch(), s.shape, sharding, **opts)

    from_slice_opts = from_slice

    @staticmethod
    def from_bytes(platform, shape: Shape, data: bytes, sharding: Optional[Sharding] = None, **opts) -> "Buffer":
        arr = np.frombuffer(data, dtype=np.uint8).copy()
        return Buffer.from_slice(platform, Slice(shape, arr), sharding, **opts)

    from_bytes_opts = from_bytes

    @staticmethod
    def scalar(platform, value, dtype=DataType.f32) -> "Buffer":
        dt = DataType.parse(dtype)
        return Buffer.from_tensor(platform, torch.tensor(value, dtype=dt.to_torch()), Shape((), dt), platform.replicated_sharding())

    @staticmethod
    def uninitialized(platform, shape: Shape, sharding: Optional[Sharding] = None) -> "Buffer":
        sharding = sharding or platform.pick_sharding(shape)
        local = sharding.sharded_shape(shape)
        shards = {d.id: torch.empty(local.dims, dtype=shape.dtype.to_torch(), device=d.torch_device)
                  for d in platform.local_devices()}
        return Buffer(shape, sharding, shards, platform)

    # ------------------------------------------------------------------ access
    def shape(self) -> Shape:
        return self._shape

    def dtype(self) -> DataType:
        return self._shape.dtype

    def num_shards(self) -> int:
        """Shards this process holds (zml/buffer.zig:93)."""
        return len(self.shards)

    def byte_size(self) -> int:
        """Bytes over all devices: shard bytes x devices of the sharding (zml/buffer.zig:314-317)."""
        return self.placement.shape.byte_size() * len(self.sharding.devices_in_canonical_order())

    def iter_shards(self):
        """(device id, shard tensor, device pointer) per local shard, in device order (zml/buffer.zig:49-66)."""
        for d in sorted(self.shards):
            t = self.shards[d]
            yield d, t, t.data_ptr()

    def memory_kind(self) -> str:
        t = self.local()
        if t.is_cuda or not torch.cuda.is_available():
            return "device"
        return "host_pinned" if t.is_pinned() else "host_unpinned"

    @staticmethod
    def deinit_all(tree) -> None:
        """`deinit` on every Buffer of a pytree (zml/buffer.zig:80-90)."""
        from . import meta
        meta.visit(lambda b, _path: b.deinit(), tree, lambda x: isinstance(x, Buffer))

    def local(self, device_id: Optional[int] = None) -> torch.Tensor:
        """The shard held on `device_id` (default: this process's first local device)."""
        if device_id is None:
            device_id = next(iter(self.shards))
        return self.shards[device_id]

    def await_(self) -> "Buffer":
        for t in self.shards.values():
            if t.is_cuda:
                torch.cuda.current_stream(t.device).synchronize()
        return self

    def to_tensor(self) -> torch.Tensor:
        """Gathers every shard into one host tensor."""
        out = torch.empty(self._shape.dims, dtype=self._shape.dtype.to_torch())
        devices = self.sharding.devices_in_canonical_order()
        missing = [d for d in devices if d.id not in self.shards]
        if missing and self.placement.shape.dims == self._shape.dims:
            return self.local().cpu().clone()           # replicated: every process holds the whole tensor
        if missing and self.platform is not None and self.platform.comm is not None and self.platform.comm.world > 1:
            mine = self.local().contiguous()
            gathered = self.platform.comm.all_gather(mine[None])
            for rank, d in enumerate(devices):
                out[self.placement.shard_index(d)] = gathered[rank].cpu()
            return out
        if missing:
            raise RuntimeError(f"shards of devices {[d.id for d in missing]} are not addressable from this process")
        for d in devices:
            out[self.placement.shard_index(d)] = self.shards[d.id].cpu()
        return out

    def to_slice(self) -> Slice:
        t = self.to_tensor()
        raw = t.contiguous().view(torch.uint8).reshape(-1).numpy() if t.numel() else np.zeros(0, np.uint8)
        return Slice(self._shape, raw)

    to_slice_alloc = to_slice

    def get_value(self):
        return self.to_tensor().reshape(-1)[0].item() if self._shape.count() == 1 else self.to_tensor().tolist()

    def opaque_device_ptr(self, device_id: Optional[int] = None) -> int:
        return self.local(device_id).data_ptr()

    def deinit(self) -> None:
        self.shards = {}

    def __repr__(self) -> str:
        parts = ", ".join(f"dev{d}:{tuple(t.shape)}" for d, t in self.shards.items())
        return f"Buffer({self._shape}, sharding={self.sharding.name}, [{parts}])"
