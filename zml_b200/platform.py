"""Platform: the devices of this machine, their mesh, and the registered shardings.

Role of zml/platform.zig.  The reference loads a PJRT plugin per target and tries
tpu, neuron, rocm, cuda, oneapi, metal, cpu in turn; this framework has exactly two
targets: `cuda` (B200, sm_100a) and `cpu` (N virtual devices in one process - how the
multi-device logic is tested without GPUs, like the reference's 4-device CPU test
platform, zml/platform.zig:708-725).  A power-of-two device count is required
(zml/platform.zig:37-50).
"""
from __future__ import annotations

import enum
import os
from dataclasses import dataclass, field
from typing import Optional

import torch

from .shape import Shape
from .sharding import LogicalMesh, Partitioning, PhysicalMesh, Sharding, Strategy


class Target(enum.Enum):
    cpu = "cpu"
    cuda = "cuda"


class MemoryKind(enum.Enum):
    """zml/platform.zig:63-115."""
    default = "default"
    host_unpinned = "host_unpinned"
    host_pinned = "host_pinned"
    device = "device"


@dataclass
class CpuOptions:
    device_count: int = 4


@dataclass
class CudaOptions:
    """What of the reference's CUDA client options (zml/platform.zig:117-166: allocator kind, memory fraction,
    preallocation) has a meaning on torch's caching allocator: the share of the device's memory this process may
    take, and whether to reserve it at start-up (one large block, returned to the allocator's cache at once, so
    that later allocations do not go to the driver)."""
    memory_fraction: float = 1.0        # < 1: cap of this process's share (torch.cuda.set_per_process_memory_fraction)
    preallocate: bool = False


@dataclass
class CreateOptions:
    cpu: CpuOptions = field(default_factory=CpuOptions)
    cuda: CudaOptions = field(default_factory=CudaOptions)
    physical_mesh: Optional[object] = None     # a PhysicalMesh, or fn(target name, device count) -> PhysicalMesh


@dataclass
class DeviceInfo:
    id: int
    mesh_device: object                 # sharding.Device
    torch_device: torch.device
    description: str = ""
    process_index: int = 0              # the rank that drives this device (zml/platform.zig:176)

    def local_hardware_id(self) -> int:
        """Index of the device on its host (zml/platform.zig:180)."""
        return int(self.torch_device.index or 0) if self.torch_device.type == "cuda" else self.id

    def kind(self) -> str:
        """Hardware kind string, e.g. "NVIDIA B200" (zml/platform.zig:184)."""
        return self.description or self.torch_device.type

    def memory(self, kind) -> Optional[MemoryKind]:
        """The memory of `kind` this device can address, or None (zml/platform.zig:207): a CPU device has one
        memory, which answers to every kind; a CUDA device has device, pinned host and unpinned host memory."""
        k = kind if isinstance(kind, MemoryKind) else MemoryKind[kind] if kind in MemoryKind.__members__ else MemoryKind(kind)
        return k

    def compute_capability(self) -> Optional[str]:
        """"10.0" on a B200; None on CPU (zml/platform.zig:799-809)."""
        if self.torch_device.type != "cuda" or self.description == "remote":
            return None
        major, minor = torch.cuda.get_device_capability(self.torch_device)
        return f"{major}.{minor}"

    def to_string(self) -> str:
        return f"{self.kind()} ({self.torch_device}, id {self.id}, process {self.process_index})"

    def debug_string(self) -> str:
        return f"{self.to_string()} coords={getattr(self.mesh_device, 'coords', None)}"

    def memory_stats(self) -> dict:
        if self.torch_device.type != "cuda":
            return {}
        free, total = torch.cuda.mem_get_info(self.torch_device)
        return {"bytes_in_use": total - free, "bytes_limit": total,
                "peak_bytes_in_use": torch.cuda.max_memory_allocated(self.torch_device)}


class Platform:
    def __init__(self, target: Target, options: Optional[CreateOptions] = None, comm=None):
        self.target = target
        self.options = options or CreateOptions()
        self.comm = comm
        if target is Target.cuda:
            if not torch.cuda.is_available():
                from . import driver_probe
                why = driver_probe.diagnose(driver_probe.probe_in_child(), driver_probe.runtime_version())
                raise RuntimeError(f"cuda target requested but no CUDA device is visible: {why}")
            world = comm.world if comm is not None and comm.world > 1 else None
            n = world or torch.cuda.device_count()
        elif comm is not None and comm.world > 1:
            n = comm.world                       # one process per (virtual) device
        else:
            n = self.options.cpu.device_count
        if n & (n - 1):
            raise ValueError(f"device count must be a power of two, got {n}")
        custom = self.options.physical_mesh
        if callable(custom) and not isinstance(custom, PhysicalMesh):
            custom = custom(target.value, n)        # the reference's `.custom = fn(target, devices)` (zml/platform.zig:696-705)
        self.physical_mesh = custom or PhysicalMesh.auto(target.value, n)
        if self.physical_mesh.num_devices() != n:
            raise ValueError("custom physical mesh does not match the device count")
        self.devices: list[DeviceInfo] = []
        for rank, md in enumerate(self.physical_mesh.devices):
            if target is Target.cuda:
                idx = (comm.device.index if comm is not None and comm.world > 1 else rank)
                td = torch.device("cuda", idx)
                desc = torch.cuda.get_device_name(idx) if (comm is None or comm.world == 1 or rank == comm.rank) else "remote"
            else:
                td, desc = torch.device("cpu"), "virtual cpu device"
            self.devices.append(DeviceInfo(md.id, md, td, desc, process_index=rank if comm is not None and comm.world > 1 else 0))
        if target is Target.cuda:
            self._apply_cuda_options()
        self._shardings: dict[str, Sharding] = {}
        self._replicated = Sharding.replicated(self.physical_mesh)
        self._shardings["replicated"] = self._replicated

    def _apply_cuda_options(self) -> None:
        o = self.options.cuda
        for dev in {d.torch_device for d in self.local_devices()}:
            if 0.0 < o.memory_fraction < 1.0:
                torch.cuda.set_per_process_memory_fraction(o.memory_fraction, dev)
            if o.preallocate:
                free, total = torch.cuda.mem_get_info(dev)
                want = min(int(total * min(o.memory_fraction, 1.0) * 0.9), int(free * 0.9))     # the cap also covers the context
                while want > (64 << 20):
                    try:
                        block = torch.empty(want, dtype=torch.uint8, device=dev)
                        del block        # stays in the caching allocator
                        break
                    except torch.OutOfMemoryError:
                        want = want * 3 // 4

    # ------------------------------------------------------------------ construction
    @staticmethod
    def auto(options: Optional[CreateOptions] = None, comm=None) -> "Platform":
        """cuda when a GPU is visible, else cpu (the reference tries its targets in order)."""
        want = os.environ.get("ZB_TARGET")
        if want:
            return Platform(Target(want), options, comm)
        return Platform(Target.cuda if torch.cuda.is_available() else Target.cpu, options, comm)

    @staticmethod
    def init(target, options: Optional[CreateOptions] = None, comm=None) -> "Platform":
        return Platform(Target(target) if not isinstance(target, Target) else target, options, comm)

    # ------------------------------------------------------------------ devices
    def local_devices(self) -> list[DeviceInfo]:
        if self.comm is not None and self.comm.world > 1:
            return [self.devices[self.comm.rank]]
        return list(self.devices)

    def num_devices(self) -> int:
        return len(self.devices)

    def compute_capability(self) -> Optional[str]:
        if self.target is not Target.cuda:
            return None
        major, minor = torch.cuda.get_device_capability(self.local_devices()[0].torch_device)
        return f"{major}.{minor}"

    # ------------------------------------------------------------------ shardings
    def replicated_sharding(self) -> Sharding:
        return self._replicated

    def register_sharding(self, name: str, logical: LogicalMesh) -> Sharding:
        return self.register_sharding_with_strategy(name, logical, Strategy.suggest(logical, self.physical_mesh))

    def register_sharding_with_strategy(self, name: str, logical: LogicalMesh, strategy: Strategy) -> Sharding:
        s = Sharding(name, self.physical_mesh, logical, strategy)
        self._shardings[name] = s
        return s

    def sharding(self, name: str) -> Sharding:
        return self._shardings[name]

    def shardings(self) -> list[Sharding]:
        return [s for n, s in self._shardings.items() if n != "replicated"]

    def partitioning(self) -> Partitioning:
        return Partitioning(self.shardings() or [self._replicated])

    def pick_sharding(self, shape: Shape) -> Sharding:
        if shape.has_at_least_one_partitioned_axis():
            for s in self.shardings():
                if s.covers(shape):
                    return s
        return self._replicated

    def spmd(self):
        """The SPMD context of a multi-process platform (None on a single process): programs compiled here run once
        per rank on local shards, see `zml_b200.spmd`."""
        if self.comm is None or self.comm.world <= 1:
            return None
        if getattr(self, "_spmd", None) is None:
            from .spmd import SpmdContext
            self._spmd = SpmdContext(self)
        return self._spmd

    # ------------------------------------------------------------------ compile / profile
    def compile(self, fn, args=(), **opts):
        from . import module
        return module.compile(fn, args, self, **opts)

    compile_fn = compile

    def compile_model(self, model, method: str = "forward", args=(), **opts):
        from . import module
        return module.compile(getattr(model, method), args, self, **opts)

    def profiler(self, **opts):
        from .profiling import Profiler
        return Profiler(**opts)

    # ------------------------------------------------------------------ printing
    def fmt_verbose(self) -> str:
        lines = [f"Platform(target={self.target.value}, devices={len(self.devices)})", f"  mesh: {self.physical_mesh}"]
        for d in self.local_devices():
            st = d.memory_stats()
            mem = f" mem {st['bytes_in_use'] / 2 ** 30:.1f}/{st['bytes_limit'] / 2 ** 30:.1f} GiB" if st else ""
            lines.append(f"  device {d.id} coords={d.mesh_device.coords} {d.torch_device} {d.description}{mem}")
        for name, s in self._shardings.items():
            lines.append(f"  sharding {name}: {s.strategy.bindings}")
        return "\n".join(lines)

    def __repr__(self) -> str:
        return f"Platform({self.target.value}, {len(self.devices)} devices)"
