"""Data model and back-ends of zb-smi (bin/zml-smi/info/*, platforms/nvml/*, platforms/linux/*).

`NvmlBackend` talks to NVML through the `pynvml` bindings (nvidia_ml_py) when the driver
library is present; `FakeNvml` implements the same calls for tests and for machines without
a GPU.  Only READ calls are made: clocks, power limits and other settings are never changed.
Host metrics come from /proc.
"""
from __future__ import annotations

import os
import time
from dataclasses import asdict, dataclass, field
from typing import Optional


@dataclass
class ProcessInfo:
    pid: int
    name: str = ""
    user: str = ""
    gpu_memory_bytes: Optional[int] = None
    sm_util: Optional[int] = None


@dataclass
class GpuInfo:
    """Optional metrics, as in info/device_info.zig:26-62."""
    index: int
    name: str = ""
    util_percent: Optional[int] = None
    encoder_util_percent: Optional[int] = None
    decoder_util_percent: Optional[int] = None
    power_w: Optional[float] = None
    power_limit_w: Optional[float] = None
    temperature_c: Optional[int] = None
    fan_percent: Optional[int] = None
    clock_graphics_mhz: Optional[int] = None
    clock_sm_mhz: Optional[int] = None
    clock_mem_mhz: Optional[int] = None
    clock_sm_max_mhz: Optional[int] = None
    clock_mem_max_mhz: Optional[int] = None
    mem_used_bytes: Optional[int] = None
    mem_total_bytes: Optional[int] = None
    mem_bus_width: Optional[int] = None
    pcie_tx_kbs: Optional[int] = None
    pcie_rx_kbs: Optional[int] = None
    pcie_gen: Optional[int] = None
    pcie_width: Optional[int] = None
    throttle_reasons: list = field(default_factory=list)
    processes: list = field(default_factory=list)


@dataclass
class HostInfo:
    hostname: str = ""
    cpu_percent: Optional[float] = None
    mem_used_bytes: Optional[int] = None
    mem_total_bytes: Optional[int] = None
    load1: Optional[float] = None
    driver_version: str = ""
    cuda_driver_version: str = ""


def _try(fn, *a):
    try:
        return fn(*a)
    except Exception:
        return None


class NvmlBackend:
    def __init__(self, nvml=None):
        if nvml is None:
            import pynvml as nvml
        self.n = nvml
        self.n.nvmlInit()

    def close(self) -> None:
        _try(self.n.nvmlShutdown)

    def versions(self) -> tuple[str, str]:
        d = _try(self.n.nvmlSystemGetDriverVersion) or ""
        c = _try(self.n.nvmlSystemGetCudaDriverVersion_v2)
        d = d.decode() if isinstance(d, bytes) else str(d)
        return d, (f"{c // 1000}.{(c % 1000) // 10}" if c else "")

    def count(self) -> int:
        return int(self.n.nvmlDeviceGetCount())

    def poll(self, index: int) -> GpuInfo:
        n = self.n
        h = n.nvmlDeviceGetHandleByIndex(index)
        name = _try(n.nvmlDeviceGetName, h) or ""
        g = GpuInfo(index, name.decode() if isinstance(name, bytes) else str(name))
        u = _try(n.nvmlDeviceGetUtilizationRates, h)
        if u is not None:
            g.util_percent = int(u.gpu)
        e = _try(n.nvmlDeviceGetEncoderUtilization, h)
        d = _try(n.nvmlDeviceGetDecoderUtilization, h)
        g.encoder_util_percent = int(e[0]) if e else None
        g.decoder_util_percent = int(d[0]) if d else None
        p = _try(n.nvmlDeviceGetPowerUsage, h)
        pl = _try(n.nvmlDeviceGetEnforcedPowerLimit, h)
        g.power_w = p / 1000.0 if p is not None else None
        g.power_limit_w = pl / 1000.0 if pl is not None else None
        g.temperature_c = _try(n.nvmlDeviceGetTemperature, h, getattr(n, "NVML_TEMPERATURE_GPU", 0))
        g.fan_percent = _try(n.nvmlDeviceGetFanSpeed, h)
        for attr, kind in (("clock_graphics_mhz", "NVML_CLOCK_GRAPHICS"), ("clock_sm_mhz", "NVML_CLOCK_SM"),
                           ("clock_mem_mhz", "NVML_CLOCK_MEM")):
            setattr(g, attr, _try(n.nvmlDeviceGetClockInfo, h, getattr(n, kind, 0)))
        g.clock_sm_max_mhz = _try(n.nvmlDeviceGetMaxClockInfo, h, getattr(n, "NVML_CLOCK_SM", 1))
        g.clock_mem_max_mhz = _try(n.nvmlDeviceGetMaxClockInfo, h, getattr(n, "NVML_CLOCK_MEM", 2))
        m = _try(n.nvmlDeviceGetMemoryInfo, h)
        if m is not None:
            g.mem_used_bytes, g.mem_total_bytes = int(m.used), int(m.total)
        g.mem_bus_width = _try(n.nvmlDeviceGetMemoryBusWidth, h)
        g.pcie_tx_kbs = _try(n.nvmlDeviceGetPcieThroughput, h, getattr(n, "NVML_PCIE_UTIL_TX_BYTES", 0))
        g.pcie_rx_kbs = _try(n.nvmlDeviceGetPcieThroughput, h, getattr(n, "NVML_PCIE_UTIL_RX_BYTES", 1))
        g.pcie_gen = _try(n.nvmlDeviceGetCurrPcieLinkGeneration, h)
        g.pcie_width = _try(n.nvmlDeviceGetCurrPcieLinkWidth, h)
        r = _try(n.nvmlDeviceGetCurrentClocksEventReasons, h) if hasattr(n, "nvmlDeviceGetCurrentClocksEventReasons") \
            else _try(getattr(n, "nvmlDeviceGetCurrentClocksThrottleReasons", lambda *_: None), h)
        if r:
            names = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
                     0x80: "hw_power_brake"}
            g.throttle_reasons = [v for k, v in names.items() if r & k]
        procs = _try(n.nvmlDeviceGetComputeRunningProcesses, h) or []
        for pr in procs:
            g.processes.append(ProcessInfo(int(pr.pid), *proc_name_user(int(pr.pid)),
                                           gpu_memory_bytes=getattr(pr, "usedGpuMemory", None)))
        return g


def proc_name_user(pid: int) -> tuple[str, str]:
    name, user = "", ""
    try:
        with open(f"/proc/{pid}/comm") as f:
            name = f.read().strip()
        import pwd
        user = pwd.getpwuid(os.stat(f"/proc/{pid}").st_uid).pw_name
    except Exception:
        pass
    return name, user


class HostPoller:
    """CPU and memory from /proc (platforms/linux/metrics.zig)."""

    def __init__(self):
        self._prev = self._cpu_times()

    @staticmethod
    def _cpu_times():
        try:
            with open("/proc/stat") as f:
                v = [int(x) for x in f.readline().split()[1:]]
            idle = v[3] + (v[4] if len(v) > 4 else 0)
            return sum(v), idle
        except Exception:
            return None

    def poll(self, versions=("", "")) -> HostInfo:
        h = HostInfo(hostname=os.uname().nodename, driver_version=versions[0], cuda_driver_version=versions[1])
        cur = self._cpu_times()
        if cur and self._prev and cur[0] > self._prev[0]:
            h.cpu_percent = 100.0 * (1.0 - (cur[1] - self._prev[1]) / (cur[0] - self._prev[0]))
        self._prev = cur
        try:
            mi = {}
            with open("/proc/meminfo") as f:
                for line in f:
                    k, v = line.split(":")
                    mi[k] = int(v.split()[0]) * 1024
            h.mem_total_bytes = mi.get("MemTotal")
            h.mem_used_bytes = mi.get("MemTotal", 0) - mi.get("MemAvailable", 0)
            h.load1 = os.getloadavg()[0]
        except Exception:
            pass
        return h


class FakeNvml:
    """In-memory stand-in for pynvml with the subset of calls the backend uses (tests, dry runs)."""
    NVML_TEMPERATURE_GPU, NVML_CLOCK_GRAPHICS, NVML_CLOCK_SM, NVML_CLOCK_MEM = 0, 0, 1, 2
    NVML_PCIE_UTIL_TX_BYTES, NVML_PCIE_UTIL_RX_BYTES = 0, 1

    class _Obj:
        def __init__(self, **kw):
            self.__dict__.update(kw)

    def __init__(self, devices: int = 2):
        self.devices = devices
        self.calls: list[str] = []

    def __getattr__(self, name):
        if name.startswith("nvmlDeviceSet") or "Reset" in name:
            raise AssertionError(f"zb-smi must never call {name}")
        raise AttributeError(name)

    def nvmlInit(self): self.calls.append("init")
    def nvmlShutdown(self): self.calls.append("shutdown")
    def nvmlSystemGetDriverVersion(self): return "580.159"
    def nvmlSystemGetCudaDriverVersion_v2(self): return 13000
    def nvmlDeviceGetCount(self): return self.devices
    def nvmlDeviceGetHandleByIndex(self, i): return i
    def nvmlDeviceGetName(self, h): return "NVIDIA B200"
    def nvmlDeviceGetUtilizationRates(self, h): return self._Obj(gpu=90 + h, memory=40)
    def nvmlDeviceGetEncoderUtilization(self, h): return (0, 1000)
    def nvmlDeviceGetDecoderUtilization(self, h): return (0, 1000)
    def nvmlDeviceGetPowerUsage(self, h): return 950_000
    def nvmlDeviceGetEnforcedPowerLimit(self, h): return 1_000_000
    def nvmlDeviceGetTemperature(self, h, k): return 61
    def nvmlDeviceGetFanSpeed(self, h): raise RuntimeError("not supported")
    def nvmlDeviceGetClockInfo(self, h, k): return {0: 1800, 1: 1800, 2: 3996}[k]
    def nvmlDeviceGetMaxClockInfo(self, h, k): return {1: 1965, 2: 3996}[k]
    def nvmlDeviceGetMemoryInfo(self, h): return self._Obj(used=100 << 30, total=183359 << 20, free=0)
    def nvmlDeviceGetMemoryBusWidth(self, h): return 8192
    def nvmlDeviceGetPcieThroughput(self, h, k): return 1234
    def nvmlDeviceGetCurrPcieLinkGeneration(self, h): return 5
    def nvmlDeviceGetCurrPcieLinkWidth(self, h): return 16
    def nvmlDeviceGetCurrentClocksEventReasons(self, h): return 0x4
    def nvmlDeviceGetComputeRunningProcesses(self, h): return [self._Obj(pid=os.getpid(), usedGpuMemory=5 << 30)]


class RemoteAgents:
    """Devices of other hosts, read from their agents' `/json` endpoint (`zb-smi --api` there): what
    bin/zml-smi/api/client.zig does for `--remotes`.  A host that does not answer keeps its last devices, marked stale."""

    def __init__(self, urls: list[str], timeout_s: float = 2.0):
        for u in urls:
            if not u.startswith(("http://", "https://")):
                raise ValueError(f"remote host must start with http:// or https://: {u}")
        self.urls, self.timeout_s = [u.rstrip("/") for u in urls], timeout_s
        self.last: dict[str, list[dict]] = {u: [] for u in self.urls}
        self.errors: dict[str, str] = {}

    def poll(self) -> list[dict]:
        import json
        import urllib.request
        out = []
        for u in self.urls:
            try:
                with urllib.request.urlopen(u + "/json", timeout=self.timeout_s) as r:
                    snap = json.loads(r.read())
                host = snap.get("host", {}).get("hostname", u)
                self.last[u] = [dict(g, remote=host, stale=False) for g in snap.get("gpus", [])]
                self.errors.pop(u, None)
            except Exception as e:          # unreachable agent: show what it last reported
                self.errors[u] = f"{type(e).__name__}: {e}"
                self.last[u] = [dict(g, stale=True) for g in self.last[u]]
            out.extend(self.last[u])
        return out


def snapshot(backend: Optional[NvmlBackend], host: HostPoller, remotes: Optional[RemoteAgents] = None) -> dict:
    gpus = [asdict(backend.poll(i)) for i in range(backend.count())] if backend else []
    if remotes is not None:
        for g in remotes.poll():            # remote devices follow the local ones; their own index is kept beside
            gpus.append(dict(g, remote_index=g.get("index"), index=len(gpus)))
    snap = {"timestamp": time.time(), "host": asdict(host.poll(backend.versions() if backend else ("", ""))), "gpus": gpus}
    if remotes is not None and remotes.errors:
        snap["remote_errors"] = dict(remotes.errors)
    return snap
