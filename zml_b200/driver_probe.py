"""CUDA driver probe: is the NVIDIA driver of this machine one that the CUDA runtime in use, and a B200, can run on?

The reference ships a forward-compatibility `libcuda` and, before loading its CUDA plugin, runs a small child program
that calls `cuInit` against it and turns the result into an exit code (platforms/cuda/compat_probe.zig:3-41); the
parent then decides whether to load the compatibility libraries or to stay on the system driver
(platforms/cuda/cuda.zig:30-125).  It probes in a child because a failed `cuInit` leaves the process unable to try
another `libcuda`.

Here the CUDA runtime comes with PyTorch, so there is nothing to swap in; what can still be wrong is the driver:

* no `libcuda.so.1` at all (no driver, or a container started without the NVIDIA runtime);
* `cuInit` fails - 803 (the user-mode driver and the kernel module are of different versions: a driver upgrade
  without a reboot), 804 (forward compatibility is not allowed on this GPU), anything else;
* the driver is older than the CUDA runtime PyTorch was built with, or older than CUDA 12.8, the first release that
  knows sm_100.

`probe()` does the calls in this process (ctypes, no PyTorch), `probe_in_child()` in a child as the reference does,
`diagnose()` puts the answer into a sentence.  `Platform` adds that sentence to its error when a CUDA target was asked
for and PyTorch sees no device.  `python -m zml_b200.driver_probe` prints it and exits with the code.
"""
from __future__ import annotations

import ctypes
import enum
import json
import subprocess
import sys
from dataclasses import asdict, dataclass
from typing import Optional

CUDA_SUCCESS = 0
CUDA_ERROR_NO_DEVICE = 100
CUDA_ERROR_SYSTEM_DRIVER_MISMATCH = 803
CUDA_ERROR_COMPAT_NOT_SUPPORTED_ON_DEVICE = 804

MIN_DRIVER_FOR_SM100 = 12080            # cuDriverGetVersion units (1000 * major + 10 * minor): CUDA 12.8


class ExitCode(enum.IntEnum):
    """0-3 are the reference's codes (platforms/cuda/compat_probe.zig:3-8); the others are cases it cannot meet
    because it always has a `libcuda` to open."""
    success = 0
    compat_not_supported_on_device = 1
    system_driver_mismatch = 2
    unexpected_error = 3
    no_driver = 4
    no_device = 5


@dataclass
class ProbeResult:
    code: ExitCode
    cu_result: Optional[int] = None         # what cuInit returned
    driver_version: Optional[int] = None    # e.g. 13000 for a driver that supports CUDA 13.0
    device_count: Optional[int] = None
    message: str = ""

    def ok(self) -> bool:
        return self.code is ExitCode.success

    def to_json(self) -> str:
        d = asdict(self)
        d["code"] = int(self.code)
        return json.dumps(d)

    @staticmethod
    def from_json(text: str) -> "ProbeResult":
        d = json.loads(text)
        d["code"] = ExitCode(d["code"])
        return ProbeResult(**d)


def format_version(v: Optional[int]) -> str:
    return "unknown" if v is None else f"{v // 1000}.{v % 1000 // 10}"


def _load(path: str):
    return ctypes.CDLL(path)


def probe(lib=None, path: str = "libcuda.so.1") -> ProbeResult:
    """Calls cuInit, cuDriverGetVersion and cuDeviceGetCount on `lib` (anything with those three callables; default:
    the `libcuda` found at `path`).  Creates no context."""
    if lib is None:
        try:
            lib = _load(path)
        except OSError as e:
            return ProbeResult(ExitCode.no_driver, message=f"{path} cannot be loaded: {e}")
    rc = int(lib.cuInit(0))
    if rc == CUDA_ERROR_SYSTEM_DRIVER_MISMATCH:
        return ProbeResult(ExitCode.system_driver_mismatch, rc, message="cuInit: system driver mismatch (803)")
    if rc == CUDA_ERROR_COMPAT_NOT_SUPPORTED_ON_DEVICE:
        return ProbeResult(ExitCode.compat_not_supported_on_device, rc,
                           message="cuInit: forward compatibility is not supported on this device (804)")
    if rc == CUDA_ERROR_NO_DEVICE:
        return ProbeResult(ExitCode.no_device, rc, device_count=0, message="cuInit: no CUDA-capable device (100)")
    if rc != CUDA_SUCCESS:
        text = ""
        get = getattr(lib, "cuGetErrorString", None)
        if get is not None:
            p = ctypes.c_char_p()
            if int(get(rc, ctypes.byref(p))) == CUDA_SUCCESS and p.value:
                text = ": " + p.value.decode("utf-8", "replace")
        return ProbeResult(ExitCode.unexpected_error, rc, message=f"cuInit returned {rc}{text}")
    ver, count = ctypes.c_int(0), ctypes.c_int(0)
    version = int(ver.value) if int(lib.cuDriverGetVersion(ctypes.byref(ver))) == CUDA_SUCCESS else None
    n = int(count.value) if int(lib.cuDeviceGetCount(ctypes.byref(count))) == CUDA_SUCCESS else None
    if n == 0:
        return ProbeResult(ExitCode.no_device, rc, version, 0, "the driver answers but lists no device")
    return ProbeResult(ExitCode.success, rc, version, n, "ok")


def probe_in_child(timeout_s: float = 30.0, python: Optional[str] = None) -> ProbeResult:
    """`probe()` in a child process, so that a failed cuInit does not stay with this one."""
    try:
        out = subprocess.run([python or sys.executable, "-m", "zml_b200.driver_probe", "--json"],
                             capture_output=True, text=True, timeout=timeout_s)
    except (OSError, subprocess.TimeoutExpired) as e:
        return ProbeResult(ExitCode.unexpected_error, message=f"the probe did not run: {e}")
    for line in reversed(out.stdout.splitlines()):
        if line.startswith("{"):
            try:
                return ProbeResult.from_json(line)
            except (ValueError, KeyError, TypeError):
                break
    try:
        code = ExitCode(out.returncode)
    except ValueError:
        code = ExitCode.unexpected_error
    return ProbeResult(code, message=(out.stderr or out.stdout).strip()[-200:] or f"the probe exited with {out.returncode}")


def runtime_version() -> Optional[int]:
    """The CUDA runtime PyTorch was built with, in cuDriverGetVersion units (12.8 -> 12080); None for a CPU build."""
    import torch
    v = torch.version.cuda
    if not v:
        return None
    major, _, minor = v.partition(".")
    return int(major) * 1000 + int(minor or 0) * 10


def diagnose(result: ProbeResult, runtime: Optional[int] = None) -> str:
    """One sentence: what is wrong with the driver, or that nothing is."""
    c = result.code
    if c is ExitCode.no_driver:
        return ("no NVIDIA driver library in this process's reach (" + result.message + "); on a GPU machine, start the "
                "container with the NVIDIA runtime (--gpus all)")
    if c is ExitCode.system_driver_mismatch:
        return ("the NVIDIA user-mode driver and kernel module are of different versions (cuInit 803): the driver was "
                "upgraded without reloading the module - reboot, or reload the nvidia modules")
    if c is ExitCode.compat_not_supported_on_device:
        return ("a forward-compatibility libcuda is on the library path and this GPU does not allow it (cuInit 804): "
                "take the compat directory out of LD_LIBRARY_PATH")
    if c is ExitCode.no_device:
        return "the driver loads but shows no device to this process (check CUDA_VISIBLE_DEVICES and the container's device list)"
    if c is ExitCode.unexpected_error:
        return "the driver probe failed: " + result.message
    need = max(runtime or 0, MIN_DRIVER_FOR_SM100)
    if result.driver_version is not None and result.driver_version < need:
        return (f"the driver supports CUDA {format_version(result.driver_version)}, older than CUDA {format_version(need)} "
                f"that {'this PyTorch build' if runtime and runtime >= MIN_DRIVER_FOR_SM100 else 'sm_100'} needs: upgrade the driver")
    return f"driver ok: CUDA {format_version(result.driver_version)}, {result.device_count} device(s)"


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else list(argv)
    r = probe()
    if "--json" in argv:
        print(r.to_json())
    else:
        rt = None
        if "--no-torch" not in argv:
            try:
                rt = runtime_version()
            except Exception:
                rt = None
        print(diagnose(r, rt))
    return int(r.code)


if __name__ == "__main__":
    sys.exit(main())
