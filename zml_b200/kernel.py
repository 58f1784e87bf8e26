"""Declarative user kernels: `kernel.cuda.Kernel(Config, spec)` -> `.emit(cfg)` gives the CUDA
C++ source, `.call(inputs, outputs, opts)` compiles it for sm_100a and launches it on the
current stream.

This is the B200 counterpart of zml/kernel.zig of the reference, where a kernel is declared as
a name, named inputs / outputs and a builder callback, `.emit()` returns Triton IR text and
`.call()` wraps it in a custom call.  There is no IR layer here: the callback returns CUDA C++
(with whatever inline PTX it needs: tcgen05, TMA, mbarriers), `nvcc` turns it into a cubin
(cached by content hash), and the CUDA driver API loads and launches it - no framework
recompilation, usable from inside CUDA-graph capture.

The generated kernel's parameters are, in order: one pointer per input, one pointer per
output, then the `scalars` of the call (int32 / float32 / int64 by Python type).
"""
from __future__ import annotations

import ctypes as C
import hashlib
import os
import subprocess
import tempfile
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Mapping, Optional, Sequence

import torch

from .shape import Shape
from .tensor import Tensor

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


class KernelError(RuntimeError):
    pass


def cache_dir() -> Path:
    d = Path(os.environ.get("ZB_KERNEL_CACHE_DIR", Path(tempfile.gettempdir()) / "zb_kernel_cache"))
    d.mkdir(parents=True, exist_ok=True)
    return d


def compile_cubin(source: str, extra_flags: Sequence[str] = ()) -> Path:
    """CUDA C++ -> cubin for sm_100a (cross-compiles on a machine without a GPU)."""
    from ._build import _nvcc
    nvcc = _nvcc()
    if nvcc is None:
        raise KernelError("nvcc not found")
    key = hashlib.sha256((source + "\0" + " ".join(extra_flags)).encode()).hexdigest()[:24]
    out = cache_dir() / f"{key}.cubin"
    if out.exists():
        return out
    src = cache_dir() / f"{key}.cu"
    src.write_text(source)
    csrc = Path(__file__).resolve().parent / "csrc"
    tmp = out.with_suffix(f".{os.getpid()}.tmp")
    r = subprocess.run([nvcc, *ARCH_FLAGS, "-O3", "-std=c++17", "-lineinfo", "-cubin", "-I", str(csrc), *extra_flags,
                        "-o", str(tmp), str(src)], capture_output=True, text=True)
    if r.returncode != 0:
        raise KernelError(f"nvcc failed for kernel source {src}:\n{r.stderr}")
    os.replace(tmp, out)
    return out


class _Driver:
    """The handful of CUDA driver entry points needed to load and launch a cubin."""
    _inst = None

    def __init__(self):
        self.lib = C.CDLL("libcuda.so.1")
        self.lib.cuModuleLoadData.argtypes = [C.POINTER(C.c_void_p), C.c_void_p]
        self.lib.cuModuleGetFunction.argtypes = [C.POINTER(C.c_void_p), C.c_void_p, C.c_char_p]
        self.lib.cuFuncSetAttribute.argtypes = [C.c_void_p, C.c_int, C.c_int]
        self.lib.cuLaunchKernel.argtypes = [C.c_void_p] + [C.c_uint] * 6 + [C.c_uint, C.c_void_p, C.POINTER(C.c_void_p), C.c_void_p]

    @staticmethod
    def get() -> "_Driver":
        if _Driver._inst is None:
            _Driver._inst = _Driver()
        return _Driver._inst

    def check(self, rc: int, what: str) -> None:
        if rc != 0:
            raise KernelError(f"{what} failed with CUDA driver error {rc}")


@dataclass
class Spec:
    name: str
    inputs: Sequence[str]
    outputs: Sequence[str]
    run: Callable[[Any], str]                 # cfg -> CUDA C++ defining `extern "C" __global__ void <name>(...)`


@dataclass
class CallOpts:
    cfg: Any = None
    grid: Sequence[int] = (1, 1, 1)
    block: Sequence[int] = (128, 1, 1)
    shared_bytes: int = 0
    scalars: Sequence = ()
    output_operand_aliases: Optional[Mapping[str, str]] = None      # output name -> input name written in place
    extra_flags: Sequence[str] = ()


class Kernel:
    def __init__(self, spec: Spec):
        self.spec = spec
        self.name = spec.name
        self._functions: dict = {}

    def emit(self, cfg=None) -> str:
        src = self.spec.run(cfg)
        if f"{self.name}(" not in src:
            raise KernelError(f"the source emitted for kernel {self.name!r} does not define it")
        return src

    def compile(self, cfg=None, extra_flags: Sequence[str] = ()) -> Path:
        return compile_cubin(self.emit(cfg), extra_flags)

    def _function(self, cfg, opts: CallOpts):
        key = (repr(cfg), tuple(opts.extra_flags), torch.cuda.current_device())
        fn = self._functions.get(key)
        if fn is None:
            d = _Driver.get()
            image = self.compile(cfg, opts.extra_flags).read_bytes()
            torch.cuda.current_stream()                    # make sure the primary context exists and is current
            mod, f = C.c_void_p(), C.c_void_p()
            d.check(d.lib.cuModuleLoadData(C.byref(mod), image), "cuModuleLoadData")
            d.check(d.lib.cuModuleGetFunction(C.byref(f), mod, self.name.encode()), "cuModuleGetFunction")
            if opts.shared_bytes > 48 * 1024:
                d.check(d.lib.cuFuncSetAttribute(f, 8, int(opts.shared_bytes)), "cuFuncSetAttribute")   # max dynamic smem
            fn = (mod, f)
            self._functions[key] = fn
        return fn[1]

    def call(self, inputs: Mapping[str, Tensor], outputs: Mapping[str, Shape], opts: CallOpts) -> dict:
        """Launches on the current CUDA stream; returns {output name: Tensor}."""
        for n in self.spec.inputs:
            if n not in inputs:
                raise KernelError(f"kernel {self.name}: missing input {n!r}")
        for n in self.spec.outputs:
            if n not in outputs:
                raise KernelError(f"kernel {self.name}: missing output {n!r}")
        ins = [inputs[n].to_torch() for n in self.spec.inputs]
        if not ins or not ins[0].is_cuda:
            raise KernelError(f"kernel {self.name}: inputs must be CUDA tensors")
        dev = ins[0].device
        alias = dict(opts.output_operand_aliases or {})
        outs = {}
        for n in self.spec.outputs:
            sh = outputs[n]
            if n in alias:
                outs[n] = inputs[alias[n]].to_torch()
            else:
                outs[n] = torch.empty(tuple(sh.dims), dtype=sh.dtype.to_torch(), device=dev)
        f = self._function(opts.cfg, opts)
        args = [C.c_void_p(t.data_ptr()) for t in ins] + [C.c_void_p(outs[n].data_ptr()) for n in self.spec.outputs]
        for s in opts.scalars:
            if isinstance(s, bool) or isinstance(s, int) and -2 ** 31 <= s < 2 ** 31:
                args.append(C.c_int32(int(s)))
            elif isinstance(s, int):
                args.append(C.c_int64(s))
            else:
                args.append(C.c_float(float(s)))
        argv = (C.c_void_p * len(args))(*[C.cast(C.pointer(a), C.c_void_p) for a in args])
        g, b = list(opts.grid) + [1] * (3 - len(opts.grid)), list(opts.block) + [1] * (3 - len(opts.block))
        d = _Driver.get()
        d.check(d.lib.cuLaunchKernel(f, g[0], g[1], g[2], b[0], b[1], b[2], int(opts.shared_bytes),
                                     C.c_void_p(torch.cuda.current_stream().cuda_stream), argv, None), "cuLaunchKernel")
        from .ops import _lib
        _lib.lib().zb_launch_count_add(1)
        return {n: Tensor(outs[n], outputs[n]) for n in self.spec.outputs}


class cuda:
    """Namespace mirroring `zml.kernel.triton` of the reference."""
    Kernel = Kernel
    Spec = Spec
    CallOpts = CallOpts

    @staticmethod
    def ctype(dt) -> str:
        """CUDA C++ element type of a DataType (kernel.zig `from`)."""
        name = getattr(dt, "name", str(dt))
        table = {"bool": "bool", "i8": "int8_t", "u8": "uint8_t", "i16": "int16_t", "u16": "uint16_t", "i32": "int32_t",
                 "u32": "uint32_t", "i64": "int64_t", "u64": "uint64_t", "f16": "__half", "bf16": "__nv_bfloat16",
                 "f32": "float", "f64": "double", "f8e4m3fn": "__nv_fp8_e4m3", "f8e5m2": "__nv_fp8_e5m2"}
        if name not in table:
            raise KernelError(f"dtype {name} has no CUDA C++ equivalent")
        return table[name]

    @staticmethod
    def elementwise(name: str, inputs: Sequence[str], output: str, expr: str, dtype="f32") -> Kernel:
        """Kernel computing `output[i] = expr` where `expr` refers to the inputs by name
        (each read as float at index i)."""
        ct = cuda.ctype(dtype)

        def run(_cfg) -> str:
            params = ", ".join([f"const {ct}* __restrict__ {n}_p" for n in inputs] + [f"{ct}* __restrict__ {output}_p", "int n"])
            loads = "\n    ".join(f"const float {n} = static_cast<float>({n}_p[i]);" for n in inputs)
            return (f"#include <cuda_bf16.h>\n#include <cuda_fp16.h>\n#include <stdint.h>\n"
                    f"extern \"C\" __global__ void {name}({params}) {{\n"
                    f"  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {{\n"
                    f"    {loads}\n    {output}_p[i] = static_cast<{ct}>({expr});\n  }}\n}}\n")
        return Kernel(Spec(name, list(inputs), [output], run))
