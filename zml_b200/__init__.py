"""zml_b200: a Blackwell-native inference framework with the capabilities of ZML.

Tagged-axis `Shape` / `Tensor`, logical-mesh sharding, safetensors streaming,
paged-KV attention, fused MoE, tokenizers and LLM serving, built on PyTorch plus
hand-written sm_100a CUDA kernels and in-kernel NVLink collectives.
"""
from __future__ import annotations

import importlib

__version__ = "0.1.0"

_LAZY = {
    "DataType": ("dtype", "DataType"),
    "Shape": ("shape", "Shape"),
    "Tensor": ("tensor", "Tensor"),
    "Slice": ("slice", "Slice"),
    "Buffer": ("buffer", "Buffer"),
    "Platform": ("platform", "Platform"),
    "Target": ("platform", "Target"),
    "Memory": ("platform", "MemoryKind"),
    "Exe": ("exe", "Exe"),
    "FnExe": ("exe", "FnExe"),
    "CompilationOptions": ("module", "CompilationOptions"),
    "Bufferized": ("mem", "Bufferized"),
    "Sharding": ("sharding", "Sharding"),
    "tracer": ("profiling.tracer", None),
}
_SUBMODULES = {
    "dtype", "floats", "shape", "tensor", "slice", "meta", "buffer", "mem", "exe", "module",
    "platform", "sharding", "io", "safetensors", "nn", "ops", "attention", "moe", "tokenizer",
    "testing", "profiling", "models", "parallel", "utils", "serving", "flags", "kernel", "logo", "stdx", "vfs", "spmd", "driver_probe",
}

# sizes, as the reference exports them (zml/zml.zig:59-62)
KiB = 1024
MiB = 1024 * KiB
GiB = 1024 * MiB
TiB = 1024 * GiB


def __getattr__(name):
    if name in _LAZY:
        mod, attr = _LAZY[name]
        m = importlib.import_module(f"{__name__}.{mod}")
        return m if attr is None else getattr(m, attr)
    if name in _SUBMODULES:
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
