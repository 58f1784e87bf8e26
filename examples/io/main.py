#!/usr/bin/env python
"""File and checkpoint tooling over the VFS (the reference's examples/io).

    io cat <uri> | tree <dir> | ls <uri> | cp <src> <dst> | stat <uri> | realpath <uri>
    io safetensors <file|index|dir>      list tensors (name, dtype, shape, bytes) and metadata
    io load <file|index|dir> [--device=cpu|cuda]   stream every tensor to the device, report GiB/s
URIs: plain paths, file://, http(s)://, hf://org/repo[@rev]/file, s3://bucket/key, gs://bucket/key.
"""
from __future__ import annotations

import os
import sys
import time
from dataclasses import dataclass
from typing import Optional

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from zml_b200 import flags, safetensors  # noqa: E402
from zml_b200.vfs import Vfs  # noqa: E402


@dataclass
class One:
    path: str


@dataclass
class OneArg:
    positional: One


@dataclass
class Two:
    src: str
    dst: str


@dataclass
class TwoArgs:
    positional: Two


@dataclass
class LoadArgs:
    positional: One
    device: str = "cpu"


def tree(vfs, path, prefix=""):
    for name in vfs.list(path):
        full = os.path.join(path, name)
        print(prefix + name)
        if vfs.stat(full).kind == "directory":
            tree(vfs, full, prefix + "  ")


def main(argv=None) -> int:
    cmds = {"cat": OneArg, "tree": OneArg, "ls": OneArg, "stat": OneArg, "realpath": OneArg, "cp": TwoArgs,
            "safetensors": OneArg, "load": LoadArgs}
    name, a = flags.parse(argv, cmds, __doc__)
    vfs = Vfs.default()
    if name == "cat":
        sys.stdout.buffer.write(vfs.read(a.positional.path))
    elif name == "tree":
        tree(vfs, a.positional.path)
    elif name == "ls":
        print("\n".join(vfs.list(a.positional.path)))
    elif name == "stat":
        st = vfs.stat(a.positional.path)
        print(f"{a.positional.path}: {st.kind}, {st.size} bytes")
    elif name == "realpath":
        print(vfs.realpath(a.positional.path))
    elif name == "cp":
        n = vfs.copy(a.positional.src, a.positional.dst)
        print(f"copied {n} bytes")
    elif name == "safetensors":
        reg = safetensors.TensorRegistry.from_path(a.positional.path)
        for k in sorted(reg.keys()):
            t = reg.get(k)
            print(f"{k}: {t.shape.dtype.value} {list(t.shape.dims)} {t.byte_size()} B  [{os.path.basename(t.file)}]")
        for k, v in reg.metadata.items():
            print(f"metadata {k} = {v}")
        print(f"{len(reg)} tensors, {reg.total_bytes() / 2 ** 20:.2f} MiB")
    elif name == "load":
        from zml_b200.io import TensorStore
        store = TensorStore.from_path(a.positional.path)
        t0 = time.perf_counter()
        total = 0
        for k in store.registry.keys():
            if store.registry.get(k).shape.dtype.bit_size_of() < 8:
                continue
            t = store.load_tensor(k, device=a.device)
            total += t.numel() * t.element_size()
        if a.device.startswith("cuda"):
            import torch
            torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        print(f"loaded {total / 2 ** 30:.3f} GiB in {dt:.2f}s: {total / 2 ** 30 / max(dt, 1e-9):.2f} GiB/s")
    return 0


if __name__ == "__main__":
    sys.exit(main())
