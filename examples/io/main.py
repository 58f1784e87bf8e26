#!/usr/bin/env python
"""File and checkpoint tooling over the VFS (the reference's examples/io).

    io cat <uri> | tree <dir> | ls <uri> | cp <src> <dst> | stat <uri> | realpath <uri>
    io safetensors <file|index|dir>      list tensors (name, dtype, shape, bytes) and metadata
    io load <file|index|dir> [--device=cpu|cuda] [--chunk-mib=32] [--chunks=8] [--parallelism=16]
                                         every tensor through the Loader (pinned staging ring, asynchronous
                                         host-to-device copies) to the device, report GiB/s
    io synth <dir> [--gib=16] [--tensor-mib=512]   write a synthetic bf16 checkpoint of that size (sharded files)
URIs: plain paths, file://, http(s)://, hf://org/repo[@rev]/file, s3://bucket/key, gs://bucket/key.
"""
from __future__ import annotations

import os
import sys
import time
from dataclasses import dataclass

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
    chunk_mib: int = 32
    chunks: int = 8
    parallelism: int = 16


@dataclass
class SynthArgs:
    positional: One
    gib: float = 16.0
    tensor_mib: int = 512


def tree(vfs, path, prefix=""):
    for name in vfs.list(path):
        full = os.path.join(path, name)
        print(prefix + name)
        if vfs.stat(full).kind == "directory":
            tree(vfs, full, prefix + "  ")


def main(argv=None) -> int:
    cmds = {"cat": OneArg, "tree": OneArg, "ls": OneArg, "stat": OneArg, "realpath": OneArg, "cp": TwoArgs,
            "safetensors": OneArg, "load": LoadArgs, "synth": SynthArgs}
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
        import torch
        from zml_b200.io import Loader, TensorStore
        from zml_b200.platform import CpuOptions, CreateOptions, Platform, Target
        store = TensorStore.from_path(a.positional.path)
        on_gpu = a.device.startswith("cuda")
        platform = Platform.init(Target.cuda) if on_gpu else Platform.init(Target.cpu, CreateOptions(cpu=CpuOptions(1)))
        view = store.view()
        model = {k: view.create_tensor(k) for k in store.registry.keys()}
        loader = Loader(platform, parallelism=a.parallelism, dma_chunk_size=a.chunk_mib << 20, dma_chunks=a.chunks)
        t0 = time.perf_counter()
        bufs = loader.load(model, store, [])
        dt = time.perf_counter() - t0
        st = loader.stats()
        print(f"loaded {st['bytes_loaded'] / 2 ** 30:.3f} GiB ({len(bufs)} tensors) in {dt:.2f}s: "
              f"{st['bytes_loaded'] / 2 ** 30 / max(dt, 1e-9):.2f} GiB/s  [staging {st['staging_bytes'] >> 20} MiB pinned, "
              f"{st['chunk_waits']} waits for a free chunk, {st['read_seconds']:.2f} reader-seconds]")
        loader.close()
        del torch
    elif name == "synth":
        import torch
        os.makedirs(a.positional.path, exist_ok=True)
        per = a.tensor_mib << 20
        n = max(1, int(a.gib * 2 ** 30) // per)
        g = torch.Generator().manual_seed(0)
        base = torch.randn(per // 2, generator=g).bfloat16()
        t0 = time.perf_counter()
        # one file per 8 tensors; the same values rotated so that files differ and no page is shared
        names = {}
        for f0 in range(0, n, 8):
            part = {f"w.{i}": torch.roll(base, i).reshape(-1, 4096) for i in range(f0, min(n, f0 + 8))}
            fname = f"model-{f0 // 8 + 1:05d}.safetensors"
            safetensors.save_file(part, os.path.join(a.positional.path, fname))
            names.update({k: fname for k in part})
        import json
        with open(os.path.join(a.positional.path, safetensors.INDEX_NAME), "w") as f:
            json.dump({"metadata": {"total_size": n * per}, "weight_map": names}, f)
        print(f"wrote {n} tensors of {a.tensor_mib} MiB ({n * per / 2 ** 30:.2f} GiB) in {time.perf_counter() - t0:.1f}s")
    return 0


if __name__ == "__main__":
    sys.exit(main())
