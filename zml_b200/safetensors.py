"""safetensors checkpoints: header parsing, sharded repos, range reads, and a writer.

Reading follows the reference (zml/safetensors.zig): a checkpoint is either a single
``model.safetensors`` or a ``model.safetensors.index.json`` whose ``weight_map`` lists
the shard files; each file starts with an 8-byte little-endian header length followed
by a JSON header ``{name: {dtype, shape, data_offsets}, "__metadata__": {...}}``; only
headers are read up front, tensor bytes are streamed on demand (one tensor, or just
the byte ranges of one device's shard).  Metadata is flattened to dotted keys.

The writer produces the same format and is used for the synthetic random-init
checkpoints of the benchmarks and tests.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import struct
from dataclasses import dataclass
from typing import Mapping, Optional, Sequence

import numpy as np
import torch

from .dtype import DataType
from .shape import Shape

BYTES_HEADER = 8
INDEX_NAME = "model.safetensors.index.json"
MODEL_NAME = "model.safetensors"


class SafetensorsError(ValueError):
    pass


@dataclass
class TensorInfo:
    name: str
    shape: Shape
    file: str
    start: int          # absolute byte offset in `file`
    end: int

    def byte_size(self) -> int:
        return self.end - self.start


# ---------------------------------------------------------------------- native reader
_HOST = None


def _host_lib():
    global _HOST
    if _HOST is None:
        from . import _build
        p = _build.OUT / "libzb_host.so"
        if not p.exists():
            try:
                _build.build_host()
            except Exception:
                _HOST = False
                return None
        try:
            lib = C.CDLL(str(p))
            lib.zbh_pread_spans.restype = C.c_longlong
            lib.zbh_pread_spans.argtypes = [C.c_int, C.POINTER(C.c_longlong), C.POINTER(C.c_longlong), C.c_int,
                                            C.c_void_p, C.c_int]
            _HOST = lib
        except OSError:
            _HOST = False
    return _HOST or None


def read_spans(fd: int, spans: Sequence[tuple[int, int]], dst: np.ndarray, threads: int = 8) -> int:
    """Reads byte ranges of `fd` back to back into `dst` (uint8).  Multi-threaded pread in
    libzb_host.so when it is built, else os.preadv."""
    total = sum(l for _, l in spans)
    if dst.nbytes < total:
        raise SafetensorsError("destination too small")
    lib = _host_lib()
    if lib is not None and total > 0:
        n = len(spans)
        offs = (C.c_longlong * n)(*[s[0] for s in spans])
        lens = (C.c_longlong * n)(*[s[1] for s in spans])
        r = lib.zbh_pread_spans(fd, offs, lens, n, dst.ctypes.data_as(C.c_void_p), threads)
        if r < 0:
            raise OSError(-r, os.strerror(-r))
        if r != total:
            raise SafetensorsError(f"short read: {r} of {total} bytes")
        return int(r)
    pos = 0
    mv = memoryview(dst).cast("B")
    for off, ln in spans:
        got = 0
        while got < ln:
            r = os.preadv(fd, [mv[pos + got:pos + ln]], off + got)
            if r <= 0:
                raise SafetensorsError("unexpected end of file")
            got += r
        pos += ln
    return total


# ---------------------------------------------------------------------- metadata
def flatten_metadata(val, prefix: str = "", out: Optional[dict] = None) -> dict:
    """Nested JSON -> {dotted.key: scalar | homogeneous list}; empty arrays are dropped,
    heterogeneous arrays are expanded by index (zml/safetensors.zig:778-850)."""
    out = {} if out is None else out
    if isinstance(val, dict):
        for k, v in val.items():
            flatten_metadata(v, f"{prefix}.{k}" if prefix else str(k), out)
    elif isinstance(val, list):
        if not val:
            return out
        kinds = {type(x) for x in val}
        if len(kinds) == 1 and next(iter(kinds)) in (bool, int, float, str):
            out[prefix] = list(val)
        else:
            for i, item in enumerate(val):
                flatten_metadata(item, f"{prefix}.{i}" if prefix else str(i), out)
    else:
        out[prefix] = val
    return out


# ---------------------------------------------------------------------- registry
def is_uri(path: str) -> bool:
    """True for http(s):// hf:// s3:// gs:// locations (read through `zml_b200.vfs`), False for local paths."""
    return "://" in path and not path.startswith("file://")


_VFS = None


def _vfs():
    global _VFS
    if _VFS is None:
        from .vfs import Vfs
        _VFS = Vfs.default()
    return _VFS


def _read_header_remote(uri: str) -> tuple[dict, int, int]:
    v = _vfs()
    size = v.stat(uri).size
    raw = v.read_range(uri, 0, BYTES_HEADER)
    if len(raw) != BYTES_HEADER:
        raise SafetensorsError(f"{uri}: too short for a safetensors header")
    (n,) = struct.unpack("<Q", raw)
    if n <= 0 or n > size - BYTES_HEADER:
        raise SafetensorsError(f"{uri}: header length {n} is inconsistent with file size {size}")
    try:
        header = json.loads(v.read_range(uri, BYTES_HEADER, n))
    except json.JSONDecodeError as e:
        raise SafetensorsError(f"{uri}: invalid header json: {e}") from None
    return header, BYTES_HEADER + n, size


def read_header(path: str) -> tuple[dict, int]:
    """(header json, offset of the data section).  `path` may be a remote location."""
    if is_uri(path):
        h, off, _ = _read_header_remote(path)
        return h, off
    with open(path, "rb") as f:
        raw = f.read(BYTES_HEADER)
        if len(raw) != BYTES_HEADER:
            raise SafetensorsError(f"{path}: too short for a safetensors header")
        (n,) = struct.unpack("<Q", raw)
        size = os.fstat(f.fileno()).st_size
        if n <= 0 or n > size - BYTES_HEADER:
            raise SafetensorsError(f"{path}: header length {n} is inconsistent with file size {size}")
        try:
            header = json.loads(f.read(n))
        except json.JSONDecodeError as e:
            raise SafetensorsError(f"{path}: invalid header json: {e}") from None
    return header, BYTES_HEADER + n


def resolve_model_repo(path: str) -> str:
    """Directory (or, for a URI, the prefix) that holds the checkpoint: a file path resolves to its directory."""
    if path.endswith(".safetensors.index.json") or path.endswith(".safetensors"):
        d = path.rsplit("/", 1)[0] if is_uri(path) else (os.path.dirname(path) or ".")
    else:
        d = path.rstrip("/") if is_uri(path) else path
    if not is_uri(d) and not os.path.isdir(d):
        raise FileNotFoundError(d)
    return d


def repo_file_exists(repo: str, name: str) -> bool:
    if not is_uri(repo):
        return os.path.exists(os.path.join(repo, name))
    try:
        return _vfs().stat(f"{repo}/{name}").kind == "file"
    except (OSError, ValueError):            # urllib's HTTPError / URLError are OSErrors
        return False


def read_repo_file(repo: str, name: str) -> bytes:
    """Bytes of a small file of a repository (config.json, tokenizer.json), local or behind the VFS."""
    if is_uri(repo):
        return _vfs().read(f"{repo}/{name}")
    with open(os.path.join(repo, name), "rb") as f:
        return f.read()


def resolve_model_entrypoint(repo: str) -> str:
    for name in (INDEX_NAME, MODEL_NAME):
        if repo_file_exists(repo, name):
            return f"{repo}/{name}" if is_uri(repo) else os.path.join(repo, name)
    raise FileNotFoundError(f"{repo}: neither {INDEX_NAME} nor {MODEL_NAME}")


class TensorRegistry:
    """Every tensor of a checkpoint (name -> TensorInfo) plus flattened metadata."""

    def __init__(self):
        self.tensors: dict[str, TensorInfo] = {}
        self.metadata: dict = {}
        self.files: list[str] = []

    # ------------------------------------------------------------------ construction
    @staticmethod
    def from_path(path: str) -> "TensorRegistry":
        """`path` is a .safetensors file, an index json, or a repo directory; files may also be remote
        (`https://...`, `hf://org/repo/model.safetensors.index.json`, `s3://...`, `gs://...`): then only headers are
        fetched here and tensors are read later as range requests."""
        if (not is_uri(path) and os.path.isdir(path)) or (is_uri(path) and not path.endswith((".safetensors", ".index.json"))):
            path = resolve_model_entrypoint(path.rstrip("/") if is_uri(path) else path)
        reg = TensorRegistry()
        if path.endswith(".index.json"):
            if is_uri(path):
                idx = json.loads(_vfs().read(path))
            else:
                with open(path) as f:
                    idx = json.load(f)
            if "weight_map" not in idx:
                raise SafetensorsError(f"{path}: no weight_map")
            reg.metadata.update(flatten_metadata(idx.get("metadata", {})))
            repo = path.rsplit("/", 1)[0] if is_uri(path) else (os.path.dirname(path) or ".")
            for fname in sorted(set(idx["weight_map"].values())):
                reg._add_file(f"{repo}/{fname}" if is_uri(path) else os.path.join(repo, fname))
            missing = [k for k in idx["weight_map"] if k not in reg.tensors]
            if missing:
                raise SafetensorsError(f"{path}: tensors listed but absent from the shards: {missing[:3]}")
        elif path.endswith(".safetensors"):
            reg._add_file(path)
        else:
            raise SafetensorsError(f"{path}: not a safetensors file or index")
        return reg

    from_repo = from_path

    def _add_file(self, path: str) -> None:
        if is_uri(path):
            header, data_off, size = _read_header_remote(path)
        else:
            header, data_off = read_header(path)
            size = os.path.getsize(path)
        self.files.append(path)
        for name, ent in header.items():
            if name == "__metadata__":
                self.metadata.update(flatten_metadata(ent))
                continue
            dt = DataType.from_safetensors(ent["dtype"])
            a, b = ent["data_offsets"]
            shape = Shape(tuple(int(d) for d in ent["shape"]), dt)
            if a > b or data_off + b > size:
                raise SafetensorsError(f"{path}: tensor {name} offsets [{a},{b}) exceed the file")
            if b - a != shape.byte_size():
                raise SafetensorsError(f"{path}: tensor {name} has {b - a} bytes, shape {shape} needs {shape.byte_size()}")
            self.tensors[name] = TensorInfo(name, shape, path, data_off + a, data_off + b)

    # ------------------------------------------------------------------ queries
    def __contains__(self, name: str) -> bool:
        return name in self.tensors

    def __len__(self) -> int:
        return len(self.tensors)

    def keys(self):
        return self.tensors.keys()

    def get(self, name: str) -> TensorInfo:
        try:
            return self.tensors[name]
        except KeyError:
            raise KeyError(f"tensor {name!r} not found in checkpoint") from None

    def total_bytes(self) -> int:
        return sum(t.byte_size() for t in self.tensors.values())

    def reader(self, name: str) -> "TensorReader":
        return TensorReader(self.get(name))


class TensorReader:
    """Streams the bytes of exactly one tensor (whole, or a list of byte ranges)."""

    def __init__(self, info: TensorInfo):
        self.info = info
        self._fd: Optional[int] = None

    def __enter__(self):
        if not is_uri(self.info.file):
            self._fd = os.open(self.info.file, os.O_RDONLY)
        return self

    def __exit__(self, *exc):
        if self._fd is not None:
            os.close(self._fd)
            self._fd = None

    def read_into(self, dst: np.ndarray, spans: Optional[Sequence[tuple[int, int]]] = None, threads: int = 8) -> int:
        """`spans` are (offset, length) relative to the tensor's first byte."""
        if is_uri(self.info.file):
            if spans is None:
                spans = [(0, self.info.byte_size())]
            for off, ln in spans:
                if off < 0 or off + ln > self.info.byte_size():
                    raise SafetensorsError(f"span [{off},{off + ln}) outside tensor {self.info.name}")
            _vfs().read_spans(self.info.file, [(self.info.start + o, l) for o, l in spans], dst, parallelism=threads)
            return sum(l for _, l in spans)
        own = self._fd is None
        fd = os.open(self.info.file, os.O_RDONLY) if own else self._fd
        try:
            if spans is None:
                spans = [(0, self.info.byte_size())]
            for off, ln in spans:
                if off < 0 or off + ln > self.info.byte_size():
                    raise SafetensorsError(f"span [{off},{off + ln}) outside tensor {self.info.name}")
            return read_spans(fd, [(self.info.start + o, l) for o, l in spans], dst, threads)
        finally:
            if own:
                os.close(fd)

    def read_all(self) -> np.ndarray:
        buf = np.empty(self.info.byte_size(), dtype=np.uint8)
        self.read_into(buf)
        return buf


def bytes_to_torch(buf: np.ndarray, shape: Sequence[int], dtype: DataType) -> torch.Tensor:
    """Reinterprets raw little-endian bytes as a torch tensor of the storage dtype."""
    t = torch.from_numpy(buf)
    if dtype is DataType.f4e2m1 or dtype.bit_size_of() < 8:
        return t            # packed sub-byte data stays as bytes
    td = dtype.to_torch()
    return t.view(td).reshape(tuple(shape))


# ---------------------------------------------------------------------- writer
_TORCH_TO_ST = {torch.float64: "F64", torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
                torch.float8_e4m3fn: "F8_E4M3", torch.float8_e5m2: "F8_E5M2", torch.int64: "I64",
                torch.int32: "I32", torch.int16: "I16", torch.int8: "I8", torch.uint8: "U8",
                torch.uint16: "U16", torch.uint32: "U32", torch.uint64: "U64", torch.bool: "BOOL"}


def save_file(tensors: Mapping[str, torch.Tensor], path: str, metadata: Optional[Mapping[str, str]] = None,
              dtype_names: Optional[Mapping[str, str]] = None, shapes: Optional[Mapping[str, Sequence[int]]] = None) -> None:
    """Writes one .safetensors file.  `dtype_names` / `shapes` override the header entry of a
    tensor whose bytes are given as uint8 (e.g. packed F4_E2M1 with its logical shape)."""
    header, blobs, off = {}, [], 0
    for name in sorted(tensors):
        t = tensors[name].detach().contiguous().cpu()
        st = (dtype_names or {}).get(name) or _TORCH_TO_ST.get(t.dtype)
        if st is None:
            raise SafetensorsError(f"cannot store dtype {t.dtype}")
        raw = t.reshape(-1).view(torch.uint8).numpy() if t.dtype != torch.bool else t.to(torch.uint8).reshape(-1).numpy()
        shp = list((shapes or {}).get(name, t.shape))
        header[name] = {"dtype": st, "shape": [int(x) for x in shp], "data_offsets": [off, off + raw.nbytes]}
        blobs.append(raw)
        off += raw.nbytes
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b.tobytes())


def save_sharded(tensors: Mapping[str, torch.Tensor], repo: str, max_shard_bytes: int = 4 << 30,
                 metadata: Optional[Mapping[str, str]] = None) -> list[str]:
    """Writes `model-0000i-of-0000n.safetensors` shards plus `model.safetensors.index.json`
    (or a single model.safetensors when everything fits one shard)."""
    os.makedirs(repo, exist_ok=True)
    groups, cur, size = [], {}, 0
    for name in sorted(tensors):
        nb = tensors[name].numel() * tensors[name].element_size()
        if cur and size + nb > max_shard_bytes:
            groups.append(cur)
            cur, size = {}, 0
        cur[name] = tensors[name]
        size += nb
    if cur:
        groups.append(cur)
    if len(groups) == 1:
        p = os.path.join(repo, MODEL_NAME)
        save_file(groups[0], p, metadata)
        return [p]
    weight_map, files = {}, []
    for i, g in enumerate(groups):
        fname = f"model-{i + 1:05d}-of-{len(groups):05d}.safetensors"
        save_file(g, os.path.join(repo, fname), metadata)
        files.append(os.path.join(repo, fname))
        for k in g:
            weight_map[k] = fname
    total = sum(t.numel() * t.element_size() for t in tensors.values())
    with open(os.path.join(repo, INDEX_NAME), "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f)
    return files
