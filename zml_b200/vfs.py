"""Virtual file system: open files by URI scheme (vfs/*.zig of the reference).

Schemes: plain paths and `file://`; `http(s)://` with ranged reads; `hf://org/repo[@rev]/path`
(Hugging Face hub, token from HF_TOKEN); `s3://bucket/key` and `gs://bucket/key` through
their public HTTPS endpoints (anonymous or pre-signed access).  Remote files are read with
parallel HTTP range requests (vfs/parallel_read.zig:55-211).  Every backend exposes the same
small interface: `stat`, `read_range`, `list`, `open` (a seekable file object).
"""
from __future__ import annotations

import concurrent.futures as cf
import io
import os
import sys
import urllib.error
import urllib.parse
import urllib.request
from dataclasses import dataclass
from typing import Optional


@dataclass
class Stat:
    size: int
    kind: str = "file"          # file | directory


class Backend:
    def stat(self, path: str) -> Stat:
        raise NotImplementedError

    def read_range(self, path: str, offset: int, length: int) -> bytes:
        raise NotImplementedError

    def list(self, path: str) -> list[str]:
        raise NotImplementedError("listing is not supported by this backend")

    def realpath(self, path: str) -> str:
        return path


class FileBackend(Backend):
    def stat(self, path):
        st = os.stat(path)
        return Stat(st.st_size, "directory" if os.path.isdir(path) else "file")

    def read_range(self, path, offset, length):
        with open(path, "rb") as f:
            f.seek(offset)
            return f.read(length)

    def list(self, path):
        return sorted(os.listdir(path))

    def realpath(self, path):
        return os.path.realpath(path)


class HttpBackend(Backend):
    def __init__(self, headers: Optional[dict] = None, timeout: float = 60.0):
        self.headers = headers or {}
        self.timeout = timeout

    def url(self, path: str) -> str:
        return path

    def _req(self, path: str, method: str = "GET", extra: Optional[dict] = None):
        h = dict(self.headers)
        h.update(extra or {})
        return urllib.request.urlopen(urllib.request.Request(self.url(path), method=method, headers=h), timeout=self.timeout)

    def stat(self, path):
        try:
            with self._req(path, "HEAD") as r:
                n = r.headers.get("Content-Length")
                if n is not None:
                    return Stat(int(n))
        except urllib.error.HTTPError:
            pass
        with self._req(path, "GET", {"Range": "bytes=0-0"}) as r:
            cr = r.headers.get("Content-Range", "")
            return Stat(int(cr.rsplit("/", 1)[1]) if "/" in cr else int(r.headers.get("Content-Length", 0)))

    def read_range(self, path, offset, length):
        if length <= 0:
            return b""
        with self._req(path, "GET", {"Range": f"bytes={offset}-{offset + length - 1}"}) as r:
            data = r.read()
        if len(data) > length:            # server ignored the range
            data = data[offset:offset + length]
        return data


def hf_token_path() -> str:
    home = os.environ.get("HF_HOME", os.path.join(os.path.expanduser("~"), ".cache", "huggingface"))
    return os.path.join(home, "token")


def hf_token() -> Optional[str]:
    """HF_TOKEN from the environment, else the token stored by `python -m zml_b200.vfs auth login`
    (the reference's `bazel run //tools/hf -- auth login`)."""
    tok = os.environ.get("HF_TOKEN")
    if tok:
        return tok.strip()
    try:
        with open(hf_token_path(), "r") as f:
            return f.read().strip() or None
    except OSError:
        return None


class HfBackend(HttpBackend):
    """hf://org/repo[@revision]/path/in/repo"""

    def __init__(self, endpoint: str = "https://huggingface.co"):
        tok = hf_token()
        super().__init__({"Authorization": f"Bearer {tok}"} if tok else {})
        self.endpoint = endpoint.rstrip("/")

    @staticmethod
    def split(path: str) -> tuple[str, str, str]:
        rest = path[len("hf://"):]
        parts = rest.split("/")
        if len(parts) < 2:
            raise ValueError(f"hf uri needs org/repo: {path}")
        repo, rev = parts[1], "main"
        if "@" in repo:
            repo, rev = repo.split("@", 1)
        return f"{parts[0]}/{repo}", rev, "/".join(parts[2:])

    def url(self, path):
        repo, rev, file = self.split(path)
        return f"{self.endpoint}/{repo}/resolve/{rev}/{file}"


class BucketBackend(HttpBackend):
    def __init__(self, template: str):
        super().__init__()
        self.template = template

    def url(self, path):
        u = urllib.parse.urlparse(path)
        return self.template.format(bucket=u.netloc, key=u.path.lstrip("/"))


class Vfs:
    """Scheme multiplexer (vfs/vfs.zig:49-90)."""

    def __init__(self):
        self.backends: dict[str, Backend] = {}
        self.register("file", FileBackend())

    def register(self, scheme: str, backend: Backend) -> None:
        self.backends[scheme] = backend

    @staticmethod
    def default() -> "Vfs":
        v = Vfs()
        v.register("http", HttpBackend())
        v.register("https", HttpBackend())
        v.register("hf", HfBackend())
        v.register("s3", BucketBackend("https://{bucket}.s3.amazonaws.com/{key}"))
        v.register("gs", BucketBackend("https://storage.googleapis.com/{bucket}/{key}"))
        return v

    def resolve(self, uri: str) -> tuple[Backend, str]:
        if "://" not in uri:
            return self.backends["file"], uri
        scheme = uri.split("://", 1)[0]
        if scheme not in self.backends:
            raise ValueError(f"no backend registered for scheme {scheme!r}")
        return self.backends[scheme], (uri[len("file://"):] if scheme == "file" else uri)

    def stat(self, uri: str) -> Stat:
        b, p = self.resolve(uri)
        return b.stat(p)

    def list(self, uri: str) -> list[str]:
        b, p = self.resolve(uri)
        return b.list(p)

    def realpath(self, uri: str) -> str:
        b, p = self.resolve(uri)
        return b.realpath(p)

    def read_range(self, uri: str, offset: int, length: int) -> bytes:
        b, p = self.resolve(uri)
        return b.read_range(p, offset, length)

    def read(self, uri: str, chunk: int = 8 << 20, parallelism: int = 8) -> bytes:
        """Whole file; remote files are fetched as parallel range requests."""
        b, p = self.resolve(uri)
        size = b.stat(p).size
        if isinstance(b, FileBackend) or size <= chunk:
            return b.read_range(p, 0, size)
        offs = list(range(0, size, chunk))
        with cf.ThreadPoolExecutor(max_workers=parallelism) as ex:
            parts = list(ex.map(lambda o: b.read_range(p, o, min(chunk, size - o)), offs))
        return b"".join(parts)

    def read_spans(self, uri: str, spans, dst=None, chunk: int = 8 << 20, parallelism: int = 8):
        """Byte ranges `spans` = [(offset, length), ...] of one file, back to back, as parallel range requests:
        neighbouring ranges are fetched as one request, long ones are cut into `chunk`-sized requests.  Writes into
        `dst` (a writable buffer of at least the total length) or returns the bytes.  This is what loads one rank's
        shard of a checkpoint tensor from a remote repository."""
        b, p = self.resolve(uri)
        total = sum(l for _, l in spans)
        out = memoryview(dst).cast("B") if dst is not None else memoryview(bytearray(total))
        if len(out) < total:
            raise ValueError("destination too small")
        reqs, pos = [], 0                    # (file offset, length, position in the output)
        for off, ln in spans:
            if reqs and reqs[-1][0] + reqs[-1][1] == off and reqs[-1][1] + ln <= chunk:
                reqs[-1] = (reqs[-1][0], reqs[-1][1] + ln, reqs[-1][2])
            else:
                done = 0
                while done < ln:
                    take = min(chunk, ln - done)
                    reqs.append((off + done, take, pos + done))
                    done += take
            pos += ln

        def fetch(r):
            data = b.read_range(p, r[0], r[1])
            if len(data) != r[1]:
                raise IOError(f"{uri}: short read at {r[0]}: {len(data)} of {r[1]} bytes")
            out[r[2]:r[2] + r[1]] = data

        if len(reqs) <= 1 or parallelism <= 1:
            for r in reqs:
                fetch(r)
        else:
            with cf.ThreadPoolExecutor(max_workers=parallelism) as ex:
                list(ex.map(fetch, reqs))
        return None if dst is not None else bytes(out)

    def open(self, uri: str) -> "VfsFile":
        return VfsFile(self, uri)

    def copy(self, src: str, dst: str, chunk: int = 8 << 20, parallelism: int = 8) -> int:
        """Streams `src` into the local file `dst`: `parallelism` range requests of `chunk` bytes in flight, written
        at their offsets (a large remote file never sits in memory as a whole)."""
        b, p = self.resolve(dst)
        if not isinstance(b, FileBackend):
            raise ValueError("copy destination must be a local path")
        sb, sp = self.resolve(src)
        size = sb.stat(sp).size
        with open(p, "wb") as f:
            f.truncate(size)
        fd = os.open(p, os.O_WRONLY)
        try:
            def piece(off):
                data = sb.read_range(sp, off, min(chunk, size - off))
                os.pwrite(fd, data, off)
                return len(data)
            offs = list(range(0, size, chunk))
            if len(offs) <= 1:
                n = sum(piece(o) for o in offs)
            else:
                with cf.ThreadPoolExecutor(max_workers=parallelism) as ex:
                    n = sum(ex.map(piece, offs))
        finally:
            os.close(fd)
        return n


class VfsFile(io.RawIOBase):
    """Seekable read-only file over any backend."""

    def __init__(self, vfs: Vfs, uri: str):
        self.vfs, self.uri = vfs, uri
        self.size = vfs.stat(uri).size
        self.pos = 0

    def readable(self):
        return True

    def seekable(self):
        return True

    def seek(self, off, whence=0):
        self.pos = off if whence == 0 else (self.pos + off if whence == 1 else self.size + off)
        return self.pos

    def tell(self):
        return self.pos

    def read(self, n=-1):
        n = self.size - self.pos if n is None or n < 0 else min(n, self.size - self.pos)
        data = self.vfs.read_range(self.uri, self.pos, n) if n > 0 else b""
        self.pos += len(data)
        return data


def _auth_main(argv) -> int:
    """`python -m zml_b200.vfs auth login [--token=...]` / `auth logout` / `auth whoami`."""
    import getpass
    if len(argv) < 2 or argv[0] != "auth" or argv[1] not in ("login", "logout", "whoami"):
        print(_auth_main.__doc__, file=sys.stderr)
        return 1
    path = hf_token_path()
    if argv[1] == "logout":
        if os.path.exists(path):
            os.remove(path)
        print("logged out")
        return 0
    if argv[1] == "whoami":
        tok = hf_token()
        print("token: " + (tok[:6] + "..." if tok else "none"))
        return 0
    tok = next((a.split("=", 1)[1] for a in argv[2:] if a.startswith("--token=")), None) or getpass.getpass("HF token: ")
    os.makedirs(os.path.dirname(path), exist_ok=True)
    with open(path, "w") as f:
        f.write(tok.strip())
    os.chmod(path, 0o600)
    print(f"token stored in {path}")
    return 0


if __name__ == "__main__":
    import sys
    sys.exit(_auth_main(sys.argv[1:]))
