"""Host trace spans (zml/profiling/tracer.zig).

`span(name)` opens a span recorded by the native tracer of libzb_host.so (ring buffer +
NVTX push/pop when libnvToolsExt is present); names may carry metadata in the reference's
`name#k=v,k=v#` encoding, which ends up in the event's args.  `encode` builds such names.
"""
from __future__ import annotations

import contextlib
import ctypes as C
import time

_lib = None
_fallback_events: list = []
_fallback_on = False


def _load():
    global _lib
    if _lib is None:
        try:
            from .. import _build
            p = _build.OUT / "libzb_host.so"
            if not p.exists():
                _build.build_host()
            l = C.CDLL(str(p))
            l.zbh_trace_begin.restype = C.c_ulonglong
            l.zbh_trace_begin.argtypes = [C.c_char_p]
            l.zbh_trace_end.argtypes = [C.c_ulonglong]
            l.zbh_trace_instant.argtypes = [C.c_char_p]
            l.zbh_trace_start.argtypes = [C.c_size_t]
            l.zbh_trace_count.restype = C.c_longlong
            l.zbh_trace_write_json.argtypes = [C.c_char_p]
            _lib = l
        except Exception:
            _lib = False
    return _lib or None


def encode(name: str, **metadata) -> str:
    """`name#k=v,k2=v2#` (tracer.zig:41-102)."""
    if not metadata:
        return name
    return name + "#" + ",".join(f"{k}={v}" for k, v in metadata.items()) + "#"


format_span_name = encode           # the reference's name for it (zml/profiling/tracer.zig:63)

_recording = False


def enabled() -> bool:
    """True while a recording session is open (zml/profiling/tracer.zig:35): callers use it to skip building span
    metadata that nobody would record."""
    return _recording


def start(capacity: int = 1 << 20) -> None:
    global _fallback_on, _recording
    _recording = True
    l = _load()
    if l:
        l.zbh_trace_start(capacity)
    else:
        _fallback_on = True
        _fallback_events.clear()


def stop() -> None:
    global _fallback_on, _recording
    _recording = False
    l = _load()
    if l:
        l.zbh_trace_stop()
    _fallback_on = False


def count() -> int:
    l = _load()
    return int(l.zbh_trace_count()) if l else len(_fallback_events)


def write_json(path: str) -> None:
    l = _load()
    if l:
        if l.zbh_trace_write_json(path.encode()) != 0:
            raise OSError(f"cannot write {path}")
        return
    import json
    with open(path, "w") as f:
        json.dump({"traceEvents": _fallback_events}, f)


class Span:
    __slots__ = ("name", "_id", "_t0")

    def __init__(self, name: str):
        self.name = name
        self._id = 0
        self._t0 = 0.0

    @staticmethod
    def start(name: str) -> "Span":
        s = Span(name)
        l = _load()
        if l:
            s._id = l.zbh_trace_begin(name.encode())
        else:
            s._t0 = time.perf_counter()
        return s

    def end(self) -> None:
        l = _load()
        if l:
            l.zbh_trace_end(self._id)
        elif _fallback_on:
            _fallback_events.append({"name": self.name, "ph": "X", "ts": self._t0 * 1e6,
                                     "dur": (time.perf_counter() - self._t0) * 1e6, "pid": 0, "tid": 0})


@contextlib.contextmanager
def span(name: str, **metadata):
    s = Span.start(encode(name, **metadata) if metadata else name)
    try:
        yield s
    finally:
        s.end()


def instant(name: str) -> None:
    l = _load()
    if l:
        l.zbh_trace_instant(name.encode())
