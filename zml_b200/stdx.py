"""Small general-purpose pieces the reference keeps in its `stdx` package (stdx/*.zig) and that the framework or its
users need in Python too: a task group with a concurrency limit, a lap timer, bounded containers, tagged-union JSON
records, and the slice formatter behind `Slice.pretty_print`.  (`stdx.flags` is `zml_b200.flags`.)
"""
from __future__ import annotations

import dataclasses
import threading
import time
from concurrent.futures import Future, ThreadPoolExecutor
from typing import Any, Callable, Generic, Iterator, Mapping, Optional, Sequence, TypeVar

T = TypeVar("T")


# ---------------------------------------------------------------------------- concurrency
class LimitedGroup:
    """Tasks submitted with `spawn` run on worker threads, at most `limit` at a time; `wait` joins them and re-raises
    the first failure; `cancel` drops what has not started (stdx/Io.zig:25-81)."""

    def __init__(self, limit: int):
        if limit < 1:
            raise ValueError("limit must be at least 1")
        self.limit = limit
        self._pool = ThreadPoolExecutor(max_workers=limit, thread_name_prefix="zb-group")
        self._futures: list[Future] = []
        self._lock = threading.Lock()
        self._in_flight = 0
        self.max_in_flight = 0

    def _run(self, fn, args, kwargs):
        with self._lock:
            self._in_flight += 1
            self.max_in_flight = max(self.max_in_flight, self._in_flight)
        try:
            return fn(*args, **kwargs)
        finally:
            with self._lock:
                self._in_flight -= 1

    def spawn(self, fn: Callable, *args, **kwargs) -> Future:
        f = self._pool.submit(self._run, fn, args, kwargs)
        self._futures.append(f)
        return f

    concurrent = spawn

    def wait(self) -> list:
        """Results in submission order; the first exception (in submission order) is raised after all tasks ended."""
        futures, self._futures = self._futures, []
        results, first_error = [], None
        for f in futures:
            try:
                results.append(f.result() if not f.cancelled() else None)
            except BaseException as e:           # noqa: BLE001 - re-raised below
                results.append(None)
                first_error = first_error or e
        if first_error is not None:
            raise first_error
        return results

    def cancel(self) -> int:
        """Cancels the tasks that have not started; returns how many."""
        return sum(1 for f in self._futures if f.cancel())

    def close(self) -> None:
        self._pool.shutdown(wait=True, cancel_futures=True)

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc, tb):
        try:
            if exc_type is None:
                self.wait()
        finally:
            self.close()
        return False


# ---------------------------------------------------------------------------- time
@dataclasses.dataclass(frozen=True)
class Duration:
    """Nanoseconds with the helpers of stdx/time.zig: `div`, `hz` (events per second for one event per duration)."""
    ns: int

    def div(self, n: int) -> "Duration":
        return Duration(self.ns // max(int(n), 1))

    def hz(self) -> int:
        return 0 if self.ns == 0 else int(1_000_000_000 // self.ns)

    def hz_float(self) -> float:
        return 0.0 if self.ns == 0 else 1e9 / self.ns

    def seconds(self) -> float:
        return self.ns / 1e9

    def __str__(self) -> str:
        ns = self.ns
        for unit, scale in (("s", 1_000_000_000), ("ms", 1_000_000), ("us", 1_000)):
            if ns >= scale:
                return f"{ns / scale:.3f}{unit}"
        return f"{ns}ns"


class Timer:
    """`lap()` returns the time since the last lap (or start) and restarts; `read()` only looks (stdx/time.zig:25-43)."""

    def __init__(self, clock: Callable[[], int] = time.perf_counter_ns):
        self._clock = clock
        self._t0 = clock()

    @staticmethod
    def start() -> "Timer":
        return Timer()

    def read(self) -> Duration:
        return Duration(self._clock() - self._t0)

    def lap(self) -> Duration:
        now = self._clock()
        d, self._t0 = Duration(now - self._t0), now
        return d

    def reset(self) -> None:
        self._t0 = self._clock()


# ---------------------------------------------------------------------------- containers
class BoundedArray(Generic[T]):
    """A list that never grows past `capacity`: appending to a full one raises `OverflowError`
    (stdx/bounded_array.zig)."""

    def __init__(self, capacity: int, items: Sequence[T] = ()):
        self.capacity = capacity
        self._items: list[T] = []
        self.append_slice(items)

    def append(self, v: T) -> None:
        if len(self._items) >= self.capacity:
            raise OverflowError(f"BoundedArray of capacity {self.capacity} is full")
        self._items.append(v)

    def append_slice(self, vs: Sequence[T]) -> None:
        if len(self._items) + len(vs) > self.capacity:
            raise OverflowError(f"BoundedArray of capacity {self.capacity} cannot take {len(vs)} more items")
        self._items.extend(vs)

    def pop(self) -> T:
        return self._items.pop()

    def const_slice(self) -> tuple:
        return tuple(self._items)

    def resize(self, n: int, fill: Optional[T] = None) -> None:
        if n > self.capacity:
            raise OverflowError(f"BoundedArray of capacity {self.capacity} cannot hold {n} items")
        self._items = self._items[:n] + [fill] * max(0, n - len(self._items))

    def __len__(self) -> int:
        return len(self._items)

    def __getitem__(self, i):
        return self._items[i]

    def __setitem__(self, i, v) -> None:
        self._items[i] = v

    def __iter__(self) -> Iterator[T]:
        return iter(self._items)

    def __eq__(self, other) -> bool:
        return list(self) == list(other)

    def __repr__(self) -> str:
        return f"BoundedArray({self._items}, capacity={self.capacity})"


class SegmentedList(Generic[T]):
    """Append-only list stored in segments that double in size, so growing never moves an element and a reference
    to a slot (segment, offset) stays valid (stdx/segmented_list.zig)."""

    def __init__(self, first_segment: int = 16):
        self._first = first_segment
        self._segments: list[list] = []
        self._len = 0

    def _locate(self, i: int) -> tuple[int, int]:
        seg, size, base = 0, self._first, 0
        while i >= base + size:
            base += size
            size *= 2
            seg += 1
        return seg, i - base

    def append(self, v: T) -> tuple[int, int]:
        seg, off = self._locate(self._len)
        if seg == len(self._segments):
            self._segments.append([None] * (self._first << seg))
        self._segments[seg][off] = v
        self._len += 1
        return seg, off

    def at(self, i: int) -> T:
        if not 0 <= i < self._len:
            raise IndexError(i)
        seg, off = self._locate(i)
        return self._segments[seg][off]

    __getitem__ = at

    def set(self, i: int, v: T) -> None:
        if not 0 <= i < self._len:
            raise IndexError(i)
        seg, off = self._locate(i)
        self._segments[seg][off] = v

    def __len__(self) -> int:
        return self._len

    def __iter__(self) -> Iterator[T]:
        for i in range(self._len):
            yield self.at(i)

    def segment_count(self) -> int:
        return len(self._segments)


class ArrayQueue(Generic[T]):
    """Fixed-size FIFO ring: `push` on a full queue raises `OverflowError`, `pop` on an empty one returns None
    (stdx/queue.zig:235-300)."""

    def __init__(self, size: int):
        self._buf: list = [None] * size
        self._head = 0
        self._len = 0

    def __len__(self) -> int:
        return self._len

    def available(self) -> int:
        return len(self._buf) - self._len

    def push(self, v: T) -> None:
        if self._len == len(self._buf):
            raise OverflowError("ArrayQueue is full")
        self._buf[(self._head + self._len) % len(self._buf)] = v
        self._len += 1

    def pop(self) -> Optional[T]:
        if self._len == 0:
            return None
        v, self._buf[self._head] = self._buf[self._head], None
        self._head = (self._head + 1) % len(self._buf)
        self._len -= 1
        return v


# ---------------------------------------------------------------------------- json
def tagged_union(variants: Mapping[str, type], tag_name: str = "type"):
    """Parser / writer pair for JSON objects whose `tag_name` field selects the dataclass the other fields fill, e.g.
    tokenizer pipeline steps {"type": "Replace", "pattern": ..., "content": ...} (stdx/json.zig:102-163).
    Returns (parse, dump): parse(dict) -> instance of the selected dataclass; dump(instance) -> dict with the tag."""
    by_type = {cls: name for name, cls in variants.items()}

    def parse(obj: Mapping[str, Any]):
        if not isinstance(obj, Mapping):
            raise ValueError(f"expected an object, got {type(obj).__name__}")
        if tag_name not in obj:
            raise KeyError(f"missing field {tag_name!r}")
        tag = obj[tag_name]
        if not isinstance(tag, str):
            raise ValueError(f"field {tag_name!r} must be a string")
        cls = variants.get(tag)
        if cls is None:
            raise ValueError(f"unknown {tag_name} {tag!r}; known: {sorted(variants)}")
        names = {f.name for f in dataclasses.fields(cls)}
        unknown = [k for k in obj if k != tag_name and k not in names]
        if unknown:
            raise ValueError(f"{tag}: unknown fields {unknown}")
        return cls(**{k: v for k, v in obj.items() if k != tag_name})

    def dump(value) -> dict:
        name = by_type.get(type(value))
        if name is None:
            raise ValueError(f"{type(value).__name__} is not a variant of this union")
        return {tag_name: name, **dataclasses.asdict(value)}

    return parse, dump


def fill_default_struct_values(cls: type, values: Mapping[str, Any]):
    """Builds the dataclass `cls` from `values`, leaving fields that are absent or null at their defaults
    (`NeverNull` / `fillDefaultStructValues`, stdx/json.zig:166-200); unknown keys are ignored, as for the HF
    `config.json` files this is used on."""
    kwargs = {}
    for f in dataclasses.fields(cls):
        v = values.get(f.name)
        if v is not None:
            kwargs[f.name] = v
        elif f.default is dataclasses.MISSING and f.default_factory is dataclasses.MISSING:
            raise KeyError(f"{cls.__name__}: required field {f.name!r} is missing")
    return cls(**kwargs)


# ---------------------------------------------------------------------------- formatting
def format_slice(values, fmt: Callable[[Any], str] = str, num_cols: int = 12, stride: int = 1) -> str:
    """`{a,b,c}` for up to `num_cols` items, else the first and last num_cols / 2 around ` ..., `
    (stdx/fmt.zig:81-110)."""
    vals = list(values)[::stride]
    n = len(vals)
    if n <= num_cols:
        return "{" + ",".join(fmt(v) for v in vals) + "}"
    half = num_cols // 2
    return "{" + "".join(fmt(v) + "," for v in vals[:half]) + " ..., " + ",".join(fmt(v) for v in vals[n - half:]) + "}"
