"""General-purpose helpers (stdx/*.zig counterparts): task group with a limit, timer, bounded containers, tagged-union
JSON records, slice formatting."""
import dataclasses
import threading
import time

import pytest

from zml_b200 import stdx


def test_limited_group_bounds_concurrency_and_reports_failures():
    gate = threading.Event()
    running, peak, lock = [0], [0], threading.Lock()

    def task(i):
        with lock:
            running[0] += 1
            peak[0] = max(peak[0], running[0])
        time.sleep(0.01)
        with lock:
            running[0] -= 1
        return i * i

    with stdx.LimitedGroup(3) as g:
        for i in range(12):
            g.spawn(task, i)
        assert g.wait() == [i * i for i in range(12)]
        assert peak[0] <= 3 and g.max_in_flight <= 3

    g = stdx.LimitedGroup(1)
    g.spawn(gate.wait, 5)
    for i in range(4):
        g.spawn(task, i)
    assert g.cancel() == 4                      # the worker is busy with the first task: the rest never start
    gate.set()
    assert g.wait()[0] is True
    g.spawn(lambda: 1 / 0)
    g.spawn(task, 2)
    with pytest.raises(ZeroDivisionError):
        g.wait()
    g.close()
    with pytest.raises(ValueError):
        stdx.LimitedGroup(0)


def test_timer_and_duration():
    ticks = iter([0, 1_500_000, 4_000_000, 4_000_000, 9_000_000])
    t = stdx.Timer(clock=lambda: next(ticks))
    assert t.lap() == stdx.Duration(1_500_000) and t.read() == stdx.Duration(2_500_000)
    t.reset()
    assert t.lap().ns == 5_000_000
    d = stdx.Duration(2_000_000)
    assert d.hz() == 500 and d.div(4).ns == 500_000 and abs(d.hz_float() - 500.0) < 1e-9 and str(d) == "2.000ms"
    assert stdx.Duration(0).hz() == 0 and str(stdx.Duration(12)) == "12ns" and str(stdx.Duration(3_210_000_000)) == "3.210s"


def test_bounded_containers():
    a = stdx.BoundedArray(4, [1, 2])
    a.append(3)
    a.append_slice([4])
    assert len(a) == 4 and a.const_slice() == (1, 2, 3, 4) and a == [1, 2, 3, 4]
    with pytest.raises(OverflowError):
        a.append(5)
    assert a.pop() == 4
    a.resize(2)
    assert list(a) == [1, 2]
    with pytest.raises(OverflowError):
        a.resize(5)

    s = stdx.SegmentedList(first_segment=2)
    slots = [s.append(i * 10) for i in range(15)]
    assert len(s) == 15 and list(s) == [i * 10 for i in range(15)] and s.segment_count() == 4      # 2 + 4 + 8 + 16
    assert slots[0] == (0, 0) and slots[2] == (1, 0) and slots[6] == (2, 0) and slots[14] == (3, 0)
    s.set(7, -1)
    assert s[7] == -1
    with pytest.raises(IndexError):
        s.at(15)

    q = stdx.ArrayQueue(3)
    for v in "abc":
        q.push(v)
    with pytest.raises(OverflowError):
        q.push("d")
    assert q.pop() == "a" and q.available() == 1
    q.push("d")
    assert [q.pop() for _ in range(4)] == ["b", "c", "d", None] and len(q) == 0


def test_tagged_union_and_struct_defaults():
    @dataclasses.dataclass
    class Replace:
        pattern: str
        content: str = ""

    @dataclasses.dataclass
    class Lowercase:
        pass

    parse, dump = stdx.tagged_union({"Replace": Replace, "Lowercase": Lowercase})
    r = parse({"type": "Replace", "pattern": " ", "content": "_"})
    assert r == Replace(" ", "_") and dump(r) == {"type": "Replace", "pattern": " ", "content": "_"}
    assert parse({"type": "Lowercase"}) == Lowercase() and dump(Lowercase()) == {"type": "Lowercase"}
    with pytest.raises(KeyError):
        parse({"pattern": "x"})
    with pytest.raises(ValueError):
        parse({"type": "Strip"})
    with pytest.raises(ValueError):
        parse({"type": "Replace", "pattern": "x", "extra": 1})
    with pytest.raises(ValueError):
        dump(3)

    @dataclasses.dataclass
    class Config:
        hidden_size: int
        rms_norm_eps: float = 1e-5
        tie_word_embeddings: bool = False

    c = stdx.fill_default_struct_values(Config, {"hidden_size": 64, "rms_norm_eps": None, "unknown": 1})
    assert c == Config(64, 1e-5, False)
    with pytest.raises(KeyError):
        stdx.fill_default_struct_values(Config, {})


def test_format_slice():
    assert stdx.format_slice([1, 2, 3]) == "{1,2,3}"
    assert stdx.format_slice(range(20), num_cols=4) == "{0,1, ..., 18,19}"
    assert stdx.format_slice(range(10), stride=5) == "{0,5}"
    assert stdx.format_slice([0.5, 0.25], fmt=lambda v: f"{v:.1f}") == "{0.5,0.2}"
    assert stdx.format_slice([]) == "{}"
