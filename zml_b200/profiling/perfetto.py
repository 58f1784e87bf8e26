"""Trace post-processing: merges the host-span trace and the device (CUPTI) trace of a
profiling session into one Chrome / Perfetto trace-event file, with one process lane per
source and a summary table of span and kernel times.

The reference ships tools/xspace_to_perfetto, which converts the XSpace protobuf written by
the PJRT profiler into trace-event JSON; here both inputs already are trace-event JSON, so the
tool's job is the merge, the time-base alignment and the summary.

    python -m zml_b200.profiling.perfetto <session dir or host.json> [device.json] -o merged.json
    python -m zml_b200.profiling.perfetto <session dir or host.json> [device.json] -o merged.pftrace   # protobuf
"""
from __future__ import annotations

import json
import os
import sys
from collections import defaultdict
from typing import Iterable, Optional


def _events(path: str) -> list[dict]:
    with open(path, "r") as f:
        data = json.load(f)
    return data["traceEvents"] if isinstance(data, dict) else list(data)


def merge_traces(host_json: str, device_json: Optional[str], out_json: str) -> dict:
    """Writes the merged trace and returns {"events": n, "host_spans": n, "device_events": n}."""
    host = _events(host_json)
    dev = _events(device_json) if device_json and os.path.exists(device_json) else []
    merged = [{"ph": "M", "name": "process_name", "pid": 1, "args": {"name": "host spans"}}]
    ts = [e["ts"] for e in host if "ts" in e]
    t0_host = min(ts) if ts else 0
    for e in host:
        e = dict(e)
        e["pid"] = 1
        if "ts" in e:
            e["ts"] = e["ts"] - t0_host
        merged.append(e)
    ts = [e["ts"] for e in dev if "ts" in e and e.get("ph") in ("X", "B", "E", "i")]
    t0_dev = min(ts) if ts else 0
    pids = {}
    for e in dev:
        e = dict(e)
        pid = e.get("pid", 0)
        if pid not in pids:
            pids[pid] = 100 + len(pids)
        e["pid"] = pids[pid]
        if "ts" in e:
            e["ts"] = e["ts"] - t0_dev
        merged.append(e)
    for old, new in pids.items():
        merged.append({"ph": "M", "name": "process_name", "pid": new, "args": {"name": f"device trace ({old})"}})
    os.makedirs(os.path.dirname(os.path.abspath(out_json)), exist_ok=True)
    with open(out_json, "w") as f:
        json.dump({"traceEvents": merged, "displayTimeUnit": "ms"}, f)
    return {"events": len(merged), "host_spans": sum(1 for e in host if e.get("ph") in ("X", "B")),
            "device_events": len(dev)}


def summarize(events: Iterable[dict], top: int = 20) -> list[tuple[str, int, float]]:
    """(name, count, total microseconds) of complete events, largest first."""
    tot, cnt = defaultdict(float), defaultdict(int)
    open_b: dict = {}
    for e in events:
        ph = e.get("ph")
        if ph == "X":
            tot[e["name"]] += float(e.get("dur", 0))
            cnt[e["name"]] += 1
        elif ph == "B":
            open_b[(e.get("pid"), e.get("tid"), e["name"])] = e["ts"]
        elif ph == "E":
            k = (e.get("pid"), e.get("tid"), e.get("name"))
            if k in open_b:
                tot[k[2]] += e["ts"] - open_b.pop(k)
                cnt[k[2]] += 1
    rows = sorted(((n, cnt[n], tot[n]) for n in tot), key=lambda r: -r[2])
    return rows[:top]


# ---------------------------------------------------------------------- native Perfetto traces (protobuf)
# The reference's converter (tools/xspace_to_perfetto) writes Perfetto's own format; so does this writer, without a
# protobuf dependency: a `Trace` is a sequence of `TracePacket`s (field 1), each either a `TrackDescriptor` (60) that
# names a process / thread track, or a `TrackEvent` (11) slice begin / end / instant on a track at a timestamp (8, ns).
# Field numbers are those of perfetto/protos/perfetto/trace/{trace,trace_packet}.proto and track_event/*.proto.
def _varint(v: int) -> bytes:
    v &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        out.append(b | (0x80 if v else 0))
        if not v:
            return bytes(out)


def _f_varint(field: int, v: int) -> bytes:
    return _varint(field << 3) + _varint(v)


def _f_bytes(field: int, data: bytes) -> bytes:
    return _varint((field << 3) | 2) + _varint(len(data)) + data


def _f_str(field: int, s: str) -> bytes:
    return _f_bytes(field, s.encode("utf-8"))


_SEQ = 1
TYPE_SLICE_BEGIN, TYPE_SLICE_END, TYPE_INSTANT = 1, 2, 3


def _track_descriptor(uuid: int, name: str, pid: int, tid: Optional[int], parent: Optional[int]) -> bytes:
    body = _f_varint(1, uuid) + _f_str(2, name)
    if tid is None:
        body += _f_bytes(3, _f_varint(1, pid) + _f_str(6, name))                         # ProcessDescriptor
    else:
        body += _f_bytes(4, _f_varint(1, pid) + _f_varint(2, tid) + _f_str(5, name))     # ThreadDescriptor
    if parent is not None:
        body += _f_varint(5, parent)
    return _f_bytes(1, _f_bytes(60, body) + _f_varint(10, _SEQ))


def _track_event(ts_ns: int, kind: int, track: int, name: Optional[str], args: Optional[dict]) -> bytes:
    ev = _f_varint(9, kind) + _f_varint(11, track)
    if name is not None:
        ev += _f_str(23, name)
    for k, v in (args or {}).items():
        ev += _f_bytes(4, _f_str(10, str(k)) + _f_str(6, str(v)))                        # DebugAnnotation
    return _f_bytes(1, _f_varint(8, ts_ns) + _f_varint(10, _SEQ) + _f_bytes(11, ev))


def write_perfetto(events: Iterable[dict], out_path: str) -> int:
    """Trace-event dicts (`ph` X / B / E / i / M with `ts` / `dur` in microseconds, `pid`, `tid`, `name`, `args`) ->
    a native Perfetto trace file (`.perfetto-trace` / `.pftrace`, opens in ui.perfetto.dev).  Returns the packet count."""
    events = list(events)
    proc_names, thread_names = {}, {}
    for e in events:
        if e.get("ph") == "M":
            if e.get("name") == "process_name":
                proc_names[e.get("pid", 0)] = e.get("args", {}).get("name", "")
            elif e.get("name") == "thread_name":
                thread_names[(e.get("pid", 0), e.get("tid", 0))] = e.get("args", {}).get("name", "")
    out = bytearray()
    packets = 0
    tracks: dict = {}

    def track_of(pid: int, tid: int) -> int:
        nonlocal packets
        if ("p", pid) not in tracks:
            tracks[("p", pid)] = len(tracks) + 1
            out.extend(_track_descriptor(tracks[("p", pid)], proc_names.get(pid, f"process {pid}"), pid, None, None))
            packets += 1
        if (pid, tid) not in tracks:
            tracks[(pid, tid)] = len(tracks) + 1
            out.extend(_track_descriptor(tracks[(pid, tid)], thread_names.get((pid, tid), f"thread {tid}"), pid, tid, tracks[("p", pid)]))
            packets += 1
        return tracks[(pid, tid)]

    timed = []
    for e in events:
        ph = e.get("ph")
        if ph not in ("X", "B", "E", "i", "I"):
            continue
        tr = track_of(int(e.get("pid", 0)), int(e.get("tid", 0)))
        ts = int(round(float(e.get("ts", 0)) * 1000))
        if ph == "X":
            timed.append((ts, 0, TYPE_SLICE_BEGIN, tr, e.get("name", ""), e.get("args")))
            timed.append((ts + int(round(float(e.get("dur", 0)) * 1000)), -1, TYPE_SLICE_END, tr, None, None))
        elif ph == "B":
            timed.append((ts, 0, TYPE_SLICE_BEGIN, tr, e.get("name", ""), e.get("args")))
        elif ph == "E":
            timed.append((ts, -1, TYPE_SLICE_END, tr, None, None))
        else:
            timed.append((ts, 1, TYPE_INSTANT, tr, e.get("name", ""), e.get("args")))
    timed.sort(key=lambda t: (t[0], t[1]))          # ends before begins at equal times keep slices nested
    for ts, _, kind, tr, name, args in timed:
        out.extend(_track_event(ts, kind, tr, name, args))
        packets += 1
    os.makedirs(os.path.dirname(os.path.abspath(out_path)), exist_ok=True)
    with open(out_path, "wb") as f:
        f.write(bytes(out))
    return packets


def read_perfetto(path: str) -> list[dict]:
    """Decodes what `write_perfetto` writes (descriptors and track events) back into dicts: for tests and quick looks."""
    data = open(path, "rb").read()

    def fields(buf: bytes):
        i = 0
        while i < len(buf):
            key = 0
            shift = 0
            while True:
                b = buf[i]; i += 1
                key |= (b & 0x7F) << shift
                shift += 7
                if not b & 0x80:
                    break
            field, wt = key >> 3, key & 7
            if wt == 0:
                v, shift = 0, 0
                while True:
                    b = buf[i]; i += 1
                    v |= (b & 0x7F) << shift
                    shift += 7
                    if not b & 0x80:
                        break
                yield field, v
            elif wt == 2:
                n, shift = 0, 0
                while True:
                    b = buf[i]; i += 1
                    n |= (b & 0x7F) << shift
                    shift += 7
                    if not b & 0x80:
                        break
                yield field, buf[i:i + n]
                i += n
            else:
                raise ValueError(f"unexpected wire type {wt}")

    out = []
    for f, packet in fields(data):
        if f != 1:
            continue
        rec: dict = {}
        for pf, pv in fields(packet):
            if pf == 8:
                rec["ts_ns"] = pv
            elif pf == 60:
                d = dict(fields(pv))
                rec.update(kind="track", uuid=d.get(1), name=d.get(2, b"").decode(), parent=d.get(5),
                           is_thread=4 in d)
            elif pf == 11:
                ev: dict = {"args": {}}
                for ef, evv in fields(pv):
                    if ef == 9:
                        ev["type"] = evv
                    elif ef == 11:
                        ev["track"] = evv
                    elif ef == 23:
                        ev["name"] = evv.decode()
                    elif ef == 4:
                        a = dict(fields(evv))
                        ev["args"][a.get(10, b"").decode()] = a.get(6, b"").decode()
                rec.update(kind="event", **ev)
        out.append(rec)
    return out


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or "-o" not in argv:
        print(__doc__, file=sys.stderr)
        return 1
    out = argv[argv.index("-o") + 1]
    pos = [a for i, a in enumerate(argv) if a != "-o" and (i == 0 or argv[i - 1] != "-o")]
    if os.path.isdir(pos[0]):
        host, dev = os.path.join(pos[0], "profiling.trace.json"), os.path.join(pos[0], "profiling.device.trace.json")
    else:
        host, dev = pos[0], pos[1] if len(pos) > 1 else None
    if out.endswith(".json"):
        info = merge_traces(host, dev, out)
        events = _events(out)
    else:                                   # .pftrace / .perfetto-trace: Perfetto's own protobuf format
        tmp = out + ".merge.json"
        info = merge_traces(host, dev, tmp)
        events = _events(tmp)
        os.remove(tmp)
        info["packets"] = write_perfetto(events, out)
    print(f"wrote {out}: {info}")
    for name, n, us in summarize(events):
        print(f"{us / 1e3:12.3f} ms  {n:8d}  {name}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
