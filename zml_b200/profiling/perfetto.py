"""Trace post-processing: merges the host-span trace and the device (CUPTI) trace of a
profiling session into one Chrome / Perfetto trace-event file, with one process lane per
source and a summary table of span and kernel times.

The reference ships tools/xspace_to_perfetto, which converts the XSpace protobuf written by
the PJRT profiler into trace-event JSON; here both inputs already are trace-event JSON, so the
tool's job is the merge, the time-base alignment and the summary.

    python -m zml_b200.profiling.perfetto <session dir or host.json> [device.json] -o merged.json
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
    info = merge_traces(host, dev, out)
    print(f"wrote {out}: {info}")
    for name, n, us in summarize(_events(out)):
        print(f"{us / 1e3:12.3f} ms  {n:8d}  {name}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
