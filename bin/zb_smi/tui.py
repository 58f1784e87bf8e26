"""Terminal pages of `zb-smi --top` (the reference's bin/zml-smi/tui/*: overview, per-process table, history charts).

Pure rendering: `render(snap, history, page, width)` returns the text of a page, so the pages are testable without
a terminal; `run` is the interactive loop (keys: 1 overview, 2 processes, 3 charts, s change the process sort key,
q quit; without a TTY it just refreshes the chosen page).
"""
from __future__ import annotations

import collections
import select
import sys
import time
from typing import Optional

PAGES = ("overview", "processes", "charts")
SORT_KEYS = ("gpu_memory_bytes", "pid", "gpu")
_BLOCKS = " ▁▂▃▄▅▆▇█"


def bar(frac: Optional[float], width: int) -> str:
    if frac is None:
        return "-" * width
    n = max(0, min(width, int(round(frac * width))))
    return "█" * n + "░" * (width - n)


def sparkline(values, width: int, top: float) -> str:
    vals = list(values)[-width:]
    out = []
    for v in vals:
        if v is None or top <= 0:
            out.append(" ")
        else:
            out.append(_BLOCKS[max(0, min(8, int(round(v / top * 8))))])
    return "".join(out).rjust(width)


class History:
    """Last `depth` samples of utilisation, power, memory and SM clock per GPU."""

    def __init__(self, depth: int = 120):
        self.depth = depth
        self.series: dict = collections.defaultdict(lambda: collections.deque(maxlen=depth))

    def add(self, snap: dict) -> None:
        for g in snap["gpus"]:
            for key in ("util_percent", "power_w", "mem_used_bytes", "clock_sm_mhz"):
                self.series[(g["index"], key)].append(g.get(key))

    def get(self, index: int, key: str):
        return self.series[(index, key)]


def _header(snap: dict, page: str) -> str:
    h = snap["host"]
    tabs = "  ".join(f"[{i + 1}:{p}]" if p == page else f" {i + 1}:{p} " for i, p in enumerate(PAGES))
    mem = f"{(h.get('mem_used_bytes') or 0) / 2 ** 30:.0f}/{(h.get('mem_total_bytes') or 0) / 2 ** 30:.0f} GiB"
    return (f"zb-smi  {h['hostname']}  driver {h['driver_version']}  cuda {h['cuda_driver_version']}  "
            f"cpu {h['cpu_percent'] if h['cpu_percent'] is not None else '-'}%  mem {mem}  load {h.get('load1')}\n{tabs}")


def processes(snap: dict, sort_key: str = "gpu_memory_bytes") -> list[dict]:
    rows = []
    for g in snap["gpus"]:
        for p in g["processes"]:
            rows.append(dict(p, gpu=g["index"]))
    rev = sort_key == "gpu_memory_bytes"
    rows.sort(key=lambda r: (r.get(sort_key) or 0), reverse=rev)
    return rows


def render(snap: dict, history: Optional[History] = None, page: str = "overview", width: int = 100,
           sort_key: str = "gpu_memory_bytes") -> str:
    lines = [_header(snap, page), ""]
    bw = max(10, min(30, (width - 60) // 2))
    if page == "overview":
        lines.append(f"{'GPU':>3} {'name':<12} {'util':<{bw + 5}} {'memory':<{bw + 16}} {'power W':>11} {'temp':>5} {'sm MHz':>10}  reasons")
        for g in snap["gpus"]:
            util = g.get("util_percent")
            used, total = g.get("mem_used_bytes"), g.get("mem_total_bytes")
            mfrac = used / total if used is not None and total else None
            mem = f"{(used or 0) / 2 ** 30:6.1f}/{(total or 0) / 2 ** 30:6.1f}G"
            pw = f"{g['power_w']:.0f}/{g['power_limit_w']:.0f}" if g.get("power_w") is not None and g.get("power_limit_w") else "-"
            lines.append(f"{g['index']:>3} {g['name'].replace('NVIDIA ', '')[:12]:<12} {bar(None if util is None else util / 100, bw)} "
                         f"{'-' if util is None else util:>3}% {bar(mfrac, bw)} {mem:>14} {pw:>11} "
                         f"{'-' if g.get('temperature_c') is None else g['temperature_c']:>4}C "
                         f"{'-' if g.get('clock_sm_mhz') is None else g['clock_sm_mhz']:>5}/{g.get('clock_sm_max_mhz') or '-':<4}  "
                         f"{','.join(g['throttle_reasons'])}")
        procs = processes(snap, sort_key)
        lines.append("")
        lines.append(f"{len(procs)} compute process(es); press 2 for the table")
    elif page == "processes":
        lines.append(f"{'GPU':>3} {'pid':>8} {'user':<12} {'GPU memory':>12} {'sm %':>5}  command      (sorted by {sort_key}; s changes)")
        for p in processes(snap, sort_key):
            mem = "-" if p.get("gpu_memory_bytes") is None else f"{p['gpu_memory_bytes'] / 2 ** 20:.0f} MiB"
            sm = "-" if p.get("sm_util") is None else p["sm_util"]
            lines.append(f"{p['gpu']:>3} {p['pid']:>8} {p['user'][:12]:<12} {mem:>12} {sm:>5}  {p['name']}")
    elif page == "charts":
        cw = max(20, width - 40)
        for g in snap["gpus"]:
            lines.append(f"GPU {g['index']} {g['name']}")
            hist = history or History()
            for key, label, top in (("util_percent", "util %", 100.0), ("power_w", "power W", g.get("power_limit_w") or 1000.0),
                                    ("mem_used_bytes", "memory", float(g.get("mem_total_bytes") or 1)),
                                    ("clock_sm_mhz", "sm MHz", float(g.get("clock_sm_max_mhz") or 2000))):
                series = hist.get(g["index"], key)
                last = series[-1] if series else None
                shown = "-" if last is None else (f"{last / 2 ** 30:.1f}G" if key == "mem_used_bytes" else f"{last:.0f}")
                lines.append(f"  {label:<8} {sparkline(series, cw, top)} {shown:>8}")
    else:
        raise ValueError(f"unknown page {page!r}; one of {PAGES}")
    return "\n".join(lines)


def _read_key(timeout: float) -> Optional[str]:
    if not sys.stdin.isatty():
        time.sleep(timeout)
        return None
    r, _, _ = select.select([sys.stdin], [], [], timeout)
    return sys.stdin.read(1) if r else None


def run(get_snapshot, interval: float = 1.0, count: int = 0, page: str = "overview") -> None:
    """Interactive loop of `--top`."""
    import shutil
    hist = History()
    sort_i = 0
    restore = None
    if sys.stdin.isatty():
        try:
            import termios
            import tty
            restore = (termios, termios.tcgetattr(sys.stdin))
            tty.setcbreak(sys.stdin.fileno())
        except Exception:
            restore = None
    n = 0
    try:
        while True:
            snap = get_snapshot()
            hist.add(snap)
            width = shutil.get_terminal_size((100, 30)).columns
            sys.stdout.write("\x1b[2J\x1b[H" + render(snap, hist, page, width, SORT_KEYS[sort_i]) + "\n")
            sys.stdout.flush()
            n += 1
            if count and n >= count:
                break
            key = _read_key(interval)
            if key in ("q", "Q"):
                break
            if key in ("1", "2", "3"):
                page = PAGES[int(key) - 1]
            elif key == "s":
                sort_i = (sort_i + 1) % len(SORT_KEYS)
    except KeyboardInterrupt:
        pass
    finally:
        if restore is not None:
            restore[0].tcsetattr(sys.stdin, restore[0].TCSADRAIN, restore[1])
