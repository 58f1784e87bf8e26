"""Output formats of zb-smi: one-shot table, CSV, JSON, Prometheus exposition, HTTP endpoints
(bin/zml-smi/{csv,json,prometheus,api}/*)."""
from __future__ import annotations

import http.server
import json
import threading
from typing import Callable

GPU_GAUGES = [("util_percent", "zml_device_utilization_percent"), ("power_w", "zml_device_power_watts"),
              ("power_limit_w", "zml_device_power_limit_watts"), ("temperature_c", "zml_device_temperature_celsius"),
              ("clock_sm_mhz", "zml_device_clock_sm_mhz"), ("clock_mem_mhz", "zml_device_clock_mem_mhz"),
              ("clock_sm_max_mhz", "zml_device_clock_sm_max_mhz"), ("mem_used_bytes", "zml_device_memory_used_bytes"),
              ("mem_total_bytes", "zml_device_memory_total_bytes"), ("pcie_tx_kbs", "zml_device_pcie_tx_kilobytes_per_second"),
              ("pcie_rx_kbs", "zml_device_pcie_rx_kilobytes_per_second"), ("fan_percent", "zml_device_fan_percent")]
HOST_GAUGES = [("cpu_percent", "zml_host_cpu_percent"), ("mem_used_bytes", "zml_host_memory_used_bytes"),
               ("mem_total_bytes", "zml_host_memory_total_bytes"), ("load1", "zml_host_load1")]
CSV_FIELDS = ["index", "name", "util_percent", "power_w", "power_limit_w", "temperature_c", "clock_sm_mhz",
              "clock_sm_max_mhz", "clock_mem_mhz", "mem_used_bytes", "mem_total_bytes", "pcie_gen", "pcie_width",
              "throttle_reasons"]


def to_json(snap: dict) -> str:
    return json.dumps(snap)


def csv_header() -> str:
    return "timestamp," + ",".join(CSV_FIELDS)


def to_csv(snap: dict) -> str:
    lines = []
    for g in snap["gpus"]:
        vals = []
        for f in CSV_FIELDS:
            v = g.get(f)
            vals.append("|".join(v) if isinstance(v, list) else ("" if v is None else str(v)))
        lines.append(f"{snap['timestamp']:.3f}," + ",".join(vals))
    return "\n".join(lines)


def to_prometheus(snap: dict) -> str:
    out = []
    for field, metric in GPU_GAUGES:
        rows = [(g, g.get(field)) for g in snap["gpus"] if g.get(field) is not None]
        if not rows:
            continue
        out.append(f"# TYPE {metric} gauge")
        for g, v in rows:
            where = f',host="{g["remote"]}"' if g.get("remote") else ""
            out.append(f'{metric}{{device="{g["index"]}",name="{g["name"]}"{where}}} {v}')
    host = snap["host"]
    for field, metric in HOST_GAUGES:
        if host.get(field) is not None:
            out.append(f"# TYPE {metric} gauge")
            out.append(f'{metric}{{host="{host["hostname"]}"}} {host[field]}')
    return "\n".join(out) + "\n"


def to_table(snap: dict) -> str:
    h = snap["host"]
    lines = [f"zb-smi  host {h['hostname']}  driver {h['driver_version']}  cuda {h['cuda_driver_version']}  "
             f"cpu {h['cpu_percent'] if h['cpu_percent'] is not None else '-'}%"]
    lines.append(f"{'GPU':>3} {'name':<14} {'util':>5} {'power':>12} {'temp':>5} {'sm MHz':>11} {'memory GiB':>15}  reasons")
    for g in snap["gpus"]:
        gi = lambda k, d="-": d if g.get(k) is None else g[k]
        mem = f"{(g['mem_used_bytes'] or 0) / 2 ** 30:6.1f}/{(g['mem_total_bytes'] or 0) / 2 ** 30:6.1f}"
        lines.append(f"{g['index']:>3} {g['name'][:14]:<14} {gi('util_percent'):>4}% {gi('power_w'):>5}/{gi('power_limit_w'):<5}W "
                     f"{gi('temperature_c'):>4}C {gi('clock_sm_mhz'):>5}/{gi('clock_sm_max_mhz'):<5} {mem:>15}  "
                     f"{','.join(g['throttle_reasons'])}"
                     + (f"  @{g['remote']}#{g.get('remote_index')}{' (stale)' if g.get('stale') else ''}" if g.get("remote") else ""))
        for p in g["processes"]:
            lines.append(f"      pid {p['pid']} {p['name']} {p['user']} {(p['gpu_memory_bytes'] or 0) / 2 ** 20:.0f} MiB")
    for url, err in snap.get("remote_errors", {}).items():
        lines.append(f"remote {url}: {err}")
    return "\n".join(lines)


def serve(get_snapshot: Callable[[], dict], host: str, port: int) -> http.server.ThreadingHTTPServer:
    """HTTP agent: /metrics (Prometheus text), /json, / (table)."""
    class H(http.server.BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def do_GET(self):
            snap = get_snapshot()
            if self.path.startswith("/metrics"):
                body, ctype = to_prometheus(snap), "text/plain; version=0.0.4"
            elif self.path.startswith("/json"):
                body, ctype = to_json(snap), "application/json"
            else:
                body, ctype = to_table(snap) + "\n", "text/plain"
            data = body.encode()
            self.send_response(200)
            self.send_header("Content-Type", ctype)
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)
    srv = http.server.ThreadingHTTPServer((host, port), H)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    return srv
