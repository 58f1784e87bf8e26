#!/usr/bin/env python
"""zb-smi: device monitor in the spirit of the reference's zml-smi (NVIDIA only).

    zb-smi                      one-shot table
    zb-smi --top [--interval=1] [--page=overview|processes|charts]
                                terminal pages: bars per GPU, the process table, history charts
                                (keys 1 / 2 / 3 switch pages, s changes the process sort, q quits)
    zb-smi --csv | --json       one line per sample (streams with --interval)
    zb-smi --prometheus-listen=127.0.0.1:9400   serve /metrics, /json
    zb-smi --api [--api-port=9090]              the same agent on every interface (what --remotes reads)
    zb-smi --remotes=http://hostA:9090,http://hostB:9090   add the devices of other hosts' agents to every view
    zb-smi --fake               use the built-in fake NVML (no GPU needed)
Read-only: it never changes clocks, power limits or any other device setting.
"""
from __future__ import annotations

import os
import sys
import threading
import time
from dataclasses import dataclass
from typing import Optional

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import metrics  # noqa: E402
import outputs  # noqa: E402

from zml_b200 import flags  # noqa: E402


@dataclass
class Args:
    top: bool = False
    csv: bool = False
    json: bool = False
    fake: bool = False
    interval: float = 0.0
    count: int = 0
    prometheus_listen: Optional[str] = None
    page: str = "overview"
    api: bool = False
    api_port: int = 9090
    remotes: Optional[str] = None
    help = __doc__


class Collector:
    """Polls in a background thread and publishes the latest snapshot by swapping a reference
    (the double buffer of bin/zml-smi/collector/collector.zig)."""

    def __init__(self, backend, interval: float, remotes=None):
        self.backend, self.host, self.remotes = backend, metrics.HostPoller(), remotes
        self.interval = max(interval, 0.1)
        self.front = metrics.snapshot(backend, self.host, remotes)
        self._stop = threading.Event()
        self._t = threading.Thread(target=self._run, daemon=True)

    def start(self):
        self._t.start()
        return self

    def _run(self):
        while not self._stop.wait(self.interval):
            self.front = metrics.snapshot(self.backend, self.host, self.remotes)

    def latest(self) -> dict:
        return self.front

    def stop(self):
        self._stop.set()


def make_backend(fake: bool):
    if fake:
        return metrics.NvmlBackend(metrics.FakeNvml())
    try:
        return metrics.NvmlBackend()
    except Exception as e:
        print(f"zb-smi: NVML unavailable ({e}); host metrics only", file=sys.stderr)
        return None


def main(argv=None) -> int:
    args = flags.parse(argv, Args)
    backend = make_backend(args.fake)
    host = metrics.HostPoller()
    remotes = metrics.RemoteAgents([u for u in args.remotes.split(",") if u]) if args.remotes else None
    if args.prometheus_listen or args.api:
        if args.prometheus_listen:
            h, _, p = args.prometheus_listen.rpartition(":")
        else:
            h, p = "0.0.0.0", args.api_port
        coll = Collector(backend, args.interval or 1.0, remotes).start()
        srv = outputs.serve(coll.latest, h or "127.0.0.1", int(p))
        print(f"serving http://{srv.server_address[0]}:{srv.server_address[1]}/metrics", flush=True)
        try:
            n = 0
            while not args.count or n < args.count:
                time.sleep(args.interval or 1.0)
                n += 1
        except KeyboardInterrupt:
            pass
        srv.shutdown()
        coll.stop()
        return 0
    if args.top and not (args.csv or args.json):
        import tui
        tui.run(lambda: metrics.snapshot(backend, host, remotes), args.interval or 1.0, args.count, args.page)
        if backend:
            backend.close()
        return 0
    n = 0
    if args.csv:
        print(outputs.csv_header())
    while True:
        snap = metrics.snapshot(backend, host, remotes)
        if args.csv:
            print(outputs.to_csv(snap), flush=True)
        elif args.json:
            print(outputs.to_json(snap), flush=True)
        else:
            print(outputs.to_table(snap), flush=True)
        n += 1
        if not (args.top or args.interval > 0) or (args.count and n >= args.count):
            break
        try:
            time.sleep(args.interval or 1.0)
        except KeyboardInterrupt:
            break
    if backend:
        backend.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
