"""Tracing and profiling (zml/profiling/*): host spans + device timelines.

`Profiler` is the session object behind `llm --profile` (examples/llm/chat.zig:74-93):
it records host spans with the native tracer and, on CUDA, device activity through
`torch.profiler` (CUPTI), and writes trace-event JSON files plus one merged native Perfetto trace
(`profiling.pftrace`) under `<logdir>/plugins/profile/<session>/`.  Setting SKIP_DEVICE_PROFILER=1 keeps only the host
spans, which is what an external profiler wrapper wants (the reference's SKIP_PJRT_PROFILER).
"""
from __future__ import annotations

import os
import time
from typing import Optional

from . import tracer
from .tracer import Span, span  # noqa: F401


class Profiler:
    def __init__(self, logdir: str = "/tmp/xprof", device: bool = True, session: Optional[str] = None):
        self.session = session or time.strftime("%Y_%m_%d_%H_%M_%S")
        self.dir = os.path.join(logdir, "plugins", "profile", self.session)
        self.device = device and os.environ.get("SKIP_DEVICE_PROFILER", os.environ.get("SKIP_PJRT_PROFILER", "")) in ("", "0", "false")
        self._tp = None
        self.host_trace = os.path.join(self.dir, "profiling.trace.json")
        self.device_trace = os.path.join(self.dir, "profiling.device.trace.json")

    def start(self) -> "Profiler":
        os.makedirs(self.dir, exist_ok=True)
        tracer.start()
        if self.device:
            try:
                import torch
                if torch.cuda.is_available():
                    from torch.profiler import ProfilerActivity, profile
                    self._tp = profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA])
                    self._tp.__enter__()
            except Exception:
                self._tp = None
        return self

    def stop(self) -> dict:
        out = {"host": self.host_trace}
        if self._tp is not None:
            self._tp.__exit__(None, None, None)
            self._tp.export_chrome_trace(self.device_trace)
            out["device"] = self.device_trace
            self._tp = None
        tracer.stop()
        tracer.write_json(self.host_trace)
        try:                                    # one file for ui.perfetto.dev: host spans and device activity merged
            from . import perfetto
            merged = os.path.join(self.dir, "profiling.merged.json")
            perfetto.merge_traces(self.host_trace, out.get("device"), merged)
            self.perfetto_trace = os.path.join(self.dir, "profiling.pftrace")
            perfetto.write_perfetto(perfetto._events(merged), self.perfetto_trace)
            os.remove(merged)
            out["perfetto"] = self.perfetto_trace
        except (OSError, ValueError, KeyError):
            pass
        return out

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        self.stop()
