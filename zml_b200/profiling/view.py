"""Trace viewer launcher (the reference starts the xprof UI on a log directory, tools/xprof/main.py): finds the newest
profiling session under a log directory, prints a summary of its spans and kernels, and serves its trace files on
127.0.0.1 with the CORS header ui.perfetto.dev asks for, so that the printed link opens the trace in the browser.

    python -m zml_b200.profiling.view [logdir=/tmp/xprof] [--port=9001] [--session=<name>] [--no-serve]
"""
from __future__ import annotations

import http.server
import json
import os
import sys
from dataclasses import dataclass
from typing import Optional

from .. import flags
from . import perfetto


@dataclass
class Positional:
    logdir: str = "/tmp/xprof"


@dataclass
class Args:
    positional: Positional
    port: int = 9001
    session: Optional[str] = None
    no_serve: bool = False
    help = __doc__


def sessions(logdir: str) -> list[str]:
    """Session directories under `<logdir>/plugins/profile`, oldest first."""
    root = os.path.join(logdir, "plugins", "profile")
    if not os.path.isdir(root):
        return []
    names = [n for n in os.listdir(root) if os.path.isdir(os.path.join(root, n))]
    return [os.path.join(root, n) for n in sorted(names, key=lambda n: os.path.getmtime(os.path.join(root, n)))]


def pick_trace(session_dir: str) -> Optional[str]:
    for name in ("profiling.pftrace", "profiling.device.trace.json", "profiling.trace.json"):
        p = os.path.join(session_dir, name)
        if os.path.isfile(p):
            return p
    return None


def summary(session_dir: str, top: int = 15) -> list[tuple[str, int, float]]:
    events = []
    for name in ("profiling.trace.json", "profiling.device.trace.json"):
        p = os.path.join(session_dir, name)
        if os.path.isfile(p):
            with open(p) as f:
                data = json.load(f)
            events += data["traceEvents"] if isinstance(data, dict) else data
    return perfetto.summarize(events, top)


def make_server(directory: str, port: int) -> http.server.ThreadingHTTPServer:
    class Handler(http.server.SimpleHTTPRequestHandler):
        def __init__(self, *a, **kw):
            super().__init__(*a, directory=directory, **kw)

        def end_headers(self):
            self.send_header("Access-Control-Allow-Origin", "https://ui.perfetto.dev")
            self.send_header("Cache-Control", "no-cache")
            super().end_headers()

        def log_message(self, *a):
            pass
    return http.server.ThreadingHTTPServer(("127.0.0.1", port), Handler)


def main(argv=None) -> int:
    args = flags.parse(argv, Args)
    found = sessions(args.positional.logdir)
    if args.session:
        found = [s for s in found if os.path.basename(s) == args.session]
    if not found:
        print(f"no profiling session under {args.positional.logdir}/plugins/profile", file=sys.stderr)
        return 1
    session = found[-1]
    trace = pick_trace(session)
    print(f"session {os.path.basename(session)} ({session})")
    for name, n, us in summary(session):
        print(f"{us / 1e3:12.3f} ms  {n:8d}  {name}")
    if trace is None:
        print("no trace file in the session", file=sys.stderr)
        return 1
    if args.no_serve:
        print(f"trace: {trace}")
        return 0
    srv = make_server(session, args.port)
    url = f"http://127.0.0.1:{srv.server_address[1]}/{os.path.basename(trace)}"
    print(f"serving {trace}\nopen https://ui.perfetto.dev/#!/?url={url}   (Ctrl-C to stop)", flush=True)
    try:
        srv.serve_forever()
    except KeyboardInterrupt:
        pass
    srv.server_close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
