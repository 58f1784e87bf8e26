"""Trace post-processing: the native Perfetto (protobuf) writer against its own decoder."""
import json
import os


def test_perfetto_protobuf_writer_round_trip(tmp_path):
    from zml_b200.profiling import perfetto
    host = tmp_path / "h.json"
    host.write_text(json.dumps({"traceEvents": [
        {"ph": "M", "name": "thread_name", "pid": 1, "tid": 7, "args": {"name": "main"}},
        {"ph": "X", "name": "outer", "ts": 10.0, "dur": 100.0, "pid": 1, "tid": 7, "args": {"step": 3}},
        {"ph": "X", "name": "inner", "ts": 20.0, "dur": 30.0, "pid": 1, "tid": 7},
        {"ph": "i", "name": "mark", "ts": 60.0, "pid": 1, "tid": 7},
    ]}))
    out = tmp_path / "t.pftrace"
    assert perfetto.main([str(host), "-o", str(out)]) == 0
    recs = perfetto.read_perfetto(str(out))
    tracks = [r for r in recs if r.get("kind") == "track"]
    events = [r for r in recs if r.get("kind") == "event"]
    assert [t["name"] for t in tracks] == ["host spans", "main"] and tracks[1]["parent"] == tracks[0]["uuid"]
    assert [(e["type"], e.get("name"), e["ts_ns"]) for e in events] == [
        (1, "outer", 0), (1, "inner", 10_000), (2, None, 40_000), (3, "mark", 50_000), (2, None, 100_000)]
    assert events[0]["args"] == {"step": "3"} and all(e["track"] == tracks[1]["uuid"] for e in events)
    # varints longer than one byte survive (a timestamp of hours, in ns)
    n = perfetto.write_perfetto([{"ph": "X", "name": "late", "ts": 3.6e9, "dur": 1.0, "pid": 0, "tid": 0}], str(out))
    assert n == 4 and perfetto.read_perfetto(str(out))[2]["ts_ns"] == 3_600_000_000_000


def test_tracer_enabled_and_span_names():
    from zml_b200.profiling import tracer
    assert not tracer.enabled()
    tracer.start()
    try:
        assert tracer.enabled()
        with tracer.span("zml.exe.call", wait=True, arg_count=3):
            pass
        assert tracer.count() >= 1
    finally:
        tracer.stop()
    assert not tracer.enabled()
    assert tracer.format_span_name("zml.exe.call", wait=True, arg_count=3) == "zml.exe.call#wait=True,arg_count=3#"
    assert tracer.format_span_name("plain") == "plain"


def test_profiler_session_writes_host_trace_and_perfetto_file(tmp_path):
    from zml_b200.profiling import Profiler, perfetto, tracer
    with Profiler(logdir=str(tmp_path), device=False, session="s1") as prof:
        with tracer.span("step", n=1):
            with tracer.span("inner"):
                pass
    assert os.path.isfile(prof.host_trace) and prof.dir.endswith(os.path.join("plugins", "profile", "s1"))
    recs = perfetto.read_perfetto(prof.perfetto_trace)
    names = [r.get("name") for r in recs if r.get("kind") == "event" and r.get("type") == 1]
    assert any(n and n.startswith("step") for n in names) and "inner" in names


def test_trace_viewer_finds_the_session_and_serves_it_with_cors(tmp_path, capsys):
    import threading
    import urllib.request
    from zml_b200.profiling import Profiler, tracer, view
    for name in ("old", "new"):
        with Profiler(logdir=str(tmp_path), device=False, session=name):
            with tracer.span(f"work_{name}"):
                pass
        os.utime(os.path.join(str(tmp_path), "plugins", "profile", name), (1000 if name == "old" else 2000,) * 2)
    found = view.sessions(str(tmp_path))
    assert [os.path.basename(s) for s in found] == ["old", "new"]
    assert view.pick_trace(found[-1]).endswith("profiling.pftrace")
    assert view.main([str(tmp_path), "--no-serve"]) == 0
    out = capsys.readouterr().out
    assert "session new" in out and "work_new" in out and "work_old" not in out
    assert view.main([str(tmp_path), "--no-serve", "--session=old"]) == 0 and "work_old" in capsys.readouterr().out
    assert view.main([str(tmp_path / "nothing"), "--no-serve"]) == 1
    srv = view.make_server(found[-1], 0)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    try:
        with urllib.request.urlopen(f"http://127.0.0.1:{srv.server_address[1]}/profiling.pftrace") as r:
            assert r.headers["Access-Control-Allow-Origin"] == "https://ui.perfetto.dev" and len(r.read()) > 0
    finally:
        srv.shutdown()
        srv.server_close()
