"""zb-smi against the fake NVML: formats, HTTP endpoints, and that no setter is ever called."""
import json
import os
import subprocess
import sys
import urllib.request

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "bin", "zb_smi"))

import metrics  # noqa: E402
import outputs  # noqa: E402


def test_snapshot_and_formats():
    fake = metrics.FakeNvml(devices=2)
    be = metrics.NvmlBackend(fake)
    snap = metrics.snapshot(be, metrics.HostPoller())
    assert len(snap["gpus"]) == 2 and snap["gpus"][1]["util_percent"] == 91
    g = snap["gpus"][0]
    assert g["fan_percent"] is None and g["power_w"] == 950.0 and g["throttle_reasons"] == ["sw_power_cap"]
    assert g["processes"][0]["pid"] == os.getpid() and snap["host"]["driver_version"] == "580.159"
    prom = outputs.to_prometheus(snap)
    assert 'zml_device_power_watts{device="0",name="NVIDIA B200"} 950.0' in prom and "zml_host_memory_total_bytes" in prom
    assert "zml_device_fan_percent" not in prom
    assert outputs.to_csv(snap).count("\n") == 1 and outputs.csv_header().startswith("timestamp,index")
    assert json.loads(outputs.to_json(snap))["gpus"][0]["name"] == "NVIDIA B200"
    assert "NVIDIA B200" in outputs.to_table(snap)
    srv = outputs.serve(lambda: snap, "127.0.0.1", 0)
    try:
        port = srv.server_address[1]
        assert b"zml_device_utilization_percent" in urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics").read()
        assert json.loads(urllib.request.urlopen(f"http://127.0.0.1:{port}/json").read())["gpus"]
    finally:
        srv.shutdown()
    be.close()
    assert fake.calls == ["init", "shutdown"]


def test_cli_fake_one_shot():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "zb_smi", "main.py"), "--fake", "--json"],
                       capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and json.loads(r.stdout.strip())["gpus"][0]["clock_sm_max_mhz"] == 1965
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "zb_smi", "main.py"), "--fake", "--csv", "--interval=0.1", "--count=2"],
                       capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and len(r.stdout.strip().splitlines()) == 5


def test_tui_pages_render_bars_process_table_and_charts():
    import tui
    fake = metrics.FakeNvml(devices=2)
    be = metrics.NvmlBackend(fake)
    host = metrics.HostPoller()
    hist = tui.History(depth=8)
    for _ in range(3):
        snap = metrics.snapshot(be, host)
        hist.add(snap)
    over = tui.render(snap, hist, "overview", 120)
    assert "[1:overview]" in over and "█" in over and "950/1000" in over and "sw_power_cap" in over
    procs = tui.render(snap, hist, "processes", 120)
    assert str(os.getpid()) in procs and "MiB" in procs and "sorted by gpu_memory_bytes" in procs
    assert [p["gpu"] for p in tui.processes(snap, "gpu")] == [0, 1]
    charts = tui.render(snap, hist, "charts", 120)
    assert charts.count("util %") == 2 and any(c in charts for c in "▁▂▃▄▅▆▇█")
    assert tui.sparkline([0, 50, 100, None], 6, 100.0) == "   ▄█ "
    assert tui.bar(0.5, 10) == "█████░░░░░" and tui.bar(None, 4) == "----"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "zb_smi", "main.py"), "--fake", "--top", "--count=2", "--interval=0.1",
                        "--page=processes"], capture_output=True, text=True, timeout=60, stdin=subprocess.DEVNULL)
    assert r.returncode == 0 and "[2:processes]" in r.stdout
    be.close()
    assert fake.calls == ["init", "shutdown"]


def test_remote_agent_devices_join_the_local_ones():
    """An agent serves its snapshot over HTTP; a second monitor started with --remotes shows the agent's devices after
    its own, keeps their host and index, and marks them stale when the agent goes away (bin/zml-smi/api/{server,client}.zig)."""
    agent_backend = metrics.NvmlBackend(metrics.FakeNvml(devices=2))
    agent_host = metrics.HostPoller()
    srv = outputs.serve(lambda: metrics.snapshot(agent_backend, agent_host), "127.0.0.1", 0)
    url = f"http://127.0.0.1:{srv.server_address[1]}"
    try:
        remotes = metrics.RemoteAgents([url])
        snap = metrics.snapshot(metrics.NvmlBackend(metrics.FakeNvml(devices=1)), metrics.HostPoller(), remotes)
        assert [g["index"] for g in snap["gpus"]] == [0, 1, 2]
        assert [g.get("remote_index") for g in snap["gpus"]] == [None, 0, 1]
        assert snap["gpus"][1]["remote"] == snap["host"]["hostname"] and snap["gpus"][1]["stale"] is False
        assert "remote_errors" not in snap
        table = outputs.to_table(snap)
        assert f"@{snap['host']['hostname']}#1" in table
        assert f'device="2",name="NVIDIA B200",host="{snap["host"]["hostname"]}"' in outputs.to_prometheus(snap)
        # the command line: one JSON sample that includes the remote devices
        r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "zb_smi", "main.py"), "--fake", "--json", f"--remotes={url}"],
                           capture_output=True, text=True, timeout=120)
        assert r.returncode == 0, r.stderr
        assert len(json.loads(r.stdout)["gpus"]) == 4
    finally:
        srv.shutdown()
        srv.server_close()
    snap = metrics.snapshot(None, metrics.HostPoller(), remotes)
    assert len(snap["gpus"]) == 2 and all(g["stale"] for g in snap["gpus"]) and url in snap["remote_errors"]
    import pytest
    with pytest.raises(ValueError):
        metrics.RemoteAgents(["hostA:9090"])
