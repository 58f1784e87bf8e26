"""Activation fixtures (collector + test_layer), profiler command lines, trace merging."""
import json
import os

import pytest
import torch

from zml_b200.profiling import perfetto, wrappers
from zml_b200.testing import NotClose
from zml_b200.utils import activations as acts


class _Block(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.fc = torch.nn.Linear(8, 8)

    def forward(self, x):
        return torch.relu(self.fc(x))


class _Net(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.layers = torch.nn.ModuleList([_Block(), _Block(), _Block()])

    def forward(self, x):
        for l in self.layers:
            x = l(x)
        return x


def test_collector_records_first_layer_and_test_layer_checks_it(tmp_path):
    torch.manual_seed(0)
    net = _Net()
    x = torch.randn(4, 8)
    out, a = acts.ActivationCollector(net)(x)
    assert out.shape == (4, 8)
    assert "layers.0.fc.in.0" in a and "layers.0.out.0" in a
    assert not any(k.startswith("layers.1.") or k.startswith("layers.2.") for k in a)     # default blacklist
    torch.testing.assert_close(a["layers.0.in.0"], x)
    path = str(tmp_path / "acts.safetensors")
    acts.save_activations(path, a)
    back = acts.load_activations(path)
    assert set(back) == set(a)
    fc = net.layers[0].fc
    acts.test_layer(lambda t: t @ fc.weight.t() + fc.bias, back, "layers.0.fc", atol=1e-5)
    with pytest.raises(NotClose):
        acts.test_layer(lambda t: t @ fc.weight.t(), back, "layers.0.fc", atol=1e-5)
    with pytest.raises(KeyError):
        acts.test_layer(lambda t: t, back, "layers.9.fc")
    _, all_layers = acts.ActivationCollector(net, blacklist_regexes=(), max_layers=3)(x)
    assert len({k.split(".in.")[0].split(".out.")[0] for k in all_layers}) == 3


def test_profiler_command_lines(monkeypatch):
    cmd = wrappers.ncu_command(["python", "x.py"], kernel_regex="zb_gemm", launch_count=2, skip=5, output="o")
    assert cmd[0] == "ncu" and cmd[cmd.index("--clock-control") + 1] == "none"
    assert cmd[cmd.index("-k") + 1] == "regex:zb_gemm" and cmd[-2:] == ["python", "x.py"]
    monkeypatch.setenv("ZB_NCU_ARGS", "--section SpeedOfLight")
    assert "--clock-control" in wrappers.ncu_command(["p"])
    monkeypatch.setenv("ZML_NSYS_ARGS", "profile -t cuda")
    assert wrappers.nsys_command(["p"], "out") == ["nsys", "profile", "-t", "cuda", "-o", "out", "p"]
    assert wrappers.main(["bogus"]) == 1


def test_trace_merge_and_summary(tmp_path):
    host = [{"ph": "X", "name": "zml.exe.call", "ts": 1000, "dur": 50, "pid": 7, "tid": 1},
            {"ph": "B", "name": "prefill", "ts": 1100, "pid": 7, "tid": 1}, {"ph": "E", "name": "prefill", "ts": 1400, "pid": 7, "tid": 1}]
    dev = {"traceEvents": [{"ph": "X", "name": "zb_gemm_bf16_kernel", "ts": 5000, "dur": 20, "pid": 0, "tid": 7},
                           {"ph": "X", "name": "zb_gemm_bf16_kernel", "ts": 5030, "dur": 22, "pid": 0, "tid": 7}]}
    h, d, o = tmp_path / "h.json", tmp_path / "d.json", tmp_path / "m" / "merged.json"
    h.write_text(json.dumps(host)); d.write_text(json.dumps(dev))
    info = perfetto.merge_traces(str(h), str(d), str(o))
    assert info["host_spans"] == 2 and info["device_events"] == 2
    ev = json.loads(o.read_text())["traceEvents"]
    assert min(e["ts"] for e in ev if e.get("pid") == 1 and "ts" in e) == 0
    rows = dict((n, (c, us)) for n, c, us in perfetto.summarize(ev))
    assert rows["zb_gemm_bf16_kernel"] == (2, 42.0) and rows["prefill"] == (1, 300.0)
    assert perfetto.main([str(h), "-o", str(tmp_path / "only_host.json")]) == 0
