"""The llm CLI end to end on CPU: synthetic repo (config.json, safetensors, tokenizer.json)."""
import json
import os
import subprocess
import sys

import pytest
import torch

from zml_b200 import safetensors
from zml_b200.models import hub
from zml_b200.models.llama import PRESETS, LlamaConfig, LlamaModel
from zml_b200.serving import Engine

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
tokenizers = pytest.importorskip("tokenizers")


def make_repo(path):
    from tokenizers import Tokenizer as HfTok, decoders, models, pre_tokenizers, trainers
    cfg = dict(PRESETS["tiny-llama-test"], model_type="llama", vocab_size=512)
    model = LlamaModel(LlamaConfig.from_hf(cfg), device="cpu", dtype=torch.float32).init_random(seed=9, std=0.08)
    safetensors.save_sharded({k: v.contiguous() for k, v in model.state_dict_hf().items()}, path, max_shard_bytes=1 << 20)
    json.dump(cfg, open(os.path.join(path, "config.json"), "w"))
    t = HfTok(models.BPE())
    t.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    t.decoder = decoders.ByteLevel()
    t.train_from_iterator(["hello world the quick brown fox"] * 10,
                          trainers.BpeTrainer(vocab_size=300, initial_alphabet=pre_tokenizers.ByteLevel.alphabet(),
                                              special_tokens=["<|begin_of_text|>", "<|start_header_id|>", "<|end_header_id|>", "<|eot_id|>"]))
    t.save(os.path.join(path, "tokenizer.json"))
    return model


def test_load_model_from_repo_reproduces_weights(tmp_path):
    ref_model = make_repo(str(tmp_path))
    model, tok = hub.load_model(str(tmp_path), device="cpu", dtype=torch.float32)
    assert tok is not None and torch.equal(model.layers[1].qkv, ref_model.layers[1].qkv)
    assert torch.equal(model.layers[0].gate_up, ref_model.layers[0].gate_up)
    a, _ = Engine(model, 32, 16, 2, 128).generate([[1, 2, 3]], 4)
    b, _ = Engine(ref_model, 32, 16, 2, 128).generate([[1, 2, 3]], 4)
    assert a == b
    ids = hub.tokenize_prompt(tok, "hello", "llama3", 0)
    assert ids[:2] == [0, tok.token_id("<|start_header_id|>")] and ids.count(tok.token_id("<|eot_id|>")) == 1


def test_cli_prompt_mode(tmp_path):
    make_repo(str(tmp_path))
    r = subprocess.run([sys.executable, os.path.join(ROOT, "examples", "llm", "main.py"), f"--model={tmp_path}",
                        "--prompt=hello world", "--seqlen=128", "--max-new-tokens=5", "--cpu"],
                       capture_output=True, text=True, timeout=180)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "tok/s" in r.stdout and "Loaded weights" in r.stderr
    # a system message changes the prompt the model sees (more prefill tokens; the run still succeeds)
    s = subprocess.run([sys.executable, os.path.join(ROOT, "examples", "llm", "main.py"), f"--model={tmp_path}",
                        "--prompt=hello world", "--system=the quick brown fox", "--seqlen=128", "--max-new-tokens=5", "--cpu"],
                       capture_output=True, text=True, timeout=180)
    assert s.returncode == 0 and "tok/s" in s.stdout, s.stderr[-2000:]


_CHAT_WORKER = r"""
import os, sys
sys.path.insert(0, os.path.join(os.environ["ZB_ROOT"], "examples", "llm"))
sys.path.insert(0, os.environ["ZB_ROOT"])
import main as llm
sys.exit(llm.main([f"--model={os.environ['ZB_REPO']}", "--seqlen=128", "--max-new-tokens=3", "--cpu", "--backend=vanilla"]))
"""


def test_cli_chat_loop_on_two_ranks_reads_stdin_on_rank_0_only(tmp_path):
    """Two gloo ranks, interactive mode: only rank 0 sees the terminal; the line and the end of input reach rank 1 by
    broadcast, so both run the same turns and leave together.  The attention backend flag is honoured."""
    repo = tmp_path / "repo"
    repo.mkdir()
    make_repo(str(repo))
    script = tmp_path / "w.py"
    script.write_text(_CHAT_WORKER)
    env = dict(os.environ, ZB_ROOT=ROOT, ZB_REPO=str(repo))
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29661", "--local-ranks-filter", "0", str(script)],
                       input="hello\nworld\n", capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-2500:]
    assert r.stdout.count("tok/s") == 2 and "attention backend: vanilla" in r.stderr


def test_load_model_from_a_remote_repository(tmp_path):
    """The same repository behind an HTTP server: config, tokenizer and the index come through the VFS, tensors as
    range requests; the loaded model equals the local one."""
    import http.server
    import threading
    ref_model = make_repo(str(tmp_path))
    files = {n: (tmp_path / n).read_bytes() for n in os.listdir(tmp_path)}

    class Repo(http.server.BaseHTTPRequestHandler):
        ranged = []

        def log_message(self, *a):
            pass

        def _serve(self, head):
            data = files.get(self.path.rsplit("/", 1)[1])
            if data is None or not self.path.startswith("/models/tiny/"):
                self.send_response(404)
                self.send_header("Content-Length", "0")
                self.end_headers()
                return
            rng = self.headers.get("Range")
            if rng:
                a, b = (int(v) for v in rng.split("=")[1].split("-"))
                body = data[a:b + 1]
                self.send_response(206)
                self.send_header("Content-Range", f"bytes {a}-{a + len(body) - 1}/{len(data)}")
                if self.path.endswith(".safetensors"):
                    Repo.ranged.append(len(body))
            else:
                body = data
                self.send_response(200)
            self.send_header("Content-Length", str(len(data) if head and not rng else len(body)))
            self.end_headers()
            if not head:
                self.wfile.write(body)

        def do_HEAD(self):
            self._serve(True)

        def do_GET(self):
            self._serve(False)

    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), Repo)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    try:
        uri = f"http://127.0.0.1:{srv.server_address[1]}/models/tiny"
        model, tok = hub.load_model(uri, device="cpu", dtype=torch.float32)
        assert tok is not None and tok.token_id("<|eot_id|>") is not None
        assert torch.equal(model.layers[1].qkv, ref_model.layers[1].qkv) and torch.equal(model.embed, ref_model.embed)
        a, _ = Engine(model, 32, 16, 2, 128).generate([[1, 2, 3]], 4)
        b, _ = Engine(ref_model, 32, 16, 2, 128).generate([[1, 2, 3]], 4)
        assert a == b
        assert Repo.ranged and max(Repo.ranged) < max(len(v) for k, v in files.items() if k.endswith(".safetensors"))
        # the index file itself is accepted too
        cfg, store, repo = hub.open_repo(f"{uri}/{safetensors.INDEX_NAME}")
        assert repo == uri and cfg["model_type"] == "llama" and len(store.registry) == len(ref_model.state_dict_hf())
    finally:
        srv.shutdown()
        srv.server_close()


def test_serve_cli_answers_and_stops_on_sigterm(tmp_path):
    """examples/llm/serve.py on CPU: starts on a free port, answers a completion and the health route, leaves cleanly
    on SIGTERM."""
    import re
    import signal
    import time
    import urllib.request
    make_repo(str(tmp_path))
    p = subprocess.Popen([sys.executable, os.path.join(ROOT, "examples", "llm", "serve.py"), f"--model={tmp_path}", "--cpu",
                          "--port=0", "--max-batch=2", "--seqlen=64"], stderr=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        port, t0 = None, time.time()
        while port is None and time.time() - t0 < 120:
            line = p.stderr.readline()
            if not line and p.poll() is not None:
                break
            m = re.search(r"http://127\.0\.0\.1:(\d+)", line)
            if m:
                port = int(m.group(1))
        assert port, "the server did not come up"
        req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/completions",
                                     data=json.dumps({"prompt": "hello world", "max_tokens": 4}).encode())
        with urllib.request.urlopen(req, timeout=60) as r:
            body = json.loads(r.read())
        assert body["usage"]["completion_tokens"] == 4 and isinstance(body["choices"][0]["text"], str)
        with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=10) as r:
            assert json.loads(r.read())["status"] == "ok"
        p.send_signal(signal.SIGTERM)
        assert p.wait(timeout=60) == 0
    finally:
        if p.poll() is None:
            p.kill()
