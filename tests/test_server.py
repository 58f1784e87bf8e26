"""The HTTP front end over Engine.serve: completions, chat, batching of concurrent requests, errors, metrics."""
import json
import threading
import urllib.error
import urllib.request

import pytest
import torch

from zml_b200.models.llama import PRESETS, LlamaConfig, LlamaModel
from zml_b200.serving import Engine
from zml_b200.serving.server import Server

tokenizers = pytest.importorskip("tokenizers")


def _tokenizer():
    from tokenizers import Tokenizer as HfTok, decoders, models, pre_tokenizers, trainers
    from zml_b200.tokenizer import Tokenizer
    t = HfTok(models.BPE())
    t.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    t.decoder = decoders.ByteLevel()
    t.train_from_iterator(["hello world the quick brown fox jumps over the lazy dog"] * 10,
                          trainers.BpeTrainer(vocab_size=300, initial_alphabet=pre_tokenizers.ByteLevel.alphabet(),
                                              special_tokens=["<|begin_of_text|>", "<|start_header_id|>", "<|end_header_id|>", "<|eot_id|>"]))
    return Tokenizer.from_bytes(t.to_str().encode())


def _post(base, route, body):
    req = urllib.request.Request(base + route, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    try:
        with urllib.request.urlopen(req, timeout=60) as r:
            return r.status, json.loads(r.read())
    except urllib.error.HTTPError as e:
        return e.code, json.loads(e.read())


def test_server_completions_chat_batching_errors_and_metrics():
    cfg = LlamaConfig.from_hf(dict(PRESETS["tiny-llama-test"], vocab_size=512))
    model = LlamaModel(cfg, device="cpu", dtype=torch.float32).init_random(seed=2, std=0.08)
    tok = _tokenizer()
    engine = Engine(model, num_pages=64, page_size=16, max_batch=4, max_seq_len=128)
    server = Server(engine, tok, model_name="tiny", template="llama3", bos=0, eos_ids=(3,), batch_window_s=0.3,
                    default_max_tokens=5, idle_tick_s=0.05)
    host, port = server.start_http("127.0.0.1", 0)
    base = f"http://{host}:{port}"
    loop = threading.Thread(target=server.run, daemon=True)
    loop.start()
    try:
        prompts = ["hello world", "the quick brown fox", "lazy dog", "hello", "fox jumps over", "dog"]
        results = {}

        def ask(i):
            results[i] = _post(base, "/v1/completions", {"prompt": prompts[i], "max_tokens": 6})
        threads = [threading.Thread(target=ask, args=(i,)) for i in range(len(prompts))]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        # six concurrent requests fall into one or two batches and equal one-at-a-time generation
        ref = Engine(model, num_pages=64, page_size=16, max_batch=4, max_seq_len=128)
        for i, p in enumerate(prompts):
            code, body = results[i]
            assert code == 200 and body["object"] == "text_completion" and body["model"] == "tiny"
            ids = [0] + tok.encode(p)
            want, _ = ref.generate([ids], 6, eos_ids=(3,))
            want_ids = want[0][:-1] if want[0] and want[0][-1] == 3 else want[0]
            assert body["choices"][0]["text"] == tok.decode(want_ids)
            assert body["usage"] == {"prompt_tokens": len(ids), "completion_tokens": len(want[0]), "total_tokens": len(ids) + len(want[0])}
            assert body["choices"][0]["finish_reason"] in ("length", "stop")
        assert 1 <= server.stats.batches <= 3 and server.stats.requests == 6

        code, body = _post(base, "/v1/completions", {"prompt": [0, 5, 6, 7]})                     # token ids, default budget
        assert code == 200 and body["usage"]["prompt_tokens"] == 4 and body["usage"]["completion_tokens"] <= 5
        code, body = _post(base, "/v1/chat/completions", {"messages": [{"role": "user", "content": "hello world"}], "max_tokens": 4})
        assert code == 200 and body["object"] == "chat.completion" and body["choices"][0]["message"]["role"] == "assistant"
        assert body["usage"]["prompt_tokens"] == len(__import__("zml_b200.models.hub", fromlist=["x"]).tokenize_prompt(tok, "hello world", "llama3", 0))

        for bad in ({}, {"prompt": []}, {"prompt": "hi", "max_tokens": 0}, {"prompt": "hi", "max_tokens": 10_000},
                    {"prompt": 3}):
            assert _post(base, "/v1/completions", bad)[0] == 400, bad
        assert _post(base, "/v1/chat/completions", {"messages": []})[0] == 400
        assert _post(base, "/v1/nothing", {})[0] == 404
        with urllib.request.urlopen(base + "/health") as r:
            assert json.loads(r.read())["status"] == "ok"
        with urllib.request.urlopen(base + "/v1/models") as r:
            assert json.loads(r.read())["data"][0]["id"] == "tiny"
        with urllib.request.urlopen(base + "/metrics") as r:
            text = r.read().decode()
        assert "zml_server_requests_total 8" in text and "zml_server_output_tokens_total" in text and "zml_server_requests_failed_total 0" in text
    finally:
        server.shutdown()
        loop.join(timeout=10)
    assert not loop.is_alive()


_TP_SERVER_WORKER = r"""
import json, os, sys, threading, time, urllib.request, torch
sys.path.insert(0, os.environ["ZB_ROOT"])
sys.path.insert(0, os.path.join(os.environ["ZB_ROOT"], "tests"))
from test_server import _tokenizer
from zml_b200.models.llama import PRESETS, LlamaConfig, LlamaModel
from zml_b200.parallel.comm import Comm
from zml_b200.serving import Engine
from zml_b200.serving.server import Server
c = Comm.from_env(backend="gloo")
cfg = LlamaConfig.from_hf(dict(PRESETS["tiny-llama-test"], vocab_size=512))
model = LlamaModel(cfg, c, device="cpu", dtype=torch.float32).init_random(seed=2, std=0.08)
tok = _tokenizer()
server = Server(Engine(model, num_pages=64, page_size=16, max_batch=4, max_seq_len=128), tok, c, model_name="tiny", bos=0,
                batch_window_s=0.2, idle_tick_s=0.05)
if c.rank == 0:
    host, port = server.start_http("127.0.0.1", 0)
    def client():
        outs = {}
        def ask(i, p):
            req = urllib.request.Request(f"http://{host}:{port}/v1/completions", data=json.dumps({"prompt": p, "max_tokens": 5}).encode())
            with urllib.request.urlopen(req, timeout=120) as r:
                outs[i] = json.loads(r.read())
        ts = [threading.Thread(target=ask, args=(i, p)) for i, p in enumerate(["hello world", "the lazy dog", "fox"])]
        [t.start() for t in ts]; [t.join() for t in ts]
        single = LlamaModel(cfg, Comm.single(torch.device("cpu")), device="cpu", dtype=torch.float32).init_random(seed=2, std=0.08)
        ref = Engine(single, num_pages=64, page_size=16, max_batch=4, max_seq_len=128)
        for i, p in enumerate(["hello world", "the lazy dog", "fox"]):
            want, _ = ref.generate([[0] + tok.encode(p)], 5)
            assert outs[i]["choices"][0]["text"] == tok.decode(want[0]), (p, outs[i])
        print("SERVER_TP_CLIENT_OK", flush=True)
        server.shutdown()
    threading.Thread(target=client, daemon=True).start()
server.run()
print("SERVER_TP_OK", c.rank, flush=True)
c.finish(0)
"""


def test_server_on_two_tensor_parallel_ranks(tmp_path):
    """Rank 0 owns the socket, both gloo ranks run every batch; answers equal one rank holding the whole model."""
    import os
    import subprocess
    import sys
    script = tmp_path / "w.py"
    script.write_text(_TP_SERVER_WORKER)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29671", str(script)],
                       capture_output=True, text=True, env=dict(os.environ, ZB_ROOT=root), timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert r.stdout.count("SERVER_TP_OK") == 2 and "SERVER_TP_CLIENT_OK" in r.stdout


def test_server_streams_server_sent_events():
    cfg = LlamaConfig.from_hf(dict(PRESETS["tiny-llama-test"], vocab_size=512))
    model = LlamaModel(cfg, device="cpu", dtype=torch.float32).init_random(seed=2, std=0.08)
    tok = _tokenizer()
    server = Server(Engine(model, num_pages=64, page_size=16, max_batch=4, max_seq_len=128), tok, model_name="tiny", bos=0,
                    batch_window_s=0.05, idle_tick_s=0.05)
    host, port = server.start_http("127.0.0.1", 0)
    loop = threading.Thread(target=server.run, daemon=True)
    loop.start()
    try:
        whole = _post(f"http://{host}:{port}", "/v1/completions", {"prompt": "the quick brown fox", "max_tokens": 40})[1]
        for route, body in (("/v1/completions", {"prompt": "the quick brown fox", "max_tokens": 40, "stream": True}),
                            ("/v1/chat/completions", {"messages": [{"role": "user", "content": "hello"}], "max_tokens": 20, "stream": True})):
            req = urllib.request.Request(f"http://{host}:{port}{route}", data=json.dumps(body).encode())
            with urllib.request.urlopen(req, timeout=60) as r:
                assert r.headers["Content-Type"] == "text/event-stream"
                lines = [l for l in r.read().decode().split("\n\n") if l]
            assert lines[-1] == "data: [DONE]" and len(lines) >= 3                  # several decode blocks, then the end
            events = [json.loads(l[len("data: "):]) for l in lines[:-1]]
            assert events[-1]["choices"][0]["finish_reason"] in ("length", "stop")
            assert all(e["choices"][0]["finish_reason"] is None for e in events[:-1])
            if route == "/v1/completions":
                assert "".join(e["choices"][0]["text"] for e in events) == whole["choices"][0]["text"]
            else:
                assert events[0]["object"] == "chat.completion.chunk"
                assert isinstance("".join(e["choices"][0]["delta"].get("content", "") for e in events), str)
    finally:
        server.shutdown()
        loop.join(timeout=10)


def test_server_reports_a_failed_batch_and_keeps_serving():
    """A batch whose `serve` raises (a collective that timed out, pages that ran out) answers 500 to its requests - an
    error event to streaming ones - and the next batch runs normally; a full queue answers 429."""
    tok = _tokenizer()

    class FlakyEngine:
        max_pages, page_size = 8, 16
        calls = 0

        def serve(self, prompts, budgets, strategy, eos_ids, seed=0, on_tokens=None):
            FlakyEngine.calls += 1
            if FlakyEngine.calls == 1:
                raise RuntimeError("collective timed out")
            outs = [[7] * b for b in budgets]
            if on_tokens:
                for i, o in enumerate(outs):
                    on_tokens(i, o, True)
            return outs, None

    server = Server(FlakyEngine(), tok, model_name="fake", bos=0, batch_window_s=0.01, idle_tick_s=0.02, max_queue=2)
    host, port = server.start_http("127.0.0.1", 0)
    base = f"http://{host}:{port}"
    loop = threading.Thread(target=server.run, daemon=True)
    loop.start()
    try:
        code, body = _post(base, "/v1/completions", {"prompt": "hello", "max_tokens": 3})
        assert code == 500 and "collective timed out" in body["error"]["message"]
        code, body = _post(base, "/v1/completions", {"prompt": "hello", "max_tokens": 3})
        assert code == 200 and body["usage"]["completion_tokens"] == 3
        assert server.stats.failed == 1 and server.stats.requests == 2 and server.stats.batches == 2
    finally:
        server.shutdown()
        loop.join(timeout=10)
    # with the scheduler stopped, requests pile up: the third one is refused
    for _ in range(2):
        server.submit({"prompt": "x", "max_tokens": 1}, chat=False)
    with pytest.raises(OverflowError):
        server.submit({"prompt": "x", "max_tokens": 1}, chat=False)


class _RecordingEngine:
    """Stands in for an Engine: records what `serve` was called with and answers token 7 for every budgeted step."""
    max_pages, page_size = 64, 16

    def __init__(self):
        self.calls = []

    def serve(self, prompts, budgets, strategy, eos_ids, seed=0, on_tokens=None):
        self.calls.append((len(prompts), strategy.topk, strategy.temperature, seed))
        return [[7] * b for b in budgets], None


def test_server_batches_by_sampling_settings_and_validates_them():
    from zml_b200.models.common import SamplingStrategy
    eng = _RecordingEngine()
    server = Server(eng, _tokenizer(), bos=0, eos_ids=(3,), batch_window_s=0.0, idle_tick_s=0.01,
                    strategy=SamplingStrategy(topk=1, temperature=1.0))
    a = server.submit({"prompt": "hello", "max_tokens": 2}, chat=False)                                     # the server's strategy
    b = server.submit({"prompt": "hello", "max_tokens": 2, "temperature": 0.7, "top_k": 40, "seed": 5}, chat=False)
    c = server.submit({"prompt": "dog", "max_tokens": 3, "temperature": 0}, chat=False)                     # greedy = the default here
    d = server.submit({"prompt": "fox", "max_tokens": 2, "top_k": 40, "temperature": 0.7, "seed": 5}, chat=False)
    e = server.submit({"prompt": "fox", "max_tokens": 2, "temperature": 1.5}, chat=False)                   # no top_k: the widest
    f = server.submit({"prompt": "fox", "max_tokens": 2, "top_k": 1000}, chat=False)                        # capped
    g = server.submit({"prompt": "fox", "max_tokens": 2, "top_k": -1, "temperature": 1.5}, chat=False)
    assert a.sampling == (1, 1.0, 0) and b.sampling == (40, 0.7, 5) and c.sampling == (1, 1.0, 0)
    assert e.sampling == (128, 1.5, 0) and f.sampling == (128, 1.0, 0) and g.sampling == e.sampling
    assert server.waiting() == 7
    for _ in range(4):
        assert server.step()
    # four batches, oldest first: {a, c}, {b, d}, {e, g}, {f}; nobody is left behind
    assert eng.calls == [(2, 1, 1.0, 0), (2, 40, 0.7, 5), (2, 128, 1.5, 0), (1, 128, 1.0, 0)]
    assert all(r.done.is_set() for r in (a, b, c, d, e, f, g)) and server.waiting() == 0
    assert len(c.tokens) == 3 and len(d.tokens) == 2 and server.stats.batches == 4 and server.stats.requests == 7
    # a server that samples by default keeps its k when a request only sets the temperature
    warm = Server(eng, _tokenizer(), bos=0, strategy=SamplingStrategy(topk=8, temperature=0.9))
    assert warm._sampling({}) == (8, 0.9, 0) and warm._sampling({"temperature": 0.5}) == (8, 0.5, 0)
    assert warm._sampling({"top_k": 3}) == (3, 0.9, 0) and warm._sampling({"temperature": 0, "top_k": 9}) == (1, 1.0, 0)
    for bad in ({"temperature": -1}, {"temperature": "hot"}, {"temperature": True}, {"temperature": float("nan")},
                {"top_k": 0}, {"top_k": 2.5}, {"top_k": -2}, {"seed": "x"}, {"seed": 1.5}):
        with pytest.raises(ValueError):
            server.submit(dict({"prompt": "hello"}, **bad), chat=False)
    for unsupported in ({"n": 2}, {"best_of": 4}, {"logprobs": 5}, {"logprobs": True}, {"top_logprobs": 3}, {"echo": True}):
        with pytest.raises(ValueError, match="not supported"):
            server.submit(dict({"prompt": "hello"}, **unsupported), chat=False)
    server.submit({"prompt": "hello", "n": 1, "logprobs": None, "echo": False, "best_of": 1, "logprobs": False}, chat=False)
    assert server.waiting() == 1 and server.step() and server.waiting() == 0


def test_server_sampled_request_matches_the_engine_with_the_same_settings():
    from zml_b200.models.common import SamplingStrategy
    cfg = LlamaConfig.from_hf(dict(PRESETS["tiny-llama-test"], vocab_size=512))
    model = LlamaModel(cfg, device="cpu", dtype=torch.float32).init_random(seed=2, std=0.08)
    tok = _tokenizer()
    server = Server(Engine(model, num_pages=64, page_size=16, max_batch=4, max_seq_len=128), tok, bos=0, eos_ids=(3,),
                    batch_window_s=0.0, idle_tick_s=0.01)
    r = server.submit({"prompt": "hello world", "max_tokens": 6, "temperature": 0.8, "top_k": 5, "seed": 11}, chat=False)
    greedy = server.submit({"prompt": "hello world", "max_tokens": 6}, chat=False)
    assert server.step() and server.step() and r.done.is_set() and greedy.done.is_set() and not r.error
    ref = Engine(model, num_pages=64, page_size=16, max_batch=4, max_seq_len=128)
    want, _ = ref.serve([[0] + tok.encode("hello world")], 6, SamplingStrategy(topk=5, temperature=0.8), (3,), seed=11)
    assert r.tokens == want[0]
    want_greedy, _ = ref.serve([[0] + tok.encode("hello world")], 6, SamplingStrategy(), (3,))
    assert greedy.tokens == want_greedy[0]


def test_server_stop_strings_cut_the_answer_streamed_or_not():
    tok = _tokenizer()
    text = "hello world the quick brown fox jumps over the lazy dog"
    ids = tok.encode(text)
    assert tok.decode(ids) == text

    class Scripted:
        """Answers every request with the tokens of `text`, in blocks of two tokens."""
        max_pages, page_size = 64, 16

        def serve(self, prompts, budgets, strategy, eos_ids, seed=0, on_tokens=None):
            outs = [ids[:b] for b in budgets]
            if on_tokens:
                for i, o in enumerate(outs):
                    for j in range(0, len(o), 2):
                        on_tokens(i, o[j:j + 2], j + 2 >= len(o))
            return outs, None

    server = Server(Scripted(), tok, bos=0, eos_ids=(3,), batch_window_s=0.0, idle_tick_s=0.01, default_max_tokens=len(ids))
    host, port = server.start_http("127.0.0.1", 0)
    base = f"http://{host}:{port}"
    loop = threading.Thread(target=server.run, daemon=True)
    loop.start()
    try:
        code, body = _post(base, "/v1/completions", {"prompt": "x"})
        assert code == 200 and body["choices"][0]["text"] == text and body["choices"][0]["finish_reason"] == "length"
        code, body = _post(base, "/v1/completions", {"prompt": "x", "stop": " brown"})
        assert body["choices"][0]["text"] == "hello world the quick" and body["choices"][0]["finish_reason"] == "stop"
        assert body["usage"]["completion_tokens"] == len(ids)                    # generation is not cut short, the answer is
        code, body = _post(base, "/v1/chat/completions", {"messages": [{"role": "user", "content": "x"}], "stop": ["lazy", "fox", "never"]})
        assert body["choices"][0]["message"]["content"] == "hello world the quick brown " and body["choices"][0]["finish_reason"] == "stop"
        code, body = _post(base, "/v1/completions", {"prompt": "x", "stop": ["zebra"]})
        assert body["choices"][0]["text"] == text and body["choices"][0]["finish_reason"] == "length"
        # token counting for clients: the ids a completion or a chat request would run with, and back to text
        code, body = _post(base, "/tokenize", {"prompt": "hello world"})
        assert code == 200 and body["tokens"] == [0] + tok.encode("hello world") and body["count"] == len(body["tokens"])
        assert body["max_model_len"] == 64 * 16
        code, plain = _post(base, "/tokenize", {"prompt": "hello world", "add_special_tokens": False})
        assert plain["tokens"] == tok.encode("hello world")
        code, back = _post(base, "/detokenize", {"tokens": plain["tokens"]})
        assert code == 200 and back["prompt"] == "hello world"
        from zml_b200.models import hub
        msgs = [{"role": "system", "content": "quick"}, {"role": "user", "content": "fox"}]
        code, body = _post(base, "/tokenize", {"messages": msgs})
        assert code == 200 and body["tokens"] == hub.tokenize_chat(tok, msgs, "llama3", 0)
        for route, bad in (("/tokenize", {}), ("/tokenize", {"prompt": 5}), ("/tokenize", {"messages": [{"role": "user"}]}),
                           ("/detokenize", {"tokens": "abc"}), ("/detokenize", {"tokens": [1.5]})):
            assert _post(base, route, bad)[0] == 400
        for bad in ("", [""], [1], ["a"] * 9, 5, {"a": 1}):
            code, body = _post(base, "/v1/completions", {"prompt": "x", "stop": bad})
            assert code == 400 and "stop" in body["error"]["message"]

        def stream(payload):
            req = urllib.request.Request(base + "/v1/completions", data=json.dumps(dict(payload, stream=True)).encode())
            events = []
            with urllib.request.urlopen(req, timeout=60) as resp:
                for line in resp:
                    line = line.decode().strip()
                    if line.startswith("data: "):
                        events.append(line[6:])
            assert events[-1] == "[DONE]"
            chunks = [json.loads(e)["choices"][0] for e in events[:-1]]
            return "".join(c["text"] for c in chunks), [c["finish_reason"] for c in chunks]

        got, reasons = stream({"prompt": "x"})
        assert got == text and reasons[-1] == "length" and all(r is None for r in reasons[:-1]) and len(reasons) > 2
        # a stop string that straddles two blocks is still found, and nothing of it is sent
        got, reasons = stream({"prompt": "x", "stop": ["ck brown f"]})
        assert got == "hello world the qui" and reasons[-1] == "stop" and all(r is None for r in reasons[:-1])
        got, reasons = stream({"prompt": "x", "stop": ["zebra crossing"]})
        assert got == text and reasons[-1] == "length"
    finally:
        server.shutdown()
        loop.join(timeout=10)


def test_tokenize_chat_equals_the_sessions_turn_by_turn_tokens_and_knows_roles():
    from zml_b200.models import hub
    tok = _tokenizer()
    convo = [{"role": "user", "content": "hello world"}, {"role": "assistant", "content": "the fox"},
             {"role": "user", "content": "lazy dog"}]
    turn_by_turn = (hub.tokenize_prompt(tok, "hello world", "llama3", 0, True) + tok.encode("the fox")
                    + hub.tokenize_prompt(tok, "lazy dog", "llama3", 0, False))
    assert hub.tokenize_chat(tok, convo, "llama3", 0) == turn_by_turn
    assert hub.tokenize_chat(tok, convo[:1], "llama3", 0) == hub.tokenize_prompt(tok, "hello world", "llama3", 0, True)
    sh, eh, eot = (tok.token_id(t) for t in ("<|start_header_id|>", "<|end_header_id|>", "<|eot_id|>"))
    with_system = hub.tokenize_chat(tok, [{"role": "system", "content": "quick"}] + convo[:1], "llama3", 0)
    nl = tok.encode("\n")
    assert with_system[:2] == [0, sh] and with_system[2:2 + len(tok.encode("system"))] == tok.encode("system")
    assert with_system == [0, sh] + tok.encode("system") + [eh] + nl + tok.encode("quick") + [eot] + nl + \
        hub.tokenize_prompt(tok, "hello world", "llama3", None, True)
    # a vocabulary without the ChatML markers: the contents, concatenated
    assert hub.tokenize_chat(tok, convo, "chatml", None) == tok.encode("hello world") + tok.encode("the fox") + tok.encode("lazy dog")
    with pytest.raises(ValueError, match="unknown role"):
        hub.tokenize_chat(tok, [{"role": "narrator", "content": "x"}], "llama3", 0)
