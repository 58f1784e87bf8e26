"""HTTP front end for an `Engine`: OpenAI-style `/v1/completions` and `/v1/chat/completions`, `/tokenize` and
`/detokenize`, `/health`, and Prometheus gauges under `/metrics`.

The reference stops at the chat CLI (examples/llm); this is the small piece a deployment needs on top of
`Engine.serve`.  Requests are collected for a short window (`batch_window_s`) or until `max_queue` of them wait, then
run as one `Engine.serve` call, which batches them continuously on the device; requests that arrive while a batch runs
wait for the next one.  `"stream": true` answers with server-sent events, one per decode block.  A request may set
`stop` (strings that end the answer), `temperature`, `top_k` (at most 128, the widest the sampler draws from) and
`seed`; requests of one batch share their sampling settings, so a batch is the waiting requests whose settings equal those of the oldest one, and the others run
in a later batch.  On a multi-rank job every rank calls `Server.run()`: rank 0 owns the socket and the queue and
broadcasts each batch (token ids, budgets, sampling settings) so that all ranks enter `Engine.serve` with the same
arguments; an idle tick is broadcast too, so that the heartbeat of `Comm.check_peers` keeps running while no request is
in flight.

    python examples/llm/serve.py --model=/models/Llama-3.1-8B-Instruct --port=8000
    curl -s localhost:8000/v1/completions -d '{"prompt": "The capital of France is", "max_tokens": 16}'
"""
from __future__ import annotations

import http.server
import json
import queue
import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import Optional

from ..models import hub
from ..models.common import SamplingStrategy


MAX_TOP_K = 128          # the sampling kernel keeps at most this many candidates per row
MAX_STOP = 8             # stop strings per request


def _first_stop(text: str, stops) -> int:
    """Offset of the earliest occurrence of any stop string, or -1.  Generation is not cut short (every rank runs the
    batch to its budgets); the answer is."""
    hits = [i for i in (text.find(s) for s in stops) if i >= 0]
    return min(hits) if hits else -1


class StopFilter:
    """Cuts a text that arrives in pieces at the first stop string: `feed(piece, last)` returns (text that can be
    sent now, whether a stop string was met).  The last len(longest stop) - 1 characters are kept back until more text
    shows whether they begin a stop string; the pieces sent add up to the whole text cut at `_first_stop`."""

    def __init__(self, stops):
        self.stops = tuple(stops)
        self.keep = max((len(x) for x in self.stops), default=1) - 1
        self.held = ""
        self.stopped = False

    def feed(self, piece: str, last: bool = False) -> tuple:
        if self.stopped:
            return "", True
        self.held += piece
        cut = _first_stop(self.held, self.stops)
        if cut >= 0:
            out, self.held, self.stopped = self.held[:cut], "", True
            return out, True
        out = self.held if last or self.keep == 0 else self.held[:max(len(self.held) - self.keep, 0)]
        self.held = self.held[len(out):]
        return out, False


@dataclass
class _Request:
    ids: list
    max_tokens: int
    chat: bool
    model: str
    done: threading.Event = field(default_factory=threading.Event)
    tokens: list = field(default_factory=list)
    error: Optional[str] = None
    arrived: float = field(default_factory=time.perf_counter)
    finished: float = 0.0
    stream: bool = False
    chunks: "queue.Queue" = field(default_factory=queue.Queue)       # (new tokens, finished) per decode block
    sampling: tuple = (1, 1.0, 0)                                    # (top-k, temperature, seed)
    stop: tuple = ()                                                 # strings that end the answer (not included in it)


@dataclass
class ServerStats:
    requests: int = 0
    failed: int = 0
    batches: int = 0
    prompt_tokens: int = 0
    output_tokens: int = 0
    busy_s: float = 0.0
    last_batch: int = 0
    last_tok_s: float = 0.0


class Server:
    def __init__(self, engine, tokenizer, comm=None, model_name: str = "model", template: Optional[str] = None,
                 bos: Optional[int] = None, eos_ids=(), strategy: Optional[SamplingStrategy] = None,
                 batch_window_s: float = 0.02, max_queue: int = 256, default_max_tokens: int = 128,
                 idle_tick_s: float = 0.5):
        self.engine, self.tok, self.comm = engine, tokenizer, comm
        self.model_name, self.template, self.bos = model_name, template, bos
        self.eos_ids = tuple(int(e) for e in eos_ids)
        self.strategy = strategy or SamplingStrategy()
        self.batch_window_s, self.max_queue = batch_window_s, max_queue
        self.default_max_tokens, self.idle_tick_s = default_max_tokens, idle_tick_s
        self.queue: "queue.Queue[_Request]" = queue.Queue()
        self.stats = ServerStats()
        self._stop = threading.Event()
        self._httpd: Optional[http.server.ThreadingHTTPServer] = None
        self.rank = comm.rank if comm is not None else 0
        self._held: list = []                    # requests taken off the queue whose sampling settings differed from their batch's

    # ------------------------------------------------------------------ request handling (rank 0)
    def _limit(self) -> int:
        return self.engine.max_pages * self.engine.page_size

    def waiting(self) -> int:
        return self.queue.qsize() + len(self._held)

    def _sampling(self, body: dict) -> tuple:
        """(top-k, temperature, seed) of a request.  Without `temperature` and `top_k` the server's strategy applies;
        `temperature: 0` is greedy; a positive temperature without `top_k` draws from the server's k when that is more
        than 1, else from the MAX_TOP_K best tokens."""
        k, t = None, None
        if body.get("temperature") is not None:
            t = body["temperature"]
            if isinstance(t, bool) or not isinstance(t, (int, float)) or t < 0 or t != t:
                raise ValueError("'temperature' must be a number >= 0")
            t = round(float(t), 2)                  # a decode graph is captured per setting: keep their number small
        if body.get("top_k") is not None:
            k = body["top_k"]
            if isinstance(k, bool) or not isinstance(k, int) or k == 0 or k < -1:
                raise ValueError("'top_k' must be a positive integer (or -1 for the widest supported)")
            k = MAX_TOP_K if k == -1 else min(k, MAX_TOP_K)
        seed = body.get("seed", 0)
        if seed is None:
            seed = 0
        if isinstance(seed, bool) or not isinstance(seed, int):
            raise ValueError("'seed' must be an integer")
        if t is None and k is None:
            return int(self.strategy.topk), float(self.strategy.temperature), int(seed)
        if t == 0.0:
            return 1, 1.0, int(seed)
        if k is None:
            k = int(self.strategy.topk) if self.strategy.topk > 1 else MAX_TOP_K
        return int(k), float(self.strategy.temperature if t is None else t), int(seed)

    def submit(self, body: dict, chat: bool) -> _Request:
        """Validates a request body and queues it; raises ValueError with the message for a 400 answer."""
        if chat:
            msgs = body.get("messages")
            if not isinstance(msgs, list) or not msgs:
                raise ValueError("'messages' must be a non-empty list")
            for m in msgs:
                if not isinstance(m, dict) or not isinstance(m.get("content"), str):
                    raise ValueError("every message needs a 'content' string")
            ids = hub.tokenize_chat(self.tok, msgs, self.template or "llama3", self.bos)
        else:
            prompt = body.get("prompt")
            if isinstance(prompt, list) and prompt and all(isinstance(t, int) for t in prompt):
                ids = [int(t) for t in prompt]
            elif isinstance(prompt, str):
                ids = ([self.bos] if self.bos is not None else []) + self.tok.encode(prompt)
            else:
                raise ValueError("'prompt' must be a string or a list of token ids")
        if not ids:
            raise ValueError("the prompt is empty")
        max_tokens = int(body.get("max_tokens", body.get("max_completion_tokens", self.default_max_tokens)))
        if max_tokens < 1:
            raise ValueError("'max_tokens' must be at least 1")
        if len(ids) + max_tokens > self._limit():
            raise ValueError(f"prompt ({len(ids)} tokens) + max_tokens ({max_tokens}) exceeds the engine's limit of {self._limit()} tokens")
        for key, neutral in (("n", 1), ("best_of", 1), ("logprobs", None), ("top_logprobs", None), ("echo", False)):
            if body.get(key) not in (None, neutral, False if neutral is None else neutral):
                raise ValueError(f"'{key}' is not supported")           # refused rather than silently ignored
        sampling = self._sampling(body)
        stop = body.get("stop")
        stop = () if stop is None else (stop,) if isinstance(stop, str) else tuple(stop) if isinstance(stop, list) else None
        if stop is None or len(stop) > MAX_STOP or not all(isinstance(x, str) and x for x in stop):
            raise ValueError(f"'stop' must be a non-empty string or a list of at most {MAX_STOP} of them")
        if self.waiting() >= self.max_queue:
            raise OverflowError("the request queue is full")
        r = _Request(ids, max_tokens, chat, str(body.get("model", self.model_name)), stream=bool(body.get("stream", False)),
                     sampling=sampling, stop=stop)
        self.queue.put(r)
        return r

    def _answer(self, r: _Request) -> dict:
        toks = list(r.tokens)
        finish = "length"
        if toks and toks[-1] in self.eos_ids:
            toks, finish = toks[:-1], "stop"
        text = self.tok.decode(toks)
        cut = _first_stop(text, r.stop)
        if cut >= 0:
            text, finish = text[:cut], "stop"
        usage = {"prompt_tokens": len(r.ids), "completion_tokens": len(r.tokens), "total_tokens": len(r.ids) + len(r.tokens)}
        rid, created = uuid.uuid4().hex[:24], int(time.time())
        if r.chat:
            return {"id": f"chatcmpl-{rid}", "object": "chat.completion", "created": created, "model": r.model,
                    "choices": [{"index": 0, "message": {"role": "assistant", "content": text}, "finish_reason": finish}],
                    "usage": usage}
        return {"id": f"cmpl-{rid}", "object": "text_completion", "created": created, "model": r.model,
                "choices": [{"index": 0, "text": text, "finish_reason": finish}], "usage": usage}

    def metrics(self) -> str:
        s = self.stats
        rows = [("zml_server_requests_total", "counter", s.requests), ("zml_server_requests_failed_total", "counter", s.failed),
                ("zml_server_batches_total", "counter", s.batches), ("zml_server_prompt_tokens_total", "counter", s.prompt_tokens),
                ("zml_server_output_tokens_total", "counter", s.output_tokens), ("zml_server_busy_seconds_total", "counter", round(s.busy_s, 6)),
                ("zml_server_queue_length", "gauge", self.waiting()), ("zml_server_last_batch_size", "gauge", s.last_batch),
                ("zml_server_last_batch_tokens_per_second", "gauge", round(s.last_tok_s, 3))]
        return "".join(f"# TYPE {n} {k}\n{n} {v}\n" for n, k, v in rows)

    def _handler(self):
        server = self

        class Handler(http.server.BaseHTTPRequestHandler):
            protocol_version = "HTTP/1.1"

            def log_message(self, *a):
                pass

            def _send(self, code: int, body, ctype: str = "application/json"):
                data = body.encode() if isinstance(body, str) else json.dumps(body).encode()
                self.send_response(code)
                self.send_header("Content-Type", ctype)
                self.send_header("Content-Length", str(len(data)))
                self.end_headers()
                self.wfile.write(data)

            def do_GET(self):
                if self.path.startswith("/health"):
                    return self._send(200, {"status": "ok", "queue": server.waiting()})
                if self.path.startswith("/metrics"):
                    return self._send(200, server.metrics(), "text/plain; version=0.0.4")
                if self.path.startswith("/v1/models"):
                    return self._send(200, {"object": "list", "data": [{"id": server.model_name, "object": "model"}]})
                self._send(404, {"error": {"message": f"no route {self.path}"}})

            def _tokens(self):
                """`/tokenize` {"prompt": str} or {"messages": [...]} -> {"tokens", "count", "max_model_len"};
                `/detokenize` {"tokens": [ids]} -> {"prompt"}: what a client needs to budget a request."""
                try:
                    body = json.loads(self.rfile.read(int(self.headers.get("Content-Length", 0))) or b"{}")
                    if not isinstance(body, dict):
                        raise ValueError("the body must be a JSON object")
                    if self.path.startswith("/detokenize"):
                        toks = body.get("tokens")
                        if not isinstance(toks, list) or not all(isinstance(t, int) and not isinstance(t, bool) for t in toks):
                            raise ValueError("'tokens' must be a list of token ids")
                        return self._send(200, {"prompt": server.tok.decode(toks)})
                    if isinstance(body.get("messages"), list) and body["messages"]:
                        for m in body["messages"]:
                            if not isinstance(m, dict) or not isinstance(m.get("content"), str):
                                raise ValueError("every message needs a 'content' string")
                        ids = hub.tokenize_chat(server.tok, body["messages"], server.template or "llama3", server.bos)
                    elif isinstance(body.get("prompt"), str):
                        ids = ([server.bos] if server.bos is not None and body.get("add_special_tokens", True) else []) + \
                            server.tok.encode(body["prompt"])
                    else:
                        raise ValueError("give 'prompt' (a string) or 'messages'")
                    self._send(200, {"tokens": ids, "count": len(ids), "max_model_len": server._limit()})
                except (ValueError, json.JSONDecodeError) as e:
                    self._send(400, {"error": {"message": str(e)}})

            def do_POST(self):
                if self.path.startswith(("/tokenize", "/detokenize")):
                    return self._tokens()
                chat = self.path.startswith("/v1/chat/completions")
                if not chat and not self.path.startswith("/v1/completions"):
                    return self._send(404, {"error": {"message": f"no route {self.path}"}})
                try:
                    body = json.loads(self.rfile.read(int(self.headers.get("Content-Length", 0))) or b"{}")
                    if not isinstance(body, dict):
                        raise ValueError("the body must be a JSON object")
                    r = server.submit(body, chat)
                except OverflowError as e:
                    return self._send(429, {"error": {"message": str(e)}})
                except (ValueError, json.JSONDecodeError) as e:
                    return self._send(400, {"error": {"message": str(e)}})
                if r.stream:
                    return self._stream(r)
                r.done.wait()
                if r.error:
                    return self._send(500, {"error": {"message": r.error}})
                self._send(200, server._answer(r))

            def _stream(self, r):
                """Server-sent events: one `data:` line per decode block with the text produced since the last one,
                then a final chunk with the finish reason and `data: [DONE]`."""
                self.send_response(200)
                self.send_header("Content-Type", "text/event-stream")
                self.send_header("Cache-Control", "no-cache")
                self.send_header("Connection", "close")
                self.end_headers()
                rid, created = uuid.uuid4().hex[:24], int(time.time())
                kind = "chat.completion.chunk" if r.chat else "text_completion"
                dec = server.tok.decoder()

                def event(text, finish):
                    choice = ({"index": 0, "delta": {"content": text} if text else {}, "finish_reason": finish} if r.chat
                              else {"index": 0, "text": text, "finish_reason": finish})
                    body = {"id": ("chatcmpl-" if r.chat else "cmpl-") + rid, "object": kind, "created": created,
                            "model": r.model, "choices": [choice]}
                    self.wfile.write(b"data: " + json.dumps(body).encode() + b"\n\n")
                    self.wfile.flush()
                try:
                    finish = "length"
                    stops = StopFilter(r.stop)
                    while True:
                        toks, fin = r.chunks.get()
                        if toks is None:                    # the batch failed
                            event("", "error")
                            break
                        if fin and toks and toks[-1] in server.eos_ids:
                            toks, finish = toks[:-1], "stop"
                        text, stopped = stops.feed("".join(dec.feed_one(t) for t in toks) + (dec.finalize() if fin else ""), fin)
                        if stopped:                         # the answer ends here; the batch runs on without a reader
                            event(text, "stop")
                            break
                        if text or fin:
                            event(text, finish if fin else None)
                        if fin:
                            break
                    self.wfile.write(b"data: [DONE]\n\n")
                    self.wfile.flush()
                except (BrokenPipeError, ConnectionResetError):
                    pass                                    # the client went away; the batch runs to its end
                self.close_connection = True
        return Handler

    # ------------------------------------------------------------------ scheduling (every rank)
    def _next_batch(self) -> Optional[list]:
        """Rank 0: requests to run now - the oldest waiting one, plus what follows within the batching window and has
        the same sampling settings; the others are held for a later batch, ahead of newer arrivals."""
        found, self._held = self._held, []
        if not found:
            try:
                found = [self.queue.get(timeout=self.idle_tick_s)]
            except queue.Empty:
                return None
            deadline = time.perf_counter() + self.batch_window_s
        else:
            deadline = time.perf_counter()                   # held requests have waited a batch already
        while len(found) < self.max_queue:
            left = deadline - time.perf_counter()
            try:
                found.append(self.queue.get(timeout=max(left, 0.0)) if left > 0 else self.queue.get_nowait())
            except queue.Empty:
                break
        batch = [r for r in found if r.sampling == found[0].sampling]
        self._held = [r for r in found if r.sampling != found[0].sampling]
        return batch

    def step(self) -> bool:
        """One scheduling round on every rank: wait for a batch (rank 0), share it, run it.  Returns False once
        `shutdown` was called (on every rank)."""
        batch = self._next_batch() if self.rank == 0 else None
        msg = ("stop", None, None, None) if self._stop.is_set() and batch is None else \
              ("run", [r.ids for r in batch], [r.max_tokens for r in batch], batch[0].sampling) if batch else ("idle", None, None, None)
        if self.comm is not None and self.comm.world > 1:
            msg = self.comm.broadcast_object(msg if self.rank == 0 else None)
            self.comm.check_peers()
        kind, prompts, budgets, sampling = msg
        if kind == "stop":
            return False
        if kind == "idle":
            return True
        t0 = time.perf_counter()
        on_tokens = None
        if self.rank == 0 and batch and any(r.stream for r in batch):
            def on_tokens(i, toks, fin):
                if batch[i].stream:
                    batch[i].chunks.put((list(toks), fin))
        try:
            topk, temperature, seed = sampling
            outs, _ = self.engine.serve(prompts, budgets, SamplingStrategy(topk=topk, temperature=temperature), self.eos_ids,
                                        seed=seed, on_tokens=on_tokens)
            err = None
        except Exception as e:                  # noqa: BLE001 - reported to the callers, the server keeps running
            outs, err = [[] for _ in prompts], f"{type(e).__name__}: {e}"
        dt = time.perf_counter() - t0
        if self.rank == 0 and batch:
            s = self.stats
            s.batches += 1
            s.requests += len(batch)
            s.failed += len(batch) if err else 0
            s.prompt_tokens += sum(len(p) for p in prompts)
            n_out = sum(len(o) for o in outs)
            s.output_tokens += n_out
            s.busy_s += dt
            s.last_batch, s.last_tok_s = len(batch), n_out / max(dt, 1e-9)
            for r, o in zip(batch, outs):
                r.tokens, r.error, r.finished = list(o), err, time.perf_counter()
                if err and r.stream:
                    r.chunks.put((None, True))
                r.done.set()
        return True

    def start_http(self, host: str = "127.0.0.1", port: int = 8000) -> tuple:
        """Rank 0: opens the socket (port 0 = any free port) and serves it on a thread; returns (host, port)."""
        self._httpd = http.server.ThreadingHTTPServer((host, port), self._handler())
        self._httpd.daemon_threads = True
        threading.Thread(target=self._httpd.serve_forever, daemon=True).start()
        return self._httpd.server_address[:2]

    def run(self, host: str = "127.0.0.1", port: int = 8000) -> None:
        """Serves until `shutdown()`; call on every rank."""
        if self.rank == 0 and self._httpd is None:
            self.start_http(host, port)
        while self.step():
            pass
        if self._httpd is not None:
            self._httpd.shutdown()
            self._httpd.server_close()
            self._httpd = None

    def shutdown(self) -> None:
        self._stop.set()
