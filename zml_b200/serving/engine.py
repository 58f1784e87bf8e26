"""LLM serving engine: paged KV cache, chunked varlen prefill, CUDA-graph decode.

This is the B200-first counterpart of the reference's session / inference layer
(examples/llm/models/llama/{inference,session}.zig): where the reference runs a
batch-1 dense-cache prefill executable followed by one PJRT execution per layer
per token with a 4-byte device->host read each step, this engine

* keeps K/V in 64-token pages shared by all sequences (block tables),
* prefills many prompts per launch as one flattened varlen batch, in chunks
  bounded by a token budget,
* captures one whole decode step (all layers, sampling, feeding the token back,
  advancing positions / slots on the device) in a CUDA graph per batch bucket, so
  that a decode step costs one graph launch and no host synchronisation,
* reads generated tokens back in blocks from an on-device history.

One Engine instance lives in each tensor-parallel rank; all ranks execute the same
schedule (SPMD), so no control traffic is needed.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Optional, Sequence as Seq

import torch

from .. import ops
from ..models.common import SamplingStrategy
from ..models.llama import AttnMeta
from ..ops import _lib


class OutOfPages(RuntimeError):
    pass


class PagePool:
    """Free list of KV pages.  Page 0 is reserved as the write target of padding rows."""

    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self.free = list(range(num_pages - 1, 0, -1))

    def alloc(self, n: int) -> list[int]:
        if n > len(self.free):
            raise OutOfPages(f"need {n} KV pages, {len(self.free)} free")
        out = self.free[-n:][::-1] if n else []
        del self.free[len(self.free) - n:]
        return out

    def release(self, pages: list[int]) -> None:
        self.free.extend(reversed(pages))

    @property
    def num_free(self) -> int:
        return len(self.free)


@dataclass
class Request:
    prompt: list[int]
    max_new_tokens: int
    rid: int = 0
    pages: list[int] = field(default_factory=list)
    output: list[int] = field(default_factory=list)
    computed: int = 0            # prompt tokens whose KV is in the cache
    finished: bool = False
    ttft_ms: Optional[float] = None
    slot: int = -1               # row in the model's recurrent-state pool (hybrid models)

    @property
    def total_len(self) -> int:
        return len(self.prompt) + len(self.output)


@dataclass
class GenerationStats:
    prefill_ms: float = 0.0
    decode_ms: float = 0.0
    total_ms: float = 0.0
    ttft_ms: list = field(default_factory=list)
    prompt_tokens: int = 0
    output_tokens: int = 0
    decode_steps: int = 0
    h2d_bytes: int = 0
    d2h_bytes: int = 0
    launches: int = 0

    def ttft_p50(self) -> float:
        if not self.ttft_ms:
            return 0.0
        s = sorted(self.ttft_ms)
        return s[len(s) // 2]


def _bucket(n: int) -> int:
    b = 1
    while b < n:
        b <<= 1
    return b


class Engine:
    def __init__(self, model, num_pages: int, page_size: int = 64, max_batch: int = 64,
                 max_seq_len: int = 4096, max_prefill_tokens: int = 8192, use_graphs: Optional[bool] = None,
                 history_steps: int = 1024):
        self.model = model
        self.device = model.device
        self.page_size = page_size
        self.max_batch = max_batch
        self.max_seq_len = max_seq_len
        self.max_pages = (max_seq_len + page_size - 1) // page_size
        self.max_prefill_tokens = max_prefill_tokens
        self.pool = PagePool(num_pages)
        self.kv_cache = torch.zeros(model.kv_cache_shape(num_pages, page_size), dtype=model.dtype,
                                    device=self.device)
        self.on_gpu = self.device.type == "cuda"
        self.use_graphs = self.on_gpu if use_graphs is None else (use_graphs and self.on_gpu)
        self.history_steps = history_steps
        self._graphs: dict = {}
        self.max_graphs = 64                     # captured decode graphs kept (one per batch bucket x sampling settings)
        self._next_rid = 0
        self.seed = 0
        i32 = dict(dtype=torch.int32, device=self.device)
        mb = max_batch
        # static decode buffers (graph inputs / outputs)
        self.d_ids = torch.zeros(mb, **i32)
        self.d_pos = torch.zeros(mb, **i32)
        self.d_seq = torch.zeros(mb, **i32)
        self.d_slot = torch.full((mb,), -1, **i32)
        self.d_bt = torch.zeros((mb, self.max_pages), **i32)
        self.d_hist = torch.zeros((history_steps, mb), **i32)
        self.d_step = torch.zeros(1, **i32)
        # {seed, draws so far} of the top-k sampler: on the device, so that a replayed decode graph draws fresh
        # noise at every step and follows the seed of the current request
        self.d_rng = torch.zeros(2, dtype=torch.int64, device=self.device)
        # recurrent-state slots (models with per-sequence state besides KV pages); the last slot is a
        # scratch row for padding rows of a batch bucket and for graph warm-up passes
        self.num_slots = 2 * mb
        self.scratch_slot = self.num_slots
        self.slot_free = list(range(self.num_slots - 1, -1, -1))
        self.d_sslot = torch.full((mb,), self.scratch_slot, **i32)
        self.d_qs = torch.arange(mb + 1, **i32)
        self.stateful = hasattr(model, "alloc_state")
        if self.stateful:
            model.alloc_state(self.num_slots + 1)
        if self.on_gpu:
            # read by the bounds-checking build of the library only: the extents kernel arguments do not carry
            _lib.set_bounds_extents(num_pages, self.num_slots + 1 if self.stateful else 0)

    # ------------------------------------------------------------------ helpers
    def set_seed(self, seed: int) -> None:
        """Seed of the sampler for what follows; restarts its draw counter."""
        self.seed = int(seed)
        self.d_rng.copy_(torch.tensor([self.seed, 0], dtype=torch.int64))

    def _pin(self, t: torch.Tensor) -> torch.Tensor:
        return t.pin_memory() if self.on_gpu else t

    def _to_dev(self, host: torch.Tensor, stats: Optional[GenerationStats] = None) -> torch.Tensor:
        if stats is not None:
            stats.h2d_bytes += host.numel() * host.element_size()
        return host.to(self.device, non_blocking=True) if self.on_gpu else host

    def new_request(self, prompt: Seq[int], max_new_tokens: int) -> Request:
        r = Request(list(prompt), max_new_tokens, self._next_rid)
        if not r.prompt:
            raise ValueError("empty prompt: a request needs at least one token (e.g. the begin-of-text token)")
        self._next_rid += 1
        need = (len(r.prompt) + max_new_tokens + self.page_size - 1) // self.page_size
        if need > self.max_pages:
            raise ValueError(f"request needs {need} pages, engine allows {self.max_pages} per sequence")
        r.pages = self.pool.alloc(need)
        if self.stateful:
            if not self.slot_free:
                self.pool.release(r.pages)
                raise OutOfPages("no free recurrent-state slot")
            r.slot = self.slot_free.pop()
        return r

    def release(self, r: Request) -> None:
        self.pool.release(r.pages)
        r.pages = []
        if r.slot >= 0:
            self.slot_free.append(r.slot)
            r.slot = -1

    # ------------------------------------------------------------------ prefill
    def _prefill_chunks(self, reqs: list[Request]):
        """Packs (request, start, end) prompt ranges into chunks of at most max_prefill_tokens."""
        chunks, cur, used = [], [], 0
        for r in reqs:
            pos = r.computed
            n = len(r.prompt)
            while pos < n:
                take = min(n - pos, self.max_prefill_tokens - used)
                cur.append((r, pos, pos + take))
                used += take
                pos += take
                if used == self.max_prefill_tokens:
                    chunks.append(cur)
                    cur, used = [], 0
        if cur:
            chunks.append(cur)
        return chunks

    def _run_prefill_chunk(self, chunk, strategy, stats: Optional[GenerationStats]):
        """Runs one flattened varlen prefill.  Returns (finishing requests, their first tokens)."""
        ps = self.page_size
        ids, pos, slots, qs, sl, rows, done = [], [], [], [0], [], [], []
        bt = torch.zeros((len(chunk), self.max_pages), dtype=torch.int32)
        for i, (r, a, b) in enumerate(chunk):
            ids.extend(r.prompt[a:b])
            pos.extend(range(a, b))
            pg = r.pages
            slots.extend(pg[p // ps] * ps + p % ps for p in range(a, b))
            qs.append(qs[-1] + (b - a))
            sl.append(b)
            bt[i, :len(pg)] = torch.tensor(pg, dtype=torch.int32)
            if b == len(r.prompt):
                rows.append(qs[-1] - 1)
                done.append(r)
        t = len(ids)
        host = self._pin(torch.tensor([ids, pos, slots], dtype=torch.int32))
        sslots = [max(r.slot, 0) if self.stateful else 0 for r, _, _ in chunk]
        meta_h = self._pin(torch.tensor(qs + sl + sslots + rows, dtype=torch.int32))
        bt_h = self._pin(bt)
        dev = self._to_dev(host, stats)
        meta_d = self._to_dev(meta_h, stats)
        bt_d = self._to_dev(bt_h, stats)
        nb = len(chunk)
        meta = AttnMeta(True, dev[1], dev[2], bt_d, meta_d[nb + 1:2 * nb + 1], meta_d[:nb + 1],
                        total_q_blocks=sum((b - a + 63) // 64 for _, a, b in chunk),
                        logits_rows=meta_d[3 * nb + 1:] if rows else None, q_start_host=list(qs),
                        state_slots=meta_d[2 * nb + 1:3 * nb + 1] if self.stateful else None)
        if rows:
            toks = self.model.forward(dev[0], meta, self.kv_cache, strategy, self.seed, 0, rng=self.d_rng)
            if strategy is not None and strategy.topk > 1:
                ops.advance_rng(self.d_rng)
        else:
            self.model.hidden_states(dev[0], meta, self.kv_cache)
            toks = None
        for r, a, b in chunk:
            r.computed = b
        return done, toks, t

    # ------------------------------------------------------------------ decode
    def _decode_body(self, b: int, strategy, num_splits, max_seq_len):
        meta = AttnMeta(False, self.d_pos[:b], self.d_slot[:b], self.d_bt[:b], self.d_seq[:b],
                        num_splits=num_splits, max_seq_len=max_seq_len,
                        q_start=self.d_qs[:b + 1] if self.stateful else None,
                        state_slots=self.d_sslot[:b] if self.stateful else None)
        toks = self.model.forward(self.d_ids[:b], meta, self.kv_cache, strategy, self.seed, 0, rng=self.d_rng)
        from ..ops import baseline as _baseline
        if self.on_gpu and not _baseline.enabled():
            rc = _lib.lib().zb_decode_advance_rng(
                toks.data_ptr(), self.d_ids.data_ptr(), self.d_pos.data_ptr(), self.d_seq.data_ptr(),
                self.d_slot.data_ptr(), self.d_bt.data_ptr(), self.d_hist.data_ptr(),
                self.d_step.data_ptr(), b, self.max_pages, self.page_size, self.d_hist.shape[1],
                self.d_hist.shape[0], self.d_rng.data_ptr(), _lib.stream_ptr())
            _lib.check(rc, "zb_decode_advance")
        else:
            self.d_rng[1] += 1
            self.d_ids[:b] = toks
            self.d_pos[:b] += 1
            self.d_seq[:b] = self.d_pos[:b] + 1
            pg = torch.div(self.d_pos[:b], self.page_size, rounding_mode="floor").long()
            page = self.d_bt[:b].gather(1, pg.clamp_max(self.max_pages - 1)[:, None])[:, 0]
            self.d_slot[:b] = page * self.page_size + self.d_pos[:b] % self.page_size
            # graph-capturable history write: row index comes from the device-side step counter
            row = self.d_step.long().clamp_max(self.d_hist.shape[0] - 1)
            self.d_hist[:, :b].index_copy_(0, row, toks[None, :].to(self.d_hist.dtype))
            self.d_step += 1

    def _decode_step(self, b: int, strategy, num_splits, max_seq_len, stats):
        if not self.use_graphs:
            self._decode_body(b, strategy, num_splits, max_seq_len)
            return
        key = (b, strategy.topk, float(strategy.temperature), num_splits)
        g = self._graphs.get(key)
        if g is None:
            while len(self._graphs) >= self.max_graphs:          # sampling settings come from requests: bound the cache
                self._graphs.pop(next(iter(self._graphs)))        # oldest capture first; its memory pool goes with it
            # warm up on a side stream (lazy kernel attributes, allocator), then capture
            saved = [t.clone() for t in (self.d_ids, self.d_pos, self.d_seq, self.d_slot, self.d_step, self.d_hist,
                                         self.d_sslot, self.d_rng)]
            self.d_sslot.fill_(self.scratch_slot)    # the warm-up pass must not advance any real recurrent state
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._decode_body(b, strategy, num_splits, max_seq_len)
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            before = _lib.launch_count()
            with torch.cuda.graph(graph):
                self._decode_body(b, strategy, num_splits, max_seq_len)
            nodes = _lib.launch_count() - before
            # the warm-up and capture passes must not count as decode steps: restore the state
            # (the warm-up really ran; the capture pass did not execute anything)
            for dst, src in zip((self.d_ids, self.d_pos, self.d_seq, self.d_slot, self.d_step, self.d_hist,
                                 self.d_sslot, self.d_rng), saved):
                dst.copy_(src)
            # the warm-up wrote one KV row per sequence at the slot of the next position; the
            # real step writes the same slot with the real values, so nothing needs undoing
            g = (graph, nodes)
            self._graphs[key] = g
        g[0].replay()
        _lib.lib().zb_launch_count_add(g[1])

    # ------------------------------------------------------------------ public API
    def generate(self, prompts: Seq[Seq[int]], max_new_tokens: int,
                 strategy: Optional[SamplingStrategy] = None, eos_ids: Seq[int] = (),
                 sync_interval: int = 64, seed: int = 0) -> tuple[list[list[int]], GenerationStats]:
        """Generates up to max_new_tokens per prompt.  Token ids go host -> device from pinned
        memory, generated ids come back device -> host in blocks of `sync_interval` steps.
        Returns (outputs, stats); stats times are device times (CUDA events)."""
        strategy = strategy or SamplingStrategy()
        self.set_seed(seed)
        stats = GenerationStats()
        if len(prompts) > self.max_batch:
            raise ValueError(f"{len(prompts)} prompts exceed max_batch={self.max_batch}")
        if not prompts:
            return [], stats
        launches0 = _lib.launch_count() if self.on_gpu else 0
        reqs: list[Request] = []
        try:
            for p in prompts:
                reqs.append(self.new_request(p, max_new_tokens))
        except Exception:
            for r in reqs:                       # a request that does not fit must not strand the pages of the others
                self.release(r)
            raise
        stats.prompt_tokens = sum(len(p) for p in prompts)
        ev = (lambda: torch.cuda.Event(enable_timing=True)) if self.on_gpu else None
        t_host0 = time.perf_counter()
        if self.on_gpu:
            e_start = ev(); e_start.record()
        first_tok: dict[int, torch.Tensor] = {}
        ttft_events = []
        # ---------------- prefill
        for chunk in self._prefill_chunks(reqs):
            done, toks, _ = self._run_prefill_chunk(chunk, strategy, stats)
            if self.on_gpu:
                e = ev(); e.record()
            else:
                e = time.perf_counter()
            for i, r in enumerate(done):
                first_tok[r.rid] = toks[i:i + 1]
                ttft_events.append((r, e))
        if self.on_gpu:
            e_prefill = ev(); e_prefill.record()
        t_host1 = time.perf_counter()
        # ---------------- decode set-up: device state of every running sequence
        b = len(reqs)
        bb = _bucket(b) if self.use_graphs else b
        bb = min(bb, self.max_batch)
        ps = self.page_size
        pos = [len(r.prompt) for r in reqs]                # position of the first generated token
        st = torch.zeros((4, bb), dtype=torch.int32)
        st[3, :] = -1
        bt = torch.zeros((bb, self.max_pages), dtype=torch.int32)
        for i, r in enumerate(reqs):
            st[1, i] = pos[i]
            st[2, i] = pos[i] + 1
            st[3, i] = r.pages[pos[i] // ps] * ps + pos[i] % ps
            bt[i, :len(r.pages)] = torch.tensor(r.pages, dtype=torch.int32)
        st_d = self._to_dev(self._pin(st), stats)
        self.d_bt[:bb].copy_(self._to_dev(self._pin(bt), stats))
        self.d_pos[:bb].copy_(st_d[1]); self.d_seq[:bb].copy_(st_d[2]); self.d_slot[:bb].copy_(st_d[3])
        self.d_ids[:bb].zero_()
        self.d_ids[:b].copy_(torch.cat([first_tok[r.rid] for r in reqs]))
        if self.stateful:
            ss = torch.full((bb,), self.scratch_slot, dtype=torch.int32)
            ss[:b] = torch.tensor([r.slot for r in reqs], dtype=torch.int32)
            self.d_sslot[:bb].copy_(self._to_dev(self._pin(ss), stats))
        self.d_step.zero_()
        max_total = max(pos) + max_new_tokens
        num_splits = ops.decode_plan_splits(bb, self.model.hkv, max_total) if self.on_gpu else 1
        # ---------------- decode loop
        outputs = [[] for _ in reqs]
        first_host = self.d_ids[:b].cpu() if max_new_tokens > 0 else None
        if first_host is not None:
            stats.d2h_bytes += b * 4
            for i in range(b):
                outputs[i].append(int(first_host[i]))
        eos = set(int(e) for e in eos_ids)
        alive = [not (eos and outputs[i] and outputs[i][-1] in eos) for i in range(b)]
        steps_total = max_new_tokens - 1
        done_steps = 0
        comm = getattr(self.model, "comm", None)
        while done_steps < steps_total and any(alive):
            if comm is not None:
                comm.check_peers()       # a rank that stopped is noticed here, before kernels that wait on it launch
            n = min(sync_interval, steps_total - done_steps, self.history_steps)
            self.d_step.zero_()
            for _ in range(n):
                self._decode_step(bb, strategy, num_splits, max_total, stats)
            hist = self.d_hist[:n, :b].cpu()              # device -> host read (synchronises)
            stats.d2h_bytes += n * b * 4
            for i in range(b):
                if not alive[i]:
                    continue
                for s in range(n):
                    tok = int(hist[s, i])
                    outputs[i].append(tok)
                    if tok in eos:
                        alive[i] = False
                        break
            done_steps += n
            stats.decode_steps += n
        if self.on_gpu:
            e_end = ev(); e_end.record()
            torch.cuda.synchronize()
            stats.prefill_ms = e_start.elapsed_time(e_prefill)
            stats.decode_ms = e_prefill.elapsed_time(e_end)
            stats.total_ms = e_start.elapsed_time(e_end)
            stats.ttft_ms = [e_start.elapsed_time(e) for _, e in ttft_events]
            stats.launches = _lib.launch_count() - launches0
        else:
            t_end = time.perf_counter()
            stats.prefill_ms = (t_host1 - t_host0) * 1e3
            stats.total_ms = (t_end - t_host0) * 1e3
            stats.decode_ms = stats.total_ms - stats.prefill_ms
            stats.ttft_ms = [(e - t_host0) * 1e3 for _, e in ttft_events]
        for (r, _), t in zip(ttft_events, stats.ttft_ms):
            r.ttft_ms = t
        stats.output_tokens = sum(len(o) for o in outputs)
        for r, o in zip(reqs, outputs):
            r.output = o
            r.finished = True
            self.release(r)
        if self.on_gpu:
            ops.raise_on_status()
        return outputs, stats


    # ------------------------------------------------------------------ continuous batching
    def serve(self, prompts: Seq[Seq[int]], max_new_tokens, strategy: Optional[SamplingStrategy] = None,
              eos_ids: Seq[int] = (), sync_interval: int = 16, seed: int = 0,
              arrivals: Optional[Seq[int]] = None, on_tokens=None) -> tuple[list[list[int]], GenerationStats]:
        """Continuous batching over any number of prompts: at most `max_batch` sequences decode together; between two
        decode blocks (`sync_interval` steps, one device -> host read) finished sequences leave - their batch row,
        KV pages and recurrent-state slot are free again - and waiting prompts are admitted as soon as a row and
        enough pages are free: they are prefilled and join the next block.  `max_new_tokens` is one number or one per
        prompt; `arrivals[i]` (optional) is the first block at which prompt i may be admitted.  `on_tokens(i, new_tokens,
        finished)` (optional) is called on the host after every block with what prompt i produced since the last call.

        On a multi-rank job every rank calls this with the same arguments; a rank that stopped or left is noticed
        on the host before the next block is launched (`Comm.check_peers`)."""
        strategy = strategy or SamplingStrategy()
        self.set_seed(seed)
        stats = GenerationStats()
        n_req = len(prompts)
        budget = [int(max_new_tokens)] * n_req if isinstance(max_new_tokens, int) else [int(m) for m in max_new_tokens]
        for i, (p, m) in enumerate(zip(prompts, budget)):     # reject what can never run before anything is admitted
            if len(p) == 0:
                raise ValueError(f"prompt {i} is empty: a request needs at least one token")
            need = (len(p) + m + self.page_size - 1) // self.page_size
            if need > self.max_pages:
                raise ValueError(f"prompt {i} needs {need} pages, engine allows {self.max_pages} per sequence")
        eos = set(int(e) for e in eos_ids)
        cap = min(self.max_batch, max(1, n_req))
        bb = min(_bucket(cap) if self.use_graphs else cap, self.max_batch)
        cap = min(cap, bb)
        ps = self.page_size
        max_total = max((len(p) + m for p, m in zip(prompts, budget)), default=1)
        num_splits = ops.decode_plan_splits(bb, self.model.hkv, max_total) if self.on_gpu else 1
        launches0 = _lib.launch_count() if self.on_gpu else 0
        outputs: list[list[int]] = [[] for _ in range(n_req)]
        waiting = list(range(n_req))
        running: dict[int, tuple[int, Request]] = {}          # batch row -> (prompt index, request)
        free_rows = list(range(cap - 1, -1, -1))
        # host mirror of the decode state; rows without a sequence point at the reserved page 0 and write no KV
        ids_h = torch.zeros(bb, dtype=torch.int32)
        pos_h = torch.zeros(bb, dtype=torch.int32)
        bt_h = torch.zeros((bb, self.max_pages), dtype=torch.int32)
        ss_h = torch.full((bb,), self.scratch_slot if self.stateful else 0, dtype=torch.int32)
        t0 = time.perf_counter()
        admitted_at: dict[int, float] = {}
        ttft: dict[int, float] = {}
        block = 0
        dirty = False                                         # a row's owner changed since the last upload
        comm = getattr(self.model, "comm", None)

        reported = [0] * n_req
        finished_idx: set = set()

        def report() -> None:
            if on_tokens is None:
                return
            for i in range(n_req):
                if reported[i] < 0:                                       # the final call has been made
                    continue
                new = outputs[i][reported[i]:]
                fin = i in finished_idx
                if new or fin:
                    reported[i] = -1 if fin else len(outputs[i])
                    on_tokens(i, new, fin)

        def finish(row: int) -> None:
            nonlocal dirty
            dirty = True
            idx, r = running.pop(row)
            finished_idx.add(idx)
            r.output, r.finished = outputs[idx], True
            self.release(r)
            free_rows.append(row)
            ids_h[row], pos_h[row] = 0, 0
            bt_h[row].zero_()
            ss_h[row] = self.scratch_slot if self.stateful else 0

        while waiting or running:
            if comm is not None:
                comm.check_peers()
            # ---------------- admission
            fresh: list[tuple[int, int, Request]] = []
            while waiting and free_rows and (arrivals is None or arrivals[waiting[0]] <= block):
                idx = waiting[0]
                try:
                    r = self.new_request(prompts[idx], budget[idx])
                except OutOfPages:
                    if not running and not fresh:
                        raise
                    break
                waiting.pop(0)
                fresh.append((free_rows.pop(), idx, r))
                admitted_at[idx] = time.perf_counter()
            if fresh:
                dirty = True
                stats.prompt_tokens += sum(len(r.prompt) for _, _, r in fresh)
                first: dict[int, int] = {}
                for chunk in self._prefill_chunks([r for _, _, r in fresh]):
                    done, toks, _ = self._run_prefill_chunk(chunk, strategy, stats)
                    if done:
                        host = toks.cpu()
                        stats.d2h_bytes += len(done) * 4
                        for i, r in enumerate(done):
                            first[r.rid] = int(host[i])
                now = time.perf_counter()
                for row, idx, r in fresh:
                    tok = first[r.rid]
                    ttft[idx] = (now - admitted_at[idx]) * 1e3
                    running[row] = (idx, r)
                    if budget[idx] > 0:
                        outputs[idx].append(tok)
                    n0 = len(r.prompt)
                    ids_h[row], pos_h[row] = tok, n0
                    bt_h[row].zero_()
                    bt_h[row, :len(r.pages)] = torch.tensor(r.pages, dtype=torch.int32)
                    ss_h[row] = r.slot if self.stateful else 0
                    if len(outputs[idx]) >= budget[idx] or tok in eos:
                        finish(row)
            if not running:
                block += 1
                report()
                continue
            # ---------------- device state (only when the set of sequences changed: a row that lost its sequence
            # must stop writing KV before its pages go to another request)
            if dirty:
                dirty = False
                pg = torch.div(pos_h, ps, rounding_mode="floor").long().clamp_max(self.max_pages - 1)
                slot_h = bt_h.gather(1, pg[:, None])[:, 0] * ps + pos_h % ps
                live = torch.zeros(bb, dtype=torch.bool)
                live[list(running)] = True
                slot_h = torch.where(live, slot_h, torch.full_like(slot_h, -1))
                st = self._to_dev(self._pin(torch.stack([ids_h, pos_h, pos_h + 1, slot_h.to(torch.int32), ss_h])), stats)
                self.d_ids[:bb].copy_(st[0]); self.d_pos[:bb].copy_(st[1]); self.d_seq[:bb].copy_(st[2])
                self.d_slot[:bb].copy_(st[3])
                if self.stateful:
                    self.d_sslot[:bb].copy_(st[4])
                self.d_bt[:bb].copy_(self._to_dev(self._pin(bt_h), stats))
            # ---------------- one decode block
            left = max(budget[idx] - len(outputs[idx]) for idx, _ in running.values())
            n = max(1, min(sync_interval, self.history_steps, left))
            self.d_step.zero_()
            for _ in range(n):
                self._decode_step(bb, strategy, num_splits, max_total, stats)
            hist = self.d_hist[:n, :bb].cpu()                  # device -> host read (synchronises)
            stats.d2h_bytes += n * bb * 4
            stats.decode_steps += n
            pos_h += n                                         # every row advanced n positions on the device
            ids_h.copy_(hist[n - 1])
            for row in list(running):
                idx, _ = running[row]
                for s_ in range(n):
                    tok = int(hist[s_, row])
                    outputs[idx].append(tok)
                    if tok in eos or len(outputs[idx]) >= budget[idx]:
                        finish(row)
                        break
            block += 1
            report()
        if self.on_gpu:
            torch.cuda.synchronize()
            stats.launches = _lib.launch_count() - launches0
            ops.raise_on_status()
        stats.total_ms = (time.perf_counter() - t0) * 1e3
        stats.ttft_ms = [ttft[i] for i in range(n_req)]
        stats.output_tokens = sum(len(o) for o in outputs)
        return outputs, stats


class Session:
    """One multi-turn conversation on an Engine (examples/llm/models/llama/session.zig of the
    reference: `runPrefill` / `runDecode` over a KV cache that persists across turns).
    The KV pages for `max_tokens` are reserved when the session is created."""

    def __init__(self, engine: Engine, max_tokens: int, strategy: Optional[SamplingStrategy] = None,
                 eos_ids: Seq[int] = (), seed: int = 0):
        self.engine = engine
        self.max_tokens = min(max_tokens, engine.max_pages * engine.page_size)
        self.strategy = strategy or SamplingStrategy()
        self.eos = set(int(e) for e in eos_ids)
        self.tokens: list[int] = []
        self.req = Request([], 0, -1)
        self.req.pages = engine.pool.alloc((self.max_tokens + engine.page_size - 1) // engine.page_size)
        if engine.stateful:
            self.req.slot = engine.slot_free.pop()
        self._next: Optional[int] = None
        engine.set_seed(seed)

    def close(self) -> None:
        self.engine.release(self.req)

    def remaining(self) -> int:
        return self.max_tokens - len(self.tokens)

    def run_prefill(self, new_tokens: Seq[int]) -> int:
        """Appends `new_tokens` to the conversation, computes their KV, returns the next token."""
        if len(self.tokens) + len(new_tokens) >= self.max_tokens:
            raise ValueError("PromptTooLong: not enough tokens remaining; use a higher seqlen")
        eng = self.engine
        self.tokens.extend(int(t) for t in new_tokens)
        self.req.prompt = self.tokens
        tok = None
        for chunk in eng._prefill_chunks([self.req]):
            _, toks, _ = eng._run_prefill_chunk(chunk, self.strategy, None)
            if toks is not None:
                tok = int(toks[0])
        self._next = tok
        return tok

    def run_decode(self, on_token=None, max_new_tokens: Optional[int] = None, stream_interval: int = 1) -> list[int]:
        """Generates until EOS or the token budget; `on_token(id)` is called per token.  The host reads the generated
        ids every `stream_interval` decode steps: 1 is the reference's loop (one device -> host read per token, lowest
        latency to the first character), larger values let the GPU run ahead (steps past an EOS inside a block are
        discarded)."""
        eng = self.engine
        out: list[int] = []
        if self._next is None:
            return out
        budget = self.remaining() - 1 if max_new_tokens is None else min(max_new_tokens, self.remaining() - 1)
        ps = eng.page_size
        pos = len(self.tokens)
        i32 = dict(dtype=torch.int32, device=eng.device)
        eng.d_ids[:1] = torch.tensor([self._next], **i32)
        eng.d_pos[:1] = torch.tensor([pos], **i32)
        eng.d_seq[:1] = torch.tensor([pos + 1], **i32)
        eng.d_slot[:1] = torch.tensor([self.req.pages[pos // ps] * ps + pos % ps], **i32)
        eng.d_bt[:1].zero_()
        eng.d_bt[0, :len(self.req.pages)] = torch.tensor(self.req.pages, **i32)
        if eng.stateful:
            eng.d_sslot[:1] = torch.tensor([self.req.slot], **i32)
        splits = ops.decode_plan_splits(1, eng.model.hkv, self.max_tokens) if eng.on_gpu else 1
        pending = [self._next]
        done = False
        while not done:
            for tok in pending:
                out.append(tok)
                self.tokens.append(tok)
                if on_token is not None:
                    on_token(tok)
                if tok in self.eos or len(out) >= budget:
                    done = True
                    break
            if done:
                break
            n = max(1, min(stream_interval, budget - len(out), eng.history_steps))
            eng.d_step.zero_()
            for _ in range(n):
                eng._decode_step(1, self.strategy, splits, self.max_tokens, None)
            pending = eng.d_hist[:n, 0].cpu().tolist() if n > 1 else [int(eng.d_ids[0])]
        self._next = None
        self.req.computed = len(self.tokens) - 1
        return out
