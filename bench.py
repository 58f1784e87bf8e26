#!/usr/bin/env python
"""Headline benchmark: LLM serving throughput (output tokens/s per box) and p50 TTFT.

    python bench.py --gpus N --steps K --warmup W            # N == 1
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

One "step" is one complete serving job of the named configuration: all prompts are
prefilled (varlen, chunked) and then decoded greedily for the configured number of
new tokens through `zml_b200.serving.Engine.generate`, the call a user makes.  The
default configuration is the tensor-parallel one that exists at every N
(Llama-3.1-8B architecture, bf16, 32 concurrent sequences, prompt lengths uniform
in [128, 2048], 512 new tokens, 64-token KV pages); `--model llama-3.1-70b` selects
the 70B / 64 x 2048 / 256 configuration (needs N >= 2 for memory).  Token ids are
synthetic and weights random-init N(0, 0.02): there is no dataset or checkpoint here.

`value` is device-timed (CUDA events around every job, max over ranks).  `e2e` is the
wall-clock figure of the same jobs, from prompts in pinned host memory to generated
ids back on the host.  Inputs (16 GB+ of weights per step) are far larger than L2,
so no explicit L2 flush is needed between iterations.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

WORKLOADS = {
    "llama-3.2-1b": dict(batch=1, prompt=(512, 512), new_tokens=256),
    "llama-3.1-8b": dict(batch=32, prompt=(128, 2048), new_tokens=512),
    "llama-3.1-70b": dict(batch=64, prompt=(2048, 2048), new_tokens=256),
    "qwen3-30b-a3b": dict(batch=128, prompt=(1024, 1024), new_tokens=256),
    "qwen3-30b-a3b-nvfp4": dict(batch=128, prompt=(1024, 1024), new_tokens=256),
    "qwen3.5-9b": dict(batch=32, prompt=(128, 2048), new_tokens=512),
    "qwen3.5-35b-a3b": dict(batch=64, prompt=(1024, 1024), new_tokens=256),
    "lfm2-1.2b": dict(batch=32, prompt=(128, 2048), new_tokens=512),
    "tiny-llama-test": dict(batch=4, prompt=(16, 64), new_tokens=8),
    "tiny-qwen35-test": dict(batch=4, prompt=(16, 64), new_tokens=8),
    "tiny-lfm2-test": dict(batch=4, prompt=(16, 64), new_tokens=8),
}


def reference_unavailable() -> None:
    print(json.dumps({
        "impl": "reference",
        "unavailable": "zml/zml is a Zig+Bazel project (no setup.py/pyproject; pip install fails: "
                       "'Neither setup.py nor pyproject.toml found'); building needs Bazel 9, Zig 0.16 "
                       "and network downloads of PJRT/XLA, flash-attention and flashinfer binaries",
    }))


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs (read-only)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, enabled: bool):
        self.proc = None
        self.path = None
        if enabled:
            try:
                fd, self.path = tempfile.mkstemp(suffix=".csv")
                os.close(fd)
                self.proc = subprocess.Popen(
                    ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200"],
                    stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
            except Exception:
                self.proc = None

    def stop(self, device_index: int = 0) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9 or not f[0].isdigit() or int(f[0]) != device_index:
                    continue
                try:
                    sm.append(float(f[1])); mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            busy = sorted(sm)[len(sm) // 3:] or sm      # drop the idle third (host-side gaps)
            out["sm_mhz"] = sorted(busy)[len(busy) // 2]
            out["sm_max_mhz"] = max(mx)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


def tp_collectives(comm, args, baseline: bool) -> str:
    if comm.world == 1:
        return "none"
    fused = getattr(comm, "fused", None)
    if fused is None or baseline or not args.fused:
        return "nccl"
    tuned = fused.tuned or {}
    note = (f" (measured at start, us per decoder layer: fused {tuned.get('fused_us')}, GEMM + tagged-slot all-reduce "
            f"{tuned.get('ll_us')}, GEMM + NCCL {tuned.get('nccl_us')})") if tuned else ""
    above = "in-kernel two-shot all-reduce over peer memory after the GEMM" if fused.ll_enabled else "NCCL after the GEMM"
    if fused.fused_max_tokens > 0:
        return (f"in-kernel (fused GEMM+all-reduce over peer memory) up to {fused.fused_max_tokens} tokens, {above} up to 256, "
                "NCCL for prefill" + note)
    return f"{above} for decode, NCCL for prefill" + note


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "baseline"])
    ap.add_argument("--model", default="llama-3.1-8b", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--new-tokens", type=int, default=0)
    ap.add_argument("--fused", type=int, default=1, help="fused GEMM+collective kernels for TP (0: NCCL)")
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args()

    if args.impl == "reference":
        reference_unavailable()
        return

    import torch
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from zml_b200.models.common import SamplingStrategy
    from zml_b200.models.registry import build_model
    from zml_b200.parallel.comm import Comm
    from zml_b200.serving import Engine

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200)")
    comm = Comm.from_env()
    if comm.world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={comm.world}: launch with torch.distributed.run")
    wl = dict(WORKLOADS[args.model])
    if args.batch:
        wl["batch"] = args.batch
    if args.new_tokens:
        wl["new_tokens"] = args.new_tokens
    baseline = args.impl == "baseline"
    model = build_model(args.model, comm, device=comm.device, seed=args.seed, baseline=baseline,
                        fused=bool(args.fused) and not baseline)
    lo, hi = wl["prompt"]
    g = torch.Generator().manual_seed(args.seed + 1)
    lens = torch.randint(lo, hi + 1, (wl["batch"],), generator=g).tolist()
    vocab = model.config.vocab_size
    prompts = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]
    page = 64
    per_seq = (hi + wl["new_tokens"] + page - 1) // page + 1
    engine = Engine(model, num_pages=wl["batch"] * per_seq + 8, page_size=page, max_batch=max(wl["batch"], 1),
                    max_seq_len=per_seq * page, max_prefill_tokens=8192)
    strat = SamplingStrategy(topk=1)

    def job():
        return engine.generate(prompts, wl["new_tokens"], strat)

    for _ in range(max(args.warmup, 0)):
        job()
    comm.barrier()
    torch.cuda.synchronize()
    from zml_b200.ops import _lib
    sampler = ClockSampler(comm.rank == 0)
    launches0 = _lib.launch_count()
    dev_ms, ttfts, out_tokens, h2d, d2h = 0.0, [], 0, 0, 0
    t0 = time.perf_counter()
    for _ in range(args.steps):
        _, st = job()
        dev_ms += st.total_ms
        ttfts.extend(st.ttft_ms)
        out_tokens += st.output_tokens
        h2d += st.h2d_bytes
        d2h += st.d2h_bytes
    torch.cuda.synchronize()
    comm.barrier()
    wall_ms = (time.perf_counter() - t0) * 1e3
    launches = _lib.launch_count() - launches0
    clocks = sampler.stop(comm.device.index or 0)
    dev_ms = comm.max_over_ranks(dev_ms)
    wall_ms = comm.max_over_ranks(wall_ms)
    ttfts.sort()
    ttft_p50 = comm.max_over_ranks(ttfts[len(ttfts) // 2] if ttfts else 0.0)
    if comm.rank == 0:
        steps = max(args.steps, 1)
        value = out_tokens / (dev_ms / 1e3)
        tp = f"tp{comm.world}" if comm.world > 1 else "single"
        print(json.dumps({
            "metric": "output tokens/sec/box",
            "value": value,
            "unit": "tokens/s",
            "n_gpus": comm.world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": dev_ms / steps,
            "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic token ids, random-init weights N(0,0.02)",
            "impl": args.impl,
            "ttft_p50_ms": ttft_p50,
            "config": {
                "model": args.model, "global_batch": wl["batch"], "seq_len": [lo, hi],
                "new_tokens": wl["new_tokens"], "parallelism": tp, "kv_page": page,
                "step": "one full serving job (prefill of all prompts + greedy decode)",
                "l2": "inputs larger than L2 (weights streamed every decode step); no flush",
                "tp_collectives": tp_collectives(comm, args, baseline),
            },
            "clocks": clocks,
            "e2e": {"value": out_tokens / (wall_ms / 1e3), "unit": "tokens/s",
                    "h2d_bytes_per_step": h2d // steps, "d2h_bytes_per_step": d2h // steps,
                    "ms_per_step": wall_ms / steps},
            "gpu_launches": int(launches),
        }))
    comm.finish(0)


if __name__ == "__main__":
    main()
