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
import threading
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
    parts = [f"row-parallel GEMM + all-reduce in one kernel over peer memory up to {fused.fused_max_tokens} tokens"]
    if fused.ll_enabled:
        parts.append("GEMM then in-kernel two-shot all-reduce over peer memory up to 256 tokens")
    parts.append("prefill: " + fused.prefill_collective())
    return "; ".join(parts)


# Headline configurations of the benchmark suite, measured in the same process group after the scaling
# configuration: which ones run at which number of GPUs.
HEADLINE = {8: ["llama-3.1-70b", "qwen3-30b-a3b-nvfp4"], 4: ["qwen3-30b-a3b-nvfp4"], 2: ["qwen3-30b-a3b-nvfp4"]}


_T0 = time.perf_counter()


def progress(comm, msg: str) -> None:
    """One line on stderr (rank 0): where the run is, in seconds since start - what a log of a run that was cut
    short has to show."""
    if comm.rank == 0:
        print(f"[bench +{time.perf_counter() - _T0:6.1f}s] {msg}", file=sys.stderr, flush=True)


def run_workload(name: str, comm, args, steps: int, warmup: int, sample_clocks: bool):
    """Builds the named model, runs `warmup` untimed and `steps` timed serving jobs, tears everything down.
    Returns the metrics on every rank (times are the max over ranks)."""
    import gc

    import torch
    from zml_b200.models.common import SamplingStrategy
    from zml_b200.models.registry import build_model
    from zml_b200.ops import _lib
    from zml_b200.serving import Engine

    wl = dict(WORKLOADS[name])
    if args.batch and name == args.model:
        wl["batch"] = args.batch
    if args.new_tokens and name == args.model:
        wl["new_tokens"] = args.new_tokens
    baseline = args.impl == "baseline"
    progress(comm, f"{name}: building the model on {comm.world} rank(s)")
    model = build_model(name, comm, device=comm.device, seed=args.seed, baseline=baseline,
                        fused=bool(args.fused) and not baseline)
    progress(comm, f"{name}: model built, collectives: {tp_collectives(comm, args, baseline)}")
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

    for i in range(max(warmup, 0)):
        job()
        progress(comm, f"{name}: warm-up job {i + 1} of {warmup} done")
    comm.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(sample_clocks and comm.rank == 0)
    launches0 = _lib.launch_count()
    dev_ms, ttfts, out_tokens, h2d, d2h = 0.0, [], 0, 0, 0
    t0 = time.perf_counter()
    for i in range(steps):
        _, st = job()
        progress(comm, f"{name}: timed job {i + 1} of {steps}: {st.total_ms:.0f} ms")
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
    res = dict(wl=wl, lo=lo, hi=hi, page=page, dev_ms=dev_ms, wall_ms=wall_ms, ttft_p50=ttft_p50, out_tokens=out_tokens,
               h2d=h2d, d2h=d2h, launches=int(launches), clocks=clocks, collectives=tp_collectives(comm, args, baseline))
    # free the model, its KV cache and the symmetric heap before the next configuration is built
    del engine, model
    if getattr(comm, "fused", None) is not None:
        comm.fused.close()
        comm.fused = None
    gc.collect()
    torch.cuda.empty_cache()
    return res


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
    ap.add_argument("--headline", default="auto", choices=["auto", "none"],
                    help="auto: after the scaling configuration also measure the headline configurations that fit this "
                         "number of GPUs (Llama-3.1-70B and the NVFP4 MoE at 8, the MoE at 2 and 4), 3 timed jobs each")
    args = ap.parse_args()

    if args.impl == "reference":
        reference_unavailable()
        return

    import torch
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from zml_b200.parallel.comm import Comm

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200)")
    import faulthandler
    # a run that takes this long prints the Python stack of every thread of every rank (and again later): a cut-off
    # log then shows where each rank was
    faulthandler.dump_traceback_later(float(os.environ.get("ZB_BENCH_STACKS_AFTER_S", "420")), repeat=True, file=sys.stderr)
    comm = Comm.from_env()
    if comm.world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={comm.world}: launch with torch.distributed.run")
    progress(comm, f"process group of {comm.world} rank(s) is up")
    r = run_workload(args.model, comm, args, args.steps, args.warmup, True)
    headline = {}
    printed = threading.Event()

    def emit() -> None:
        """Rank 0 prints the one JSON line (once)."""
        if comm.rank != 0 or printed.is_set():
            return
        printed.set()
        steps = max(args.steps, 1)
        wl, dev_ms, wall_ms = r["wl"], r["dev_ms"], r["wall_ms"]
        tp = f"tp{comm.world}" if comm.world > 1 else "single"
        line = {
            "metric": "output tokens/sec/box",
            "value": r["out_tokens"] / (dev_ms / 1e3),
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
            "ttft_p50_ms": r["ttft_p50"],
            "config": {
                "model": args.model, "global_batch": wl["batch"], "seq_len": [r["lo"], r["hi"]],
                "new_tokens": wl["new_tokens"], "parallelism": tp, "kv_page": r["page"],
                "step": "one full serving job (prefill of all prompts + greedy decode)",
                "l2": "inputs larger than L2 (weights streamed every decode step); no flush",
                "tp_collectives": r["collectives"],
            },
            "clocks": r["clocks"],
            "e2e": {"value": r["out_tokens"] / (wall_ms / 1e3), "unit": "tokens/s",
                    "h2d_bytes_per_step": r["h2d"] // steps, "d2h_bytes_per_step": r["d2h"] // steps,
                    "ms_per_step": wall_ms / steps},
            "gpu_launches": r["launches"],
        }
        if headline:
            line["headline"] = dict(headline)
        print(json.dumps(line), flush=True)

    if args.headline == "auto" and args.impl == "ours" and args.model == "llama-3.1-8b" and HEADLINE.get(comm.world):
        budget_s = float(os.environ.get("ZB_BENCH_HEADLINE_BUDGET_S", "420"))
        deadline_s = float(os.environ.get("ZB_BENCH_DEADLINE_S", "760"))
        current = {"name": None}

        def give_up() -> None:
            # the scaling configuration has been measured; a headline configuration that does not finish must not
            # cost the whole run its result: report what there is and leave (every rank has the same timer)
            if current["name"] is not None:
                headline[current["name"]] = {"aborted": f"not finished {deadline_s:.0f} s into the run"}
            progress(comm, f"deadline: leaving with {current['name']} unfinished")
            emit()
            sys.stdout.flush()
            sys.stderr.flush()
            os._exit(0)

        timer = threading.Timer(max(1.0, deadline_s - (time.perf_counter() - _T0)), give_up)
        timer.daemon = True
        timer.start()
        for name in HEADLINE.get(comm.world, []):
            # every rank takes the same decision: rank 0's clock decides
            go = comm.broadcast_object(time.perf_counter() - _T0 < budget_s)
            if not go:
                headline[name] = {"skipped": f"the run had used its {budget_s:.0f} s when this configuration came up"}
                progress(comm, f"{name}: skipped (time budget)")
                continue
            current["name"] = name
            h = run_workload(name, comm, args, 3, 3, False)
            headline[name] = {"tok_s": h["out_tokens"] / (h["dev_ms"] / 1e3), "ttft_p50_ms": h["ttft_p50"],
                              "ms_per_step": h["dev_ms"] / 3, "steps": 3, "warmup": 3,
                              "e2e_tok_s": h["out_tokens"] / (h["wall_ms"] / 1e3), "global_batch": h["wl"]["batch"],
                              "seq_len": [h["lo"], h["hi"]], "new_tokens": h["wl"]["new_tokens"],
                              "tp_collectives": h["collectives"]}
            current["name"] = None
        timer.cancel()
    emit()
    faulthandler.cancel_dump_traceback_later()
    comm.finish(0)


if __name__ == "__main__":
    main()
