"""Layer-by-layer check of a model against activations captured from its PyTorch implementation.

    # 1. capture (any machine with transformers):
    #      from zml_b200.utils.activations import ActivationCollector, save_activations
    #      _, acts = ActivationCollector(hf_model, max_layers=..., stop_after_first_step=True)(input_ids)
    #      save_activations("acts.safetensors", acts)
    # 2. compare:
    python examples/llm/model_tests.py --model=/path/to/hf_repo --activations=acts.safetensors

Every decoder layer whose input and output were recorded (`model.layers.N.in.0` / `.out.0`, shape
[batch, seq, hidden]) is run on this framework's weights as a prefill of `batch` sequences of `seq` tokens and
compared with `expect_close`; so is the final norm (`model.norm`).  The reference ships the same check as the
binaries `llama_tests` / `lfm2_tests` (examples/llm/models/llama_tests.zig:56-125, zml/testing.zig:341-455).
"""
from __future__ import annotations

import os
import sys
from dataclasses import dataclass

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from zml_b200 import flags, ops  # noqa: E402
from zml_b200.models import hub  # noqa: E402
from zml_b200.models.llama import AttnMeta  # noqa: E402
from zml_b200.testing import expect_close  # noqa: E402
from zml_b200.utils.activations import load_activations  # noqa: E402


@dataclass
class Args:
    model: str = ""
    activations: str = ""
    device: str = "cuda" if torch.cuda.is_available() else "cpu"
    atol: float = 2e-2
    rtol: float = 2e-2
    min_close: float = 0.99
    help = __doc__


def prefill_meta(batch: int, seq: int, page: int, device) -> tuple[AttnMeta, int]:
    """Metadata of a prefill of `batch` fresh sequences of `seq` tokens; page 0 stays unused."""
    pages_per = (seq + page - 1) // page
    bt = (torch.arange(batch * pages_per, dtype=torch.int32) + 1).view(batch, pages_per)
    pos = torch.arange(seq, dtype=torch.int32).repeat(batch)
    tok = torch.arange(seq)
    slots = torch.cat([bt[b, tok // page].long() * page + tok % page for b in range(batch)]).to(torch.int32)
    qs = [b * seq for b in range(batch + 1)]
    meta = AttnMeta(True, pos.to(device), slots.to(device), bt.to(device),
                    torch.full((batch,), seq, dtype=torch.int32, device=device),
                    torch.tensor(qs, dtype=torch.int32, device=device),
                    total_q_blocks=batch * ((seq + 63) // 64), q_start_host=qs)
    return meta, batch * pages_per + 1


def run(args: Args) -> int:
    if not args.model or not args.activations:
        print(__doc__)
        return 2
    acts = load_activations(args.activations)
    dtype = torch.bfloat16 if args.device != "cpu" else torch.float32
    model, _ = hub.load_model(args.model, device=args.device, dtype=dtype)
    failures, checked = [], 0
    for l in range(model.config.num_hidden_layers):
        name = f"model.layers.{l}"
        if f"{name}.in.0" not in acts or f"{name}.out.0" not in acts:
            continue
        x = acts[f"{name}.in.0"]
        batch, seq, d = x.shape
        page = 64
        meta, pages = prefill_meta(batch, seq, page, args.device)
        kv = torch.zeros(model.kv_cache_shape(pages, page), dtype=dtype, device=args.device)
        if hasattr(model, "alloc_state"):
            print(f"{name}: skipped (layers with recurrent state are checked through the engine)")
            continue
        y = model.layer(l, x.reshape(batch * seq, d).to(args.device, dtype), meta, kv)
        checked += 1
        try:
            expect_close(y.float().cpu().view(batch, seq, d), acts[f"{name}.out.0"].float(), atol=args.atol, rtol=args.rtol,
                         min_close=args.min_close)
            print(f"{name}: ok")
        except AssertionError as e:
            failures.append(name)
            print(f"{name}: MISMATCH\n{e}")
    if "model.norm.in.0" in acts and "model.norm.out.0" in acts:
        x = acts["model.norm.in.0"]
        y = ops.rmsnorm(x.reshape(-1, x.shape[-1]).to(args.device, dtype), model.final_norm, model.config.rms_norm_eps)
        checked += 1
        try:
            expect_close(y.float().cpu().view(x.shape), acts["model.norm.out.0"].float(), atol=args.atol, rtol=args.rtol,
                         min_close=args.min_close)
            print("model.norm: ok")
        except AssertionError as e:
            failures.append("model.norm")
            print(f"model.norm: MISMATCH\n{e}")
    if args.device != "cpu":
        ops.raise_on_status()
    print(f"{checked} modules checked, {len(failures)} mismatches")
    return 1 if failures or not checked else 0


def main(argv=None) -> int:
    return run(flags.parse(sys.argv[1:] if argv is None else argv, Args))


if __name__ == "__main__":
    raise SystemExit(main())
