#!/usr/bin/env python
"""LLM CLI (the reference's `examples/llm`): load a HF-format checkpoint and chat with it.

    python examples/llm/main.py --model=<repo dir | .safetensors | index.json | hf://org/repo | s3://... | gs://... | https://...> [--prompt=...]
        [--system=...] [--seqlen=2048] [--topk=1] [--temperature=1.0] [--seed=0] [--no-chat-template] [--profile]
        [--backend=b200|vanilla|attnd] [--attnd-ip=IP:PORT]

--backend picks the attention implementation (default: this library's paged kernels; `vanilla` is PyTorch SDPA on K/V
gathered from the pages); --attnd-ip registers a remote attention daemon at IP:PORT and prefers it (dense decoder
models, one conversation).  --system puts a system message in front of the first turn (chat template only).

Without --prompt an interactive chat loop starts (history in ~/.llm_chat_history).  For
tensor / expert parallelism launch one process per GPU:
    python -m torch.distributed.run --nproc-per-node=8 --master-addr 127.0.0.1 examples/llm/main.py --model=...
Supported `model_type`s: llama, mistral, qwen2, qwen3, qwen3_moe, qwen3_5, qwen3_5_moe, lfm2.
"""
from __future__ import annotations

import logging
import os
import sys
import time
from dataclasses import dataclass
from typing import Optional

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch  # noqa: E402

from zml_b200 import flags  # noqa: E402
from zml_b200.models import hub  # noqa: E402
from zml_b200.models.common import SamplingStrategy  # noqa: E402
from zml_b200.parallel.comm import Comm  # noqa: E402
from zml_b200.profiling import Profiler  # noqa: E402
from zml_b200.serving.engine import Engine, Session  # noqa: E402

log = logging.getLogger("llm")


@dataclass
class Args:
    model: str
    prompt: Optional[str] = None
    system: Optional[str] = None
    seqlen: int = 2048
    topk: int = 1
    temperature: float = 1.0
    seed: int = 0
    max_new_tokens: int = 0
    no_chat_template: bool = False
    profile: bool = False
    cpu: bool = False
    backend: Optional[str] = None
    attnd_ip: Optional[str] = None
    help = __doc__


class Chat:
    def __init__(self, session: Session, tok, template: Optional[str], bos, rank: int, comm=None, system: Optional[str] = None):
        self.session, self.tok, self.template, self.bos, self.rank = session, tok, template, bos, rank
        self.comm = comm
        self.system = system
        self.first = True

    def run_once(self, prompt: str, max_new: Optional[int]) -> str:
        if self.tok is None:
            ids = [int(x) for x in prompt.split()]
        elif self.template is None:
            ids = self.tok.encode(prompt)
        elif self.first and self.system:
            ids = hub.tokenize_chat(self.tok, [{"role": "system", "content": self.system}, {"role": "user", "content": prompt}],
                                    self.template, self.bos)
        else:
            ids = hub.tokenize_prompt(self.tok, prompt, self.template, self.bos, self.first)
        self.first = False
        if self.rank == 0:
            sys.stdout.write("\x1b[2mprefill...\x1b[0m")
            sys.stdout.flush()
        t0 = time.perf_counter()
        self.session.run_prefill(ids)
        ttft = time.perf_counter() - t0
        if self.rank == 0:
            sys.stdout.write("\r          \r")
        dec = self.tok.decoder() if self.tok is not None else None
        pieces = []

        def on_token(t: int):
            if t in self.session.eos:
                return
            s = dec.next(t) if dec is not None else f"{t} "
            pieces.append(s)
            if self.rank == 0:
                sys.stdout.write(s)
                sys.stdout.flush()

        t0 = time.perf_counter()
        out = self.session.run_decode(on_token, max_new)
        dt = time.perf_counter() - t0
        if self.rank == 0:
            tps = len(out) / dt if dt > 0 else 0.0
            sys.stdout.write(f"\n\n\x1b[36mdecode\x1b[0m \x1b[2m{dt:.2f}s · {tps:.1f}tok/s · ttft {ttft * 1e3:.0f}ms\x1b[0m\n\n")
            sys.stdout.flush()
        return "".join(pieces)

    def loop(self, max_new: Optional[int]) -> None:
        try:
            import readline
            hist = os.path.expanduser("~/.llm_chat_history")
            if os.path.exists(hist):
                readline.read_history_file(hist)
        except Exception:
            readline, hist = None, None
        while self.session.remaining() > 8:
            # rank 0 owns the terminal; the others get the line (or the end of the chat) from it
            line = None
            if self.rank == 0:
                try:
                    line = input("> ")
                except (EOFError, KeyboardInterrupt):
                    line = None
            if self.comm is not None and self.comm.world > 1:
                line = self.comm.broadcast_object(line)
            if line is None:
                break
            if not line.strip():
                continue
            self.run_once(line, max_new)
            if readline is not None:
                try:
                    readline.write_history_file(hist)
                except OSError:
                    pass
        print(f"\x1b[2m{len(self.session.tokens)}/{self.session.max_tokens} tokens used\x1b[0m")


def main(argv=None) -> int:
    logging.basicConfig(level=logging.INFO, format="%(levelname)s(%(name)s): %(message)s")
    args = flags.parse(argv, Args)
    comm = Comm.from_env()
    if comm.rank == 0 and sys.stderr.isatty():
        from zml_b200 import logo
        logo.write(sys.stderr)
    device = torch.device("cpu") if args.cpu or not torch.cuda.is_available() else comm.device
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    model, tok = hub.load_model(args.model, comm, device, dtype)
    cfg = model.config
    backend = "attnd" if args.attnd_ip and args.backend in (None, "attnd") else (args.backend or "b200")
    if backend != "b200":
        if not hasattr(model, "set_attention_backend"):
            raise SystemExit(f"--backend={backend} is implemented for the dense decoder models, not for {type(model).__name__}")
        addr = None
        if backend == "attnd":
            if not args.attnd_ip:
                raise SystemExit("--backend=attnd needs --attnd-ip=IP:PORT")
            host, _, port = args.attnd_ip.rpartition(":")
            addr = (host or "127.0.0.1", int(port))
        model.set_attention_backend(backend, addr)
        log.info("attention backend: %s%s", backend, f" at {addr[0]}:{addr[1]}" if addr else "")
    page = 64
    engine = Engine(model, num_pages=(args.seqlen + page - 1) // page + 2, page_size=page, max_batch=1,
                    max_seq_len=args.seqlen, max_prefill_tokens=min(8192, args.seqlen),
                    use_graphs=False if backend == "attnd" else None)     # the daemon is reached from the host: no graph
    strategy = SamplingStrategy(topk=args.topk, temperature=args.temperature)
    session = Session(engine, args.seqlen, strategy, cfg.eos_ids(), args.seed)
    template = None if args.no_chat_template or tok is None else hub.chat_template(getattr(cfg, "model_type", "llama"))
    chat = Chat(session, tok, template, getattr(cfg, "bos_token_id", None), comm.rank, comm, args.system)
    max_new = args.max_new_tokens or None
    prof = Profiler().start() if args.profile else None
    if args.prompt is not None:
        chat.run_once(args.prompt, max_new)
    else:
        chat.loop(max_new)
    if prof is not None:
        log.info("profile written: %s", prof.stop())
    session.close()
    comm.finish(0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
