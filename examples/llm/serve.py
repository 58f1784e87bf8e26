#!/usr/bin/env python
"""HTTP server for a HF-format checkpoint: OpenAI-style completions on top of continuous batching.

    python examples/llm/serve.py --model=<repo dir | hf://org/repo | s3://... > [--host=127.0.0.1] [--port=8000]
        [--max-batch=32] [--seqlen=4096] [--pages=0] [--topk=1] [--temperature=1.0] [--window-ms=20]
    torchrun --nproc-per-node=8 --master-addr 127.0.0.1 examples/llm/serve.py --model=...     # tensor / expert parallel

Routes: POST /v1/completions {"prompt": "..." | [ids], "max_tokens": n}, POST /v1/chat/completions {"messages": [...]},
GET /v1/models, /health, /metrics (Prometheus).  Rank 0 owns the socket; every rank runs the same batches.
"""
from __future__ import annotations

import logging
import os
import signal
import sys
from dataclasses import dataclass
from typing import Optional

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch  # noqa: E402

from zml_b200 import flags  # noqa: E402
from zml_b200.models import hub  # noqa: E402
from zml_b200.models.common import SamplingStrategy  # noqa: E402
from zml_b200.parallel.comm import Comm  # noqa: E402
from zml_b200.serving.engine import Engine  # noqa: E402
from zml_b200.serving.server import Server  # noqa: E402

log = logging.getLogger("serve")


@dataclass
class Args:
    model: str
    host: str = "127.0.0.1"
    port: int = 8000
    max_batch: int = 32
    seqlen: int = 4096
    pages: int = 0              # 0: enough pages for max_batch sequences of seqlen tokens
    topk: int = 1
    temperature: float = 1.0
    window_ms: float = 20.0
    cpu: bool = False
    help = __doc__


def main(argv=None) -> int:
    logging.basicConfig(level=logging.INFO, format="%(levelname)s(%(name)s): %(message)s")
    args = flags.parse(argv, Args)
    comm = Comm.from_env()
    device = torch.device("cpu") if args.cpu or not torch.cuda.is_available() else comm.device
    model, tok = hub.load_model(args.model, comm, device, torch.bfloat16 if device.type == "cuda" else torch.float32)
    if tok is None:
        raise SystemExit("the repository has no tokenizer.json / tokenizer.model")
    cfg = model.config
    page = 64 if device.type == "cuda" else 16
    pages = args.pages or args.max_batch * ((args.seqlen + page - 1) // page) + 1
    engine = Engine(model, num_pages=pages, page_size=page, max_batch=args.max_batch, max_seq_len=args.seqlen)
    eos = cfg.eos_ids() if hasattr(cfg, "eos_ids") else []
    server = Server(engine, tok, comm, model_name=os.path.basename(args.model.rstrip("/")),
                    template=hub.chat_template(getattr(cfg, "model_type", "llama")), bos=getattr(cfg, "bos_token_id", None),
                    eos_ids=eos, strategy=SamplingStrategy(topk=args.topk, temperature=args.temperature),
                    batch_window_s=args.window_ms / 1e3)
    if comm.rank == 0:
        host, port = server.start_http(args.host, args.port)
        log.info("serving %s on http://%s:%d (%d rank(s), max batch %d, %d KV pages)", args.model, host, port, comm.world,
                 args.max_batch, pages)
        signal.signal(signal.SIGINT, lambda *_: server.shutdown())
        signal.signal(signal.SIGTERM, lambda *_: server.shutdown())
    server.run()
    comm.finish(0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
