"""Open a model repository (config.json + safetensors + tokenizer) and build the matching
model, as `LoadedModel.load` does in the reference (examples/llm/models.zig:27-95)."""
from __future__ import annotations

import logging
import os
import time
from typing import Optional

import torch

from ..io import TensorStore
from ..parallel.comm import Comm
from ..tokenizer import Tokenizer
from . import common
from .registry import model_class_for

log = logging.getLogger("zml_b200.llm")


def open_repo(path: str):
    """(config dict, TensorStore, repo dir) for a checkpoint path (directory, .safetensors or index)."""
    from .. import safetensors
    repo = safetensors.resolve_model_repo(path)
    cfg = common.read_config_json(repo)
    is_file = path.endswith((".safetensors", ".index.json")) if safetensors.is_uri(path) else os.path.isfile(path)
    entry = path if is_file else safetensors.resolve_model_entrypoint(repo)
    return cfg, TensorStore.from_path(entry), repo


def load_model(path: str, comm: Optional[Comm] = None, device="cpu", dtype=torch.bfloat16, fused: bool = True):
    """Returns (model, tokenizer or None).  Weights are streamed shard-by-shard for this rank."""
    cfg, store, repo = open_repo(path)
    config_cls, model_cls = model_class_for(cfg)
    config = config_cls.from_hf(cfg.get("text_config", cfg) if "hidden_size" not in cfg else cfg)
    comm = comm or Comm.single(torch.device(device))
    t0 = time.perf_counter()
    model = model_cls(config, comm, device=device, dtype=dtype)
    if model_cls.__name__ == "LlamaModel":
        # dense decoder: the generic Loader cuts the checkpoint by `Sharding.placement`
        from ..platform import CpuOptions, CreateOptions, Platform, Target
        on_gpu = torch.device(device).type == "cuda"
        if on_gpu and comm.world == 1 and torch.device(device).index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        platform = (Platform.init(Target.cuda, comm=comm) if on_gpu and comm.world > 1 else
                    Platform.init(Target.cpu, CreateOptions(cpu=CpuOptions(device_count=1)), comm=comm) if not on_gpu else None)
        model = model.load(store, platform=platform)
    else:
        model = model.load(store)
    dt = time.perf_counter() - t0
    nbytes = model.weight_bytes()
    log.info("Loaded weights [%.2f GiB, %.2fs, %.2f GiB/s]", nbytes / 2 ** 30, dt, nbytes / 2 ** 30 / max(dt, 1e-9))
    if fused and comm.world > 1 and torch.device(device).type == "cuda":
        from ..parallel import symm
        comm.fused = symm.SymmetricContext.create(comm, config.hidden_size, staging_elems=8192 * config.hidden_size)
    tok = None
    from .. import safetensors
    for name in ("tokenizer.json", "tokenizer.model"):
        if not safetensors.repo_file_exists(repo, name):
            continue
        if safetensors.is_uri(repo):
            if name.endswith(".json"):
                tok = Tokenizer.from_bytes(safetensors.read_repo_file(repo, name))
            else:                           # SentencePiece wants a file: fetch it next to the other temporaries
                import tempfile
                with tempfile.NamedTemporaryFile(suffix=".model", delete=False) as f:
                    f.write(safetensors.read_repo_file(repo, name))
                tok = Tokenizer.from_file(f.name)
        else:
            tok = Tokenizer.from_file(os.path.join(repo, name))
        break
    return model, tok


def chat_template(model_type: str) -> str:
    return "chatml" if model_type.startswith(("qwen", "lfm")) else "llama3"


def tokenize_prompt(tok: Tokenizer, prompt: str, template: str, bos: Optional[int], first_turn: bool = True) -> list[int]:
    """Chat-template tokenisation built from special tokens, as the reference's sessions do
    (llama: examples/llm/models/llama/session.zig:100-146; ChatML for the Qwen / LFM families)."""
    if template == "llama3":
        sh, eh, eot = tok.token_id("<|start_header_id|>"), tok.token_id("<|end_header_id|>"), tok.token_id("<|eot_id|>")
        if None in (sh, eh, eot):
            return ([bos] if first_turn and bos is not None else []) + tok.encode(prompt)
        nl = tok.encode("\n")
        out = [bos, sh] if first_turn and bos is not None else ([sh] if first_turn else [eot] + nl + [sh])
        out += tok.encode("user") + [eh] + nl + tok.encode(prompt) + [eot] + nl + [sh] + tok.encode("assistant") + [eh] + nl
        return out
    ims, ime = tok.token_id("<|im_start|>"), tok.token_id("<|im_end|>")
    if None in (ims, ime):
        return tok.encode(prompt)
    nl = tok.encode("\n")
    pre = [] if first_turn else [ime] + nl
    return pre + [ims] + tok.encode("user") + nl + tok.encode(prompt) + [ime] + nl + [ims] + tok.encode("assistant") + nl


CHAT_ROLES = ("system", "user", "assistant", "tool")


def tokenize_chat(tok: Tokenizer, messages, template: str, bos: Optional[int]) -> list[int]:
    """A whole conversation - [{"role": "system" | "user" | "assistant" | "tool", "content": str}, ...] - in the same
    token layout as `tokenize_prompt` builds turn by turn, ending with the header of the assistant's next turn.  A
    conversation of user and assistant turns gives exactly the tokens the chat session accumulates."""
    msgs = []
    for m in messages:
        role = str(m.get("role", "user"))
        if role not in CHAT_ROLES:
            raise ValueError(f"unknown role {role!r}; one of {', '.join(CHAT_ROLES)}")
        msgs.append((role, str(m["content"])))
    nl = tok.encode("\n")
    if template == "llama3":
        sh, eh, eot = tok.token_id("<|start_header_id|>"), tok.token_id("<|end_header_id|>"), tok.token_id("<|eot_id|>")
        if None in (sh, eh, eot):
            return ([bos] if bos is not None else []) + [t for _, c in msgs for t in tok.encode(c)]
        out = [bos] if bos is not None else []
        for role, content in msgs:
            out += [sh] + tok.encode(role) + [eh] + nl + tok.encode(content) + [eot] + nl
        return out + [sh] + tok.encode("assistant") + [eh] + nl
    ims, ime = tok.token_id("<|im_start|>"), tok.token_id("<|im_end|>")
    if None in (ims, ime):
        return [t for _, c in msgs for t in tok.encode(c)]
    out = []
    for role, content in msgs:
        out += [ims] + tok.encode(role) + nl + tok.encode(content) + [ime] + nl
    return out + [ims] + tok.encode("assistant") + nl
