"""Pieces shared by the model zoo: config parsing, generation options, TP helpers.

Mirrors examples/llm/models/common.zig and examples/llm/models.zig of the
reference: `parse_config` reads a HF ``config.json`` ignoring unknown fields,
`detect_model_type` dispatches on ``model_type``, `Shardings` names the two
logical shardings (``model`` and ``experts``) used by every LLM.
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass, field
from enum import Enum
from typing import Optional, Union

import torch


class Phase(Enum):
    prefill = "prefill"
    decode = "decode"

    def is_prefill(self) -> bool:
        return self is Phase.prefill

    def program_name(self, model_name: str, component: str) -> str:
        return f"llm_{model_name}_{self.value}_{component}"


@dataclass
class SamplingStrategy:
    """topk == 1 is greedy; otherwise top-k then Gumbel-max at `temperature` (zml/nn.zig:1999-2005)."""
    topk: int = 1
    temperature: float = 1.0


@dataclass
class GenerationOptions:
    sampling_strategy: SamplingStrategy = field(default_factory=SamplingStrategy)


def read_config_json(repo: str) -> dict:
    """config.json of a repository: a local directory or a URI the VFS can read (hf://, s3://, gs://, https://)."""
    from ..safetensors import read_repo_file
    return json.loads(read_repo_file(repo, "config.json").decode("utf-8"))


def parse_config(cls, source: Union[str, dict]):
    """Builds dataclass `cls` from a HF config (path to a repo, or a dict), ignoring unknown
    fields and raising on missing mandatory ones."""
    obj = read_config_json(source) if isinstance(source, str) else dict(source)
    if hasattr(cls, "from_hf"):
        return cls.from_hf(obj)
    names = {f.name for f in dataclasses.fields(cls)}
    return cls(**{k: v for k, v in obj.items() if k in names})


MODEL_TYPES = {
    "llama": "llama", "qwen3_5": "qwen3_5", "qwen3_5_text": "qwen3_5", "qwen3_5_moe": "qwen3_5_moe",
    "qwen3_5_moe_text": "qwen3_5_moe", "lfm2": "lfm2", "qwen3": "qwen3", "qwen2": "qwen3",
    "qwen3_moe": "qwen3_moe", "mistral": "llama",
}


def detect_model_type(config: dict) -> str:
    """examples/llm/models.zig:189-194: pick the implementation from `model_type`."""
    mt = config.get("model_type")
    if mt is None and "text_config" in config:
        mt = config["text_config"].get("model_type")
    if mt not in MODEL_TYPES:
        raise ValueError(f"unsupported model_type {mt!r}; known: {sorted(set(MODEL_TYPES))}")
    return MODEL_TYPES[mt]


def eos_list(eos: Union[int, list, None]) -> list[int]:
    """`eos_token_id` is an int or a list in HF configs (llama/model.zig:13-16)."""
    if eos is None:
        return []
    return [int(eos)] if isinstance(eos, int) else [int(e) for e in eos]


def shard_range(n: int, rank: int, world: int) -> tuple[int, int]:
    if n % world != 0:
        raise ValueError(f"axis of size {n} is not divisible by {world} partitions")
    per = n // world
    return rank * per, (rank + 1) * per


def kv_head_shard(num_kv_heads: int, rank: int, world: int) -> tuple[int, int]:
    """KV heads of `rank`.  When there are fewer KV heads than partitions each head is
    replicated on world / num_kv_heads consecutive ranks (the reference's `shardableDim`
    stutter, zml/Sharding.zig:230-245)."""
    if num_kv_heads >= world:
        return shard_range(num_kv_heads, rank, world)
    if world % num_kv_heads != 0:
        raise ValueError(f"{num_kv_heads} kv heads cannot be spread over {world} partitions")
    rep = world // num_kv_heads
    return rank // rep, rank // rep + 1


def randn_weight(shape, std: float, seed: int, device, dtype=torch.bfloat16, rows: Optional[tuple[int, int]] = None,
                 cols: Optional[tuple[int, int]] = None, full: bool = True) -> torch.Tensor:
    """Random-init N(0, std) weight.  With `full` the whole tensor is drawn from `seed` and then
    sliced, so every TP degree sees the same global weights; otherwise only the shard is drawn
    (seed mixed with the slice), which is what the large benchmark configs use."""
    g = torch.Generator(device=device)
    if full:
        g.manual_seed(seed)
        w = torch.empty(shape, dtype=dtype, device=device).normal_(0.0, std, generator=g)
        if rows is not None:
            w = w[rows[0]:rows[1]]
        if cols is not None:
            w = w[:, cols[0]:cols[1]]
        return w.contiguous()
    r0, r1 = rows if rows is not None else (0, shape[0])
    sub = [r1 - r0] + list(shape[1:])
    c0 = 0
    if cols is not None:
        c0 = cols[0]
        sub[1] = cols[1] - cols[0]
    g.manual_seed((seed * 1000003 + r0 * 7919 + c0) % (2 ** 63))
    return torch.empty(sub, dtype=dtype, device=device).normal_(0.0, std, generator=g)
