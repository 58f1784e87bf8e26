"""Name -> model construction for the CLIs and the benchmark.

`model_type` dispatch mirrors examples/llm/models.zig:189-194 of the reference.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..parallel.comm import Comm
from . import common
from .llama import PRESETS as LLAMA_PRESETS, LlamaConfig, LlamaModel


def _families():
    """(presets, config class, model class) of every model family, imported lazily."""
    from .lfm2 import PRESETS as P_LFM2, Lfm2Config, Lfm2Model
    from .qwen3_5 import PRESETS as P_Q35, Qwen35Config, Qwen35Model
    from .qwen3_5_moe import PRESETS as P_Q35M, Qwen35MoeConfig, Qwen35MoeModel
    from .qwen3_moe import PRESETS as P_MOE, Qwen3MoeConfig, Qwen3MoeModel
    return [(LLAMA_PRESETS, LlamaConfig, LlamaModel), (P_MOE, Qwen3MoeConfig, Qwen3MoeModel),
            (P_Q35, Qwen35Config, Qwen35Model), (P_Q35M, Qwen35MoeConfig, Qwen35MoeModel),
            (P_LFM2, Lfm2Config, Lfm2Model)]


def preset_names() -> list[str]:
    return [n for presets, _, _ in _families() for n in presets]


def build_model(name: str, comm: Optional[Comm] = None, device="cuda", seed: int = 0,
                baseline: bool = False, fused: bool = True, dtype=torch.bfloat16):
    """Random-init model of a named architecture on `device` (this rank's shard).  With `fused` and more than
    one rank the symmetric heap of the in-kernel collectives is set up and the row-parallel projections use them."""
    comm = comm or Comm.single(torch.device(device))
    for presets, cfg_cls, model_cls in _families():
        if name in presets:
            model = model_cls(cfg_cls.from_hf(presets[name]), comm, device=device, dtype=dtype).init_random(seed)
            break
    else:
        raise KeyError(f"unknown model {name!r}; known: {preset_names()}")
    if baseline:
        from ..ops import baseline as _baseline
        _baseline.enable(True)
    elif fused and comm.world > 1 and torch.device(device).type == "cuda":
        from ..parallel import symm
        is_moe = getattr(model.config, "num_experts", 0) > 0
        comm.fused = symm.SymmetricContext.create(comm, model.config.hidden_size, staging_elems=512 * model.config.hidden_size,
                                                  combine_tokens=256 if is_moe else 0)
    return model


def model_class_for(config: dict):
    """Implementation for a HF config.json (by `model_type`)."""
    kind = common.detect_model_type(config)
    if kind in ("llama", "qwen3"):
        return LlamaConfig, LlamaModel
    if kind == "qwen3_moe":
        from .qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
        return Qwen3MoeConfig, Qwen3MoeModel
    if kind == "qwen3_5":
        from .qwen3_5 import Qwen35Config, Qwen35Model
        return Qwen35Config, Qwen35Model
    if kind == "qwen3_5_moe":
        from .qwen3_5_moe import Qwen35MoeConfig, Qwen35MoeModel
        return Qwen35MoeConfig, Qwen35MoeModel
    if kind == "lfm2":
        from .lfm2 import Lfm2Config, Lfm2Model
        return Lfm2Config, Lfm2Model
    raise ValueError(kind)
