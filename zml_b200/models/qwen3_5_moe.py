"""Qwen3.5-MoE: the Qwen3.5 hybrid decoder (gated full attention / gated delta net layers)
with a routed mixture of SwiGLU experts plus a gated shared expert in place of the dense MLP.

As in examples/llm/models/qwen3_5_moe/model.zig of the reference: router = linear -> float32
-> top-k -> softmax over the selected k (model.zig:727-754); experts stored fused as
`mlp.experts.gate_up_proj [E, 2F, d]` ([gate | up] rows) and `mlp.experts.down_proj [E, d, F]`
(model.zig:763-776); the shared expert is a dense SwiGLU MLP whose output is scaled by
sigmoid(shared_expert_gate(x)) and added to the routed output (model.zig:810-821).

Experts are expert parallel (rank r owns a contiguous block of experts), the shared expert is
tensor parallel; its local partial sum joins the routed partial sum before the single
all-reduce of the layer, so the MoE block costs one collective.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import moe, ops
from ..parallel.comm import Comm
from .llama import LayerWeights
from .qwen3_5 import PRESETS as _DENSE_PRESETS, Qwen35Config, Qwen35Model


@dataclass
class Qwen35MoeConfig(Qwen35Config):
    num_experts: int = 256
    num_experts_per_tok: int = 8
    moe_intermediate_size: int = 512
    shared_expert_intermediate_size: int = 512
    norm_topk_prob: bool = True

    @classmethod
    def from_hf(cls, obj: dict):
        c = super().from_hf(obj)
        c.model_type = "qwen3_5_moe"
        c.intermediate_size = c.shared_expert_intermediate_size
        return c

    def num_params(self) -> int:
        base = super().num_params() - self.num_hidden_layers * 3 * self.hidden_size * self.intermediate_size
        d = self.hidden_size
        per = self.num_experts * 3 * d * self.moe_intermediate_size + self.num_experts * d \
            + 3 * d * self.shared_expert_intermediate_size + d
        return base + self.num_hidden_layers * per


PRESETS = {
    "qwen3.5-35b-a3b": dict(hidden_size=2048, num_hidden_layers=40, num_attention_heads=16, num_key_value_heads=2,
                            head_dim=256, vocab_size=248320, rms_norm_eps=1e-6,
                            rope_parameters=dict(rope_theta=1e7, partial_rotary_factor=0.25, mrope_section=[11, 11, 10]),
                            linear_conv_kernel_dim=4, linear_key_head_dim=128, linear_num_key_heads=16,
                            linear_num_value_heads=32, linear_value_head_dim=128, full_attention_interval=4,
                            num_experts=256, num_experts_per_tok=8, moe_intermediate_size=512,
                            shared_expert_intermediate_size=512, tie_word_embeddings=False,
                            max_position_embeddings=262144, eos_token_id=[248046, 248044]),
    "tiny-qwen35-moe-test": dict(_DENSE_PRESETS["tiny-qwen35-test"], num_experts=8, num_experts_per_tok=2,
                                 moe_intermediate_size=128, shared_expert_intermediate_size=128),
}


class Qwen35MoeModel(Qwen35Model):
    def __init__(self, config: Qwen35MoeConfig, comm: Optional[Comm] = None, device="cpu", dtype=torch.bfloat16):
        super().__init__(config, comm, device, dtype)
        p = self.comm.world
        if config.num_experts % p != 0:
            raise ValueError(f"{config.num_experts} experts not divisible by EP={p}")
        self.e_local = config.num_experts // p
        self.e0 = self.comm.rank * self.e_local

    # ------------------------------------------------------------------ weights
    def _pack_moe(self, lw: LayerWeights, router, gate_up, down, sh_gate, sh_up, sh_down, sh_gate_w) -> None:
        f = gate_up.shape[1] // 2
        gw = torch.zeros((8, sh_gate_w.shape[-1]), dtype=sh_gate_w.dtype, device=sh_gate_w.device)
        gw[:1] = sh_gate_w.reshape(1, -1)
        extra = dict(lw.extra or {})
        extra.update(router=router, gate_up=moe.interleave_gate_up(gate_up[:, :f], gate_up[:, f:]), down=down.contiguous(),
                     shared_gate_up=torch.cat([sh_gate, sh_up], 0), shared_down=sh_down, shared_gate_w=gw)
        lw.extra = extra

    def _init_mlp(self, lw: LayerWeights, rw, b: int) -> None:
        c, d, f = self.config, self.config.hidden_size, self.config.moe_intermediate_size
        erng = (self.e0, self.e0 + self.e_local)
        fs = c.shared_expert_intermediate_size
        self._pack_moe(lw, rw((c.num_experts, d), b + 15), rw((c.num_experts, 2 * f, d), b + 16, rows=erng),
                       rw((c.num_experts, d, f), b + 17, rows=erng), rw((fs, d), b + 18, rows=self.f_rng),
                       rw((fs, d), b + 19, rows=self.f_rng), rw((d, fs), b + 20, cols=self.f_rng), rw((1, d), b + 21))

    def _load_mlp(self, lw: LayerWeights, get, has, p: str) -> None:
        erng = (self.e0, self.e0 + self.e_local)
        m = p + "mlp."
        self._pack_moe(lw, get(m + "gate.weight"), get(m + "experts.gate_up_proj", rows=erng),
                       get(m + "experts.down_proj", rows=erng), get(m + "shared_expert.gate_proj.weight", rows=self.f_rng),
                       get(m + "shared_expert.up_proj.weight", rows=self.f_rng),
                       get(m + "shared_expert.down_proj.weight", cols=self.f_rng), get(m + "shared_expert_gate.weight"))

    def _mlp_state_dict(self, lw: LayerWeights, p: str, out: dict) -> None:
        e, m = lw.extra, p + "mlp."
        g, u = moe.deinterleave_gate_up(e["gate_up"])
        out[m + "gate.weight"] = e["router"]
        out[m + "experts.gate_up_proj"] = torch.cat([g, u], 1).contiguous()
        out[m + "experts.down_proj"] = e["down"]
        out[m + "shared_expert.gate_proj.weight"] = e["shared_gate_up"][:self.f_local]
        out[m + "shared_expert.up_proj.weight"] = e["shared_gate_up"][self.f_local:]
        out[m + "shared_expert.down_proj.weight"] = e["shared_down"]
        out[m + "shared_expert_gate.weight"] = e["shared_gate_w"][:1]

    def weight_bytes(self) -> int:
        n = super().weight_bytes()
        for lw in self.layers:
            n += sum(t.numel() * t.element_size() for k, t in lw.extra.items() if isinstance(t, torch.Tensor))
        return n

    # ------------------------------------------------------------------ forward
    def mlp(self, lw: LayerWeights, x, n2):
        c, e = self.config, lw.extra
        logits = ops.gemm(n2, e["router"], out_dtype=torch.float32, static_w=True)
        ids, w = moe.router_topk(logits, c.num_experts_per_tok, True)
        act = ops.swiglu(ops.gemm(n2, e["shared_gate_up"], static_w=True))
        shared = ops.gemm(act, e["shared_down"], static_w=True)                       # this rank's partial sum
        gate = torch.sigmoid(ops.gemm(n2, e["shared_gate_w"], out_dtype=torch.float32, static_w=True)[:, :1])
        shared = (shared.float() * gate).to(shared.dtype)
        return moe.forward_moe(n2, ids, w, e["gate_up"], e["down"], self.comm, c.num_experts, residual=x,
                               extra_partial=shared)
