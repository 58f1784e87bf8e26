"""Qwen3-MoE-style decoder (the Qwen3-30B-A3B shape of the benchmark suite): Llama-like
attention with per-head q/k RMSNorm, and a routed mixture of SwiGLU experts in place of
the dense MLP.  Router = linear -> float32 -> top-k -> softmax over the selected k, as in
the reference's MoE models (examples/llm/models/qwen3_5_moe/model.zig:727-754).

Parallelism: attention is tensor parallel (KV heads replicated when there are fewer than
ranks); experts are expert parallel, rank r owning experts [r * E/P, (r + 1) * E/P)
(examples/llm/models/qwen3_5_moe/model.zig:766-775 shards `.expert` on `.experts`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import moe, ops
from ..parallel.comm import Comm
from . import common
from .llama import LayerWeights, LlamaConfig, LlamaModel


@dataclass
class Qwen3MoeConfig(LlamaConfig):
    num_experts: int = 128
    num_experts_per_tok: int = 8
    moe_intermediate_size: int = 768
    norm_topk_prob: bool = True
    expert_dtype: str = "bf16"          # bf16 | nvfp4

    @staticmethod
    def from_hf(obj: dict) -> "Qwen3MoeConfig":
        names = set(Qwen3MoeConfig.__dataclass_fields__)
        kw = {k: v for k, v in obj.items() if k in names and v is not None}
        if "num_experts" not in kw and obj.get("num_local_experts") is not None:
            kw["num_experts"] = obj["num_local_experts"]      # transformers >= 5 serialises it under this name
        kw.setdefault("qk_norm", True)
        kw.setdefault("intermediate_size", kw.get("moe_intermediate_size", 768))
        kw.setdefault("num_key_value_heads", kw.get("num_attention_heads"))
        kw.setdefault("model_type", "qwen3_moe")
        return Qwen3MoeConfig(**kw)

    def num_params(self) -> int:
        d, l = self.hidden_size, self.num_hidden_layers
        attn = d * self.hd * (self.num_attention_heads * 2 + self.num_key_value_heads * 2)
        experts = self.num_experts * 3 * d * self.moe_intermediate_size + self.num_experts * d
        return l * (attn + experts + 2 * d) + self.vocab_size * d * (1 if self.tie_word_embeddings else 2)


PRESETS = {
    "qwen3-30b-a3b": dict(hidden_size=2048, num_hidden_layers=48, num_attention_heads=32, num_key_value_heads=4,
                          head_dim=128, intermediate_size=768, moe_intermediate_size=768, num_experts=128,
                          num_experts_per_tok=8, vocab_size=151936, rms_norm_eps=1e-6, rope_theta=1e6,
                          tie_word_embeddings=False, max_position_embeddings=40960, norm_topk_prob=True,
                          bos_token_id=151643, eos_token_id=[151645, 151643], model_type="qwen3_moe"),
    "qwen3-30b-a3b-nvfp4": None,     # filled below: same shape, NVFP4 expert weights
    "tiny-moe-test": dict(hidden_size=256, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2,
                          head_dim=64, intermediate_size=128, moe_intermediate_size=128, num_experts=8,
                          num_experts_per_tok=2, vocab_size=1024, rms_norm_eps=1e-6, rope_theta=10000.0,
                          tie_word_embeddings=True, max_position_embeddings=4096, norm_topk_prob=True,
                          bos_token_id=1, eos_token_id=2, model_type="qwen3_moe"),
}


PRESETS["qwen3-30b-a3b-nvfp4"] = dict(PRESETS["qwen3-30b-a3b"], expert_dtype="nvfp4")


class Qwen3MoeModel(LlamaModel):
    def __init__(self, config: Qwen3MoeConfig, comm: Optional[Comm] = None, device="cpu", dtype=torch.bfloat16):
        super().__init__(config, comm, device, dtype)
        p = self.comm.world
        if config.num_experts % p != 0:
            raise ValueError(f"{config.num_experts} experts not divisible by EP={p}")
        self.e_local = config.num_experts // p
        self.e0 = self.comm.rank * self.e_local

    # ------------------------------------------------------------------ weights
    def init_random(self, seed: int = 0, std: float = 0.02, full: Optional[bool] = None) -> "Qwen3MoeModel":
        c, dev, dt = self.config, self.device, self.dtype
        if full is None:
            full = c.num_params() < 4e9
        d, hd, f = c.hidden_size, c.hd, c.moe_intermediate_size
        rw = lambda shape, s, **kw: common.randn_weight(shape, std, seed * 7919 + s, dev, dt, full=full, **kw)
        self.embed = rw((c.vocab_size, d), 1)
        self.final_norm = torch.ones(d, dtype=dt, device=dev)
        if c.tie_word_embeddings:
            self.lm_head = self.embed[self.v_rng[0]:self.v_rng[1]] if self.comm.world > 1 else self.embed
        else:
            self.lm_head = rw((c.vocab_size, d), 2, rows=self.v_rng)
        q0, q1 = self.q_rng[0] * hd, self.q_rng[1] * hd
        k0, k1 = self.kv_rng[0] * hd, self.kv_rng[1] * hd
        erng = (self.e0, self.e0 + self.e_local)
        for l in range(c.num_hidden_layers):
            lw = LayerWeights()
            b = 100 + l * 16
            lw.input_norm = torch.ones(d, dtype=dt, device=dev)
            lw.post_norm = torch.ones(d, dtype=dt, device=dev)
            lw.qkv = torch.cat([rw((c.num_attention_heads * hd, d), b + 0, rows=(q0, q1)),
                                rw((c.num_key_value_heads * hd, d), b + 1, rows=(k0, k1)),
                                rw((c.num_key_value_heads * hd, d), b + 2, rows=(k0, k1))], 0)
            if c.qk_norm:
                lw.q_norm = torch.ones(hd, dtype=dt, device=dev)
                lw.k_norm = torch.ones(hd, dtype=dt, device=dev)
            lw.o = rw((d, c.num_attention_heads * hd), b + 3, cols=(q0, q1))
            gate = rw((c.num_experts, f, d), b + 4, rows=erng)
            up = rw((c.num_experts, f, d), b + 5, rows=erng)
            down = rw((c.num_experts, d, f), b + 6, rows=erng)
            lw.extra = {"router": rw((c.num_experts, d), b + 7), "gate_up": moe.interleave_gate_up(gate, up), "down": down}
            del gate, up
            if c.expert_dtype == "nvfp4":
                self._to_nvfp4(lw)
            self.layers.append(lw)
        return self

    def _to_nvfp4(self, lw: LayerWeights) -> None:
        """Expert weights become NVFP4 (quantised in the interleaved gate|up layout the kernels use).  The
        packed form feeds the decode-regime kernel; its de-quantised bf16 twin feeds the compute-bound
        prefill kernel, so both see the same values."""
        gu = moe.Nvfp4Experts.quantize(lw.extra["gate_up"])
        dn = moe.Nvfp4Experts.quantize(lw.extra["down"])
        lw.extra["gate_up"] = gu.dequantize(self.dtype)
        lw.extra["down"] = dn.dequantize(self.dtype)
        lw.extra["w4"] = (gu, dn)

    def load(self, store, prefix: str = "") -> "Qwen3MoeModel":
        c, hd = self.config, self.config.hd
        dev, dt = self.device, self.dtype
        q0, q1 = self.q_rng[0] * hd, self.q_rng[1] * hd
        k0, k1 = self.kv_rng[0] * hd, self.kv_rng[1] * hd
        get = lambda name, **kw: store.load_tensor(prefix + name, device=dev, dtype=dt, **kw)
        self.embed = get("model.embed_tokens.weight")
        self.final_norm = get("model.norm.weight")
        self.lm_head = get("lm_head.weight", rows=self.v_rng) if store.has_key(prefix + "lm_head.weight") else self.embed
        for l in range(c.num_hidden_layers):
            p = f"model.layers.{l}."
            lw = LayerWeights()
            lw.input_norm = get(p + "input_layernorm.weight")
            lw.post_norm = get(p + "post_attention_layernorm.weight")
            lw.qkv = torch.cat([get(p + "self_attn.q_proj.weight", rows=(q0, q1)),
                                get(p + "self_attn.k_proj.weight", rows=(k0, k1)),
                                get(p + "self_attn.v_proj.weight", rows=(k0, k1))], 0)
            if store.has_key(prefix + p + "self_attn.q_norm.weight"):
                lw.q_norm = get(p + "self_attn.q_norm.weight")
                lw.k_norm = get(p + "self_attn.k_norm.weight")
            lw.o = get(p + "self_attn.o_proj.weight", cols=(q0, q1))
            if self._has_nvfp4_experts(store, prefix + p):
                lw.extra = {"router": get(p + "mlp.gate.weight")}
                self._load_nvfp4_experts(store, prefix + p, lw)
                self.layers.append(lw)
                continue
            if store.has_key(prefix + p + "mlp.experts.gate_up_proj"):
                # fused layout: gate_up_proj [E, 2F, d] with [gate | up] rows, down_proj [E, d, F]
                gu = get(p + "mlp.experts.gate_up_proj", rows=(self.e0, self.e0 + self.e_local))
                f = gu.shape[1] // 2
                gate_s, up_s = gu[:, :f], gu[:, f:]
                down_s = get(p + "mlp.experts.down_proj", rows=(self.e0, self.e0 + self.e_local))
            else:
                gates, ups, downs = [], [], []
                for e in range(self.e0, self.e0 + self.e_local):
                    gates.append(get(p + f"mlp.experts.{e}.gate_proj.weight"))
                    ups.append(get(p + f"mlp.experts.{e}.up_proj.weight"))
                    downs.append(get(p + f"mlp.experts.{e}.down_proj.weight"))
                gate_s, up_s, down_s = torch.stack(gates), torch.stack(ups), torch.stack(downs)
            lw.extra = {"router": get(p + "mlp.gate.weight"),
                        "gate_up": moe.interleave_gate_up(gate_s, up_s), "down": down_s.contiguous()}
            self.layers.append(lw)
        return self

    # NVFP4 expert checkpoints: per expert and projection a packed u8 weight [N, K / 2], f8e4m3fn block scales
    # [N, K / 16] and one float32 matrix scale, in either of the two common spellings:
    #   weight + weight_scale + weight_scale_2          (w = code x weight_scale x weight_scale_2)
    #   weight_packed + weight_scale + weight_global_scale   (w = code x weight_scale / weight_global_scale)
    def _has_nvfp4_experts(self, store, layer_prefix: str) -> bool:
        base = layer_prefix + f"mlp.experts.{self.e0}.gate_proj."
        return store.has_key(base + "weight_scale") and (store.has_key(base + "weight_scale_2") or
                                                         store.has_key(base + "weight_global_scale"))

    def _load_nvfp4_experts(self, store, layer_prefix: str, lw: LayerWeights) -> None:
        dev = self.device

        def proj(name: str):
            codes, scales, gs = [], [], []
            for e in range(self.e0, self.e0 + self.e_local):
                base = layer_prefix + f"mlp.experts.{e}.{name}."
                packed = base + ("weight_packed" if store.has_key(base + "weight_packed") else "weight")
                codes.append(store.load_tensor(packed, device=dev).view(torch.uint8))
                scales.append(store.load_tensor(base + "weight_scale", device=dev).view(torch.float8_e4m3fn))
                if store.has_key(base + "weight_scale_2"):
                    gs.append(store.load_tensor(base + "weight_scale_2", device=dev).float().reshape(()))
                else:
                    gs.append(1.0 / store.load_tensor(base + "weight_global_scale", device=dev).float().reshape(()))
            return torch.stack(codes), torch.stack(scales), torch.stack(gs)

        gu = moe.Nvfp4Experts.from_checkpoint_gate_up(proj("gate_proj"), proj("up_proj"))
        dc, ds, dg = proj("down_proj")
        e, n, kb = dc.shape
        dn = moe.Nvfp4Experts.from_checkpoint(dc, ds, dg, e, n, kb * 2)
        lw.extra["gate_up"] = gu.dequantize(self.dtype)
        lw.extra["down"] = dn.dequantize(self.dtype)
        lw.extra["w4"] = (gu, dn)

    def state_dict_hf(self) -> dict:
        from ..moe.ops import deinterleave_gate_up
        c, hd = self.config, self.config.hd
        out = {"model.embed_tokens.weight": self.embed, "model.norm.weight": self.final_norm}
        if not c.tie_word_embeddings:
            out["lm_head.weight"] = self.lm_head
        nq, nk = self.hq * hd, self.hkv * hd
        for l, lw in enumerate(self.layers):
            p = f"model.layers.{l}."
            out[p + "input_layernorm.weight"] = lw.input_norm
            out[p + "post_attention_layernorm.weight"] = lw.post_norm
            out[p + "self_attn.q_proj.weight"] = lw.qkv[:nq]
            out[p + "self_attn.k_proj.weight"] = lw.qkv[nq:nq + nk]
            out[p + "self_attn.v_proj.weight"] = lw.qkv[nq + nk:]
            if lw.q_norm is not None:
                out[p + "self_attn.q_norm.weight"] = lw.q_norm
                out[p + "self_attn.k_norm.weight"] = lw.k_norm
            out[p + "self_attn.o_proj.weight"] = lw.o
            out[p + "mlp.gate.weight"] = lw.extra["router"]
            g, u = deinterleave_gate_up(lw.extra["gate_up"])
            for i in range(self.e_local):
                e = self.e0 + i
                out[p + f"mlp.experts.{e}.gate_proj.weight"] = g[i].contiguous()
                out[p + f"mlp.experts.{e}.up_proj.weight"] = u[i].contiguous()
                out[p + f"mlp.experts.{e}.down_proj.weight"] = lw.extra["down"][i]
        return out

    def weight_bytes(self) -> int:
        n = super().weight_bytes()
        for lw in self.layers:
            n += sum(t.numel() * t.element_size() for t in lw.extra.values() if isinstance(t, torch.Tensor))
            n += sum(q.nbytes() for q in lw.extra.get("w4", ()))
        return n

    # ------------------------------------------------------------------ forward
    def mlp(self, lw: LayerWeights, x, n2):
        c = self.config
        logits = ops.gemm(n2, lw.extra["router"], out_dtype=torch.float32, static_w=True)
        ids, w = moe.router_topk(logits, c.num_experts_per_tok, c.norm_topk_prob)
        return moe.forward_moe(n2, ids, w, lw.extra["gate_up"], lw.extra["down"], self.comm, c.num_experts, residual=x,
                               w4=lw.extra.get("w4"))
