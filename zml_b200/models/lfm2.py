"""LFM2: decoder whose layers are either a gated short convolution or GQA attention.

As in examples/llm/models/lfm2/model.zig of the reference: `layer_types` in {conv,
full_attention}; every layer is x + op(operator_norm(x)) followed by x + ffn(ffn_norm(x))
(model.zig:360-427).  `ShortConv` (model.zig:441-509): in_proj -> (B, C, x) thirds, depthwise
causal conv of B*x with `conv_L_cache` taps and a rolling cache of its inputs, C * conv,
out_proj.  Attention (model.zig:511-600): per-head RMSNorm of q and k (`q_layernorm`,
`k_layernorm`), RoPE (rotate-half layout, default scaling), out_proj.  SwiGLU MLP with HF names
w1 (gate), w3 (up), w2 (down); final norm is `model.embedding_norm`; lm_head tied.

On the B200 a conv layer is: one GEMM (in_proj), one kernel (gate, conv, gate, cache update),
one row-parallel GEMM (out_proj, fused with the all-reduce under TP).  Channels are sharded
across ranks the way attention heads are.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from .. import ops
from ..ops import linear_attn as la
from ..parallel.comm import Comm
from . import common
from .llama import AttnMeta, LayerWeights, LlamaConfig, LlamaModel


@dataclass
class Lfm2Config(LlamaConfig):
    layer_types: list = field(default_factory=list)
    conv_L_cache: int = 3
    conv_bias: bool = False
    norm_eps: float = 1e-5
    block_ff_dim: int = 0
    block_auto_adjust_ff_dim: bool = False
    block_ffn_dim_multiplier: float = 1.0
    block_multiple_of: int = 256
    full_attn_idxs: list = field(default_factory=list)

    @classmethod
    def from_hf(cls, obj: dict):
        names = set(cls.__dataclass_fields__)
        kw = {k: v for k, v in obj.items() if k in names and v is not None}
        kw.setdefault("num_key_value_heads", kw.get("num_attention_heads"))
        kw["rms_norm_eps"] = kw.get("norm_eps", 1e-5)
        kw["qk_norm"] = True
        kw["tie_word_embeddings"] = bool(obj.get("tie_embedding", obj.get("tie_word_embeddings", True)))
        kw.setdefault("model_type", "lfm2")
        if obj.get("conv_bias"):
            raise ValueError("conv_bias is not supported")
        ff = kw.get("block_ff_dim") or kw.get("intermediate_size")
        if ff is None:
            raise ValueError("config.json lacks block_ff_dim / intermediate_size")
        if kw.get("block_auto_adjust_ff_dim"):
            ff = int(2 * ff / 3)
            ff = int(kw.get("block_ffn_dim_multiplier", 1.0) * ff)
            mo = kw.get("block_multiple_of", 256)
            ff = mo * ((ff + mo - 1) // mo)
        kw["intermediate_size"] = ff
        if not kw.get("layer_types"):
            full = set(kw.get("full_attn_idxs") or [])
            kw["layer_types"] = ["full_attention" if i in full else "conv" for i in range(kw["num_hidden_layers"])]
        for t in kw["layer_types"]:
            if t not in ("conv", "full_attention"):
                raise ValueError(f"unknown layer type {t!r}")
        return cls(**kw)

    def num_params(self) -> int:
        d, f = self.hidden_size, self.intermediate_size
        conv = 4 * d * d + d * self.conv_L_cache
        attn = d * self.hd * (2 * self.num_attention_heads + 2 * self.num_key_value_heads)
        n = sum(conv if t == "conv" else attn for t in self.layer_types)
        return n + self.num_hidden_layers * (3 * d * f + 2 * d) + self.vocab_size * d


PRESETS = {
    "lfm2-1.2b": dict(hidden_size=2048, num_hidden_layers=16, num_attention_heads=32, num_key_value_heads=8,
                      vocab_size=65536, norm_eps=1e-5, rope_theta=1000000.0, conv_L_cache=3, block_ff_dim=12288,
                      block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0, block_multiple_of=256,
                      layer_types=["conv", "conv", "full_attention", "conv", "conv", "full_attention", "conv", "conv",
                                   "full_attention", "conv", "full_attention", "conv", "full_attention", "conv",
                                   "full_attention", "conv"],
                      max_position_embeddings=128000, bos_token_id=1, eos_token_id=7, tie_embedding=True),
    "tiny-lfm2-test": dict(hidden_size=256, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                           vocab_size=1024, norm_eps=1e-5, rope_theta=10000.0, conv_L_cache=3, block_ff_dim=512,
                           layer_types=["conv", "full_attention", "conv", "full_attention"],
                           max_position_embeddings=4096, bos_token_id=1, eos_token_id=2, tie_embedding=True),
}


class Lfm2Model(LlamaModel):
    def __init__(self, config: Lfm2Config, comm: Optional[Comm] = None, device="cpu", dtype=torch.bfloat16):
        super().__init__(config, comm, device, dtype)
        c = config
        self.conv_layers = [i for i, t in enumerate(c.layer_types) if t == "conv"]
        self.full_layers = [i for i, t in enumerate(c.layer_types) if t == "full_attention"]
        self.kv_index = {l: i for i, l in enumerate(self.full_layers)}
        self.conv_index = {l: i for i, l in enumerate(self.conv_layers)}
        self.c_rng = common.shard_range(c.hidden_size, self.comm.rank, self.comm.world)
        self.c_local = self.c_rng[1] - self.c_rng[0]
        self.conv_state = None

    def alloc_state(self, num_slots: int) -> None:
        self.conv_state = torch.zeros((max(len(self.conv_layers), 1), num_slots, self.config.conv_L_cache - 1,
                                       self.c_local), dtype=self.dtype, device=self.device)

    def kv_cache_shape(self, num_pages: int, page_size: int):
        return (max(len(self.full_layers), 1), 2, num_pages, page_size, self.hkv, self.config.hd)

    # ------------------------------------------------------------------ weights
    def _bcx_rows(self, w: torch.Tensor) -> torch.Tensor:
        """This rank's rows of in_proj, whose rows are [B | C | x] over all channels."""
        d = self.config.hidden_size
        c0, c1 = self.c_rng
        return torch.cat([w[c0:c1], w[d + c0:d + c1], w[2 * d + c0:2 * d + c1]], 0).contiguous()

    def init_random(self, seed: int = 0, std: float = 0.02, full: Optional[bool] = None) -> "Lfm2Model":
        c, dev, dt = self.config, self.device, self.dtype
        d, hd = c.hidden_size, c.hd
        rw = lambda shape, s, **kw: common.randn_weight(shape, std, seed * 7919 + s, dev, dt, full=True, **kw)
        self.embed = rw((c.vocab_size, d), 1)
        self.final_norm = torch.ones(d, dtype=dt, device=dev)
        self.lm_head = self.embed[self.v_rng[0]:self.v_rng[1]] if self.comm.world > 1 else self.embed
        q0, q1 = self.q_rng[0] * hd, self.q_rng[1] * hd
        k0, k1 = self.kv_rng[0] * hd, self.kv_rng[1] * hd
        for l in range(c.num_hidden_layers):
            lw = LayerWeights()
            b = 100 + l * 16
            lw.input_norm = torch.ones(d, dtype=dt, device=dev)
            lw.post_norm = torch.ones(d, dtype=dt, device=dev)
            if c.layer_types[l] == "full_attention":
                lw.qkv = torch.cat([rw((c.num_attention_heads * hd, d), b + 0, rows=(q0, q1)),
                                    rw((c.num_key_value_heads * hd, d), b + 1, rows=(k0, k1)),
                                    rw((c.num_key_value_heads * hd, d), b + 2, rows=(k0, k1))], 0)
                lw.q_norm = torch.ones(hd, dtype=dt, device=dev)
                lw.k_norm = torch.ones(hd, dtype=dt, device=dev)
                lw.o = rw((d, c.num_attention_heads * hd), b + 3, cols=(q0, q1))
            else:
                conv_w = common.randn_weight((d, c.conv_L_cache), 0.3, seed * 7919 + b + 8, dev, dt)
                lw.extra = {"in_proj": self._bcx_rows(rw((3 * d, d), b + 7)),
                            "conv_w": conv_w[self.c_rng[0]:self.c_rng[1]].contiguous(),
                            "out_proj": rw((d, d), b + 9, cols=self.c_rng)}
            g = rw((c.intermediate_size, d), b + 4, rows=self.f_rng)
            u = rw((c.intermediate_size, d), b + 5, rows=self.f_rng)
            lw.gate_up = torch.cat([g, u], 0)
            lw.down = rw((d, c.intermediate_size), b + 6, cols=self.f_rng)
            self.layers.append(lw)
        return self

    def load(self, store, prefix: str = "") -> "Lfm2Model":
        c, hd = self.config, self.config.hd
        dev, dt = self.device, self.dtype
        get = lambda name, **kw: store.load_tensor(prefix + name, device=dev, dtype=dt, **kw)
        q0, q1 = self.q_rng[0] * hd, self.q_rng[1] * hd
        k0, k1 = self.kv_rng[0] * hd, self.kv_rng[1] * hd
        self.embed = get("model.embed_tokens.weight")
        self.final_norm = get("model.embedding_norm.weight")
        if store.has_key(prefix + "lm_head.weight"):
            self.lm_head = get("lm_head.weight", rows=self.v_rng)
        else:
            self.lm_head = self.embed[self.v_rng[0]:self.v_rng[1]] if self.comm.world > 1 else self.embed
        for l in range(c.num_hidden_layers):
            p = f"model.layers.{l}."
            lw = LayerWeights()
            lw.input_norm = get(p + "operator_norm.weight")
            lw.post_norm = get(p + "ffn_norm.weight")
            if c.layer_types[l] == "full_attention":
                a = p + "self_attn."
                lw.qkv = torch.cat([get(a + "q_proj.weight", rows=(q0, q1)), get(a + "k_proj.weight", rows=(k0, k1)),
                                    get(a + "v_proj.weight", rows=(k0, k1))], 0)
                lw.q_norm = get(a + "q_layernorm.weight")
                lw.k_norm = get(a + "k_layernorm.weight")
                lw.o = get(a + "out_proj.weight", cols=(q0, q1))
            else:
                a = p + "conv."
                cw = get(a + "conv.weight")                                   # [d, 1, L]
                lw.extra = {"in_proj": self._bcx_rows(get(a + "in_proj.weight")),
                            "conv_w": cw.reshape(cw.shape[0], -1)[self.c_rng[0]:self.c_rng[1]].contiguous(),
                            "out_proj": get(a + "out_proj.weight", cols=self.c_rng)}
            f = store.shape_of(prefix + p + "feed_forward.w1.weight")[0] if hasattr(store, "shape_of") else c.intermediate_size
            if f != c.intermediate_size:
                raise ValueError(f"feed_forward width {f} in the checkpoint, {c.intermediate_size} from config.json")
            lw.gate_up = torch.cat([get(p + "feed_forward.w1.weight", rows=self.f_rng),
                                    get(p + "feed_forward.w3.weight", rows=self.f_rng)], 0)
            lw.down = get(p + "feed_forward.w2.weight", cols=self.f_rng)
            self.layers.append(lw)
        return self

    def state_dict_hf(self) -> dict:
        c, hd = self.config, self.config.hd
        out = {"model.embed_tokens.weight": self.embed, "model.embedding_norm.weight": self.final_norm}
        nq, nk = self.hq * hd, self.hkv * hd
        cl = self.c_local
        for l, lw in enumerate(self.layers):
            p = f"model.layers.{l}."
            out[p + "operator_norm.weight"] = lw.input_norm
            out[p + "ffn_norm.weight"] = lw.post_norm
            if c.layer_types[l] == "full_attention":
                a = p + "self_attn."
                out[a + "q_proj.weight"] = lw.qkv[:nq]
                out[a + "k_proj.weight"] = lw.qkv[nq:nq + nk]
                out[a + "v_proj.weight"] = lw.qkv[nq + nk:]
                out[a + "q_layernorm.weight"] = lw.q_norm
                out[a + "k_layernorm.weight"] = lw.k_norm
                out[a + "out_proj.weight"] = lw.o
            else:
                a = p + "conv."
                out[a + "in_proj.weight"] = lw.extra["in_proj"]
                out[a + "conv.weight"] = lw.extra["conv_w"].reshape(cl, 1, -1)
                out[a + "out_proj.weight"] = lw.extra["out_proj"]
            out[p + "feed_forward.w1.weight"] = lw.gate_up[:self.f_local]
            out[p + "feed_forward.w3.weight"] = lw.gate_up[self.f_local:]
            out[p + "feed_forward.w2.weight"] = lw.down
        return out

    def weight_bytes(self) -> int:
        n = super().weight_bytes()
        for lw in self.layers:
            if lw.extra:
                n += sum(t.numel() * t.element_size() for t in lw.extra.values())
        return n

    # ------------------------------------------------------------------ forward
    def short_conv(self, l: int, lw: LayerWeights, n1, meta: AttnMeta):
        e, cl = lw.extra, self.c_local
        if meta.state_slots is None:
            raise ValueError("LFM2 needs AttnMeta.state_slots (one conv-cache slot per sequence)")
        q_start = meta.q_start
        if q_start is None:
            q_start = torch.arange(n1.shape[0] + 1, dtype=torch.int32, device=n1.device)
        bcx = ops.gemm(n1, e["in_proj"], static_w=True)                # [T, B | C | x]
        return la.causal_conv1d(bcx[:, 2 * cl:3 * cl], e["conv_w"], self.conv_state[self.conv_index[l]], q_start,
                                meta.seq_lens, meta.state_slots, pre=bcx[:, :cl], post=bcx[:, cl:2 * cl])

    def layer(self, l: int, x, meta: AttnMeta, kv_cache):
        lw, c = self.layers[l], self.config
        n1 = ops.rmsnorm(x, lw.input_norm, c.rms_norm_eps)
        if c.layer_types[l] == "full_attention":
            i = self.kv_index[l]
            a = self.attention(lw, n1, meta, kv_cache[i, 0], kv_cache[i, 1])
            x = self.row_parallel(a, lw.o, x)
        else:
            if self.conv_state is None:
                self.alloc_state(int(meta.state_slots.max().item()) + 1)
            y = self.short_conv(l, lw, n1, meta)
            x = self.row_parallel(y, lw.extra["out_proj"], x)
        n2 = ops.rmsnorm(x, lw.post_norm, c.rms_norm_eps)
        return self.mlp(lw, x, n2)
