"""Qwen3.5 dense hybrid decoder: layers are either gated full attention or a gated delta net
(linear attention), chosen per layer by `layer_types`.

Architecture as in examples/llm/models/qwen3_5/model.zig of the reference:

* every RMSNorm multiplies by (1 + weight) (model.zig:982-1001);
* full attention (model.zig:538-688): q_proj emits [q | gate] per head, per-head RMSNorm of q
  and k, partial rotary (`partial_rotary_factor` of the head dim, HF rotate-half layout),
  attention, output * sigmoid(gate), o_proj;
* gated delta net (model.zig:768-980): in_proj_{qkv, z, b, a}; depthwise causal conv (kernel
  `linear_conv_kernel_dim`) + SiLU over the q|k|v mix with a rolling cache; q, k L2-normalised;
  decay exp(-exp(A_log) * softplus(a + dt_bias)), write gate sigmoid(b); delta-rule recurrence
  over a per-head [dk, dv] state; RMSNorm(out) * weight * silu(z); out_proj;
* SwiGLU MLP.

HF tensor names live under `model.language_model.` (model.zig:162).  On the B200 the four input
projections of a linear-attention layer are one GEMM ([q|k|v|z|b|a] rows), the conv + SiLU is
one kernel, and the recurrence with both normalisations is one kernel; q/k/v/gate of a full
attention layer are one GEMM.  Tensor parallelism shards heads (k and v heads of the delta
net, q and kv heads of attention); the recurrent and conv states live in a slot pool indexed
per sequence, like KV pages.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from .. import ops
from ..nn import rotary as rope_mod
from ..ops import linear_attn as la
from ..parallel.comm import Comm
from . import common
from .llama import AttnMeta, LayerWeights, LlamaConfig, LlamaModel


@dataclass
class Qwen35Config(LlamaConfig):
    layer_types: list = field(default_factory=list)
    partial_rotary_factor: float = 0.25
    mrope_section: list = field(default_factory=lambda: [11, 11, 10])
    linear_conv_kernel_dim: int = 4
    linear_key_head_dim: int = 128
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 32
    linear_value_head_dim: int = 128
    full_attention_interval: int = 4

    @classmethod
    def from_hf(cls, obj: dict):
        tc = dict(obj.get("text_config", obj))
        rp = tc.get("rope_parameters") or {}
        names = set(cls.__dataclass_fields__)
        kw = {k: v for k, v in tc.items() if k in names and v is not None}
        if "num_experts" in names and "num_experts" not in kw and tc.get("num_local_experts") is not None:
            kw["num_experts"] = tc["num_local_experts"]
        kw["rope_theta"] = rp.get("rope_theta", tc.get("rope_theta", 1e7))
        kw["partial_rotary_factor"] = rp.get("partial_rotary_factor", tc.get("partial_rotary_factor", 0.25))
        if "mrope_section" in rp:
            kw["mrope_section"] = list(rp["mrope_section"])
        kw.pop("rope_scaling", None)
        kw.setdefault("num_key_value_heads", kw.get("num_attention_heads"))
        kw.setdefault("intermediate_size", tc.get("moe_intermediate_size", 0))
        kw.setdefault("model_type", "qwen3_5")
        kw["qk_norm"] = True
        if not kw.get("layer_types"):
            n, iv = kw["num_hidden_layers"], kw.get("full_attention_interval", 4)
            kw["layer_types"] = ["full_attention" if (i + 1) % iv == 0 else "linear_attention" for i in range(n)]
        for t in kw["layer_types"]:
            if t not in ("linear_attention", "full_attention"):
                raise ValueError(f"unknown layer type {t!r}")
        if "eos_token_id" not in kw and "eos_token_id" in obj:
            kw["eos_token_id"] = obj["eos_token_id"]
        return cls(**kw)

    def rope_opts(self) -> rope_mod.RopeOpts:
        return rope_mod.RopeOpts(rope_mod.Layout.real_im_pass, rope_mod.Scaling(kind="default", rope_theta=self.rope_theta))

    @property
    def rotary_dim(self) -> int:
        return int(self.hd * self.partial_rotary_factor)

    def num_params(self) -> int:
        d, f = self.hidden_size, self.intermediate_size
        kd = self.linear_num_key_heads * self.linear_key_head_dim
        vd = self.linear_num_value_heads * self.linear_value_head_dim
        lin = d * (2 * kd + 2 * vd + 2 * self.linear_num_value_heads) + vd * d
        full = d * self.hd * (2 * self.num_attention_heads + 2 * self.num_key_value_heads) + self.num_attention_heads * self.hd * d
        n = sum(lin if t == "linear_attention" else full for t in self.layer_types)
        return n + self.num_hidden_layers * (3 * d * f + 2 * d) + self.vocab_size * d * (1 if self.tie_word_embeddings else 2)


PRESETS = {
    # the 9B-class dense hybrid shape: 3 linear-attention layers per full-attention layer
    "qwen3.5-9b": dict(hidden_size=4096, num_hidden_layers=32, num_attention_heads=16, num_key_value_heads=4,
                       head_dim=256, intermediate_size=12288, vocab_size=248320, rms_norm_eps=1e-6,
                       rope_parameters=dict(rope_theta=1e7, partial_rotary_factor=0.25, mrope_section=[11, 11, 10]),
                       linear_conv_kernel_dim=4, linear_key_head_dim=128, linear_num_key_heads=16,
                       linear_num_value_heads=32, linear_value_head_dim=128, full_attention_interval=4,
                       tie_word_embeddings=False, max_position_embeddings=262144, eos_token_id=[248046, 248044]),
    "tiny-qwen35-test": dict(hidden_size=256, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                             head_dim=64, intermediate_size=512, vocab_size=1024, rms_norm_eps=1e-6,
                             rope_parameters=dict(rope_theta=10000.0, partial_rotary_factor=0.5, mrope_section=[6, 5, 5]),
                             linear_conv_kernel_dim=4, linear_key_head_dim=64, linear_num_key_heads=2,
                             linear_num_value_heads=4, linear_value_head_dim=64, full_attention_interval=2,
                             tie_word_embeddings=True, max_position_embeddings=4096, eos_token_id=2),
}


class LinearAttnWeights:
    """Weights of one gated-delta-net layer, this rank's heads only."""
    __slots__ = ("in_proj", "conv_w", "a_log", "dt_bias", "norm_w", "out_proj")

    def __init__(self):
        for s in self.__slots__:
            setattr(self, s, None)


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


class Qwen35Model(LlamaModel):
    PREFIX = "model.language_model."

    def __init__(self, config: Qwen35Config, comm: Optional[Comm] = None, device="cpu", dtype=torch.bfloat16):
        super().__init__(config, comm, device, dtype)
        c, p, r = config, self.comm.world, self.comm.rank
        self.rot_dim = c.rotary_dim
        self.inv_freq = rope_mod.inv_freq(self.rot_dim, c.rope_opts()).to(self.device)
        self.lin_layers = [i for i, t in enumerate(c.layer_types) if t == "linear_attention"]
        self.full_layers = [i for i, t in enumerate(c.layer_types) if t == "full_attention"]
        self.kv_index = {l: i for i, l in enumerate(self.full_layers)}
        self.lin_index = {l: i for i, l in enumerate(self.lin_layers)}
        self.kh_rng = common.shard_range(c.linear_num_key_heads, r, p)
        self.vh_rng = common.shard_range(c.linear_num_value_heads, r, p)
        self.hk_l = self.kh_rng[1] - self.kh_rng[0]
        self.hv_l = self.vh_rng[1] - self.vh_rng[0]
        self.dk, self.dv = c.linear_key_head_dim, c.linear_value_head_dim
        self.key_dim_l = self.hk_l * self.dk
        self.val_dim_l = self.hv_l * self.dv
        self.conv_dim_l = 2 * self.key_dim_l + self.val_dim_l
        # column layout of the fused input projection
        self.off_z = self.conv_dim_l
        self.off_b = self.off_z + self.val_dim_l
        self.off_a = self.off_b + self.hv_l
        self.in_cols = _pad8(self.off_a + self.hv_l)
        self.conv_state = None
        self.rec_state = None

    # ------------------------------------------------------------------ state
    def alloc_state(self, num_slots: int) -> None:
        """Per-sequence state pool of the linear-attention layers (conv inputs + recurrent state)."""
        c, nl = self.config, max(len(self.lin_layers), 1)
        self.conv_state = torch.zeros((nl, num_slots, c.linear_conv_kernel_dim - 1, self.conv_dim_l),
                                      dtype=self.dtype, device=self.device)
        self.rec_state = torch.zeros((nl, num_slots, self.hv_l, self.dk, self.dv), dtype=torch.float32,
                                     device=self.device)

    def state_bytes_per_slot(self) -> int:
        c = self.config
        return len(self.lin_layers) * ((c.linear_conv_kernel_dim - 1) * self.conv_dim_l * 2 + self.hv_l * self.dk * self.dv * 4)

    def kv_cache_shape(self, num_pages: int, page_size: int):
        return (max(len(self.full_layers), 1), 2, num_pages, page_size, self.hkv, self.config.hd)

    # ------------------------------------------------------------------ weights
    def _fuse_full_attn(self, q_proj, k, v):
        """HF q_proj rows are per head [q(hd) ; gate(hd)]: split them into a q block and a gate block."""
        hd = self.config.hd
        qg = q_proj.reshape(self.hq, 2, hd, q_proj.shape[-1])
        return torch.cat([qg[:, 0].reshape(self.hq * hd, -1), k, v, qg[:, 1].reshape(self.hq * hd, -1)], 0).contiguous()

    def _fuse_in_proj(self, qkv, z, b, a):
        """qkv rows are [all q heads | all k heads | all v heads] of this rank."""
        w = torch.zeros((self.in_cols, qkv.shape[1]), dtype=qkv.dtype, device=qkv.device)
        w[:self.conv_dim_l] = qkv
        w[self.off_z:self.off_b] = z
        w[self.off_b:self.off_a] = b
        w[self.off_a:self.off_a + self.hv_l] = a
        return w

    def _mix_rows(self, full_rows: torch.Tensor) -> torch.Tensor:
        """Selects this rank's rows of a tensor laid out [q heads | k heads | v heads] over all heads."""
        c = self.config
        kd = c.linear_num_key_heads * self.dk
        k0, k1 = self.kh_rng[0] * self.dk, self.kh_rng[1] * self.dk
        v0, v1 = self.vh_rng[0] * self.dv, self.vh_rng[1] * self.dv
        return torch.cat([full_rows[k0:k1], full_rows[kd + k0:kd + k1], full_rows[2 * kd + v0:2 * kd + v1]], 0)

    def _init_mlp(self, lw: LayerWeights, rw, b: int) -> None:
        c, d = self.config, self.config.hidden_size
        g = rw((c.intermediate_size, d), b + 4, rows=self.f_rng)
        u = rw((c.intermediate_size, d), b + 5, rows=self.f_rng)
        lw.gate_up = torch.cat([g, u], 0)
        lw.down = rw((d, c.intermediate_size), b + 6, cols=self.f_rng)

    def init_random(self, seed: int = 0, std: float = 0.02, full: Optional[bool] = None) -> "Qwen35Model":
        c, dev, dt = self.config, self.device, self.dtype
        if full is None:
            full = c.num_params() < 4e9
        d, hd = c.hidden_size, c.hd
        rw = lambda shape, s, **kw: common.randn_weight(shape, std, seed * 7919 + s, dev, dt, full=full, **kw)
        self.embed = rw((c.vocab_size, d), 1)
        self.final_norm = torch.zeros(d, dtype=dt, device=dev)
        if c.tie_word_embeddings:
            self.lm_head = self.embed[self.v_rng[0]:self.v_rng[1]] if self.comm.world > 1 else self.embed
        else:
            self.lm_head = rw((c.vocab_size, d), 2, rows=self.v_rng)
        k0, k1 = self.kv_rng[0] * hd, self.kv_rng[1] * hd
        kd, vd = c.linear_num_key_heads * self.dk, c.linear_num_value_heads * self.dv
        v0, v1 = self.vh_rng[0] * self.dv, self.vh_rng[1] * self.dv
        for l in range(c.num_hidden_layers):
            lw = LayerWeights()
            b = 100 + l * 24
            lw.input_norm = torch.zeros(d, dtype=dt, device=dev)
            lw.post_norm = torch.zeros(d, dtype=dt, device=dev)
            if c.layer_types[l] == "full_attention":
                qp = rw((c.num_attention_heads * 2 * hd, d), b + 0, rows=(self.q_rng[0] * 2 * hd, self.q_rng[1] * 2 * hd))
                k = rw((c.num_key_value_heads * hd, d), b + 1, rows=(k0, k1))
                v = rw((c.num_key_value_heads * hd, d), b + 2, rows=(k0, k1))
                lw.qkv = self._fuse_full_attn(qp, k, v)
                lw.q_norm = torch.zeros(hd, dtype=dt, device=dev)
                lw.k_norm = torch.zeros(hd, dtype=dt, device=dev)
                lw.o = rw((d, c.num_attention_heads * hd), b + 3, cols=(self.q_rng[0] * hd, self.q_rng[1] * hd))
            else:
                la_w = LinearAttnWeights()
                qkv = self._mix_rows(rw((2 * kd + vd, d), b + 8))
                z = rw((vd, d), b + 9, rows=(v0, v1))
                bb = rw((c.linear_num_value_heads, d), b + 10, rows=self.vh_rng)
                aa = rw((c.linear_num_value_heads, d), b + 11, rows=self.vh_rng)
                la_w.in_proj = self._fuse_in_proj(qkv, z, bb, aa)
                conv = common.randn_weight((2 * kd + vd, c.linear_conv_kernel_dim), 0.3, seed * 7919 + b + 12, dev, dt)
                la_w.conv_w = self._mix_rows(conv).contiguous()
                g = torch.Generator(device="cpu").manual_seed(seed * 7919 + b + 13)
                a_log = torch.log(torch.empty(c.linear_num_value_heads).uniform_(1.0, 16.0, generator=g))
                dtb = torch.empty(c.linear_num_value_heads).uniform_(-1.0, 1.0, generator=g)
                la_w.a_log = a_log[self.vh_rng[0]:self.vh_rng[1]].float().to(dev).contiguous()
                la_w.dt_bias = dtb[self.vh_rng[0]:self.vh_rng[1]].float().to(dev).contiguous()
                la_w.norm_w = torch.ones(self.dv, dtype=dt, device=dev)
                la_w.out_proj = rw((d, vd), b + 14, cols=(v0, v1))
                lw.extra = {"linear_attn": la_w}
            self._init_mlp(lw, rw, b)
            self.layers.append(lw)
        return self

    def _load_mlp(self, lw: LayerWeights, get, has, p: str) -> None:
        lw.gate_up = torch.cat([get(p + "mlp.gate_proj.weight", rows=self.f_rng),
                                get(p + "mlp.up_proj.weight", rows=self.f_rng)], 0)
        lw.down = get(p + "mlp.down_proj.weight", cols=self.f_rng)

    def load(self, store, prefix: Optional[str] = None) -> "Qwen35Model":
        c, hd = self.config, self.config.hd
        dev, dt = self.device, self.dtype
        prefix = self.PREFIX if prefix is None else prefix
        get = lambda name, **kw: store.load_tensor(prefix + name, device=dev, dtype=dt, **kw)
        has = lambda name: store.has_key(prefix + name)
        self.embed = get("embed_tokens.weight")
        self.final_norm = get("norm.weight")
        if store.has_key("lm_head.weight"):
            self.lm_head = store.load_tensor("lm_head.weight", device=dev, dtype=dt, rows=self.v_rng)
        else:
            self.lm_head = self.embed[self.v_rng[0]:self.v_rng[1]] if self.comm.world > 1 else self.embed
        k0, k1 = self.kv_rng[0] * hd, self.kv_rng[1] * hd
        v0, v1 = self.vh_rng[0] * self.dv, self.vh_rng[1] * self.dv
        for l in range(c.num_hidden_layers):
            p = f"layers.{l}."
            lw = LayerWeights()
            lw.input_norm = get(p + "input_layernorm.weight")
            lw.post_norm = get(p + "post_attention_layernorm.weight")
            if c.layer_types[l] == "full_attention":
                a = p + "self_attn."
                qp = get(a + "q_proj.weight", rows=(self.q_rng[0] * 2 * hd, self.q_rng[1] * 2 * hd))
                lw.qkv = self._fuse_full_attn(qp, get(a + "k_proj.weight", rows=(k0, k1)), get(a + "v_proj.weight", rows=(k0, k1)))
                lw.q_norm = get(a + "q_norm.weight")
                lw.k_norm = get(a + "k_norm.weight")
                lw.o = get(a + "o_proj.weight", cols=(self.q_rng[0] * hd, self.q_rng[1] * hd))
            else:
                a = p + "linear_attn."
                la_w = LinearAttnWeights()
                la_w.in_proj = self._fuse_in_proj(self._mix_rows(get(a + "in_proj_qkv.weight")),
                                                  get(a + "in_proj_z.weight", rows=(v0, v1)),
                                                  get(a + "in_proj_b.weight", rows=self.vh_rng),
                                                  get(a + "in_proj_a.weight", rows=self.vh_rng))
                conv = get(a + "conv1d.weight")                     # [conv_dim, 1, K]
                la_w.conv_w = self._mix_rows(conv.reshape(conv.shape[0], -1)).contiguous()
                la_w.a_log = store.load_tensor(prefix + a + "A_log", device=dev, dtype=torch.float32)[self.vh_rng[0]:self.vh_rng[1]].contiguous()
                la_w.dt_bias = store.load_tensor(prefix + a + "dt_bias", device=dev, dtype=torch.float32)[self.vh_rng[0]:self.vh_rng[1]].contiguous()
                la_w.norm_w = get(a + "norm.weight")
                la_w.out_proj = get(a + "out_proj.weight", cols=(v0, v1))
                lw.extra = {"linear_attn": la_w}
            self._load_mlp(lw, get, has, p)
            self.layers.append(lw)
        return self

    def _mlp_state_dict(self, lw: LayerWeights, p: str, out: dict) -> None:
        out[p + "mlp.gate_proj.weight"] = lw.gate_up[:self.f_local]
        out[p + "mlp.up_proj.weight"] = lw.gate_up[self.f_local:]
        out[p + "mlp.down_proj.weight"] = lw.down

    def state_dict_hf(self) -> dict:
        """This rank's weights under HF names; a complete checkpoint when TP == 1."""
        c, hd, pre = self.config, self.config.hd, self.PREFIX
        out = {pre + "embed_tokens.weight": self.embed, pre + "norm.weight": self.final_norm}
        if not c.tie_word_embeddings:
            out["lm_head.weight"] = self.lm_head
        nq, nk = self.hq * hd, self.hkv * hd
        for l, lw in enumerate(self.layers):
            p = pre + f"layers.{l}."
            out[p + "input_layernorm.weight"] = lw.input_norm
            out[p + "post_attention_layernorm.weight"] = lw.post_norm
            if c.layer_types[l] == "full_attention":
                q, g = lw.qkv[:nq], lw.qkv[nq + 2 * nk:]
                qp = torch.stack([q.reshape(self.hq, hd, -1), g.reshape(self.hq, hd, -1)], 1).reshape(2 * nq, -1)
                out[p + "self_attn.q_proj.weight"] = qp.contiguous()
                out[p + "self_attn.k_proj.weight"] = lw.qkv[nq:nq + nk]
                out[p + "self_attn.v_proj.weight"] = lw.qkv[nq + nk:nq + 2 * nk]
                out[p + "self_attn.q_norm.weight"] = lw.q_norm
                out[p + "self_attn.k_norm.weight"] = lw.k_norm
                out[p + "self_attn.o_proj.weight"] = lw.o
            else:
                w = lw.extra["linear_attn"]
                a = p + "linear_attn."
                out[a + "in_proj_qkv.weight"] = w.in_proj[:self.conv_dim_l]
                out[a + "in_proj_z.weight"] = w.in_proj[self.off_z:self.off_b]
                out[a + "in_proj_b.weight"] = w.in_proj[self.off_b:self.off_a]
                out[a + "in_proj_a.weight"] = w.in_proj[self.off_a:self.off_a + self.hv_l]
                out[a + "conv1d.weight"] = w.conv_w.reshape(w.conv_w.shape[0], 1, -1)
                out[a + "A_log"] = w.a_log
                out[a + "dt_bias"] = w.dt_bias
                out[a + "norm.weight"] = w.norm_w
                out[a + "out_proj.weight"] = w.out_proj
            self._mlp_state_dict(lw, p, out)
        return out

    def weight_bytes(self) -> int:
        n = super().weight_bytes()
        for lw in self.layers:
            if lw.extra and "linear_attn" in lw.extra:
                w = lw.extra["linear_attn"]
                n += sum(getattr(w, s).numel() * getattr(w, s).element_size() for s in w.__slots__)
        return n

    # ------------------------------------------------------------------ forward
    def _seq_meta(self, meta: AttnMeta, tokens: int):
        """(q_start, seq_lens, slots) of this launch; decode steps are one token per sequence."""
        if meta.state_slots is None:
            raise ValueError("hybrid models need AttnMeta.state_slots (one state slot per sequence)")
        q_start = meta.q_start
        if q_start is None:
            q_start = torch.arange(tokens + 1, dtype=torch.int32, device=meta.seq_lens.device)
        return q_start, meta.seq_lens, meta.state_slots

    def full_attention(self, l: int, lw: LayerWeights, n1, meta: AttnMeta, kv_cache):
        c = self.config
        kc, vc = kv_cache[self.kv_index[l], 0], kv_cache[self.kv_index[l], 1]
        nqkv = (self.hq + 2 * self.hkv) * c.hd
        qkvg = ops.gemm(n1, lw.qkv, static_w=True)
        q = ops.rope_kvwrite(qkvg[:, :nqkv], meta.positions, meta.slot_mapping, self.inv_freq, kc, vc, self.hq,
                             self.hkv, c.hd, self.rope_layout, self.rot_dim, 1.0, lw.q_norm, lw.k_norm,
                             c.rms_norm_eps, True)
        if meta.is_prefill:
            a = ops.paged_prefill(q, kc, vc, meta.block_table, meta.seq_lens, meta.q_start,
                                  total_q_blocks=meta.total_q_blocks)
        else:
            a = ops.paged_decode(q, kc, vc, meta.block_table, meta.seq_lens, num_splits=meta.num_splits,
                                 max_seq_len=meta.max_seq_len)
        a = a.reshape(a.shape[0], self.hq * c.hd)
        return la.sigmoid_gate_mul(a, qkvg[:, nqkv:])

    def linear_attention(self, l: int, lw: LayerWeights, n1, meta: AttnMeta):
        c, w = self.config, lw.extra["linear_attn"]
        i = self.lin_index[l]
        q_start, seq_lens, slots = self._seq_meta(meta, n1.shape[0])
        proj = ops.gemm(n1, w.in_proj, static_w=True)                   # [T, q|k|v|z|b|a]
        mix = la.causal_conv1d(proj[:, :self.conv_dim_l], w.conv_w, self.conv_state[i], q_start, seq_lens, slots,
                               silu=True)
        return la.gated_delta_scan(mix, proj[:, self.off_z:self.off_b], proj[:, self.off_a:self.off_a + self.hv_l],
                                   proj[:, self.off_b:self.off_a], w.a_log, w.dt_bias, w.norm_w, c.rms_norm_eps,
                                   self.rec_state[i], q_start, seq_lens, slots, self.hk_l, self.hv_l, self.dk, self.dv)

    def layer(self, l: int, x, meta: AttnMeta, kv_cache):
        lw, c = self.layers[l], self.config
        n1 = ops.rmsnorm(x, lw.input_norm, c.rms_norm_eps, unit_offset=True)
        if c.layer_types[l] == "full_attention":
            a = self.full_attention(l, lw, n1, meta, kv_cache)
            x = self.row_parallel(a, lw.o, x)
        else:
            if self.rec_state is None:
                self.alloc_state(int(meta.state_slots.max().item()) + 1 if meta.state_slots is not None else 1)
            a = self.linear_attention(l, lw, n1, meta)
            x = self.row_parallel(a, lw.extra["linear_attn"].out_proj, x)
        n2 = ops.rmsnorm(x, lw.post_norm, c.rms_norm_eps, unit_offset=True)
        return self.mlp(lw, x, n2)

    def logits(self, x, rows=None):
        if rows is not None:
            x = x.index_select(0, rows.long() if rows.dtype != torch.int64 else rows)
        n = ops.rmsnorm(x, self.final_norm, self.config.rms_norm_eps, unit_offset=True)
        return ops.gemm(n, self.lm_head, out_dtype=torch.float32, static_w=True)
