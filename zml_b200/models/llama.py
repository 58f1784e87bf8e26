"""Llama 3.1 / 3.2 (and architecturally identical dense decoders: Mistral, Qwen2/3 dense).

Same model as examples/llm/models/llama/model.zig of the reference: HF tensor
names (``model.embed_tokens``, ``model.layers.N.{input_layernorm, self_attn.{q,k,v,o}_proj,
post_attention_layernorm, mlp.{gate,up,down}_proj}``, ``model.norm``, optional ``lm_head``
else tied), RMSNorm -> attention -> residual -> RMSNorm -> SwiGLU MLP -> residual,
RoPE in the HF `rotate_half` layout with llama3 frequency scaling.

Tensor parallelism is Megatron style as in the reference (model.zig:474-479,516-519):
q/k/v/gate/up are split on their output axis, o/down on their input axis, the
residual stream is replicated and each layer ends in two all-reduces - here issued
from inside the row-parallel GEMM kernel when fused kernels are enabled.
q, k, v are stored fused ([q | k | v] rows) and gate, up fused ([gate | up] rows),
so a layer is 4 GEMMs, and the B200 kernels never materialise a transpose.
"""
from __future__ import annotations

import os

from dataclasses import dataclass, field
from typing import Optional

import torch

from .. import ops
from ..nn import rotary as rope_mod
from ..parallel.comm import Comm
from . import common


@dataclass
class LlamaConfig:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    max_position_embeddings: int = 8192
    head_dim: Optional[int] = None
    tie_word_embeddings: bool = False
    rope_scaling: Optional[dict] = None
    bos_token_id: int = 1
    eos_token_id: object = 2
    hf_rope_impl: bool = True
    attention_bias: bool = False      # Qwen2-style q/k/v bias
    qk_norm: bool = False             # Qwen3-style per-head RMSNorm of q and k
    sliding_window: int = 0
    model_type: str = "llama"

    @staticmethod
    def from_hf(obj: dict) -> "LlamaConfig":
        names = set(LlamaConfig.__dataclass_fields__)
        kw = {k: v for k, v in obj.items() if k in names and v is not None}
        mt = obj.get("model_type", "llama")
        if mt in ("qwen3", "qwen3_moe"):
            kw.setdefault("qk_norm", True)
        if mt == "qwen2":
            kw.setdefault("attention_bias", True)
        if "sliding_window" in kw and not obj.get("use_sliding_window", mt == "mistral"):
            kw["sliding_window"] = 0
        for need in ("hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size",
                     "vocab_size"):
            if need not in kw:
                raise ValueError(f"config.json lacks {need}")
        kw.setdefault("num_key_value_heads", kw["num_attention_heads"])
        return LlamaConfig(**kw)

    @property
    def hd(self) -> int:
        return self.head_dim or self.hidden_size // self.num_attention_heads

    def rope_opts(self) -> rope_mod.RopeOpts:
        layout = rope_mod.Layout.real_im_pass if self.hf_rope_impl else rope_mod.Layout.interleaved
        return rope_mod.RopeOpts(layout, rope_mod.Scaling.from_hf(self.rope_scaling, self.rope_theta))

    def eos_ids(self) -> list[int]:
        return common.eos_list(self.eos_token_id)

    def num_params(self) -> int:
        d, f, v, l = self.hidden_size, self.intermediate_size, self.vocab_size, self.num_hidden_layers
        attn = d * self.hd * (self.num_attention_heads * 2 + self.num_key_value_heads * 2)
        per_layer = attn + 3 * d * f + 2 * d
        return l * per_layer + v * d * (1 if self.tie_word_embeddings else 2) + d


# Named configurations of the benchmark suite (architecture only; weights are random-init).
PRESETS = {
    "llama-3.2-1b": dict(hidden_size=2048, num_hidden_layers=16, num_attention_heads=32,
                         num_key_value_heads=8, head_dim=64, intermediate_size=8192,
                         vocab_size=128256, rms_norm_eps=1e-5, rope_theta=500000.0,
                         tie_word_embeddings=True, max_position_embeddings=131072,
                         rope_scaling=dict(rope_type="llama3", factor=32.0, high_freq_factor=4.0,
                                           low_freq_factor=1.0, original_max_position_embeddings=8192),
                         bos_token_id=128000, eos_token_id=[128001, 128008, 128009]),
    "llama-3.1-8b": dict(hidden_size=4096, num_hidden_layers=32, num_attention_heads=32,
                         num_key_value_heads=8, head_dim=128, intermediate_size=14336,
                         vocab_size=128256, rms_norm_eps=1e-5, rope_theta=500000.0,
                         tie_word_embeddings=False, max_position_embeddings=131072,
                         rope_scaling=dict(rope_type="llama3", factor=8.0, high_freq_factor=4.0,
                                           low_freq_factor=1.0, original_max_position_embeddings=8192),
                         bos_token_id=128000, eos_token_id=[128001, 128008, 128009]),
    "llama-3.1-70b": dict(hidden_size=8192, num_hidden_layers=80, num_attention_heads=64,
                          num_key_value_heads=8, head_dim=128, intermediate_size=28672,
                          vocab_size=128256, rms_norm_eps=1e-5, rope_theta=500000.0,
                          tie_word_embeddings=False, max_position_embeddings=131072,
                          rope_scaling=dict(rope_type="llama3", factor=8.0, high_freq_factor=4.0,
                                            low_freq_factor=1.0, original_max_position_embeddings=8192),
                          bos_token_id=128000, eos_token_id=[128001, 128008, 128009]),
    "tiny-llama-test": dict(hidden_size=256, num_hidden_layers=2, num_attention_heads=8,
                            num_key_value_heads=2, head_dim=64, intermediate_size=512, vocab_size=1024,
                            rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=True,
                            max_position_embeddings=4096, bos_token_id=1, eos_token_id=2),
}


@dataclass
class AttnMeta:
    """Per-step attention metadata in the shapes of the reference's paged API
    (zml/attention/paged_attention.zig:19-293): block_table {b,p}, seq_lens {b},
    query_start_len {b+1}, slot_mapping {tokens}."""
    is_prefill: bool
    positions: torch.Tensor
    slot_mapping: torch.Tensor
    block_table: torch.Tensor
    seq_lens: torch.Tensor
    q_start: Optional[torch.Tensor] = None
    total_q_blocks: Optional[int] = None
    num_splits: Optional[int] = None
    max_seq_len: Optional[int] = None
    logits_rows: Optional[torch.Tensor] = None    # rows of the hidden state that need logits
    state_slots: Optional[torch.Tensor] = None    # {b} slot of every sequence in a model's recurrent-state pool
    q_start_host: Optional[list] = None           # host copy of q_start (prefill), for splitting a chunk by sequences


class LayerWeights:
    __slots__ = ("input_norm", "qkv", "qkv_bias", "q_norm", "k_norm", "o", "post_norm", "gate_up", "down",
                 "extra")

    def __init__(self):
        for s in self.__slots__:
            setattr(self, s, None)


class LlamaModel:
    """Weights of one tensor-parallel rank plus the forward pass over a flattened token batch."""

    def __init__(self, config: LlamaConfig, comm: Optional[Comm] = None, device="cpu",
                 dtype=torch.bfloat16):
        self.config = config
        self.comm = comm or Comm.single()
        self.device = torch.device(device)
        self.dtype = dtype
        c, p, r = config, self.comm.world, self.comm.rank
        if c.num_attention_heads % p != 0:
            raise ValueError(f"{c.num_attention_heads} heads not divisible by TP={p}")
        self.hq = c.num_attention_heads // p
        self.q_rng = common.shard_range(c.num_attention_heads, r, p)
        self.kv_rng = common.kv_head_shard(c.num_key_value_heads, r, p)
        self.hkv = self.kv_rng[1] - self.kv_rng[0]
        self.f_rng = common.shard_range(c.intermediate_size, r, p)
        self.f_local = self.f_rng[1] - self.f_rng[0]
        # vocab-parallel lm_head: every rank holds v_per rows; rows past the vocabulary (last ranks, when the
        # vocabulary does not divide) are zero rows whose logits are masked to -inf
        self.v_per = (c.vocab_size + p - 1) // p
        self.v_rng = (min(c.vocab_size, r * self.v_per), min(c.vocab_size, (r + 1) * self.v_per))
        self.v_pad = self.v_per - (self.v_rng[1] - self.v_rng[0])
        self.fused_layout = False     # see prepare_fused
        opts = c.rope_opts()
        self.rope_layout = opts.layout.value
        self.rot_dim = opts.scaling.partial_rotary_dim(c.hd)
        self.attn_factor = opts.scaling.attention_scaling()
        self.inv_freq = rope_mod.inv_freq(c.hd, opts).to(self.device)
        self.embed = None
        self.final_norm = None
        self.lm_head = None
        self.layers: list[LayerWeights] = []

    # ------------------------------------------------------------------ weights
    def init_random(self, seed: int = 0, std: float = 0.02, full: Optional[bool] = None) -> "LlamaModel":
        """Random-init N(0, std) weights of this architecture (norm weights are ones)."""
        c, dev, dt = self.config, self.device, self.dtype
        if full is None:
            full = c.num_params() < 12e9
        d, hd = c.hidden_size, c.hd
        rw = lambda shape, s, **kw: common.randn_weight(shape, std, seed * 7919 + s, dev, dt, full=full, **kw)
        self.embed = rw((c.vocab_size, d), 1)
        self.final_norm = torch.ones(d, dtype=dt, device=dev)
        if c.tie_word_embeddings:
            self.lm_head = self.embed[self.v_rng[0]:self.v_rng[1]] if self.comm.world > 1 else self.embed
        else:
            self.lm_head = rw((c.vocab_size, d), 2, rows=self.v_rng)
        self._pad_lm_head()
        q0, q1 = self.q_rng[0] * hd, self.q_rng[1] * hd
        k0, k1 = self.kv_rng[0] * hd, self.kv_rng[1] * hd
        for l in range(c.num_hidden_layers):
            lw = LayerWeights()
            b = 100 + l * 16
            lw.input_norm = torch.ones(d, dtype=dt, device=dev)
            lw.post_norm = torch.ones(d, dtype=dt, device=dev)
            q = rw((c.num_attention_heads * hd, d), b + 0, rows=(q0, q1))
            k = rw((c.num_key_value_heads * hd, d), b + 1, rows=(k0, k1))
            v = rw((c.num_key_value_heads * hd, d), b + 2, rows=(k0, k1))
            lw.qkv = torch.cat([q, k, v], 0)
            del q, k, v
            if c.attention_bias:
                lw.qkv_bias = torch.zeros(lw.qkv.shape[0], dtype=dt, device=dev)
            if c.qk_norm:
                lw.q_norm = torch.ones(hd, dtype=dt, device=dev)
                lw.k_norm = torch.ones(hd, dtype=dt, device=dev)
            lw.o = rw((d, c.num_attention_heads * hd), b + 3, cols=(q0, q1))
            g = rw((c.intermediate_size, d), b + 4, rows=self.f_rng)
            u = rw((c.intermediate_size, d), b + 5, rows=self.f_rng)
            lw.gate_up = torch.cat([g, u], 0)
            del g, u
            lw.down = rw((d, c.intermediate_size), b + 6, cols=self.f_rng)
            self.layers.append(lw)
        return self

    def _pad_lm_head(self) -> None:
        if self.v_pad > 0 and self.comm.world > 1 and self.lm_head.shape[0] < self.v_per:
            pad = torch.zeros((self.v_pad, self.lm_head.shape[1]), dtype=self.lm_head.dtype, device=self.lm_head.device)
            self.lm_head = torch.cat([self.lm_head, pad], 0)

    def load(self, store, prefix: str = "", platform=None) -> "LlamaModel":
        """Loads this rank's shards from a TensorStore view (HF names).  Only the byte ranges
        of the shard are read.  With a `platform`, the weights are described as tagged tensors with partition
        specs and cut by the generic `Loader` (`Sharding.placement` decides each rank's rows and columns) when the
        layout allows it; otherwise the ranges come from this model's own head / vocabulary split."""
        if platform is not None:
            from . import tagged_llama
            try:
                return tagged_llama.load_serving_weights(self, platform, store, prefix)
            except ValueError:
                pass
        c, hd = self.config, self.config.hd
        dev, dt = self.device, self.dtype
        q0, q1 = self.q_rng[0] * hd, self.q_rng[1] * hd
        k0, k1 = self.kv_rng[0] * hd, self.kv_rng[1] * hd
        get = lambda name, **kw: store.load_tensor(prefix + name, device=dev, dtype=dt, **kw)
        self.embed = get("model.embed_tokens.weight")
        self.final_norm = get("model.norm.weight")
        if store.has_key(prefix + "lm_head.weight"):
            self.lm_head = get("lm_head.weight", rows=self.v_rng)
        else:
            self.lm_head = self.embed[self.v_rng[0]:self.v_rng[1]] if self.comm.world > 1 else self.embed
        self._pad_lm_head()
        for l in range(c.num_hidden_layers):
            p = f"model.layers.{l}."
            lw = LayerWeights()
            lw.input_norm = get(p + "input_layernorm.weight")
            lw.post_norm = get(p + "post_attention_layernorm.weight")
            lw.qkv = torch.cat([get(p + "self_attn.q_proj.weight", rows=(q0, q1)),
                                get(p + "self_attn.k_proj.weight", rows=(k0, k1)),
                                get(p + "self_attn.v_proj.weight", rows=(k0, k1))], 0)
            if store.has_key(prefix + p + "self_attn.q_proj.bias"):
                lw.qkv_bias = torch.cat([get(p + "self_attn.q_proj.bias", rows=(q0, q1)),
                                         get(p + "self_attn.k_proj.bias", rows=(k0, k1)),
                                         get(p + "self_attn.v_proj.bias", rows=(k0, k1))], 0)
            if store.has_key(prefix + p + "self_attn.q_norm.weight"):
                lw.q_norm = get(p + "self_attn.q_norm.weight")
                lw.k_norm = get(p + "self_attn.k_norm.weight")
            lw.o = get(p + "self_attn.o_proj.weight", cols=(q0, q1))
            lw.gate_up = torch.cat([get(p + "mlp.gate_proj.weight", rows=self.f_rng),
                                    get(p + "mlp.up_proj.weight", rows=self.f_rng)], 0)
            lw.down = get(p + "mlp.down_proj.weight", cols=self.f_rng)
            self.layers.append(lw)
        return self

    def state_dict_hf(self) -> dict:
        """This rank's weights under HF names (un-fused); with TP=1 this is a full checkpoint."""
        c, hd = self.config, self.config.hd
        if self.fused_layout:
            raise RuntimeError("the weights are in the fused-kernel layout (norms folded, gate / up interleaved); "
                               "export before the first forward pass on a GPU")
        out = {"model.embed_tokens.weight": self.embed, "model.norm.weight": self.final_norm}
        if not c.tie_word_embeddings:
            out["lm_head.weight"] = self.lm_head[:self.v_rng[1] - self.v_rng[0]]
        nq, nk = self.hq * hd, self.hkv * hd
        for l, lw in enumerate(self.layers):
            p = f"model.layers.{l}."
            out[p + "input_layernorm.weight"] = lw.input_norm
            out[p + "post_attention_layernorm.weight"] = lw.post_norm
            out[p + "self_attn.q_proj.weight"] = lw.qkv[:nq]
            out[p + "self_attn.k_proj.weight"] = lw.qkv[nq:nq + nk]
            out[p + "self_attn.v_proj.weight"] = lw.qkv[nq + nk:]
            if lw.qkv_bias is not None:
                out[p + "self_attn.q_proj.bias"] = lw.qkv_bias[:nq]
                out[p + "self_attn.k_proj.bias"] = lw.qkv_bias[nq:nq + nk]
                out[p + "self_attn.v_proj.bias"] = lw.qkv_bias[nq + nk:]
            if lw.q_norm is not None:
                out[p + "self_attn.q_norm.weight"] = lw.q_norm
                out[p + "self_attn.k_norm.weight"] = lw.k_norm
            out[p + "self_attn.o_proj.weight"] = lw.o
            out[p + "mlp.gate_proj.weight"] = lw.gate_up[:self.f_local]
            out[p + "mlp.up_proj.weight"] = lw.gate_up[self.f_local:]
            out[p + "mlp.down_proj.weight"] = lw.down
        return out

    def weight_bytes(self) -> int:
        n = self.embed.numel() + self.final_norm.numel()
        if self.lm_head is not None and self.lm_head.data_ptr() != self.embed.data_ptr():
            n += self.lm_head.numel()
        for lw in self.layers:
            for s in LayerWeights.__slots__:
                t = getattr(lw, s)
                if isinstance(t, torch.Tensor):
                    n += t.numel()
        return n * 2

    # ------------------------------------------------------------------ forward
    def kv_cache_shape(self, num_pages: int, page_size: int):
        return (self.config.num_hidden_layers, 2, num_pages, page_size, self.hkv, self.config.hd)

    def row_parallel(self, a, w, residual, emit_stats: bool = False, next_w=None):
        """Row-parallel linear + all-reduce + residual add: the o_proj / down_proj pattern.  With `emit_stats`
        returns (x, RowStats of x): the partial sums of squares the next GEMM normalises its input with.
        `next_w`: the weights of the GEMM that follows, which the fused kernel pulls into L2 while it
        exchanges partial sums with the peers."""
        comm = self.comm
        if comm.world == 1:
            return ops.gemm(a, w, residual=residual, out=residual if residual.is_cuda else None, static_w=True,
                            emit_stats=emit_stats)
        if comm.fused is not None and a.is_cuda and a.shape[0] <= comm.fused.fused_max_tokens:
            return comm.fused.gemm_allreduce(a, w, residual, emit_stats=emit_stats,
                                             prefetch=next_w if self.prefetch_next else None)
        if comm.fused is not None and a.is_cuda and comm.fused.can_all_reduce_ll(a.shape[0], w.shape[0]):
            x = comm.fused.all_reduce_ll(ops.gemm(a, w, static_w=True), residual)
        elif comm.fused is not None and a.is_cuda and comm.fused.can_all_reduce_mm(a.shape[0], w.shape[0]):
            # prefill-sized: partial sums go straight into the symmetric heap, NVSwitch adds them up
            part = ops.gemm(a, w, static_w=True, out=comm.fused.partial_buffer(a.shape[0], w.shape[0]))
            x = comm.fused.all_reduce_mm(part, residual)
        else:
            part = ops.gemm(a, w, residual=residual if comm.rank == 0 else None, static_w=True)
            x = comm.all_reduce_(part)
        return (x, ops.row_sumsq(x)) if emit_stats else x

    def mlp(self, lw: LayerWeights, x, n2):
        gu = ops.gemm(n2, lw.gate_up, static_w=True)
        act = ops.swiglu(gu)
        return self.row_parallel(act, lw.down, x)

    # Attention backend (the reference's `zml.attention.Backend`, zml/attention/attention.zig:9-27):
    #   "b200"     the paged tcgen05 / flash-decoding kernels of this library (on CPU: their float32 restatements)
    #   "vanilla"  PyTorch SDPA on K/V gathered from the pages (what the reference's `vanilla` tensor formulation is)
    #   "attnd"    a remote attention daemon that owns the KV cache (one UDP datagram per token and KV head)
    attn_backend = "b200"
    _attnd = None

    def set_attention_backend(self, name: str, attnd_address=None, model_id: int = 0, conversation_id: int = 749,
                              mtu: int = 1500) -> None:
        if name not in ("b200", "vanilla", "attnd"):
            raise ValueError(f"unknown attention backend {name!r}; known: b200, vanilla, attnd")
        if name == "attnd":
            from ..attention import attnd
            if attnd_address is None:
                raise ValueError("the attnd backend needs the daemon's address (IP:PORT)")
            attnd.register(attnd.Config(tuple(attnd_address), mtu), num_devices=1)
            c = self.config
            mk = lambda prefill: attnd.Parameters.init(model_id, c.hd, c.num_attention_heads, c.num_key_value_heads, prefill)
            self._attnd = (attnd, mk(True), mk(False), conversation_id)
        self.attn_backend = name

    def _attention_attnd(self, lw: LayerWeights, qkv, meta: AttnMeta):
        """One sequence at a time (a chat session): q, k, v of the new tokens go to the daemon, which keeps the KV."""
        from ..ops import reference as R
        from ..tensor import Tensor
        attnd, p_prefill, p_decode, conv = self._attnd
        c, hd = self.config, self.config.hd
        t = qkv.shape[0]
        q, k, v = qkv.split([self.hq * hd, self.hkv * hd, self.hkv * hd], dim=-1)
        q, k, v = q.reshape(t, self.hq, hd), k.reshape(t, self.hkv, hd), v.reshape(t, self.hkv, hd)
        if lw.q_norm is not None:
            q = R.rmsnorm(q, lw.q_norm, c.rms_norm_eps)
            k = R.rmsnorm(k, lw.k_norm, c.rms_norm_eps)
        q = R.rope_rotate(q, meta.positions, self.inv_freq, self.rope_layout, self.rot_dim, self.attn_factor)
        k = R.rope_rotate(k, meta.positions, self.inv_freq, self.rope_layout, self.rot_dim, self.attn_factor)
        b16 = lambda x: x.to(torch.bfloat16)
        md = attnd.Metadata(conv, self.layers.index(lw), t)
        start = int(meta.positions[0])
        if meta.is_prefill:
            # the client sends rows 0..t-1 of k / v as positions start..start+t-1
            out = attnd.causal_attention(Tensor(b16(q), None, ("q", "h", "hd")), Tensor(b16(k), None, ("k", "h", "hd")),
                                         Tensor(b16(v), None, ("k", "h", "hd")), start, md, p_prefill,
                                         self.comm.rank, self.comm.world)
        else:
            out = attnd.causal_attention(Tensor(b16(q), None, ("q", "h", "hd")), Tensor(b16(k), None, ("k", "h", "hd")),
                                         Tensor(b16(v), None, ("k", "h", "hd")), start, md, p_decode,
                                         self.comm.rank, self.comm.world, new_rows_only=True)
        return out.to_torch().to(qkv.dtype).reshape(t, self.hq * hd)

    def attention_from_qkv(self, lw: LayerWeights, qkv, meta: AttnMeta, kc, vc):
        c = self.config
        if self.attn_backend == "attnd":
            return self._attention_attnd(lw, qkv, meta)
        q = ops.rope_kvwrite(qkv, meta.positions, meta.slot_mapping, self.inv_freq, kc, vc, self.hq,
                             self.hkv, c.hd, self.rope_layout, self.rot_dim, self.attn_factor,
                             lw.q_norm, lw.k_norm, c.rms_norm_eps, False)
        impl = ops
        if self.attn_backend == "vanilla":
            from ..ops import baseline as impl
        if meta.is_prefill:
            a = impl.paged_prefill(q, kc, vc, meta.block_table, meta.seq_lens, meta.q_start,
                                   window=c.sliding_window, total_q_blocks=meta.total_q_blocks)
        else:
            a = impl.paged_decode(q, kc, vc, meta.block_table, meta.seq_lens, window=c.sliding_window,
                                  num_splits=meta.num_splits, max_seq_len=meta.max_seq_len)
        return a.reshape(a.shape[0], self.hq * c.hd)

    def attention(self, lw: LayerWeights, n1, meta: AttnMeta, kc, vc):
        qkv = ops.gemm(n1, lw.qkv, bias=lw.qkv_bias, static_w=True)
        return self.attention_from_qkv(lw, qkv, meta, kc, vc)

    # ---- fused-kernel layout: a decoder layer is 6 launches (qkv GEMM, rope + KV write, attention, o GEMM
    # (+ all-reduce), gate|up GEMM with SwiGLU, down GEMM (+ all-reduce)) instead of 9: the two RMSNorms
    # become a per-row scale in the epilogue of the GEMM that consumes the normalised activation (the norm
    # weight is folded into that GEMM's weight columns, the row statistics come out of the epilogue of the
    # GEMM that produced the residual stream), and SwiGLU runs in the gate|up GEMM's epilogue on interleaved
    # gate / up rows.  The reference leaves these fusions to XLA (examples/llm/models/llama/model.zig:414-443).
    # ZB_PREFETCH_NEXT=0: the fused GEMM + all-reduce does not pull the next GEMM's weights into L2
    prefetch_next = os.environ.get("ZB_PREFETCH_NEXT", "1") != "0"

    def wants_fused_layout(self) -> bool:
        from ..ops import baseline as _baseline
        return (type(self).layer is LlamaModel.layer and type(self).mlp is LlamaModel.mlp and self.device.type == "cuda"
                and not _baseline.enabled() and os.environ.get("ZB_FOLD_NORMS", "1") != "0")

    def prepare_fused(self) -> None:
        """In place, once: qkv[:, j] *= input_norm[j], gate_up[:, j] *= post_norm[j], gate / up rows interleaved."""
        if self.fused_layout:
            return
        for lw in self.layers:
            lw.qkv.mul_(lw.input_norm[None, :].to(lw.qkv.dtype))
            gu = ops.interleave_gate_up(lw.gate_up)
            gu.mul_(lw.post_norm[None, :].to(gu.dtype))
            lw.gate_up.copy_(gu)
            del gu
        self.fused_layout = True

    def _layer_fused(self, l: int, x, stats, meta: AttnMeta, kv_cache):
        lw, c = self.layers[l], self.config
        qkv = ops.gemm(x, lw.qkv, bias=lw.qkv_bias, static_w=True, row_stats=stats, eps=c.rms_norm_eps)
        a = self.attention_from_qkv(lw, qkv, meta, kv_cache[l, 0], kv_cache[l, 1])
        x, stats = self.row_parallel(a, lw.o, x, emit_stats=True, next_w=lw.gate_up)
        act = ops.gemm(x, lw.gate_up, static_w=True, row_stats=stats, eps=c.rms_norm_eps, swiglu=True)
        nxt = self.layers[l + 1].qkv if l + 1 < len(self.layers) else None
        return self.row_parallel(act, lw.down, x, emit_stats=True, next_w=nxt)

    def layer(self, l: int, x, meta: AttnMeta, kv_cache):
        if self.fused_layout:
            return self._layer_fused(l, x, ops.row_sumsq(x), meta, kv_cache)[0]
        lw, c = self.layers[l], self.config
        kc, vc = kv_cache[l, 0], kv_cache[l, 1]
        n1 = ops.rmsnorm(x, lw.input_norm, c.rms_norm_eps)
        a = self.attention(lw, n1, meta, kc, vc)
        x = self.row_parallel(a, lw.o, x)
        n2 = ops.rmsnorm(x, lw.post_norm, c.rms_norm_eps)
        return self.mlp(lw, x, n2)

    def _layers_banded(self, x, meta: AttnMeta, kv_cache):
        """Prefill-sized step under tensor parallelism: the all-reduce after o_proj / down_proj never runs on its
        own.  The row-parallel GEMM leaves partial sums in the symmetric heap and announces them band by band
        (128 tokens); a few CTAs of the column-parallel GEMM that follows (gate|up, next layer's qkv) pull them from
        the peers' heaps, add them up with the residual and hand the bands with their RMSNorm statistics to every
        rank, the other CTAs multiply the bands as they arrive.  Only the last down_proj of the stack is followed by
        a stand-alone sum."""
        c, fused = self.config, self.comm.fused
        t, n_layers = x.shape[0], len(self.layers)
        stats, owed = ops.row_sumsq(x), False
        for l, lw in enumerate(self.layers):
            if owed:
                qkv, x = fused.band_consumer(t, lw.qkv, x, bias=lw.qkv_bias, eps=c.rms_norm_eps)
            else:
                qkv = ops.gemm(x, lw.qkv, bias=lw.qkv_bias, static_w=True, row_stats=stats, eps=c.rms_norm_eps)
            a = self.attention_from_qkv(lw, qkv, meta, kv_cache[l, 0], kv_cache[l, 1])
            fused.band_producer(a, lw.o)
            act, x = fused.band_consumer(t, lw.gate_up, x, swiglu=True, eps=c.rms_norm_eps)
            if l + 1 < n_layers:
                fused.band_producer(act, lw.down)
                owed = True
            else:
                x, stats = self.row_parallel(act, lw.down, x, emit_stats=True)
                owed = False
        return x

    def hidden_states(self, ids, meta: AttnMeta, kv_cache):
        x = ops.embedding(ids, self.embed)
        if not self.fused_layout and self.wants_fused_layout():
            self.prepare_fused()
        if self.fused_layout and self.comm.world > 1 and self.comm.fused is not None and \
                self.comm.fused.can_band(x.shape[0], self.config.hidden_size):
            return self._layers_banded(x, meta, kv_cache)
        if self.fused_layout:
            stats = ops.row_sumsq(x)
            for l in range(self.config.num_hidden_layers):
                x, stats = self._layer_fused(l, x, stats, meta, kv_cache)
            return x
        for l in range(self.config.num_hidden_layers):
            x = self.layer(l, x, meta, kv_cache)
        return x

    def logits(self, x, rows=None):
        """float32 logits of this rank's vocab shard for the selected rows."""
        if rows is not None:
            x = x.index_select(0, rows.long() if rows.dtype != torch.int64 else rows)
        n = ops.rmsnorm(x, self.final_norm, self.config.rms_norm_eps)
        if self.v_pad > 0 and self.comm.world > 1 and self.lm_head.shape[0] < self.v_per:
            self._pad_lm_head()         # model families that fill `lm_head` themselves
        lg = ops.gemm(n, self.lm_head, out_dtype=torch.float32, static_w=True)
        if self.v_pad > 0 and self.comm.world > 1:
            lg[:, self.v_per - self.v_pad:] = float("-inf")
        return lg

    def sample(self, logits, strategy: common.SamplingStrategy, seed: int = 0, step: int = 0, rng=None):
        """Token ids int32 [B] from vocab-parallel logits.  `rng`: device-side {seed, draw counter} of
        `ops.topk_sample` (the serving engine's, so that graph replays draw fresh noise)."""
        comm = self.comm
        rng = rng if (rng is not None and logits.is_cuda) else None
        if comm.world == 1:
            if strategy.topk <= 1:
                return ops.argmax(logits)
            return ops.topk_sample(logits, strategy.topk, strategy.temperature, seed, step, rng=rng)
        if strategy.topk <= 1:
            if comm.fused is not None and logits.is_cuda and comm.fused.can_argmax_tp(logits.shape[0]):
                return comm.fused.argmax_tp(logits, comm.rank * self.v_per)     # candidates exchanged inside the kernel
            idx = ops.argmax(logits)
            val = logits.gather(1, idx.long()[:, None])[:, 0]
            vals = comm.all_gather(val[None])                   # [P, B]
            idxs = comm.all_gather((idx + self.comm.rank * self.v_per)[None])
            best = vals.argmax(0)
            return idxs.gather(0, best[None])[0].to(torch.int32)
        # Every rank ranks its own columns (column j of rank r is token r * v_per + j; padding columns are -inf) and
        # only the k best (value, token) pairs per row travel: the k best of their union are the k best of the whole
        # vocabulary, in the same order, so the draw below equals the draw on gathered logits at 1 / (v_per / k) of the bytes.
        k = min(strategy.topk, logits.shape[1])
        vals, idx = ops.topk(logits, k)
        cand_v = comm.all_gather(vals.contiguous(), dim=1).contiguous()
        cand_i = comm.all_gather((idx + comm.rank * self.v_per).to(torch.int32).contiguous(), dim=1)
        pos = ops.topk_sample(cand_v, strategy.topk if strategy.topk <= cand_v.shape[1] else cand_v.shape[1],
                              strategy.temperature, seed, step, rng=rng)
        return cand_i.gather(1, pos.long()[:, None])[:, 0].to(torch.int32)

    def forward(self, ids, meta: AttnMeta, kv_cache, strategy: Optional[common.SamplingStrategy] = None,
                seed: int = 0, step: int = 0, rng=None):
        """ids int32 [T] -> sampled tokens int32 [rows] (one per sequence)."""
        x = self.hidden_states(ids, meta, kv_cache)
        lg = self.logits(x, meta.logits_rows)
        return self.sample(lg, strategy or common.SamplingStrategy(), seed, step, rng)
