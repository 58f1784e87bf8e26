"""Llama written on the tagged Tensor API, the way the reference writes its models
(examples/llm/models/llama/model.zig: weights created from a `TensorStore.View` with axis tags and partition
specs, `forward` on tagged tensors, loaded with `io.load` under the platform's shardings, compiled with
`platform.compile`, called through `Exe`).

It reads the same Hugging Face checkpoint as the serving model (`zml_b200.models.llama.LlamaModel`).  That one is
the fast path: fused kernels, paged KV cache, CUDA graphs.  This one is the generic path: every projection is a
`Tensor.dot`, the layout is carried by partition specs, and on a multi-process platform the program runs SPMD on
the shards the `Loader` cut out of the checkpoint (`Sharding.placement`), with the collectives issued where a
layout changes:

    q/k/v, gate, up   weight {dout, d}, dout sharded over `model`   column parallel: the heads / the ffn are split
    o_proj, down      weight {d, din},  din  sharded over `model`   row parallel: partial sums, all-reduce
    lm_head           weight {voc, d},  voc  sharded over `model`   vocabulary parallel: logits all-gathered

Prefill only (whole sequences, causal attention, no KV cache): the serving path owns decoding.
"""
from __future__ import annotations


import torch

from ..io import Loader, TensorStore, View
from ..nn import attention_ref, layers
from ..ops import reference as _ref
from ..tensor import Tensor
from .llama import LlamaConfig

MODEL_AXIS = "model"


class TaggedLlamaLayer:
    def __init__(self, view: View, cfg: LlamaConfig):
        col = {"dout": MODEL_AXIS}
        row = {"din": MODEL_AXIS}
        a, m = view.with_prefix("self_attn"), view.with_prefix("mlp")
        self.input_norm = view.create_tensor("input_layernorm.weight", ("d",))
        self.post_norm = view.create_tensor("post_attention_layernorm.weight", ("d",))
        self.q = a.create_tensor("q_proj.weight", ("dout", "d"), col)
        self.k = a.create_tensor("k_proj.weight", ("dout", "d"), col)
        self.v = a.create_tensor("v_proj.weight", ("dout", "d"), col)
        self.o = a.create_tensor("o_proj.weight", ("d", "din"), row)
        self.gate = m.create_tensor("gate_proj.weight", ("dout", "d"), col)
        self.up = m.create_tensor("up_proj.weight", ("dout", "d"), col)
        self.down = m.create_tensor("down_proj.weight", ("d", "din"), row)
        # Qwen2-style projection biases and Qwen3-style per-head q / k norms, where the checkpoint has them
        self.q_bias = a.maybe_create_tensor("q_proj.bias", ("dout",), col)
        self.k_bias = a.maybe_create_tensor("k_proj.bias", ("dout",), col)
        self.v_bias = a.maybe_create_tensor("v_proj.bias", ("dout",), col)
        self.q_norm = a.maybe_create_tensor("q_norm.weight", ("hd",))
        self.k_norm = a.maybe_create_tensor("k_norm.weight", ("hd",))


class TaggedLlama:
    """`forward(weights, tokens {s} i32) -> logits {s, voc}` of one sequence."""

    def __init__(self, view: View, cfg: LlamaConfig):
        self.cfg = cfg
        model = view.with_prefix("model")
        self.embed = model.create_tensor("embed_tokens.weight", ("voc", "d"))
        self.layers = [TaggedLlamaLayer(model.with_prefix("layers").with_layer(i), cfg) for i in range(cfg.num_hidden_layers)]
        self.norm = model.create_tensor("norm.weight", ("d",))
        head = "model.embed_tokens.weight" if cfg.tie_word_embeddings or not view.has_key("lm_head.weight") else "lm_head.weight"
        self.lm_head = view.create_tensor(head, ("voc", "d"), {"voc": MODEL_AXIS})
        opts = cfg.rope_opts()
        from ..nn import rotary
        self._inv_freq = rotary.inv_freq(cfg.hd, opts)
        self._rope_layout = opts.layout.value
        self._rot_dim = opts.scaling.partial_rotary_dim(cfg.hd)
        self._attn_factor = opts.scaling.attention_scaling()

    @staticmethod
    def from_store(store: TensorStore, cfg: LlamaConfig) -> "TaggedLlama":
        return TaggedLlama(store.view(), cfg)

    def load(self, platform, store: TensorStore, shardings=()):
        """Bufferised twin of this model: every weight cut by `Sharding.placement` and read from the checkpoint as
        byte ranges, this process's shards only."""
        loader = Loader(platform, parallelism=4)
        try:
            return loader.load(self, store, list(shardings))
        finally:
            loader.close()

    # ------------------------------------------------------------------ program
    def _rope(self, x: Tensor, positions: torch.Tensor) -> Tensor:
        """x {s, h, hd}"""
        d = x.to_torch()
        y = _ref.rope_rotate(d, positions.to(d.device), self._inv_freq.to(d.device), self._rope_layout, self._rot_dim,
                             self._attn_factor)
        return x._like(y)

    def _layer(self, w: TaggedLlamaLayer, x: Tensor, positions: torch.Tensor, mask: Tensor) -> Tensor:
        c = self.cfg
        h = layers.rms_norm(x, w.input_norm, c.rms_norm_eps)
        heads = {"h": "auto", "hd": c.hd}
        bias = lambda y, b: y if b is None else y.add(b.broad(y.shape()))
        hnorm = lambda y, g: y if g is None else layers.rms_norm(y, g, c.rms_norm_eps, ax="hd")
        q = bias(h.dot(w.q, "d"), getattr(w, "q_bias", None)).split_axis("dout", heads)
        k = bias(h.dot(w.k, "d"), getattr(w, "k_bias", None)).split_axis("dout", heads)
        v = bias(h.dot(w.v, "d"), getattr(w, "v_bias", None)).split_axis("dout", heads)
        q = self._rope(hnorm(q, getattr(w, "q_norm", None)), positions)
        k = self._rope(hnorm(k, getattr(w, "k_norm", None)), positions)
        att = attention_ref.sdpa(q.rename({"s": "q"}).transpose(("h", "q", "hd")),
                                 k.rename({"s": "k"}).transpose(("h", "k", "hd")),
                                 v.rename({"s": "k"}).transpose(("h", "k", "hd")), mask)
        att = att.transpose(("q", "h", "hd")).merge({"din": ["h", "hd"]}).rename({"q": "s"})
        # row parallel: the product holds partial sums over the model axis; asking for a replicated layout sums them
        x = x.add(att.dot(w.o, "din").with_partitioning({"d": "replicated"}))
        h = layers.rms_norm(x, w.post_norm, c.rms_norm_eps)
        act = h.dot(w.gate, "d").silu().mul(h.dot(w.up, "d")).rename({"dout": "din"})
        return x.add(act.dot(w.down, "din").with_partitioning({"d": "replicated"}))

    def forward(self, weights: "TaggedLlama", tokens: Tensor) -> Tensor:
        """`weights` is this model with Tensors holding values (the Exe passes it in); `tokens` {s} i32."""
        s = tokens.dim("s")
        dev = tokens.to_torch().device
        positions = torch.arange(s, device=dev)
        x = layers.TokenEmbedding(weights.embed).forward(tokens)               # {s, d}
        mask = attention_ref.causal_attn_mask({"q": s, "k": s}, x.dtype(), device=dev)
        for w in weights.layers:
            x = self._layer(w, x, positions, mask)
        x = layers.rms_norm(x, weights.norm, self.cfg.rms_norm_eps)
        logits = x.dot(weights.lm_head, "d")                                   # {s, voc}, voc sharded
        return logits.with_partitioning({"voc": "replicated"})                 # all-gather of the vocabulary shards


def compile_prefill(model: TaggedLlama, platform, seq_len: int, cuda_graph: bool = False):
    """Exe of `model.forward` for sequences of `seq_len` tokens: call it with (weight buffers, token buffer)."""
    from ..shape import Shape
    tokens = Tensor.from_shape(Shape({"s": seq_len}, "i32"))
    return platform.compile(model.forward, (model, tokens), cuda_graph=cuda_graph, program_name="tagged_llama.prefill")


def load_serving_weights(model, platform, store: TensorStore, prefix: str = ""):
    """Fills a `LlamaModel` (the serving path's weights: fused qkv and gate|up matrices of this rank) from the
    buffers the generic `Loader` produced for the `TaggedLlama` description of the same checkpoint: each rank's
    rows and columns are the ones `Sharding.placement` assigns to its device, read as byte ranges.

    Needs layouts a placement can express: key/value heads and the vocabulary divisible by the number of ranks
    (the range-based `LlamaModel.load` also covers replicated KV heads and a padded vocabulary)."""
    from ..sharding import LogicalMesh
    c, world = model.config, model.comm.world
    if c.num_key_value_heads % world or c.vocab_size % world or c.intermediate_size % world:
        raise ValueError("this checkpoint's head / vocabulary counts do not divide over the ranks")
    if len(platform.local_devices()) != 1 or platform.num_devices() != world:
        raise ValueError("the serving model holds one shard per process: the platform must have one device per rank")
    try:
        tp = platform.sharding("model")
    except KeyError:
        tp = platform.register_sharding("model", LogicalMesh({MODEL_AXIS: "high_bandwidth"}))
    view = store.view().with_prefix(prefix.rstrip(".")) if prefix else store.view()
    desc = TaggedLlama(view, c)
    bufs = desc.load(platform, store, [tp])
    dev, dt = model.device, model.dtype
    loc = lambda b: None if b is None else b.local().to(device=dev, dtype=dt)
    model.embed = loc(bufs.embed)
    model.final_norm = loc(bufs.norm)
    model.lm_head = loc(bufs.lm_head) if (world > 1 or not c.tie_word_embeddings) else model.embed
    from .llama import LayerWeights
    for lb in bufs.layers:
        lw = LayerWeights()
        lw.input_norm, lw.post_norm = loc(lb.input_norm), loc(lb.post_norm)
        lw.qkv = torch.cat([loc(lb.q), loc(lb.k), loc(lb.v)], 0)
        if getattr(lb, "q_bias", None) is not None:
            lw.qkv_bias = torch.cat([loc(lb.q_bias), loc(lb.k_bias), loc(lb.v_bias)], 0)
        if getattr(lb, "q_norm", None) is not None:
            lw.q_norm, lw.k_norm = loc(lb.q_norm), loc(lb.k_norm)
        lw.o = loc(lb.o)
        lw.gate_up = torch.cat([loc(lb.gate), loc(lb.up)], 0)
        lw.down = loc(lb.down)
        model.layers.append(lw)
    return model
