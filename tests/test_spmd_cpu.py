"""SPMD execution of tagged-tensor programs over gloo ranks: `Loader` cuts a checkpoint by `Sharding.placement`,
`Exe` runs the program on every rank's shards, contractions over sharded axes and `with_partitioning` issue the
collectives, and the result equals the one-process run of the same program and the serving model's logits."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_WORKER = r"""
import json, os, sys, torch
sys.path.insert(0, os.environ["ZB_ROOT"])
from zml_b200 import safetensors
from zml_b200.buffer import Buffer
from zml_b200.io import TensorStore
from zml_b200.models.llama import LlamaConfig, LlamaModel
from zml_b200.models.tagged_llama import TaggedLlama, compile_prefill
from zml_b200.parallel.comm import Comm
from zml_b200.platform import Platform, Target
from zml_b200.shape import Shape
from zml_b200.sharding import LogicalMesh
from zml_b200.tensor import Tensor

c = Comm.from_env(backend="gloo")
repo = os.environ["ZB_REPO"]
cfg = LlamaConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=4, intermediate_size=128,
                  vocab_size=256, head_dim=16, max_position_embeddings=128)
if c.rank == 0:
    ref = LlamaModel(cfg, device="cpu", dtype=torch.float32).init_random(seed=5, std=0.08)
    safetensors.save_file({k: v.contiguous() for k, v in ref.state_dict_hf().items()}, os.path.join(repo, "model.safetensors"))
c.barrier()
store = TensorStore.from_path(repo)
tokens = torch.randint(3, 250, (24,), generator=torch.Generator().manual_seed(1)).to(torch.int32)


def run(platform):
    tp = platform.register_sharding("tp", LogicalMesh({"model": "high_bandwidth"}))
    model = TaggedLlama.from_store(store, cfg)
    weights = model.load(platform, store, [tp])
    exe = compile_prefill(model, platform, len(tokens))
    tok = Buffer.from_tensor(platform, tokens, Shape({"s": len(tokens)}, "i32"))
    out = exe.call(weights, tok)
    return model, weights, out


# 1. the SPMD run: every rank holds 1/world of each projection
platform = Platform.init(Target.cpu, comm=c)
model, weights, out = run(platform)
w = c.world
q = weights.layers[0].q
assert q.shape().dims == (128, 64) and tuple(q.local().shape) == (128 // w, 64), (q, q.local().shape)
o = weights.layers[0].o
assert tuple(o.local().shape) == (64, 128 // w)
assert tuple(weights.lm_head.local().shape) == (256 // w, 64)
assert tuple(weights.embed.local().shape) == (256, 64)                       # no spec: replicated
assert out.shape().dims == (24, 256) and tuple(out.local().shape) == (24, 256)
logits = out.to_tensor()

# 2. the same program on one process holding the whole checkpoint
_, _, single = run(Platform.init(Target.cpu))
want = single.to_tensor()
err = (logits - want).abs().max().item()
assert err < 2e-4 * max(1.0, want.abs().max().item()), err
allv = c.all_gather(logits[None])
assert all(torch.equal(allv[0], allv[r]) for r in range(w))                  # identical on every rank

# 3. the serving model's prefill logits from the same checkpoint
from zml_b200.serving import Engine
from zml_b200.serving.engine import AttnMeta
serving = LlamaModel(cfg, device="cpu", dtype=torch.float32).load(store)
eng = Engine(serving, num_pages=8, page_size=16, max_batch=1, max_seq_len=64)
i32 = lambda v: torch.tensor(v, dtype=torch.int32)
n = len(tokens)
meta = AttnMeta(True, i32(list(range(n))), i32(list(range(n))), i32([[0, 1, 2, 3]]), i32([n]), i32([0, n]))
ref_logits = serving.logits(serving.hidden_states(tokens, meta, eng.kv_cache)).float()[:, :256]
err2 = (logits - ref_logits).abs().max().item()
assert err2 < 5e-4 * max(1.0, ref_logits.abs().max().item()), err2

# 3b. the serving model of this rank, filled from Loader buffers cut by `Sharding.placement`, holds exactly the
#     weights its own range-based loader reads
by_ranges = LlamaModel(cfg, c, device="cpu", dtype=torch.float32).load(store)
by_placement = LlamaModel(cfg, c, device="cpu", dtype=torch.float32).load(store, platform=platform)
assert by_placement.layers and len(by_placement.layers) == len(by_ranges.layers)
for a_, b_ in zip(by_ranges.layers, by_placement.layers):
    for name in ("input_norm", "post_norm", "qkv", "o", "gate_up", "down"):
        assert torch.equal(getattr(a_, name), getattr(b_, name)), name
assert torch.equal(by_ranges.lm_head, by_placement.lm_head) and torch.equal(by_ranges.embed, by_placement.embed)

# 4. a resharding chain on its own: rows sharded -> columns sharded -> replicated
mesh = platform.sharding("tp")
x_shape = Shape({"m": 16, "k": 32}, "f32").with_partitioning({"m": "model"})
g = torch.Generator().manual_seed(7)
xa, wb = torch.randn(16, 32, generator=g), torch.randn(32, 8, generator=g)
def prog(x, wt):
    y = x.dot(wt, "k")                                        # {m sharded, n}
    y = y.with_partitioning({"n": "model"})                   # all-gather m, keep this rank's columns
    assert y.dims() == (16, 8 // w), y
    z = y.sum("n")                                            # partial sums over the model axis
    return y.with_partitioning({"m": "replicated", "n": "replicated"}), z.with_partitioning({"m": "model"})
exe = platform.compile(prog, (Tensor.from_shape(x_shape), Tensor.from_shape(Shape({"k": 32, "n": 8}, "f32"))), cuda_graph=False)
y, z = exe.call(Buffer.from_tensor(platform, xa, x_shape, mesh), Buffer.from_tensor(platform, wb, Shape({"k": 32, "n": 8}, "f32")))
assert torch.allclose(y.to_tensor(), xa @ wb, atol=1e-5)
assert z.shape().dims == (16, 1) and tuple(z.local().shape) == (16 // w, 1)      # reduce-scattered over the rows
assert torch.allclose(z.to_tensor(), (xa @ wb).sum(1, keepdim=True), atol=1e-4)

# 5. a 2 x 2 mesh (4 ranks): the batch cut over `data`, the ffn over `model`; the row-parallel sum runs inside each
#    model group of 2 ranks only
if w == 4:
    from zml_b200.platform import CreateOptions
    from zml_b200.sharding import PhysicalMesh, Strategy
    p2 = Platform.init(Target.cpu, CreateOptions(physical_mesh=PhysicalMesh.grid([2, 2], target="cpu")), comm=c)
    dm = p2.register_sharding_with_strategy("dm", LogicalMesh({"data": "low_bandwidth", "model": "high_bandwidth"}),
                                            Strategy.parse_bindings({"data": "link_x", "model": "link_y"}))
    xs = Shape({"b": 8, "d": 16}, "f32").with_partitioning({"b": "data"})
    w1s = Shape({"f": 32, "d": 16}, "f32").with_partitioning({"f": "model"})
    w2s = Shape({"d": 16, "f": 32}, "f32").with_partitioning({"f": "model"})
    xv, w1v, w2v = torch.randn(8, 16, generator=g), torch.randn(32, 16, generator=g), torch.randn(16, 32, generator=g)
    def mlp(x, w1, w2):
        h = x.dot(w1, "d").relu()                             # {b@data, f@model}
        assert h.dims() == (4, 16), h
        return h.dot(w2, "f").with_partitioning({"b": "data", "d": "replicated"})
    exe = p2.compile(mlp, tuple(Tensor.from_shape(s_) for s_ in (xs, w1s, w2s)), cuda_graph=False)
    out2 = exe.call(*[Buffer.from_tensor(p2, v_, s_, dm) for v_, s_ in ((xv, xs), (w1v, w1s), (w2v, w2s))])
    assert out2.shape().dims == (8, 16) and tuple(out2.local().shape) == (4, 16)
    assert torch.allclose(out2.to_tensor(), torch.relu(xv @ w1v.t()) @ w2v.t(), atol=1e-4)
    assert p2.spmd().group("model") is not c.group and p2.spmd().parts("data") == 2
print("SPMD_OK", c.rank, round(err, 7), round(err2, 7), flush=True)
c.finish(0)
"""


@pytest.mark.parametrize("world", [2, 4])
def test_tagged_llama_runs_spmd_on_loader_cut_shards(tmp_path, world):
    script = tmp_path / "w.py"
    script.write_text(_WORKER)
    env = dict(os.environ, ZB_ROOT=ROOT, ZB_REPO=str(tmp_path))
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                        "--master-addr", "127.0.0.1", "--master-port", str(29671 + world), str(script)],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert r.stdout.count("SPMD_OK") == world


def test_partial_sums_cannot_leave_an_spmd_program():
    from zml_b200.tensor import Tensor
    t = Tensor(torch.ones(2, 2))
    t._partial = frozenset({"model"})
    with pytest.raises(RuntimeError, match="partial sums"):
        t.data
