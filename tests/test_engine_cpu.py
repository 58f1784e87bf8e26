"""End-to-end generation on CPU: the paged engine must reproduce, token for token, a plain
dense-attention recomputation of the same weights."""
import math

import pytest

import torch

from zml_b200.models.common import SamplingStrategy
from zml_b200.models.llama import PRESETS, LlamaConfig, LlamaModel
from zml_b200.nn import rotary as rope_mod
from zml_b200.ops import reference as ref
from zml_b200 import ops, testing
from zml_b200.serving import Engine


def dense_logits(model: LlamaModel, ids: list[int]) -> torch.Tensor:
    """Straightforward full-sequence forward (no cache, no paging) -> logits of the last token."""
    c = model.config
    x = model.embed[torch.tensor(ids)]
    t = len(ids)
    pos = torch.arange(t)
    for lw in model.layers:
        n1 = ref.rmsnorm(x, lw.input_norm, c.rms_norm_eps)
        qkv = ref.gemm(n1, lw.qkv, bias=lw.qkv_bias)
        q, k, v = qkv.split([model.hq * c.hd, model.hkv * c.hd, model.hkv * c.hd], -1)
        q = q.reshape(t, model.hq, c.hd); k = k.reshape(t, model.hkv, c.hd); v = v.reshape(t, model.hkv, c.hd)
        q = ref.rope_rotate(q, pos, model.inv_freq, model.rope_layout, model.rot_dim, model.attn_factor)
        k = ref.rope_rotate(k, pos, model.inv_freq, model.rope_layout, model.rot_dim, model.attn_factor)
        g = model.hq // model.hkv
        kk = k.float().repeat_interleave(g, 1); vv = v.float().repeat_interleave(g, 1)
        s = torch.einsum("qhd,khd->hqk", q.float(), kk) / math.sqrt(c.hd)
        s = s.masked_fill(~torch.tril(torch.ones(t, t, dtype=torch.bool)), float("-inf"))
        a = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), vv).to(x.dtype).reshape(t, -1)
        x = ref.gemm(a, lw.o, residual=x)
        n2 = ref.rmsnorm(x, lw.post_norm, c.rms_norm_eps)
        x = ref.gemm(ref.swiglu(ref.gemm(n2, lw.gate_up)), lw.down, residual=x)
    n = ref.rmsnorm(x[-1:], model.final_norm, c.rms_norm_eps)
    return ref.gemm(n, model.lm_head, out_dtype=torch.float32)[0]


def test_engine_matches_dense_recompute():
    torch.manual_seed(0)
    cfg = LlamaConfig.from_hf(PRESETS["tiny-llama-test"])
    model = LlamaModel(cfg, device="cpu", dtype=torch.float32).init_random(seed=1, std=0.08)
    eng = Engine(model, num_pages=64, page_size=16, max_batch=4, max_seq_len=256, max_prefill_tokens=48)
    prompts = [torch.randint(0, cfg.vocab_size, (n,)).tolist() for n in (5, 37, 70)]
    outs, stats = eng.generate(prompts, max_new_tokens=6)
    assert stats.output_tokens == 18 and len(stats.ttft_ms) == 3
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o:
            want = int(torch.argmax(dense_logits(model, seq)))
            assert tok == want
            seq.append(tok)
    # every page went back to the pool
    assert eng.pool.num_free == 63


def test_engine_eos_and_sampling():
    torch.manual_seed(0)
    cfg = LlamaConfig.from_hf(PRESETS["tiny-llama-test"])
    model = LlamaModel(cfg, device="cpu", dtype=torch.float32).init_random(seed=2, std=0.08)
    eng = Engine(model, num_pages=32, page_size=16, max_batch=2, max_seq_len=128)
    p = [[1, 2, 3, 4]]
    greedy, _ = eng.generate(p, 8)
    eos = greedy[0][2]
    cut, _ = eng.generate(p, 8, eos_ids=[eos], sync_interval=2)
    assert cut[0] == greedy[0][:greedy[0].index(eos) + 1]
    sampled, _ = eng.generate(p, 8, SamplingStrategy(topk=5, temperature=1.0))
    assert len(sampled[0]) == 8


def test_llama3_inv_freq_matches_hf_formula():
    """Llama-3 scaled frequencies (the reference checks the same against HF values, zml/nn.zig:882-985)."""
    cfg = LlamaConfig.from_hf(PRESETS["llama-3.1-8b"])
    f = rope_mod.inv_freq(cfg.hd, cfg.rope_opts()).double()
    base = 1.0 / (500000.0 ** (torch.arange(0, 128, 2).double() / 128))
    wavelen = 2 * math.pi / base
    low, high = 8192 / 1.0, 8192 / 4.0
    smooth = (8192 / wavelen - 1.0) / (4.0 - 1.0)
    want = torch.where(wavelen < high, base, torch.where(wavelen > low, base / 8.0,
                       (1 - smooth) * base / 8.0 + smooth * base))
    assert torch.allclose(f, want, rtol=1e-5, atol=0)


def test_moe_model_generates_and_matches_dense_expert_math():
    from zml_b200 import moe
    from zml_b200.models.qwen3_moe import PRESETS as MOE_PRESETS, Qwen3MoeConfig, Qwen3MoeModel
    torch.manual_seed(0)
    cfg = Qwen3MoeConfig.from_hf(MOE_PRESETS["tiny-moe-test"])
    model = Qwen3MoeModel(cfg, device="cpu", dtype=torch.float32).init_random(seed=4, std=0.08)
    eng = Engine(model, num_pages=32, page_size=16, max_batch=2, max_seq_len=128)
    outs, st = eng.generate([[3, 4, 5, 6, 7], list(range(20, 60))], 5)
    assert [len(o) for o in outs] == [5, 5]
    # the layer's MoE equals the per-expert dense computation
    lw = model.layers[0]
    x = torch.randn(9, cfg.hidden_size) * 0.5
    y = model.mlp(lw, torch.zeros_like(x), x)
    logits = ref.gemm(x, lw.extra["router"], out_dtype=torch.float32)
    ids, w = moe.router_topk(logits, cfg.num_experts_per_tok)
    g, u = moe.ops.deinterleave_gate_up(lw.extra["gate_up"])
    want = moe.reference_fused_experts(x, ids, w, g, u, lw.extra["down"])
    assert torch.allclose(y, want, atol=1e-4, rtol=1e-4)
    # HF-named state dict round trip through safetensors and the store-based loader
    import tempfile
    from zml_b200 import safetensors
    from zml_b200.io import TensorStore
    with tempfile.TemporaryDirectory() as d:
        safetensors.save_sharded(model.state_dict_hf(), d)
        m2 = Qwen3MoeModel(cfg, device="cpu", dtype=torch.float32).load(TensorStore.from_path(d))
        outs2, _ = Engine(m2, num_pages=32, page_size=16, max_batch=2, max_seq_len=128).generate([[3, 4, 5, 6, 7], list(range(20, 60))], 5)
        assert outs2 == outs


def test_moe_nvfp4_expert_weights_are_representable():
    """`expert_dtype="nvfp4"` holds expert weights at values an NVFP4 checkpoint can store."""
    from zml_b200 import moe
    from zml_b200.models.qwen3_moe import PRESETS as MOE_PRESETS, Qwen3MoeConfig, Qwen3MoeModel
    w = torch.randn(2, 32, 64).bfloat16() * 0.02
    r = moe.nvfp4_roundtrip(w)
    assert ((r.float() - w.float()).norm() / w.float().norm()).item() < 0.15
    again = moe.nvfp4_roundtrip(r)
    assert ((again.float() - r.float()).norm() / r.float().norm()).item() < 0.02      # (nearly) a fixed point
    cfg = Qwen3MoeConfig.from_hf(dict(MOE_PRESETS["tiny-moe-test"], expert_dtype="nvfp4"))
    m = Qwen3MoeModel(cfg, device="cpu").init_random(0)
    eng = Engine(m, num_pages=16, page_size=16, max_batch=2, max_seq_len=64)
    out, _ = eng.generate([[5, 6, 7, 8]], 4)
    assert len(out[0]) == 4


def test_nvfp4_experts_container_and_cpu_path():
    from zml_b200 import moe
    from zml_b200.nn import quant as Q
    torch.manual_seed(0)
    # K = 64: not a shape the kernel streams -> plain codes and scales, de-quantising fallback
    w = torch.randn(3, 128, 64).bfloat16() * 0.05
    q = moe.Nvfp4Experts.quantize(w)
    assert not q.kernel_ready and q.blocks is None
    assert q.codes.shape == (3 * 128, 32) and q.scales.shape == (3 * 128, 4) and q.gscale.shape == (3, 1)
    assert q.nbytes() == 3 * 128 * 32 + 3 * 128 * 4 + 12
    d = q.dequantize()
    assert ((d.float() - w.float()).norm() / w.float().norm()).item() < 0.15
    xs = torch.randn(10, 64).bfloat16()
    meta = torch.tensor([0, 4, 4, 10], dtype=torch.int32)
    assert torch.equal(moe.grouped_gemm_w4(xs, q, meta), moe.grouped_gemm(xs, d, meta))
    # N a multiple of 128 and K of 256: tile-major 18 KB blocks, a bijection of the checkpoint arrays
    w2 = torch.randn(2, 256, 512).bfloat16() * 0.05
    q2 = moe.Nvfp4Experts.quantize(w2)
    assert q2.kernel_ready and q2.blocks.shape == (2, 2, 2, moe.ops.W4_BLOCK_BYTES) and q2.codes is None
    c, s_, g = Q.quantize_weight_nvfp4(w2)
    codes, scales = q2.checkpoint_arrays()
    assert torch.equal(codes, c.reshape(512, 256)) and torch.equal(scales.view(torch.uint8), s_.reshape(512, 32).view(torch.uint8))
    want = Q.dequantize_nvfp4(Q.unpack_e2m1(c), s_, None) * g.reshape(2, 1, 1)
    assert torch.allclose(q2.dequantize(torch.float32), want.float(), rtol=1e-6, atol=1e-9)
    assert torch.equal(moe.ops.nvfp4_codes_from_kernel_order(moe.ops.nvfp4_codes_to_kernel_order(c[0])), c[0])
    # block layout: chunk ch of row r of block (e, tile, kchunk) sits at [ch][r][16 bytes], scales after the codes
    blk = q2.blocks[1, 1, 0]
    krow = moe.ops.nvfp4_codes_to_kernel_order(c[1])[128 + 5]            # row 5 of tile 1, kernel nibble order
    assert torch.equal(blk[(3 * 128 + 5) * 16:(3 * 128 + 5) * 16 + 16], krow[3 * 16:4 * 16])
    assert torch.equal(blk[128 * 128 + 5 * 16:128 * 128 + 5 * 16 + 16], s_[1, 128 + 5, :16].view(torch.uint8))


def test_moe_loads_nvfp4_expert_checkpoints(tmp_path):
    """Per-expert packed weights + block scales + matrix scale (both spellings) load into the NVFP4 container
    and its bf16 twin; gate and up keep their own matrix scales."""
    from zml_b200 import moe, safetensors
    from zml_b200.io import TensorStore
    from zml_b200.nn import quant as Q
    from zml_b200.models.qwen3_moe import PRESETS as MOE_PRESETS, Qwen3MoeConfig, Qwen3MoeModel
    cfg = Qwen3MoeConfig.from_hf(dict(MOE_PRESETS["tiny-moe-test"]))
    model = Qwen3MoeModel(cfg, device="cpu", dtype=torch.float32).init_random(1)
    sd = model.state_dict_hf()
    for spelling in ("modelopt", "compressed-tensors"):
        out, want = {}, {}
        for name, t in sd.items():
            if ".mlp.experts." not in name:
                out[name] = t
                continue
            base = name[:-len("weight")]
            codes, scales, g = Q.quantize_weight_nvfp4(t * (3.0 if "up_proj" in name else 1.0))
            want[name] = Q.dequantize_nvfp4(Q.unpack_e2m1(codes), scales, g)
            if spelling == "modelopt":
                out[base + "weight"], out[base + "weight_scale"], out[base + "weight_scale_2"] = codes, scales, g.reshape(())
            else:
                out[base + "weight_packed"], out[base + "weight_scale"] = codes, scales
                out[base + "weight_global_scale"] = (1.0 / g).reshape(1)
        d = tmp_path / spelling
        d.mkdir()
        safetensors.save_sharded(out, str(d))
        m2 = Qwen3MoeModel(cfg, device="cpu", dtype=torch.float32).load(TensorStore.from_path(str(d)))
        lw = m2.layers[0]
        gu, dn = lw.extra["w4"]
        assert gu.gscale.shape == (cfg.num_experts, 2) and dn.gscale.shape == (cfg.num_experts, 1)
        g_, u_ = moe.ops.deinterleave_gate_up(lw.extra["gate_up"])
        for e in (0, cfg.num_experts - 1):
            assert torch.allclose(g_[e], want[f"model.layers.0.mlp.experts.{e}.gate_proj.weight"], rtol=1e-6, atol=1e-8)
            assert torch.allclose(u_[e], want[f"model.layers.0.mlp.experts.{e}.up_proj.weight"], rtol=1e-6, atol=1e-8)
            assert torch.allclose(lw.extra["down"][e], want[f"model.layers.0.mlp.experts.{e}.down_proj.weight"], rtol=1e-6, atol=1e-8)
        outs, _ = Engine(m2, num_pages=32, page_size=16, max_batch=2, max_seq_len=128).generate([[3, 4, 5, 6, 7]], 4)
        assert len(outs[0]) == 4


def test_fused_kernel_layout_matches_plain_layers():
    """Norm weights folded into the qkv / gate|up columns, gate and up rows interleaved, row statistics handed
    from GEMM to GEMM: the same hidden states as RMSNorm -> GEMM -> SwiGLU layer by layer (float32, CPU)."""
    from zml_b200.models.llama import AttnMeta
    cfg = LlamaConfig.from_hf(PRESETS["tiny-llama-test"])
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg.vocab_size, (19,), generator=g, dtype=torch.int32)
    outs = {}
    for fused in (False, True):
        model = LlamaModel(cfg, device="cpu", dtype=torch.float32).init_random(seed=2, std=0.05)
        for lw in model.layers:             # norm weights that are not all ones
            lw.input_norm.copy_(1.0 + 0.3 * torch.randn(lw.input_norm.shape, generator=torch.Generator().manual_seed(5)))
            lw.post_norm.copy_(1.0 + 0.3 * torch.randn(lw.post_norm.shape, generator=torch.Generator().manual_seed(6)))
        if fused:
            model.prepare_fused()
            with pytest.raises(RuntimeError):
                model.state_dict_hf()
        kv = torch.zeros(model.kv_cache_shape(4, 16), dtype=torch.float32)
        meta = AttnMeta(True, torch.arange(19, dtype=torch.int32), torch.arange(16, 35, dtype=torch.int32),
                        torch.tensor([[1, 2, 3]], dtype=torch.int32), torch.tensor([19], dtype=torch.int32),
                        torch.tensor([0, 19], dtype=torch.int32), total_q_blocks=1)
        outs[fused] = model.hidden_states(ids, meta, kv)
        if fused:      # `layer` stays usable on its own in this layout
            x = ops.embedding(ids, model.embed)
            y = model.layer(0, x, meta, torch.zeros_like(kv))
            assert y.shape == x.shape
    testing.expect_close(outs[True], outs[False], atol=2e-4, rtol=2e-4)


_VOCAB_WORKER = r"""
import os, sys, torch
sys.path.insert(0, os.environ["ZB_ROOT"])
from zml_b200.models.common import SamplingStrategy
from zml_b200.models.llama import PRESETS, LlamaConfig, LlamaModel
from zml_b200.parallel.comm import Comm
from zml_b200.serving import Engine
c = Comm.from_env(backend="gloo")
single = Comm.single(torch.device("cpu"))
cfg = LlamaConfig.from_hf(dict(PRESETS["tiny-llama-test"], vocab_size=1021, tie_word_embeddings=False))
g = torch.Generator().manual_seed(3)
prompts = [torch.randint(3, cfg.vocab_size, (n,), generator=g).tolist() for n in (17, 9)]
for strat in (SamplingStrategy(topk=1), SamplingStrategy(topk=4, temperature=0.8)):
    got = {}
    for label, comm in (("tp", c), ("single", single)):
        model = LlamaModel(cfg, comm, device="cpu", dtype=torch.float32).init_random(seed=5, std=0.05)
        assert model.lm_head.shape[0] == model.v_per
        torch.manual_seed(99)
        got[label], _ = Engine(model, num_pages=32, page_size=16, max_batch=2, max_seq_len=128).generate(prompts, 6, strat)
    assert got["tp"] == got["single"], (strat, got)
    assert all(t < cfg.vocab_size for o in got["tp"] for t in o)
print("VOCAB_OK", c.rank, flush=True)
c.finish(0)
"""


def test_vocab_parallel_head_with_a_vocabulary_that_does_not_divide(tmp_path):
    """1021 tokens over 2 ranks: the last rank's missing rows are zero rows masked to -inf, greedy and top-k
    sampling give the tokens of one rank holding the whole head."""
    import os
    import subprocess
    import sys
    script = tmp_path / "w.py"
    script.write_text(_VOCAB_WORKER)
    env = dict(os.environ, ZB_ROOT=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29641", str(script)],
                       capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert r.stdout.count("VOCAB_OK") == 2


_TP_CPU_WORKER = r"""
import os, sys, torch
sys.path.insert(0, os.environ["ZB_ROOT"])
from zml_b200.models import registry
from zml_b200.parallel.comm import Comm
from zml_b200.serving import Engine
c = Comm.from_env(backend="gloo")
single = Comm.single(torch.device("cpu"))
for name in os.environ["ZB_FAMILIES"].split(","):
    prompts = [torch.randint(3, 200, (n,), generator=torch.Generator().manual_seed(11)).tolist() for n in (13, 30)]
    got = {}
    for label, comm in (("tp", c), ("single", single)):
        model = registry.build_model(name, comm, device="cpu", seed=3, dtype=torch.float32)
        eng = Engine(model, num_pages=32, page_size=16, max_batch=2, max_seq_len=128)
        got[label], _ = eng.generate(prompts, 6)
    assert got["tp"] == got["single"], (name, got)
    allo = c.all_gather_object(got["tp"])
    assert all(o == allo[0] for o in allo), name
print("TP_CPU_OK", c.rank, flush=True)
c.finish(0)
"""


@pytest.mark.parametrize("world,families", [
    (2, "tiny-llama-test,tiny-moe-test,tiny-qwen35-test,tiny-qwen35-moe-test,tiny-lfm2-test"),
    (4, "tiny-llama-test,tiny-moe-test"),           # the tiny hybrids have 2 linear-attention heads: not divisible by 4
])
def test_every_model_family_under_two_way_parallelism_on_cpu(tmp_path, world, families):
    """Tensor / expert parallel shards of every model family over gloo ranks produce the tokens of one rank
    holding the whole model (float32, CPU restatements of the kernels)."""
    import os
    import subprocess
    import sys
    script = tmp_path / "w.py"
    script.write_text(_TP_CPU_WORKER)
    env = dict(os.environ, ZB_ROOT=os.path.dirname(os.path.dirname(os.path.abspath(__file__))), ZB_FAMILIES=families)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                        "--master-addr", "127.0.0.1", "--master-port", str(29651 + world), str(script)],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert r.stdout.count("TP_CPU_OK") == world


@pytest.mark.parametrize("name", ["tiny-llama-test", "tiny-qwen35-test"])
def test_continuous_admission_matches_one_at_a_time_generation(name):
    """Seven prompts through three batch rows: sequences leave and join between decode blocks (also with staggered
    arrivals); every prompt gets the tokens it gets alone, and all pages and state slots come back."""
    import torch
    from zml_b200.models import registry
    from zml_b200.parallel.comm import Comm
    from zml_b200.serving import Engine
    m = registry.build_model(name, Comm.single(torch.device("cpu")), device="cpu", seed=3, dtype=torch.float32)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(3, 200, (n,), generator=g).tolist() for n in (5, 17, 9, 30, 12, 7, 21)]
    budgets = [6, 3, 9, 4, 1, 8, 5]
    eng = Engine(m, num_pages=16, page_size=16, max_batch=3, max_seq_len=64)
    want = [eng.generate([p], b)[0][0] for p, b in zip(prompts, budgets)]
    got, st = eng.serve(prompts, budgets, sync_interval=4)
    assert got == want and len(st.ttft_ms) == 7 and st.output_tokens == sum(budgets)
    got, _ = eng.serve(prompts, budgets, sync_interval=3, arrivals=[0, 0, 2, 2, 5, 5, 9])
    assert got == want and eng.pool.num_free == 15
    eos = want[2][3]
    got, _ = eng.serve(prompts[2:3], 9, eos_ids=[eos])
    assert got[0] == want[2][:want[2].index(eos) + 1]


def test_session_decode_in_blocks_matches_token_by_token():
    """`Session.run_decode(stream_interval=n)` reads the generated ids every n steps; the conversation (two turns)
    is the one the token-by-token loop produces, and an EOS inside a block ends the turn at that token."""
    import torch
    from zml_b200.models import registry
    from zml_b200.parallel.comm import Comm
    from zml_b200.serving import Engine
    from zml_b200.serving.engine import Session
    m = registry.build_model("tiny-llama-test", Comm.single(torch.device("cpu")), device="cpu", seed=11, dtype=torch.float32)
    outs = []
    for si in (1, 4, 7):
        s = Session(Engine(m, num_pages=16, page_size=16, max_batch=1, max_seq_len=128), 100)
        s.run_prefill([5, 6, 7, 8, 9])
        a = s.run_decode(max_new_tokens=10, stream_interval=si)
        s.run_prefill([11, 12])
        b = s.run_decode(max_new_tokens=6, stream_interval=si)
        outs.append((a, b, list(s.tokens)))
        s.close()
    assert outs[0] == outs[1] == outs[2] and len(outs[0][0]) == 10 and len(outs[0][1]) == 6
    eos = outs[0][0][4]
    s = Session(Engine(m, num_pages=16, page_size=16, max_batch=1, max_seq_len=128), 100, eos_ids=[eos])
    s.run_prefill([5, 6, 7, 8, 9])
    assert s.run_decode(stream_interval=4) == outs[0][0][:outs[0][0].index(eos) + 1]


def test_engine_rejects_bad_requests_without_stranding_pages():
    """Empty prompts, prompts that cannot fit and a batch that runs out of pages are refused with a clear error, leave
    no page allocated, and the engine keeps working; no prompts is an empty result; top-k beyond the vocabulary is capped."""
    from zml_b200.serving.engine import OutOfPages
    cfg = LlamaConfig.from_hf(dict(PRESETS["tiny-llama-test"], vocab_size=300))
    model = LlamaModel(cfg, device="cpu", dtype=torch.float32).init_random(seed=1, std=0.05)
    eng = Engine(model, num_pages=4, page_size=16, max_batch=2, max_seq_len=64)
    free0 = len(eng.pool.free)
    with pytest.raises(ValueError, match="empty prompt"):
        eng.generate([[1, 2], []], 3)
    with pytest.raises(ValueError, match="pages"):
        eng.generate([list(range(1, 80))], 5)
    with pytest.raises(OutOfPages):
        eng.generate([list(range(1, 40)), list(range(1, 40))], 4)
    with pytest.raises(ValueError, match="prompt 1 is empty"):
        eng.serve([[1], [], [2]], 3)
    with pytest.raises(ValueError, match="prompt 0 needs"):
        eng.serve([list(range(1, 80))], 5)
    assert len(eng.pool.free) == free0
    assert eng.generate([], 3)[0] == [] and eng.serve([], 3)[0] == []
    out, _ = eng.generate([[1, 2, 3]], 2, SamplingStrategy(topk=1000, temperature=1.0))
    assert len(out[0]) == 2 and len(eng.pool.free) == free0
    assert eng.generate([[1, 2, 3]], 0)[0] == [[]]


def test_serve_reports_tokens_block_by_block():
    """`on_tokens` sees every token exactly once, in order, per prompt, and one final call per prompt."""
    cfg = LlamaConfig.from_hf(dict(PRESETS["tiny-llama-test"], vocab_size=300))
    model = LlamaModel(cfg, device="cpu", dtype=torch.float32).init_random(seed=1, std=0.05)
    eng = Engine(model, num_pages=32, page_size=16, max_batch=2, max_seq_len=64)
    calls = []
    outs, _ = eng.serve([[1, 2, 3], [4, 5], [6]], [5, 9, 1], sync_interval=3,
                        on_tokens=lambda i, toks, fin: calls.append((i, list(toks), fin)))
    acc, final = {0: [], 1: [], 2: []}, set()
    for i, toks, fin in calls:
        assert i not in final
        acc[i] += toks
        if fin:
            final.add(i)
    assert [acc[i] for i in range(3)] == outs and final == {0, 1, 2}
    assert [len(o) for o in outs] == [5, 9, 1]
    assert eng.serve([[1, 2, 3], [4, 5], [6]], [5, 9, 1], sync_interval=3)[0] == outs        # the callback changes nothing


def test_a_seed_reproduces_a_sampled_generation_on_cpu():
    """Top-k sampling draws its noise from (seed, draws so far): the same seed gives the same tokens from a fresh
    engine and from one that has served before; another seed gives others; consecutive steps draw different noise."""
    from zml_b200.models.common import SamplingStrategy
    cfg = LlamaConfig.from_hf(dict(PRESETS["tiny-llama-test"], vocab_size=512))
    model = LlamaModel(cfg, device="cpu", dtype=torch.float32).init_random(seed=4, std=0.08)
    strat = SamplingStrategy(topk=16, temperature=1.5)
    prompts = [[1, 5, 9, 13], [2, 6]]
    eng = Engine(model, num_pages=32, page_size=16, max_batch=2, max_seq_len=64)
    a, _ = eng.generate(prompts, 12, strat, seed=3)
    other, _ = eng.generate(prompts, 12, strat, seed=4)
    again, _ = eng.generate(prompts, 12, strat, seed=3)
    fresh, _ = Engine(model, num_pages=32, page_size=16, max_batch=2, max_seq_len=64).generate(prompts, 12, strat, seed=3)
    assert a == again == fresh and a != other
    served, _ = eng.serve(prompts, 12, strat, seed=3)
    assert served == eng.serve(prompts, 12, strat, seed=3)[0]
    greedy, _ = eng.generate(prompts, 12)
    assert a != greedy                                   # at temperature 1.5 over 16 candidates the draw leaves the arg-max
