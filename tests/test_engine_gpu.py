"""The serving engine on a B200: kernels vs the CPU restatement on the same weights, and
CUDA-graph decode vs eager decode."""
import pytest
import torch

from zml_b200 import ops
from zml_b200.models.llama import PRESETS, AttnMeta, LlamaConfig, LlamaModel
from zml_b200.serving import Engine
from zml_b200.testing import expect_close

pytestmark = pytest.mark.gpu


def _models(std=0.05):
    cfg = LlamaConfig.from_hf(PRESETS["tiny-llama-test"])
    gpu = LlamaModel(cfg, device="cuda").init_random(seed=3, std=std)
    cpu = LlamaModel(cfg, device="cpu")
    cpu.embed, cpu.final_norm, cpu.lm_head = gpu.embed.cpu(), gpu.final_norm.cpu(), gpu.lm_head.cpu()
    for lw in gpu.layers:
        c = type(lw)()
        for s in lw.__slots__:
            t = getattr(lw, s)
            setattr(c, s, t.cpu() if isinstance(t, torch.Tensor) else t)
        cpu.layers.append(c)
    return cfg, gpu, cpu


def test_prefill_hidden_states_match_cpu():
    cfg, gpu, cpu = _models()
    t, page = 150, 64
    ids = torch.randint(0, cfg.vocab_size, (t,), dtype=torch.int32)
    pos = torch.arange(t, dtype=torch.int32)
    slots = (pos + page).to(torch.int32)                       # pages 1..3
    bt = torch.tensor([[1, 2, 3, 0]], dtype=torch.int32)
    sl = torch.tensor([t], dtype=torch.int32)
    qs = torch.tensor([0, t], dtype=torch.int32)
    outs = []
    for m, dev in ((gpu, "cuda"), (cpu, "cpu")):
        kv = torch.zeros(m.kv_cache_shape(8, page), dtype=torch.bfloat16, device=dev)
        meta = AttnMeta(True, pos.to(dev), slots.to(dev), bt.to(dev), sl.to(dev), qs.to(dev), total_q_blocks=3)
        x = m.hidden_states(ids.to(dev), meta, kv)
        lg = m.logits(x, torch.tensor([t - 1], device=dev))
        outs.append((x.float().cpu(), lg.float().cpu(), kv.float().cpu()))
    expect_close(outs[0][0], outs[1][0], atol=5e-2, rtol=5e-2, min_close=0.99)
    expect_close(outs[0][1], outs[1][1], atol=5e-2, rtol=5e-2, min_close=0.99)
    expect_close(outs[0][2], outs[1][2], atol=5e-2, rtol=5e-2, min_close=0.99)
    ops.raise_on_status()


def test_decode_step_logits_match_cpu():
    """One decode step on top of a prefilled cache: logits of the kernels against the CPU restatement."""
    cfg, gpu, cpu = _models()
    t, page = 70, 64
    ids = torch.randint(0, cfg.vocab_size, (t,), dtype=torch.int32)
    pos = torch.arange(t, dtype=torch.int32)
    bt = torch.tensor([[1, 2, 3, 0]], dtype=torch.int32)
    outs = []
    for m, dev in ((gpu, "cuda"), (cpu, "cpu")):
        kv = torch.zeros(m.kv_cache_shape(8, page), dtype=torch.bfloat16, device=dev)
        meta = AttnMeta(True, pos.to(dev), (pos + page).to(dev), bt.to(dev), torch.tensor([t], dtype=torch.int32, device=dev),
                        torch.tensor([0, t], dtype=torch.int32, device=dev), total_q_blocks=2)
        m.hidden_states(ids.to(dev), meta, kv)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        dmeta = AttnMeta(False, i32([t]), i32([page + t]), bt.to(dev), i32([t + 1]), num_splits=1, max_seq_len=t + 1)
        x = m.hidden_states(i32([5]), dmeta, kv)
        outs.append(m.logits(x).float().cpu())
    expect_close(outs[0], outs[1], atol=5e-2, rtol=5e-2, min_close=0.99)
    ops.raise_on_status()


def test_graph_decode_equals_eager():
    cfg, gpu, _ = _models(std=0.08)
    prompts = [torch.randint(0, cfg.vocab_size, (n,)).tolist() for n in (9, 64, 131)]
    eng_g = Engine(gpu, num_pages=64, page_size=64, max_batch=4, max_seq_len=512, use_graphs=True)
    eng_e = Engine(gpu, num_pages=64, page_size=64, max_batch=4, max_seq_len=512, use_graphs=False)
    out_g, st = eng_g.generate(prompts, 24, sync_interval=5)
    out_e, _ = eng_e.generate(prompts, 24)
    assert out_g == out_e
    assert st.launches > 0 and st.decode_steps == 23
    # a second job on the same engine reuses the captured graph and the freed pages
    out_g2, _ = eng_g.generate(prompts, 24)
    assert out_g2 == out_g


def test_topk_sampling_draws_fresh_noise_every_step_and_follows_the_seed():
    """The sampler's seed and draw counter live on the device: a replayed decode graph must not repeat its
    noise, and a new seed must change the draws without a new capture."""
    from zml_b200.models.common import SamplingStrategy
    # nearly flat, but distinct logits (ties would leave the choice of candidates open): the draw picks the token
    logits = (-1e-4 * torch.arange(4096, device="cuda", dtype=torch.float32)).repeat(64, 1).contiguous()
    rng = torch.tensor([7, 0], dtype=torch.int64, device="cuda")
    a = ops.topk_sample(logits, 8, 1.0, rng=rng)
    ops.advance_rng(rng)
    b = ops.topk_sample(logits, 8, 1.0, rng=rng)
    assert not torch.equal(a, b)
    rng.copy_(torch.tensor([7, 0]))
    assert torch.equal(ops.topk_sample(logits, 8, 1.0, rng=rng), a)        # same state, same draw
    rng.copy_(torch.tensor([8, 0]))
    assert not torch.equal(ops.topk_sample(logits, 8, 1.0, rng=rng), a)
    # through the engine, with CUDA graphs: a flat-ish model (tiny weights) samples by noise
    cfg, gpu, _ = _models(std=0.002)
    eng = Engine(gpu, num_pages=64, page_size=64, max_batch=4, max_seq_len=512, use_graphs=True)
    prompts = [[3, 4, 5, 6], [9, 8, 7]]
    strat = SamplingStrategy(topk=16, temperature=1.0)
    o1, _ = eng.generate(prompts, 32, strat, seed=1)
    o1b, _ = eng.generate(prompts, 32, strat, seed=1)
    o2, _ = eng.generate(prompts, 32, strat, seed=2)
    assert o1 == o1b and o1 != o2
    assert all(len(set(o)) > 4 for o in o1), o1              # not the same draw at every step


def test_smoke_entry():
    import __graft_entry__ as entry
    entry.smoke()
