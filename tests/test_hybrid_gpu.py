"""Linear-attention / short-conv kernels and the hybrid models on a B200, against the float32
PyTorch restatement of the same ops on the CPU."""
import os

import pytest
import torch

from zml_b200 import ops
from zml_b200.models import registry
from zml_b200.ops import linear_attn as la
from zml_b200.serving import Engine
from zml_b200.testing import expect_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    ops.raise_on_status()


def _seq_meta(lens, prior):
    """q_start / seq_lens / slots for sequences of `lens` new tokens after `prior` cached ones."""
    qs = [0]
    for n in lens:
        qs.append(qs[-1] + n)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32)
    return i32(qs), i32([p + n for p, n in zip(prior, lens)]), i32([3, 0, 2, 1][:len(lens)])


@pytest.mark.parametrize("k", [3, 4])
@pytest.mark.parametrize("gated,silu", [(False, True), (True, False)])
def test_causal_conv1d_two_chunks(k, gated, silu):
    torch.manual_seed(k)
    c, ld = 200, 3 * 200 + 8
    w = (torch.randn(c, k) * 0.5).bfloat16()
    st_cpu = torch.zeros((4, k - 1, c), dtype=torch.bfloat16)
    st_gpu = st_cpu.to(DEV)
    prior = [0, 0, 0]
    for lens in ([5, 1, 40], [1, 1, 1], [2, 33, 7]):
        qs, sl, slots = _seq_meta(lens, prior)
        t = int(qs[-1])
        buf = torch.randn(t, ld).bfloat16()
        x, pre, post = buf[:, :c], (buf[:, c:2 * c] if gated else None), (buf[:, 2 * c:3 * c] if gated else None)
        want = la.causal_conv1d_reference(x, w, st_cpu, qs, sl, slots, pre, post, silu)
        g = buf.to(DEV)
        got = la.causal_conv1d(g[:, :c], w.to(DEV), st_gpu, qs.to(DEV), sl.to(DEV), slots.to(DEV),
                               g[:, c:2 * c] if gated else None, g[:, 2 * c:3 * c] if gated else None, silu)
        expect_close(got.float().cpu(), want.float(), atol=2e-2, rtol=2e-2, min_close=0.999)
        expect_close(st_gpu.float().cpu(), st_cpu.float(), atol=1e-6, rtol=0, min_close=1.0)
        prior = [p + n for p, n in zip(prior, lens)]


@pytest.mark.parametrize("hk,hv,dk,dv", [(2, 4, 64, 64), (2, 2, 128, 128), (1, 2, 128, 64), (4, 8, 64, 128)])
def test_gated_delta_scan_chunks_and_decode(hk, hv, dk, dv):
    torch.manual_seed(hk * 10 + dk)
    key_dim, val_dim = hk * dk, hv * dv
    cols = 2 * key_dim + 2 * val_dim + 2 * hv
    cols = (cols + 7) // 8 * 8
    a_log = torch.log(torch.empty(hv).uniform_(1, 8))
    dtb = torch.empty(hv).uniform_(-1, 1)
    nw = (1 + 0.1 * torch.randn(dv)).bfloat16()
    st_cpu = torch.zeros((4, hv, dk, dv))
    st_gpu = st_cpu.to(DEV)
    prior = [0, 0, 0]
    off_z, off_b, off_a = 2 * key_dim + val_dim, 2 * key_dim + 2 * val_dim, 2 * key_dim + 2 * val_dim + hv
    for lens in ([37, 1, 16], [1, 1, 1], [3, 20, 0]):
        qs, sl, slots = _seq_meta(lens, prior)
        t = int(qs[-1])
        proj = torch.randn(t, cols).bfloat16()
        args = lambda p, s, d: (p[:, :off_z], p[:, off_z:off_b], p[:, off_a:off_a + hv], p[:, off_b:off_a],
                                a_log.to(d), dtb.to(d), nw.to(d), 1e-6, s, qs.to(d), sl.to(d), slots.to(d), hk, hv, dk, dv)
        want = la.gated_delta_scan_reference(*args(proj, st_cpu, "cpu"))
        got = la.gated_delta_scan(*args(proj.to(DEV), st_gpu, DEV))
        expect_close(got.float().cpu(), want.float(), atol=3e-2, rtol=3e-2, min_close=0.995)
        expect_close(st_gpu.cpu(), st_cpu, atol=2e-3, rtol=2e-2, min_close=0.999)
        prior = [p + n for p, n in zip(prior, lens)]


def test_sigmoid_gate_mul():
    buf = torch.randn(37, 256 + 128, device=DEV).bfloat16()
    x = buf[:, :128].clone()
    want = x.float() * torch.sigmoid(buf[:, 256:].float())
    got = la.sigmoid_gate_mul(x, buf[:, 256:])
    expect_close(got.float(), want, atol=1e-2, rtol=1e-2, min_close=0.999)


@pytest.mark.parametrize("name", ["tiny-qwen35-test", "tiny-qwen35-moe-test", "tiny-lfm2-test"])
def test_hybrid_model_graph_decode_equals_eager_and_chunking(name):
    m = registry.build_model(name, device=DEV, seed=5)
    torch.manual_seed(0)
    prompts = [torch.randint(3, 1000, (n,)).tolist() for n in (9, 70, 131)]
    outs = []
    for graphs, budget in ((True, 8192), (False, 8192), (False, 64)):
        eng = Engine(m, num_pages=64, page_size=64, max_batch=4, max_seq_len=512, max_prefill_tokens=budget,
                     use_graphs=graphs)
        out, st = eng.generate(prompts, 20, sync_interval=7)
        outs.append(out)
        assert st.launches > 0
    assert outs[0] == outs[1]
    same = sum(a == b for o1, o2 in zip(outs[1], outs[2]) for a, b in zip(o1, o2))
    assert same >= 0.9 * 60          # chunked prefill differs only by bf16 round-off in rare ties


def _to_cpu(obj):
    """Deep copy of a weight container (tensors, dicts, slotted objects) onto the CPU."""
    if torch.is_tensor(obj):
        return obj.cpu()
    if isinstance(obj, dict):
        return {k: _to_cpu(v) for k, v in obj.items()}
    if hasattr(obj, "__slots__"):
        c = type(obj)()
        for s in obj.__slots__:
            setattr(c, s, _to_cpu(getattr(obj, s)))
        return c
    return obj


def _cpu_twin(gpu, name):
    """CPU model with the GPU model's weights (the CUDA and CPU generators draw different streams)."""
    cpu = registry.build_model(name, device="cpu", seed=2)
    cpu.embed, cpu.final_norm, cpu.lm_head = gpu.embed.cpu(), gpu.final_norm.cpu(), gpu.lm_head.cpu()
    cpu.layers = [_to_cpu(lw) for lw in gpu.layers]
    return cpu


@pytest.mark.parametrize("name", ["tiny-qwen35-test", "tiny-qwen35-moe-test", "tiny-lfm2-test"])
def test_hybrid_prefill_logits_match_cpu(name):
    from zml_b200.models.llama import AttnMeta
    gpu = registry.build_model(name, device=DEV, seed=2)
    cpu = _cpu_twin(gpu, name)
    lens, page = [50, 7], 64
    ids = torch.randint(3, 1000, (sum(lens),), dtype=torch.int32)
    pos = torch.cat([torch.arange(n) for n in lens]).int()
    slots = torch.cat([torch.arange(n) + page * (1 + i) for i, n in enumerate(lens)]).int()
    bt = torch.tensor([[1, 0], [2, 0]], dtype=torch.int32)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32)
    outs = []
    for m, dev in ((gpu, DEV), (cpu, "cpu")):
        m.alloc_state(4)
        kv = torch.zeros(m.kv_cache_shape(4, page), dtype=torch.bfloat16, device=dev)
        meta = AttnMeta(True, pos.to(dev), slots.to(dev), bt.to(dev), i32(lens).to(dev), i32([0, 50, 57]).to(dev),
                        total_q_blocks=2, state_slots=i32([1, 2]).to(dev))
        x = m.hidden_states(ids.to(dev), meta, kv)
        outs.append(m.logits(x).float().cpu())
    expect_close(outs[0], outs[1], atol=6e-2, rtol=6e-2, min_close=0.99)


def test_quant_kernels_match_torch_formulation():
    from zml_b200.nn import quant as Q
    from zml_b200.ops import quant as opsq
    torch.manual_seed(0)
    x = (torch.randn(37, 256, device=DEV) * 3).bfloat16()
    x[0, :16] = 0                                              # an all-zero block takes the minimum scale
    codes, scales = opsq.nvfp4_quantize(x)
    rc, rs = Q.quantize_nvfp4(x.cpu())
    assert torch.equal(scales.cpu().view(torch.uint8), rs.view(torch.uint8))
    assert torch.equal(codes.cpu(), Q.pack_e2m1(rc))
    gs = torch.tensor(0.37)
    codes_g, scales_g = opsq.nvfp4_quantize(x, gs.to(DEV))
    rc_g, rs_g = Q.quantize_nvfp4(x.cpu(), gs)
    assert (codes_g.cpu() != Q.pack_e2m1(rc_g)).float().mean().item() < 0.01
    back = opsq.nvfp4_dequantize(codes, scales)
    want = Q.dequantize_nvfp4(rc, rs, None, torch.bfloat16)
    assert torch.equal(back.cpu(), want)
    err = (back.float() - x.float()).abs().mean() / x.float().abs().mean()
    assert err.item() < 0.12
    q8, s8 = opsq.fp8_group_quant(x, 128)
    rq, rsc = Q.per_token_group_quant_fp8(x.cpu(), 128)
    torch.testing.assert_close(s8.cpu(), rsc, rtol=1e-6, atol=0)
    assert (q8.cpu().view(torch.uint8) != rq.view(torch.uint8)).float().mean().item() < 0.002


def test_nvfp4_linear_runs_on_the_bf16_gemm():
    from zml_b200.nn import layers, quant as Q
    from zml_b200.shape import Shape
    from zml_b200.tensor import Tensor
    torch.manual_seed(1)
    w = torch.randn(256, 128) * 0.1
    packed, scales, gs = Q.quantize_weight_nvfp4(w)
    x = torch.randn(9, 128).bfloat16()
    def make(dev):
        lin = layers.Linear(Tensor(packed.to(dev), Shape({"dout": 256, "d": 64}, "u8")), None, "d",
                            layers.Quant(Q.QuantScheme.nvfp4, Tensor(scales.to(dev), Shape({"dout": 256, "d": 8}, "f8e4m3fn")),
                                         layers.TensorScale(Tensor(gs.reshape(1).to(dev), Shape((1,), "f32")))))
        return lin(Tensor(x.to(dev), Shape({"b": 9, "d": 128}, "bf16"))).to_torch().float().cpu()
    expect_close(make(DEV), make("cpu"), atol=3e-2, rtol=3e-2, min_close=0.995)
    exact = x.float() @ w.t()
    assert ((make("cpu") - exact).norm() / exact.norm()).item() < 0.2          # 4-bit weights: ~10 % error


@pytest.mark.parametrize("tokens,e_local,k_top,d,f", [(24, 8, 2, 256, 256), (128, 16, 4, 512, 768), (7, 4, 1, 256, 512), (300, 8, 2, 512, 256),
                                                     (9, 4, 2, 128, 128)])
def test_moe_grouped_gemm_nvfp4_weights(tokens, e_local, k_top, d, f, monkeypatch):
    """NVFP4 expert weights de-quantised inside the grouped GEMM (bf16 activations, `ZB_MOE_FP4=a16`) == the bf16
    kernels on the de-quantised weights (the last case has K = 128, which the NVFP4 kernel does not take: the bf16
    kernels run)."""
    from zml_b200 import moe
    monkeypatch.setenv("ZB_MOE_FP4", "a16")
    torch.manual_seed(tokens)
    gate = (torch.randn(e_local, f, d, device=DEV) * 0.05).bfloat16()
    up = (torch.randn(e_local, f, d, device=DEV) * 0.05).bfloat16()
    down = (torch.randn(e_local, d, f, device=DEV) * 0.05).bfloat16()
    if tokens % 2 == 0:
        gu_q = moe.Nvfp4Experts.quantize(moe.interleave_gate_up(gate, up))
    else:
        # gate and up quantised separately, as a checkpoint stores them: two matrix scales per expert
        from zml_b200.nn import quant as Q
        gu_q = moe.Nvfp4Experts.from_checkpoint_gate_up(Q.quantize_weight_nvfp4(gate), Q.quantize_weight_nvfp4(up * 4.0))
        assert gu_q.gscale.shape == (e_local, 2)
    dn_q = moe.Nvfp4Experts.quantize(down)
    gu_bf, dn_bf = gu_q.dequantize(), dn_q.dequantize()
    x = torch.randn(tokens, d, device=DEV).bfloat16()
    logits = torch.randn(tokens, e_local, device=DEV)
    ids, w = moe.router_topk(logits, k_top, True)
    want = moe.fused_experts(x, ids, w, gu_bf, dn_bf, 0, e_local)
    got = moe.fused_experts(x, ids, w, gu_bf, dn_bf, 0, e_local, w4=(gu_q, dn_q))
    expect_close(got.float(), want.float(), atol=2e-2, rtol=2e-2, min_close=0.995)
    g, u = moe.deinterleave_gate_up(gu_bf)
    ref = moe.reference_fused_experts(x.cpu(), ids.cpu(), w.cpu(), g.cpu(), u.cpu(), dn_bf.cpu(), 0)
    expect_close(got.float().cpu(), ref.float(), atol=3e-2, rtol=3e-2, min_close=0.99)


def _offsets(counts):
    off = [0]
    for c in counts:
        off.append(off[-1] + c)
    return torch.tensor(off, dtype=torch.int32, device=DEV), off[-1]


@pytest.mark.parametrize("e,n,k,counts,swiglu,avg", [
    (2, 128, 256, [5, 3], False, 8),
    (4, 256, 512, [16, 0, 7, 33], True, 8),
    (8, 512, 1024, [40, 1, 0, 64, 17, 3, 90, 8], False, 32),
    (8, 512, 1024, [40, 1, 0, 64, 17, 3, 90, 8], True, 64),
    (3, 256, 768, [200, 130, 5], False, 100),
])
def test_block_scaled_nvfp4_grouped_gemm(e, n, k, counts, swiglu, avg):
    """`tcgen05.mma.kind::mxf4nvf4.block_scale` on NVFP4 weights and NVFP4 activations == a float32 matmul of the
    de-quantised operands (`nn/quant.py`), for token tiles of 16 to 128, with and without the SwiGLU epilogue."""
    from zml_b200 import moe
    from zml_b200.nn import quant as Q
    torch.manual_seed(e * 7 + n)
    wq = moe.Nvfp4Experts.quantize((torch.randn(e, n, k, device=DEV) * 0.05).bfloat16())
    meta, cap = _offsets(counts)
    xs = torch.randn(cap, k, device=DEV).bfloat16()
    got = moe.grouped_gemm_fp4(xs, wq, meta, swiglu=swiglu, avg_tokens=avg)
    codes, scales = Q.quantize_nvfp4(xs.cpu(), None)
    xq = Q.dequantize_nvfp4(codes, scales, None, torch.float32)
    wd = wq.dequantize(torch.float32).cpu()
    off = meta.cpu().tolist()
    want = torch.zeros(cap, n // 2 if swiglu else n)
    for i in range(e):
        a, b = off[i], off[i + 1]
        y = xq[a:b] @ wd[i].t()
        if swiglu:
            y = y.reshape(b - a, n // 128, 2, 64)
            y = (torch.nn.functional.silu(y[:, :, 0]) * y[:, :, 1]).reshape(b - a, n // 2)
        want[a:b] = y
    expect_close(got.float().cpu(), want, atol=2e-2, rtol=2e-2, min_close=0.995)


def test_block_scaled_nvfp4_expert_block():
    """The whole expert block on the block-scaled path: the gather quantises the activations, the gate|up GEMM
    quantises its SwiGLU output in the epilogue (bit-equal to the stand-alone quantiser), and the result equals the
    CPU restatement of the same recipe; against bf16 activations the difference is the 4-bit activation noise."""
    from zml_b200 import moe
    torch.manual_seed(3)
    wq = moe.Nvfp4Experts.quantize((torch.randn(4, 512, 512, device=DEV) * 0.05).bfloat16())
    meta, cap = _offsets([16, 0, 7, 33])
    xq = moe.Fp4Activations.quantize(torch.randn(cap, 512, device=DEV).bfloat16())
    h = moe.grouped_gemm_fp4(xq, wq, meta, swiglu=True, avg_tokens=8)
    hq = moe.grouped_gemm_fp4(xq, wq, meta, swiglu=True, avg_tokens=8, quantize_out=True)
    want = moe.Fp4Activations.quantize(h)
    assert (hq.codes == want.codes).float().mean().item() > 0.999
    assert (hq.scales.view(torch.uint8) == want.scales.view(torch.uint8)).float().mean().item() > 0.999
    for tokens in (32, 300):
        e_local, k_top, d, f = 16, 4, 512, 768
        gate = (torch.randn(e_local, f, d, device=DEV) * 0.05).bfloat16()
        up = (torch.randn(e_local, f, d, device=DEV) * 0.05).bfloat16()
        down = (torch.randn(e_local, d, f, device=DEV) * 0.05).bfloat16()
        gu_q = moe.Nvfp4Experts.quantize(moe.interleave_gate_up(gate, up))
        dn_q = moe.Nvfp4Experts.quantize(down)
        gu_bf, dn_bf = gu_q.dequantize(), dn_q.dequantize()
        x = torch.randn(tokens, d, device=DEV).bfloat16()
        ids, wts = moe.router_topk(torch.randn(tokens, e_local, device=DEV), k_top, True)
        assert moe.fp4_activations()
        y = moe.fused_experts(x, ids, wts, gu_bf, dn_bf, 0, e_local, w4=(gu_q, dn_q))
        cpu_q = (moe.Nvfp4Experts.quantize(moe.interleave_gate_up(gate, up).cpu()), moe.Nvfp4Experts.quantize(down.cpu()))
        yc = moe.fused_experts(x.cpu(), ids.cpu(), wts.cpu(), gu_bf.cpu(), dn_bf.cpu(), 0, e_local, w4=cpu_q)
        assert ((y.float().cpu() - yc.float()).norm() / yc.float().norm()).item() < 0.05
        ybf = moe.fused_experts(x, ids, wts, gu_bf, dn_bf, 0, e_local)
        assert ((y.float() - ybf.float()).norm() / ybf.float().norm()).item() < 0.3
    ops.raise_on_status()


@pytest.mark.parametrize("activation", ["geglu", "geglu_tanh", "relu2"])
@pytest.mark.parametrize("tokens", [24, 600])
def test_expert_mlp_activations(activation, tokens):
    """geglu / geglu_tanh / relu2 in the epilogues of the grouped GEMMs (few and many tokens per expert: both tile
    orientations; bf16 weights, NVFP4 weights with bf16 and with NVFP4 activations) == the CPU restatement."""
    from zml_b200 import moe
    torch.manual_seed(tokens)
    e, f, d, k = 8, 256, 256, 2
    gate, up, down = ((torch.randn(e, f, d, device=DEV) * 0.05).bfloat16(), (torch.randn(e, f, d, device=DEV) * 0.05).bfloat16(),
                      (torch.randn(e, d, f, device=DEV) * 0.05).bfloat16())
    x = torch.randn(tokens, d, device=DEV).bfloat16()
    ids, w = moe.router_topk(torch.randn(tokens, e, device=DEV), k, True)
    w1 = up if activation == "relu2" else moe.interleave_gate_up(gate, up)
    got = moe.fused_experts(x, ids, w, w1, down, 0, e, activation=activation)
    want = moe.fused_experts(x.cpu().float(), ids.cpu(), w.cpu(), w1.cpu().float(), down.cpu().float(), 0, e, activation=activation)
    expect_close(got.float().cpu(), want, atol=2e-2, rtol=3e-2, min_close=0.99)
    if tokens <= 64:
        w4 = (moe.Nvfp4Experts.quantize(w1), moe.Nvfp4Experts.quantize(down))
        w4c = (moe.Nvfp4Experts.quantize(w1.cpu()), moe.Nvfp4Experts.quantize(down.cpu()))
        for mode in ("a16", "a4"):
            os.environ["ZB_MOE_FP4"] = mode
            try:
                y = moe.fused_experts(x, ids, w, w4[0].dequantize(), w4[1].dequantize(), 0, e, w4=w4, activation=activation)
                yc = moe.fused_experts(x.cpu(), ids.cpu(), w.cpu(), w4c[0].dequantize(), w4c[1].dequantize(), 0, e, w4=w4c, activation=activation)
            finally:
                os.environ.pop("ZB_MOE_FP4", None)
            assert ((y.float().cpu() - yc.float()).norm() / yc.float().norm()).item() < 0.06, mode
    ops.raise_on_status()
