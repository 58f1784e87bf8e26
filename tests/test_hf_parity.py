"""Architecture parity against HuggingFace transformers, the way the reference checks its
models against PyTorch activations (tools/zml_utils.py + zml/testing.zig `testLayer`): a tiny
random-init HF model is saved as safetensors, loaded through the framework's own loader under
HF tensor names, and the logits of a varlen prefill (plus a decode step through the paged
cache / recurrent state) are compared with the HF forward pass."""
import json
import os

import pytest
import torch

from zml_b200.io import TensorStore
from zml_b200.models import registry
from zml_b200.models.llama import AttnMeta
from zml_b200.safetensors import save_file

transformers = pytest.importorskip("transformers")


def _ours_logits(model, prompts, page=16, decode_tokens=None):
    """Prefill logits of every prompt token (list of [len, vocab]) and, if `decode_tokens` is
    given, the logits after feeding one more token per sequence through the decode path."""
    from zml_b200.serving.engine import Engine
    eng = Engine(model, num_pages=64, page_size=page, max_batch=4, max_seq_len=128, max_prefill_tokens=4096)
    reqs = [eng.new_request(p, 4) for p in prompts]
    ids, pos, slots, qs, sl = [], [], [], [0], []
    bt = torch.zeros((len(reqs), eng.max_pages), dtype=torch.int32)
    for i, r in enumerate(reqs):
        n = len(r.prompt)
        ids += r.prompt
        pos += list(range(n))
        slots += [r.pages[p // page] * page + p % page for p in range(n)]
        qs.append(qs[-1] + n)
        sl.append(n)
        bt[i, :len(r.pages)] = torch.tensor(r.pages, dtype=torch.int32)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32)
    ss = i32([max(r.slot, 0) for r in reqs])
    meta = AttnMeta(True, i32(pos), i32(slots), bt, i32(sl), i32(qs), total_q_blocks=sum((n + 63) // 64 for n in sl),
                    state_slots=ss)
    x = model.hidden_states(i32(ids), meta, eng.kv_cache)
    lg = model.logits(x).float()
    pre = [lg[qs[i]:qs[i + 1]] for i in range(len(reqs))]
    dec = None
    if decode_tokens is not None:
        dpos = i32(sl)
        dslot = i32([r.pages[n // page] * page + n % page for r, n in zip(reqs, sl)])
        meta = AttnMeta(False, dpos, dslot, bt, dpos + 1, i32(list(range(len(reqs) + 1))), state_slots=ss)
        x = model.hidden_states(i32(decode_tokens), meta, eng.kv_cache)
        dec = model.logits(x).float()
    return pre, dec


def _check(hf_model, hf_config_dict, tmp_path, atol):
    hf_model = hf_model.eval().to(torch.bfloat16)
    sd = {k: v.contiguous() for k, v in hf_model.state_dict().items()}
    repo = str(tmp_path)
    save_file(sd, os.path.join(repo, "model.safetensors"))
    with open(os.path.join(repo, "config.json"), "w") as f:
        json.dump(hf_config_dict, f)
    cfg_cls, model_cls = registry.model_class_for(hf_config_dict)
    cfg = cfg_cls.from_hf(hf_config_dict)
    ours = model_cls(cfg, device="cpu", dtype=torch.bfloat16).load(TensorStore.from_path(repo))
    g = torch.Generator().manual_seed(1)
    vocab = cfg.vocab_size
    prompts = [torch.randint(3, vocab, (n,), generator=g).tolist() for n in (7, 19)]
    nxt = [5, 9]
    pre, dec = _ours_logits(ours, prompts, decode_tokens=nxt)
    for p, lg, t, d in zip(prompts, pre, nxt, dec):
        with torch.no_grad():
            ref = hf_model(torch.tensor([p + [t]])).logits[0].float()
        scale = ref.abs().max().item()
        assert (lg - ref[:len(p)]).abs().max().item() <= atol * max(scale, 1.0), "prefill logits"
        assert (d - ref[len(p)]).abs().max().item() <= atol * max(scale, 1.0), "decode-step logits"
        assert int(lg[-1].argmax()) == int(ref[len(p) - 1].argmax())


def test_llama_parity(tmp_path):
    c = transformers.LlamaConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                                 num_key_value_heads=2, vocab_size=512, max_position_embeddings=256, rms_norm_eps=1e-5,
                                 rope_theta=10000.0, tie_word_embeddings=False, head_dim=32)
    torch.manual_seed(0)
    _check(transformers.LlamaForCausalLM(c), c.to_dict(), tmp_path, 0.03)


def test_qwen3_moe_parity(tmp_path):
    c = transformers.Qwen3MoeConfig(hidden_size=128, intermediate_size=256, moe_intermediate_size=128, num_hidden_layers=2,
                                    num_attention_heads=4, num_key_value_heads=2, head_dim=32, vocab_size=512,
                                    num_experts=8, num_experts_per_tok=2, norm_topk_prob=True, decoder_sparse_step=1,
                                    mlp_only_layers=[], max_position_embeddings=256, tie_word_embeddings=False)
    torch.manual_seed(0)
    _check(transformers.Qwen3MoeForCausalLM(c), c.to_dict(), tmp_path, 0.04)


def _qwen35_text_kwargs():
    return dict(hidden_size=128, intermediate_size=256, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                head_dim=64, vocab_size=512, max_position_embeddings=256, rms_norm_eps=1e-6, linear_conv_kernel_dim=4,
                linear_key_head_dim=64, linear_value_head_dim=64, linear_num_key_heads=2, linear_num_value_heads=4,
                layer_types=["linear_attention", "full_attention", "linear_attention", "full_attention"],
                tie_word_embeddings=False)


def test_qwen3_5_parity(tmp_path):
    from transformers.models.qwen3_5 import Qwen3_5ForCausalLM, Qwen3_5TextConfig
    c = Qwen3_5TextConfig(**_qwen35_text_kwargs())
    torch.manual_seed(0)
    m = Qwen3_5ForCausalLM(c)
    d = c.to_dict()
    d["model_type"] = "qwen3_5_text"
    _check_prefixed(m, d, tmp_path, 0.04)


def test_qwen3_5_moe_parity(tmp_path):
    from transformers.models.qwen3_5_moe import Qwen3_5MoeForCausalLM, Qwen3_5MoeTextConfig
    c = Qwen3_5MoeTextConfig(**_qwen35_text_kwargs(), num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64,
                             shared_expert_intermediate_size=64)
    torch.manual_seed(0)
    m = Qwen3_5MoeForCausalLM(c)
    d = c.to_dict()
    d["model_type"] = "qwen3_5_moe_text"
    _check_prefixed(m, d, tmp_path, 0.04)


def _check_prefixed(hf_model, cfg_dict, tmp_path, atol):
    """The text-only HF classes name tensors `model.*`; checkpoints of the full model (and the
    reference, examples/llm/models/qwen3_5/model.zig:162) use `model.language_model.*`."""
    class Renamed(torch.nn.Module):
        def __init__(self, inner):
            super().__init__()
            self.inner = inner

        def state_dict(self, *a, **k):
            sd = self.inner.state_dict(*a, **k)
            return {("model.language_model." + n[len("model."):] if n.startswith("model.") else n): v for n, v in sd.items()}

        def forward(self, *a, **k):
            return self.inner(*a, **k)

        def eval(self):
            self.inner.eval()
            return self

        def to(self, *a, **k):
            self.inner.to(*a, **k)
            return self
    _check(Renamed(hf_model), cfg_dict, tmp_path, atol)


def test_lfm2_parity(tmp_path):
    c = transformers.Lfm2Config(hidden_size=128, intermediate_size=256, block_ff_dim=256, block_auto_adjust_ff_dim=False,
                                num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, vocab_size=512,
                                max_position_embeddings=256, norm_eps=1e-5, conv_L_cache=3, conv_bias=False,
                                layer_types=["conv", "full_attention", "conv", "full_attention"], rope_theta=10000.0)
    torch.manual_seed(0)
    d = c.to_dict()
    _check(transformers.Lfm2ForCausalLM(c), d, tmp_path, 0.04)


def test_model_tests_runner_checks_layers_against_captured_activations(tmp_path):
    """`examples/llm/model_tests.py`: activations captured from the HF model with ActivationCollector, then every
    recorded decoder layer and the final norm re-computed on this framework's weights."""
    import importlib.util
    import sys
    from zml_b200.utils.activations import ActivationCollector, save_activations
    cfgd = dict(model_type="llama", architectures=["LlamaForCausalLM"], vocab_size=320, hidden_size=128, intermediate_size=256,
                num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-5,
                rope_theta=10000.0, max_position_embeddings=256, tie_word_embeddings=False, hidden_act="silu",
                bos_token_id=1, eos_token_id=2)
    torch.manual_seed(0)
    hf = transformers.LlamaForCausalLM(transformers.LlamaConfig(**{k: v for k, v in cfgd.items() if k not in ("architectures",)}))
    hf = hf.eval().float()
    repo = tmp_path / "repo"
    repo.mkdir()
    save_file({k: v.contiguous() for k, v in hf.state_dict().items()}, str(repo / "model.safetensors"))
    (repo / "config.json").write_text(json.dumps(cfgd))
    ids = torch.randint(3, 320, (2, 21), generator=torch.Generator().manual_seed(4))
    _, acts = ActivationCollector(hf, blacklist_regexes=())(ids)
    keep = {k: v for k, v in acts.items() if k.startswith("model.layers.") and k.count(".") == 4 or k.startswith("model.norm.")}
    assert "model.layers.2.in.0" in keep and "model.norm.out.0" in keep
    save_activations(str(tmp_path / "acts.safetensors"), keep)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("model_tests", os.path.join(root, "examples", "llm", "model_tests.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["model_tests"] = mod
    spec.loader.exec_module(mod)
    rc = mod.main([f"--model={repo}", f"--activations={tmp_path / 'acts.safetensors'}", "--device=cpu", "--atol=2e-3", "--rtol=2e-3"])
    assert rc == 0
    # a corrupted fixture is reported
    keep["model.layers.1.out.0"] = keep["model.layers.1.out.0"] + 1.0
    save_activations(str(tmp_path / "bad.safetensors"), keep)
    assert mod.main([f"--model={repo}", f"--activations={tmp_path / 'bad.safetensors'}", "--device=cpu"]) == 1
