"""Collecting PyTorch activations as test fixtures, and checking a layer of this framework
against them - the workflow of the reference's tools/zml_utils.py (`ActivationCollector`,
producing `name.in.N` / `name.out.N` entries) and zml/testing.zig (`testLayer`).

    collector = ActivationCollector(hf_model, max_layers=200)
    output, acts = collector(input_ids)                 # {"model.layers.0.mlp.in.0": tensor, ...}
    save_activations("acts.safetensors", acts)
    ...
    test_layer(lambda x: my_mlp(x), acts, "model.layers.0.mlp", atol=1e-2)
"""
from __future__ import annotations

import re
from typing import Callable, Mapping, Optional, Sequence

import torch

from .. import safetensors
from ..testing import expect_close


class ActivationCollector:
    """Wraps a torch.nn.Module; calling it runs the module and returns (output, activations).

    * max_layers: stop collecting after this many modules were recorded (-1: no limit)
    * stop_after_first_step: stop as soon as a module is entered a second time (generation loops)
    * blacklist_regexes: module names to skip (default: every layer index other than 0)
    """

    class CollectionOver(Exception):
        pass

    def __init__(self, model: torch.nn.Module, *, max_layers: int = -1, stop_after_first_step: bool = False,
                 blacklist_regexes: Sequence[str] = (r".*\.(\d\d+)\.", r".*\.[1-9]\.")):
        self.model = model
        self.max_layers = max_layers
        self.stop_after_first_step = stop_after_first_step
        self.blacklist = [re.compile(r) for r in blacklist_regexes]
        self.activations: dict[str, torch.Tensor] = {}
        self._seen: set[str] = set()
        self._count = 0

    def _skip(self, name: str) -> bool:
        return any(r.match(name + ".") for r in self.blacklist)

    def _hook(self, name: str):
        def fn(_module, args, kwargs, output):
            if name in self._seen:
                if self.stop_after_first_step:
                    raise ActivationCollector.CollectionOver()
                return
            self._seen.add(name)
            ins = [a for a in args if torch.is_tensor(a)]
            for i, a in enumerate(ins):
                self.activations[f"{name}.in.{i}"] = a.detach().cpu().contiguous()
            for k, v in kwargs.items():
                if torch.is_tensor(v):
                    self.activations[f"{name}.in.{k}"] = v.detach().cpu().contiguous()
            outs = [output] if torch.is_tensor(output) else \
                [o for o in output if torch.is_tensor(o)] if isinstance(output, (list, tuple)) else \
                [getattr(output, "last_hidden_state", None) if hasattr(output, "last_hidden_state") else getattr(output, "logits", None)]
            for i, o in enumerate(x for x in outs if torch.is_tensor(x)):
                self.activations[f"{name}.out.{i}"] = o.detach().cpu().contiguous()
            self._count += 1
            if 0 < self.max_layers <= self._count:
                raise ActivationCollector.CollectionOver()
        return fn

    def __call__(self, *args, **kwargs):
        self.activations, self._seen, self._count = {}, set(), 0
        handles = []
        for name, mod in self.model.named_modules():
            if name == "" or self._skip(name):
                continue
            handles.append(mod.register_forward_hook(self._hook(name), with_kwargs=True))
        out = None
        try:
            with torch.no_grad():
                out = self.model(*args, **kwargs)
        except ActivationCollector.CollectionOver:
            pass
        finally:
            for h in handles:
                h.remove()
        return out, dict(self.activations)


def save_activations(path: str, activations: Mapping[str, torch.Tensor]) -> None:
    """Writes the fixtures as one safetensors file (readable with `TensorStore.from_path`)."""
    safetensors.save_file({k: v for k, v in activations.items()}, path)


def load_activations(path: str) -> dict[str, torch.Tensor]:
    from ..io import TensorStore
    store = TensorStore.from_path(path)
    return {k: store.load_tensor(k) for k in store.view().keys()}


def test_layer(layer: Callable, activations: Mapping[str, torch.Tensor], name: str, atol: float = 1e-3,
               rtol: float = 1e-2, min_close: float = 0.999, device: Optional[str] = None):
    """Feeds `name.in.*` to `layer` and compares what it returns with `name.out.*`
    (zml/testing.zig `testLayer`).  Returns the outputs."""
    ins = []
    i = 0
    while f"{name}.in.{i}" in activations:
        t = activations[f"{name}.in.{i}"]
        ins.append(t.to(device) if device else t)
        i += 1
    if not ins:
        raise KeyError(f"no activation named {name}.in.0; available: {sorted(activations)[:8]} ...")
    got = layer(*ins)
    got = list(got) if isinstance(got, (list, tuple)) else [got]
    for j, g in enumerate(got):
        want = activations.get(f"{name}.out.{j}")
        if want is None:
            raise KeyError(f"layer returned {len(got)} outputs but {name}.out.{j} was not recorded")
        g = g.to_torch() if hasattr(g, "to_torch") else g
        expect_close(g.detach().float().cpu(), want.float(), atol=atol, rtol=rtol, min_close=min_close)
    return got


test_layer.__test__ = False      # not a pytest test despite the name
