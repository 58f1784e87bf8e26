"""MNIST config: random-init 784->1000->10 MLP through safetensors + Loader + compile + Exe on CPU,
against a NumPy restatement."""
import os
import subprocess
import sys

import numpy as np
import torch

from zml_b200 import safetensors
from zml_b200.models.mnist import random_checkpoint
from zml_b200.platform import Platform, Target

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "examples", "mnist"))


def test_mnist_matches_numpy(tmp_path):
    import mnist as example
    path = str(tmp_path / "m.safetensors")
    random_checkpoint(path, seed=3)
    reg = safetensors.TensorRegistry.from_path(path)
    w = {k: safetensors.bytes_to_torch(reg.reader(k).read_all(), reg.get(k).shape.dims, reg.get(k).shape.dtype).numpy() for k in reg.keys()}
    platform = Platform.init(Target.cpu)
    for seed in range(4):
        img = np.random.default_rng(seed).integers(0, 256, (28, 28), dtype=np.uint8)
        x = img.reshape(-1).astype(np.float32)
        h = np.maximum(w["fc1.weight"] @ x + w["fc1.bias"], 0)
        o = np.maximum(w["fc2.weight"] @ h + w["fc2.bias"], 0)
        assert example.classify(path, img, platform) == int(np.argmax(o))


def test_mnist_cli_synthetic():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "examples", "mnist", "mnist.py"), "--synthetic", "--seed=1"],
                       capture_output=True, text=True, timeout=120, env=dict(os.environ, ZB_TARGET="cpu"))
    assert r.returncode == 0 and "RECOGNIZED DIGIT" in r.stderr + r.stdout
