"""MNIST-shaped MLP (examples/mnist/mnist.zig:12-74): two Linear + bias + ReLU layers,
input {28, 28} u8 -> flatten -> f32 -> argmax -> u8 class.  Written on the tagged Tensor
API and run through `Platform.compile` / `Loader` - the plumbing smoke test of the framework."""
from __future__ import annotations

import torch

from ..io import Loader, TensorStore, View
from ..tensor import Tensor


class Layer:
    def __init__(self, view: View):
        self.weight = view.create_tensor("weight", ("d_out", "d"))
        self.bias = view.create_tensor("bias", ("d_out",))

    @staticmethod
    def forward(weight: Tensor, bias: Tensor, x: Tensor) -> Tensor:
        return weight.dot(x, "d").add(bias).relu().with_tags("d")


class Mnist:
    def __init__(self, view: View):
        self.fc1 = Layer(view.with_prefix("fc1"))
        self.fc2 = Layer(view.with_prefix("fc2"))

    def load(self, platform, store: TensorStore):
        loader = Loader(platform, parallelism=4)
        try:
            return loader.load(self, store, [])
        finally:
            loader.close()

    @staticmethod
    def forward(fc1_w: Tensor, fc1_b: Tensor, fc2_w: Tensor, fc2_b: Tensor, image: Tensor) -> Tensor:
        """image {28, 28} u8 -> class u8 (scalar-shaped {1})."""
        x = image.flatten().convert("f32").with_tags("d")
        x = Layer.forward(fc1_w, fc1_b, x)
        x = Layer.forward(fc2_w, fc2_b, x)
        _, idx = x.arg_max(0)
        return idx.convert("u8")

    def arg_tensors(self):
        return (self.fc1.weight, self.fc1.bias, self.fc2.weight, self.fc2.bias)


def random_checkpoint(path: str, seed: int = 0, std: float = 0.02) -> None:
    """Random-init weights of the MNIST MLP: f32 N(0, std), zero biases (784 -> 1000 -> 10)."""
    from .. import safetensors
    g = torch.Generator().manual_seed(seed)
    safetensors.save_file({
        "fc1.weight": torch.randn(1000, 784, generator=g) * std, "fc1.bias": torch.zeros(1000),
        "fc2.weight": torch.randn(10, 1000, generator=g) * std, "fc2.bias": torch.zeros(10),
    }, path)
