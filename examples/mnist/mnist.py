#!/usr/bin/env python
"""MNIST smoke test (the reference's examples/mnist): load a 2-layer MLP checkpoint,
compile it, classify one 28x28 image, print it as ASCII art.

    python examples/mnist/mnist.py <model.safetensors> <t10k-images.idx3-ubyte>
    python examples/mnist/mnist.py --synthetic [--seed=N]     # random weights + random image

Runs on CPU (default without a GPU) or on the GPU chosen by Platform.auto.
"""
from __future__ import annotations

import logging
import os
import sys
import tempfile
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import numpy as np  # noqa: E402
import torch  # noqa: E402

from zml_b200 import safetensors  # noqa: E402
from zml_b200.buffer import Buffer  # noqa: E402
from zml_b200.io import TensorStore  # noqa: E402
from zml_b200.models.mnist import Mnist, random_checkpoint  # noqa: E402
from zml_b200.platform import Platform  # noqa: E402
from zml_b200.shape import Shape  # noqa: E402
from zml_b200.slice import Slice  # noqa: E402
from zml_b200.tensor import Tensor  # noqa: E402

log = logging.getLogger("mnist")

DIGITS = ["zero", "one", "two", "three", "four", "five", "six", "seven", "eight", "nine"]


def print_digit(pixels: np.ndarray) -> str:
    ramp = " .:-=+*#%@"
    rows = []
    for r in range(28):
        rows.append("".join(ramp[int(v) * (len(ramp) - 1) // 255] * 2 for v in pixels[r]))
    return "\n".join(rows)


def classify(model_path: str, image: np.ndarray, platform=None) -> int:
    registry = safetensors.TensorRegistry.from_path(model_path)
    store = TensorStore.from_registry(registry)
    model = Mnist(store.view())
    platform = platform or Platform.auto()
    t0 = time.perf_counter()
    image_t = Tensor.init((28, 28), "u8")
    exe = platform.compile(Mnist.forward, (*model.arg_tensors(), image_t), program_name="mnist")
    log.info("Compiled model [%.3fs]", time.perf_counter() - t0)
    t0 = time.perf_counter()
    bufs = model.load(platform, store)
    log.info("Transferred weights [%.3fs]", time.perf_counter() - t0)
    inp = Buffer.from_slice(platform, Slice.init(Shape((28, 28), "u8"), image.astype(np.uint8)))
    runner = exe.runner(bufs.fc1.weight, bufs.fc1.bias, bufs.fc2.weight, bufs.fc2.bias)
    return int(runner.call(inp, wait=True).get_value())


def main(argv) -> int:
    logging.basicConfig(level=logging.INFO, format="%(levelname)s(%(name)s): %(message)s")
    if argv and argv[0] == "--synthetic":
        seed = 0
        for a in argv[1:]:
            if a.startswith("--seed="):
                seed = int(a.split("=", 1)[1])
        tmp = tempfile.mkdtemp()
        model_path = os.path.join(tmp, "mnist.safetensors")
        random_checkpoint(model_path, seed)
        image = np.random.default_rng(seed).integers(0, 256, (28, 28), dtype=np.uint8)
    elif len(argv) == 2:
        model_path, data = argv
        idx = int(time.time() * 1000) % 10000
        with open(data, "rb") as f:
            f.seek(16 + idx * 784)
            image = np.frombuffer(f.read(784), dtype=np.uint8).reshape(28, 28)
    else:
        print(__doc__)
        return 2
    print(print_digit(image))
    digit = classify(model_path, image)
    log.info("RECOGNIZED DIGIT: %d (%s)", digit, DIGITS[digit])
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
