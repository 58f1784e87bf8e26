"""Declarative user kernels: emission and sm_100a compilation run anywhere nvcc exists; the
launch is checked on a GPU."""
import shutil

import pytest
import torch

from zml_b200 import kernel
from zml_b200.shape import Shape
from zml_b200.tensor import Tensor

needs_nvcc = pytest.mark.skipif(shutil.which("nvcc") is None, reason="nvcc not installed")


def _axpy():
    def run(cfg):
        return f"""
extern "C" __global__ void axpy(const float* x, const float* y, float* out, int n, float a) {{
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = a * x[i] + y[i] + {float(cfg['bias'])}f;
}}"""
    return kernel.cuda.Kernel(kernel.cuda.Spec("axpy", ["x", "y"], ["out"], run))


@needs_nvcc
def test_emit_and_cross_compile(tmp_path, monkeypatch):
    monkeypatch.setenv("ZB_KERNEL_CACHE_DIR", str(tmp_path))
    k = _axpy()
    assert "1.5f" in k.emit({"bias": 1.5})
    cubin = k.compile({"bias": 1.5})
    assert cubin.exists() and cubin.stat().st_size > 0 and cubin.read_bytes()[:4] == b"\x7fELF"
    assert k.compile({"bias": 1.5}) == cubin                      # cached by content
    ew = kernel.cuda.elementwise("fma3", ["a", "b"], "c", "a * b + 3.0f", "bf16")
    assert "__nv_bfloat16" in ew.emit() and ew.compile().exists()
    bad = kernel.cuda.Kernel(kernel.cuda.Spec("oops", ["x"], ["y"], lambda c: 'extern "C" __global__ void oops( { }'))
    with pytest.raises(kernel.KernelError):
        bad.compile()
    with pytest.raises(kernel.KernelError):
        kernel.cuda.ctype("c64")


@pytest.mark.gpu
def test_launch_on_gpu_and_in_place_alias():
    k = _axpy()
    n = 1000
    x, y = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
    sh = Shape((n,), "f32")
    out = k.call({"x": Tensor(x, sh), "y": Tensor(y, sh)}, {"out": sh},
                 kernel.cuda.CallOpts(cfg={"bias": 0.5}, grid=((n + 127) // 128,), block=(128,), scalars=(n, 2.0)))["out"]
    torch.testing.assert_close(out.to_torch(), 2.0 * x + y + 0.5)
    y0 = y.clone()
    k.call({"x": Tensor(x, sh), "y": Tensor(y, sh)}, {"out": sh},
           kernel.cuda.CallOpts(cfg={"bias": 0.0}, grid=((n + 127) // 128,), block=(128,), scalars=(n, 1.0),
                                output_operand_aliases={"out": "y"}))
    torch.testing.assert_close(y, x + y0)
