"""Structured ops: generic reduce / reduce_window / sort with user functions, control flow,
custom calls, and all_reduce across gloo ranks."""
import os
import subprocess
import sys

import pytest
import torch

from zml_b200 import ops
from zml_b200.shape import Shape
from zml_b200.tensor import Tensor


def T(x, tags=None, dtype=None):
    x = torch.as_tensor(x)
    return Tensor.from_torch(x, tags)


def test_reduce_sum_and_argmax_like_pair():
    x = torch.arange(24, dtype=torch.float32).reshape(2, 3, 4)
    (s,) = ops.reduce([T(x, ("a", "b", "c"))], [T(torch.tensor(0.0))], ["b"], lambda acc, v: (acc[0].add(v[0]),))
    assert s.shape().tags == ("a", "c")
    torch.testing.assert_close(s.to_torch(), x.sum(1))
    # two operands reduced together: (max value, index of the max), ties to the smaller index
    torch.manual_seed(0)
    v = torch.randn(5, 17)
    idx = torch.arange(17).expand(5, 17).contiguous()

    def arg_max(a, b):
        take_a = a[0].cmp("GT", b[0]).logical("or", a[0].cmp("EQ", b[0]).logical("and", a[1].cmp("LT", b[1])))
        return take_a.select(a[0], b[0]), take_a.select(a[1], b[1])
    mv, mi = ops.reduce([T(v, ("r", "c")), T(idx, ("r", "c"))], [T(torch.tensor(float("-inf"))), T(torch.tensor(0))],
                        ["c"], arg_max)
    torch.testing.assert_close(mv.to_torch(), v.max(1).values)
    assert mi.to_torch().tolist() == v.argmax(1).tolist()


def test_reduce_window_is_max_pool():
    x = torch.randn(1, 1, 8, 8)
    (y,) = ops.reduce_window([T(x)], [T(torch.tensor(float("-inf")))],
                             ops.ReduceWindowOpts(window_dimensions=[1, 1, 2, 2], window_strides=[1, 1, 2, 2]),
                             lambda a, b: (a[0].maximum(b[0]),))
    torch.testing.assert_close(y.to_torch(), torch.nn.functional.max_pool2d(x, 2))


def test_reduce_window_padding_and_dilations():
    """A windowed sum with padding, a dilated window and a dilated base against a convolution with ones."""
    x = torch.arange(1.0, 8.0)[None]                                            # [1, 7]
    add = lambda a, b: (a[0].add(b[0]),)
    zero = T(torch.tensor(0.0))
    (y,) = ops.reduce_window([T(x)], [zero], ops.ReduceWindowOpts([1, 3], [1, 2], None, [1, 2], [(0, 0), (1, 1)]), add)
    ref = torch.nn.functional.conv1d(x[None], torch.ones(1, 1, 3), stride=2, padding=1, dilation=2)[0]
    torch.testing.assert_close(y.to_torch(), ref)
    # base dilation 2: 1 _ 2 _ 3 ... (holes hold the init value), then windows of 3
    (z,) = ops.reduce_window([T(x)], [zero], ops.ReduceWindowOpts([1, 3], [1, 1], [1, 2], None, None), add)
    holes = torch.zeros(1, 13)
    holes[:, ::2] = x
    torch.testing.assert_close(z.to_torch(), torch.nn.functional.conv1d(holes[None], torch.ones(1, 1, 3))[0])


def test_sort_by_key_and_by_comparator():
    torch.manual_seed(1)
    k = torch.randn(3, 9)
    payload = torch.arange(27).reshape(3, 9)
    ks, ps = ops.sort([T(k, ("r", "c")), T(payload, ("r", "c"))], "c", key=lambda a, b: a)
    order = torch.argsort(k, 1)
    torch.testing.assert_close(ks.to_torch(), torch.gather(k, 1, order))
    assert ps.to_torch().tolist() == torch.gather(payload, 1, order).tolist()
    kd, pd = ops.sort([T(k, ("r", "c")), T(payload, ("r", "c"))], "c", func=lambda a, b: a[0].cmp("GT", b[0]))
    torch.testing.assert_close(kd.to_torch(), torch.sort(k, 1, descending=True).values)


def test_control_flow_and_custom_call():
    st = ops.while_(lambda s: s["i"].cmp("LT", 5), lambda s: {"i": s["i"].add_constant(1), "acc": s["acc"].scale(2)},
                    {"i": T(torch.tensor(0)), "acc": T(torch.tensor(1.0))})
    assert int(st["i"].to_torch()) == 5 and float(st["acc"].to_torch()) == 32.0
    a, b = T(torch.tensor([1.0, 2.0])), T(torch.tensor([10.0, 20.0]))
    assert ops.if_(T(torch.tensor(True)), lambda x, y: x, lambda x, y: y, a, b) is a
    sel = ops.if2(T(torch.tensor(False)), lambda x, y: x, lambda x, y: y, a, b)
    assert sel.to_torch().tolist() == [10.0, 20.0]
    ops.register_custom_call("test.double", lambda ins, outs, md: ins[0].scale(md["k"]))
    out = ops.custom_call("test.double", [a], [a.shape()], {"k": 3}, ops.CustomCallOptions(compute_on_host=True))
    assert out.to_torch().tolist() == [3.0, 6.0]
    with pytest.raises(KeyError):
        ops.custom_call("nope", [a], [a.shape()])
    r = ops.manual_computation([a], [a.shape()], None, lambda ins, ctx: [ins[0].add(ins[0])])
    assert r[0].to_torch().tolist() == [2.0, 4.0]
    with pytest.raises(ValueError):
        ops.manual_computation([a], [Shape((3,), "f32")], None, lambda ins, ctx: [ins[0]])
    assert int(ops.partition_id().to_torch()) == 0


_WORKER = r"""
import os, sys, torch
sys.path.insert(0, os.environ["ZB_ROOT"])
from zml_b200 import ops
from zml_b200.parallel.comm import Comm
from zml_b200.tensor import Tensor
c = Comm.from_env(backend="gloo")
x = Tensor.from_torch(torch.full((4,), float(c.rank + 1)), ("d",))
s = ops.all_reduce(x, "add", comm=c)
m = ops.all_reduce({"v": x}, "max", comm=c)
u = ops.all_reduce(x, lambda a, b: a.mul(b), comm=c)
assert s.to_torch().tolist() == [3.0] * 4, s
assert m["v"].to_torch().tolist() == [2.0] * 4
assert u.to_torch().tolist() == [2.0] * 4
assert int(ops.partition_id(c).to_torch()) == c.rank
print("AR_OK", c.rank, flush=True)
c.finish(0)
"""


def test_all_reduce_two_gloo_ranks(tmp_path):
    script = tmp_path / "w.py"
    script.write_text(_WORKER)
    env = dict(os.environ, ZB_ROOT=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29631", str(script)],
                       capture_output=True, text=True, env=env, timeout=180)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("AR_OK") == 2
