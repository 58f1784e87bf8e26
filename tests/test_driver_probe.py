"""The CUDA driver probe against fakes of libcuda (no GPU, no driver): each cuInit outcome maps to its exit code and
to a sentence a user can act on; the child-process form and the platform's error message use it."""
import ctypes
import subprocess
import sys

import pytest

from zml_b200 import driver_probe as dp
from zml_b200.driver_probe import ExitCode


class FakeCuda:
    def __init__(self, init_rc=0, version=13000, devices=8, with_strings=True):
        self.init_rc, self.version, self.devices = init_rc, version, devices
        self.calls = []
        if not with_strings:
            self.cuGetErrorString = None

    def cuInit(self, flags):
        self.calls.append(("cuInit", flags))
        return self.init_rc

    def cuDriverGetVersion(self, ref):
        ref._obj.value = self.version
        return 0

    def cuDeviceGetCount(self, ref):
        ref._obj.value = self.devices
        return 0

    def cuGetErrorString(self, rc, ref):
        ref._obj.value = b"out of memory" if rc == 2 else None
        return 0 if rc == 2 else 1


def test_each_cuinit_outcome_maps_to_its_code():
    ok = dp.probe(FakeCuda())
    assert ok.ok() and ok.code is ExitCode.success and ok.driver_version == 13000 and ok.device_count == 8
    assert dp.probe(FakeCuda(803)).code is ExitCode.system_driver_mismatch
    assert dp.probe(FakeCuda(804)).code is ExitCode.compat_not_supported_on_device
    assert dp.probe(FakeCuda(100)).code is ExitCode.no_device
    assert dp.probe(FakeCuda(0, devices=0)).code is ExitCode.no_device
    odd = dp.probe(FakeCuda(2))
    assert odd.code is ExitCode.unexpected_error and "out of memory" in odd.message and odd.cu_result == 2
    bare = dp.probe(FakeCuda(999, with_strings=False))
    assert bare.code is ExitCode.unexpected_error and "999" in bare.message
    # the four codes the reference's probe returns keep their numbers
    assert [int(ExitCode.success), int(ExitCode.compat_not_supported_on_device), int(ExitCode.system_driver_mismatch),
            int(ExitCode.unexpected_error)] == [0, 1, 2, 3]
    fake = FakeCuda()
    dp.probe(fake)
    assert fake.calls == [("cuInit", 0)]


def test_missing_library_is_no_driver():
    r = dp.probe(path="libcuda_that_does_not_exist.so.1")
    assert r.code is ExitCode.no_driver and "libcuda_that_does_not_exist" in r.message
    assert "NVIDIA runtime" in dp.diagnose(r)


def test_diagnosis_names_the_remedy():
    assert "reboot" in dp.diagnose(dp.probe(FakeCuda(803)))
    assert "LD_LIBRARY_PATH" in dp.diagnose(dp.probe(FakeCuda(804)))
    assert "CUDA_VISIBLE_DEVICES" in dp.diagnose(dp.probe(FakeCuda(100)))
    assert dp.diagnose(dp.probe(FakeCuda(version=13000)), 12080) == "driver ok: CUDA 13.0, 8 device(s)"
    old = dp.diagnose(dp.probe(FakeCuda(version=12040)), 12080)
    assert "12.4" in old and "12.8" in old and "upgrade the driver" in old and "PyTorch" in old
    # a runtime older than sm_100's first CUDA release: the GPU sets the bar
    assert "sm_100" in dp.diagnose(dp.probe(FakeCuda(version=12040)), 12040)
    # a runtime newer than the driver
    assert "13.0" in dp.diagnose(dp.probe(FakeCuda(version=12080)), 13000)
    assert dp.format_version(12080) == "12.8" and dp.format_version(None) == "unknown"


def test_result_round_trips_as_json():
    r = dp.probe(FakeCuda(803))
    back = dp.ProbeResult.from_json(r.to_json())
    assert back == r and isinstance(back.code, ExitCode)


def test_runtime_version_parses_torch():
    import torch
    v = dp.runtime_version()
    if torch.version.cuda is None:
        assert v is None
    else:
        major, minor = torch.version.cuda.split(".")[:2]
        assert v == int(major) * 1000 + int(minor) * 10


@pytest.mark.skipif(__import__("torch").cuda.is_available(), reason="checks the answer of a machine without a GPU")
def test_child_probe_and_platform_message_on_a_machine_without_gpu():
    r = dp.probe_in_child()
    assert r.code in (ExitCode.no_driver, ExitCode.no_device, ExitCode.unexpected_error, ExitCode.success)
    out = subprocess.run([sys.executable, "-m", "zml_b200.driver_probe", "--no-torch"], capture_output=True, text=True)
    assert out.returncode == int(r.code) and out.stdout.strip()
    from zml_b200.platform import Platform, Target
    with pytest.raises(RuntimeError, match="no CUDA device is visible: ") as e:
        Platform(Target.cuda)
    assert dp.diagnose(r, dp.runtime_version()) in str(e.value)


def test_child_that_cannot_start_is_reported():
    r = dp.probe_in_child(python="/nonexistent/python")
    assert r.code is ExitCode.unexpected_error and "did not run" in r.message
