"""The reference-side adaptor (paddle-lite_b200/lite_target) driven through the reference's own
KernelRegistry and KernelBase::Launch(): the probe binary is built against the reference headers
and objects where the reference tree exists and travels prebuilt to the GPU machine."""
import os
import subprocess

import pytest

from helpers import ROOT

PROBE = os.path.join(ROOT, "oracle", "_ref", "lite_target_probe")


@pytest.mark.gpu
def test_kernels_created_by_the_reference_registry_run_on_gpu(plb):
    if not os.path.exists(PROBE):
        pytest.skip("probe not built (needs the reference tree at build time)")
    res = subprocess.run([PROBE], capture_output=True, text=True, timeout=300)
    print(res.stdout, res.stderr)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "PROBE OK" in res.stdout
    assert "conv2d:cuda/int8_t/NCHW" in res.stdout


def test_adaptor_compiles_against_reference_headers():
    if not os.path.isdir("/root/reference/lite"):
        pytest.skip("reference tree absent")
    subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), "probe", "-j8"], check=True,
                   stdout=subprocess.DEVNULL)
    assert os.path.exists(os.path.join(ROOT, "oracle", "_ref", "obj", "lite_target", "cuda_int8_kernels.o"))
