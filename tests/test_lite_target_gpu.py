"""The reference-side adaptor (paddle-lite_b200/lite_target) driven through the reference's own
KernelRegistry and KernelBase::Launch() by tests/lite_target_probe.cc: the probe binary is built against the
reference headers and objects where the reference tree exists and travels prebuilt to the GPU machine."""
import importlib
import os
import re
import subprocess

import numpy as np
import pytest

from helpers import ROOT

PROBE = os.path.join(ROOT, "oracle", "_ref", "lite_target_probe")

EXPECTED = ["conv2d int8_out", "conv2d fp32_out", "conv2d int8_out after a shape change",
            "depthwise_conv2d int8_out", "depthwise_conv2d fp32_out", "depthwise_conv2d fp32_out after a shape change",
            "fc fp32_out", "fc int8_out", "sparse_conv2d int8_int8_out", "sparse_conv2d int8_fp32_out",
            "sparse_conv2d fp32 def", "io_copy -> calib -> calib -> io_copy",
            "io_copy_once -> calib_once -> calib_once -> io_copy_once",
            "conv2d -> depthwise_conv2d -> conv2d through the kNHWC kernels",
            "conv2d -> depthwise_conv2d -> conv2d through the kNCHW kernels"]


def _need_probe():
    if not os.path.exists(PROBE):
        pytest.skip("probe not built (needs the reference tree at build time)")


@pytest.mark.gpu
def test_every_registered_kernel_runs_through_the_reference_registry(plb):
    """Every registration of the new target is created by KernelRegistry and launched: conv2d and depthwise_conv2d
    (both aliases, a second Launch, a Launch after an input-shape change), fc (both aliases), the three
    sparse_conv2d kernels on tensors from the restated weight encoder, calib / calib_once / io_copy /
    io_copy_once, softmax, and a three-layer chain through the kNHWC and the kNCHW kernels."""
    _need_probe()
    res = subprocess.run([PROBE], capture_output=True, text=True, timeout=300)
    print(res.stdout, res.stderr)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "PROBE OK" in res.stdout
    assert "conv2d:cuda/int8_t/NCHW" in res.stdout
    for what in EXPECTED:
        assert re.search(re.escape(what) + r": 0 of \d+ outputs differ", res.stdout), "missing or failing: " + what
    assert "softmax: max relative error" in res.stdout


@pytest.mark.gpu
def test_unsupported_activation_on_sparse_conv_is_fatal(plb):
    """hard_swish fused into sparse_conv2d (the ARM reference implements it) must stop the program with
    LOG(FATAL); it must never run as "no activation"."""
    _need_probe()
    res = subprocess.run([PROBE, "--hard-swish"], capture_output=True, text=True, timeout=300)
    assert res.returncode != 0
    assert "hard_swish" in res.stderr and "is not implemented" in res.stderr
    assert "ran with hard_swish" not in res.stdout


@pytest.mark.gpu
def test_chain_through_launch_against_the_python_runner(plb, ctx):
    """The same pointwise -> depthwise -> pointwise chain (128 x 56 x 56, 32 -> 64 -> 64 channels) timed through
    KernelBase::Launch() with the kNHWC and the kNCHW registrations, and through the ctypes binding the
    benchmark's network runner uses: the cost of the reference-side binding as a number."""
    import torch
    _need_probe()
    res = subprocess.run([PROBE, "--time"], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    us = dict(re.findall(r"CHAIN_US (\w+) ([\d.]+)", res.stdout))
    rng = np.random.default_rng(3)
    mk = lambda *s: rng.integers(-127, 128, s, dtype=np.int8)  # noqa: E731
    a = plb.Conv(ctx, mk(64, 32, 1, 1), [0.001], 0.02, None, in_hw=(56, 56), act=plb.ACT_RELU, out_scale=0.9)
    b = plb.Conv(ctx, mk(64, 1, 3, 3), [0.001], 0.9, None, in_hw=(56, 56), pads=(1, 1, 1, 1), groups=64,
                 act=plb.ACT_RELU, out_scale=40.0)
    c = plb.Conv(ctx, mk(64, 64, 1, 1), [0.001], 40.0, None, in_hw=(56, 56), act=plb.ACT_RELU)
    x = torch.randint(-127, 128, (128, 56, 56, 32), dtype=torch.int8, device="cuda")
    ya = torch.empty((128, 56, 56, 64), dtype=torch.int8, device="cuda")
    yb = torch.empty_like(ya)
    yc = torch.empty((128, 56, 56, 64), dtype=torch.float32, device="cuda")

    def chain():
        a.run_nhwc(x, out=ya)
        b.run_nhwc(ya, out=yb)
        c.run_nhwc(yb, out=yc)

    for _ in range(6):
        chain()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(50):
        chain()
    e1.record()
    torch.cuda.synchronize()
    py_us = e0.elapsed_time(e1) / 50 * 1e3
    ctx.sync()
    print("three-layer chain: Launch() kNHWC %.1f us, Launch() kNCHW %.1f us, python runner (channels-last) %.1f us"
          % (float(us["nhwc"]), float(us["nchw"]), py_us))
    # the kNHWC registrations run the same launches as the runner: within 25 % (host-side launch cost only)
    assert float(us["nhwc"]) < 1.25 * py_us + 20.0


def test_adaptor_compiles_against_reference_headers():
    if not os.path.isdir("/root/reference/lite"):
        pytest.skip("reference tree absent")
    subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), "probe", "-j8"], check=True,
                   stdout=subprocess.DEVNULL)
    assert os.path.exists(os.path.join(ROOT, "oracle", "_ref", "obj", "lite_target", "cuda_int8_kernels.o"))
