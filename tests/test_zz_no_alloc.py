"""plb_conv_run_static: the conv2d entry point for callers that cannot let the library allocate
device memory (its layout staging sits in a fixed 8 MiB array inside the library instead of a
cudaMalloc'ed workspace).  Called through the C ABI twice in a row and compared with
plb_conv_run; the file name makes pytest collect it last."""
import ctypes as C

import numpy as np
import pytest
import torch

from helpers import O, conv_case

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("shape", [(2, 64, 28, 28, 64, 3, 1, 1), (3, 3, 40, 40, 32, 7, 2, 3), (1, 40, 9, 9, 24, 1, 1, 0)],
                         ids=["3x3", "stem7x7", "ragged1x1"])
def test_static_scratch_entry_matches_plb_conv_run(plb, ctx, shape):
    n, cin, h, w, cout, k, s, p = shape
    xq, in_s, wq, ws, bias = conv_case(4242 + cin, n, cin, h, w, cout, k)
    kw = dict(stride=(s, s), pads=(p, p, p, p), act=plb.ACT_RELU)
    want = O.conv_int8(xq, wq, ws, in_s, bias, O.ACT_RELU, stride=(s, s), pads=(p, p, p, p))
    out_s = float(np.abs(want).max() / 127)
    want8 = O.conv_int8(xq, wq, ws, in_s, bias, O.ACT_RELU, stride=(s, s), pads=(p, p, p, p), out_scale=out_s)
    for conv, oracle_out in ((plb.Conv(ctx, wq, ws, in_s, bias, in_hw=(h, w), **kw), want),
                             (plb.Conv(ctx, wq, ws, in_s, bias, in_hw=(h, w), out_scale=out_s, **kw), want8)):
        x = dev(xq)
        ref = conv.run(x)                     # the existing entry point (ctx workspace)
        x2 = dev(np.negative(xq))             # a second, different input for the second call
        ref2 = conv.run(x2)
        got = torch.empty_like(ref)
        got2 = torch.empty_like(ref)
        conv.run_static(x, got)               # two calls in a row share the built-in scratch
        conv.run_static(x2, got2)
        ctx.sync()
        assert torch.equal(got, ref), "first call differs from plb_conv_run"
        assert torch.equal(got2, ref2), "second call differs from plb_conv_run"
        assert np.array_equal(got.cpu().numpy(), oracle_out), "differs from the oracle"


def test_static_scratch_entry_rejects_oversize(plb, ctx):
    xq, in_s, wq, ws, bias = conv_case(7, 1, 64, 56, 56, 64, 3)
    conv = plb.Conv(ctx, wq, ws, in_s, bias, in_hw=(56, 56), pads=(1, 1, 1, 1))
    batch = 16  # 16 x (64*56*56 int8 + 64*56*56 fp32) = 16 MB of staging > 8 MiB
    assert conv.workspace_bytes(batch) > 8 << 20
    x = torch.zeros((batch, 64, 56, 56), dtype=torch.int8, device="cuda")
    y = torch.zeros((batch, 64, 56, 56), dtype=torch.float32, device="cuda")
    with pytest.raises(plb.PlbError) as e:
        conv.run_static(x, y)
    assert e.value.code == plb.E_INVALID
    assert "8388608" in str(e.value) and "staging" in str(e.value)
    ctx.sync()
    assert not y.any(), "a rejected call must not launch anything"
