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


@pytest.mark.parametrize("shape", [(2, 32, 20, 20, 32, 3, 1, 1, 32), (2, 64, 15, 15, 64, 3, 2, 1, 64), (1, 16, 12, 12, 24, 3, 1, 1, 4)],
                         ids=["depthwise", "depthwise_s2", "groups4"])
def test_static_scratch_entry_depthwise_and_grouped(plb, shape):
    """The CUDA-core layers (depthwise, grouped) through the same entry, on a context of their own whose
    workspace must stay empty: the entry may not fall back to the ctx allocation."""
    n, cin, h, w, cout, k, s, p, groups = shape
    own = plb.Context(0)
    assert own.workspace_size() == 0
    xq, in_s, wq, ws, bias = conv_case(5151 + cin, n, cin, h, w, cout, k, groups=groups, w_std=0.3)
    kw = dict(stride=(s, s), pads=(p, p, p, p), groups=groups, act=plb.ACT_RELU)
    want = O.conv_int8(xq, wq, ws, in_s, bias, O.ACT_RELU, stride=(s, s), pads=(p, p, p, p), groups=groups)
    out_s = float(np.abs(want).max() / 127)
    want8 = O.conv_int8(xq, wq, ws, in_s, bias, O.ACT_RELU, stride=(s, s), pads=(p, p, p, p), groups=groups,
                        out_scale=out_s)
    x, x2 = dev(xq), dev(np.negative(xq))
    for conv, oracle_out in ((plb.Conv(own, wq, ws, in_s, bias, in_hw=(h, w), **kw), want),
                             (plb.Conv(own, wq, ws, in_s, bias, in_hw=(h, w), out_scale=out_s, **kw), want8)):
        got = torch.empty(oracle_out.shape, dtype=torch.int8 if conv.out_is_i8 else torch.float32, device="cuda")
        got2 = torch.empty_like(got)
        before = own.workspace_size()
        conv.run_static(x, got)
        conv.run_static(x2, got2)
        own.sync()
        assert own.workspace_size() == before, "plb_conv_run_static grew the ctx workspace"
        ref, ref2 = conv.run(x), conv.run(x2)   # the existing entry point (allocates the ctx workspace)
        own.sync()
        assert own.workspace_size() > 0
        assert torch.equal(got, ref) and torch.equal(got2, ref2), "differs from plb_conv_run"
        assert np.array_equal(got.cpu().numpy(), oracle_out), "differs from the oracle"
    own.close()


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
