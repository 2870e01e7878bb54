"""Depthwise 3x3 + 1x1 convolution in one launch (plb_conv_run_nhwc_dwpw): bit-identical to the oracle's
two-layer sequence  depthwise_conv2d (int8 out) -> conv2d (int8 out)  and to the library's own two launches, for
every tile shape the kernel has, both strides, ragged image sizes and the MobileNetV1 block shapes."""
import numpy as np
import pytest
import torch

from helpers import O, conv_case

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def make_pair(plb, ctx, seed, n, c, h, w, cout, stride, dw_act=1, dw_alpha=0.0, pw_act=1, pw_alpha=0.0, pad=1):
    """A depthwise layer and the 1x1 layer on its output, with the oracle's result of the sequence."""
    xq, in_s, wdw, wsdw, bdw = conv_case(seed, n, c, h, w, c, 3, groups=c, w_std=0.3)
    kw = dict(stride=(stride, stride), pads=(pad, pad, pad, pad), groups=c)
    acc1 = O.conv_acc_i32(xq, wdw, **kw)
    y1 = O.epilogue(acc1, wsdw, in_s, bdw, dw_act, dw_alpha)
    mid_s = float(max(np.abs(y1).max(), 1e-6) / 127.0)
    q1 = O.epilogue(acc1, wsdw, in_s, bdw, dw_act, dw_alpha, out_scale=mid_s)
    rng = np.random.default_rng(seed + 1)
    wf = (rng.standard_normal((cout, c, 1, 1)) * 0.05).astype(np.float32)
    wpw, wspw = O.quantize_per_channel(wf)
    bpw = (rng.standard_normal(cout) * 0.1).astype(np.float32)
    acc2 = O.conv_acc_i32(q1, wpw)
    y2 = O.epilogue(acc2, wspw, mid_s, bpw, pw_act, pw_alpha)
    out_s = float(max(np.abs(y2).max(), 1e-6) / 127.0)
    q2 = O.epilogue(acc2, wspw, mid_s, bpw, pw_act, pw_alpha, out_scale=out_s)
    dw = plb.Conv(ctx, wdw, wsdw, in_s, bdw, in_hw=(h, w), act=dw_act, alpha=dw_alpha, out_scale=mid_s, **kw)
    pw = plb.Conv(ctx, wpw, wspw, mid_s, bpw, in_hw=(dw.ho, dw.wo), act=pw_act, alpha=pw_alpha, out_scale=out_s)
    x = dev(np.ascontiguousarray(xq.transpose(0, 2, 3, 1)))
    return dw, pw, x, q1, q2


def check_pair(plb, ctx, *args, **kw):
    dw, pw, x, q1, q2 = make_pair(plb, ctx, *args, **kw)
    assert dw.dwpw_fusable(pw)
    before = ctx.dwpw_launch_count()
    y = dw.run_nhwc_dwpw(pw, x)
    ctx.sync()
    assert ctx.dwpw_launch_count() == before + 1
    got = y.cpu().numpy().transpose(0, 3, 1, 2)
    assert np.array_equal(got, q2), "fused output differs from the oracle's two-layer sequence (%d of %d)" % (
        int((got != q2).sum()), q2.size)
    # and the library's own two launches give the same bytes
    mid = dw.run_nhwc(x)
    two = pw.run_nhwc(mid)
    ctx.sync()
    assert np.array_equal(mid.cpu().numpy().transpose(0, 3, 1, 2), q1)
    assert torch.equal(two, y)


# (n, c, h, w, cout, stride): every channel count, ragged sizes, images smaller than a tile, several tiles per strip
SHAPES = [
    (2, 32, 20, 20, 64, 1),
    (3, 32, 37, 23, 32, 1),
    (2, 64, 30, 30, 128, 2),
    (2, 64, 17, 40, 64, 1),
    (3, 128, 28, 28, 128, 1),
    (2, 128, 29, 31, 256, 2),
    (2, 256, 14, 14, 256, 1),
    (2, 256, 28, 28, 512, 2),
    (1, 128, 7, 7, 128, 1),
    (5, 256, 9, 5, 64, 1),
]


@pytest.mark.parametrize("shape", SHAPES)
def test_fused_equals_the_two_layer_sequence(plb, ctx, shape):
    n, c, h, w, cout, s = shape
    check_pair(plb, ctx, 100 + c + h, n, c, h, w, cout, s)


FORCED = [(shape, tw, seg)
          for shape in [(3, 128, 40, 36, 128, 1), (2, 256, 33, 18, 128, 2), (4, 64, 45, 45, 64, 1)]
          for tw, seg in [(16, 8), (16, 0), (8, 16), (8, 32), (4, 32), (4, 0)]
          if shape[1] * tw >= 512 and not (tw == 4 and shape[1] < 128)]  # a strip needs at least one warp of threads


@pytest.mark.parametrize("shape,tw,seg", FORCED)
def test_forced_tile_shapes(plb, ctx, shape, tw, seg, monkeypatch):
    """Tile columns and rows per work item forced through the tuning switches: partial last tiles, work items
    with several tiles, the alternating swizzle phase of 4-column tiles, more items than groups."""
    n, c, h, w, cout, s = shape
    monkeypatch.setenv("PLB_DWPW_TW", str(tw))
    if seg:
        monkeypatch.setenv("PLB_DWPW_SEG", str(seg))
    check_pair(plb, ctx, 7 + tw + seg, n, c, h, w, cout, s)


@pytest.mark.parametrize("dw_act,dw_alpha,pw_act,pw_alpha", [(0, 0.0, 0, 0.0), (2, 6.0, 2, 6.0), (1, 0.0, 3, 0.1), (2, 3.0, 1, 0.0)])
def test_activations(plb, ctx, dw_act, dw_alpha, pw_act, pw_alpha):
    check_pair(plb, ctx, 55, 2, 64, 19, 22, 128, 1, dw_act=dw_act, dw_alpha=dw_alpha, pw_act=pw_act, pw_alpha=pw_alpha)


def test_many_images_more_items_than_slots(plb, ctx):
    """More work items than the GPU has depthwise groups: several rounds per CTA, a ragged last round."""
    check_pair(plb, ctx, 77, 70, 32, 24, 24, 64, 1)


@pytest.mark.parametrize("c,cout,hw,stride", [(32, 64, 112, 1), (64, 128, 112, 2), (128, 128, 56, 1), (128, 256, 56, 2),
                                              (256, 256, 28, 1), (256, 512, 28, 2)])
def test_mobilenet_v1_block_shapes(plb, ctx, c, cout, hw, stride):
    """The first six blocks of MobileNetV1 at their real sizes, batch 2, against the oracle's two-layer sequence."""
    dw, pw, x, q1, q2 = make_pair(plb, ctx, 900 + c + hw, 2, c, hw, hw, cout, stride)
    y = dw.run_nhwc_dwpw(pw, x)
    ctx.sync()
    assert np.array_equal(y.cpu().numpy().transpose(0, 3, 1, 2), q2)


def test_pairs_that_do_not_qualify(plb, ctx):
    xq, in_s, wdw, wsdw, bdw = conv_case(5, 1, 48, 10, 10, 48, 3, groups=48, w_std=0.3)
    dw = plb.Conv(ctx, wdw, wsdw, in_s, bdw, in_hw=(10, 10), pads=(1, 1, 1, 1), groups=48, act=1, out_scale=0.05)
    _, _, wpw, wspw, bpw = conv_case(6, 1, 48, 10, 10, 64, 1)
    pw = plb.Conv(ctx, wpw, wspw, 0.05, bpw, in_hw=(10, 10), act=1, out_scale=0.1)
    assert not dw.dwpw_fusable(pw)  # 48 channels
    x = torch.zeros((1, 10, 10, 48), dtype=torch.int8, device="cuda")
    with pytest.raises(plb.PlbError):
        dw.run_nhwc_dwpw(pw, x)
    # a leaky depthwise layer keeps the two-launch path
    xq, in_s, wdw, wsdw, bdw = conv_case(7, 1, 64, 10, 10, 64, 3, groups=64, w_std=0.3)
    dwl = plb.Conv(ctx, wdw, wsdw, in_s, bdw, in_hw=(10, 10), pads=(1, 1, 1, 1), groups=64, act=3, alpha=0.1, out_scale=0.05)
    _, _, wpw, wspw, bpw = conv_case(8, 1, 64, 10, 10, 64, 1)
    pw64 = plb.Conv(ctx, wpw, wspw, 0.05, bpw, in_hw=(10, 10), act=1, out_scale=0.1)
    assert not dwl.dwpw_fusable(pw64)
    # fp32-out 1x1 layer
    pwf = plb.Conv(ctx, wpw, wspw, 0.05, bpw, in_hw=(10, 10), act=1)
    dwr = plb.Conv(ctx, wdw, wsdw, in_s, bdw, in_hw=(10, 10), pads=(1, 1, 1, 1), groups=64, act=1, out_scale=0.05)
    assert not dwr.dwpw_fusable(pwf)
    assert dwr.dwpw_fusable(pw64)
