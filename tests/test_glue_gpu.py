"""Layout staging, calib and pooling kernels against their oracle restatements."""
import numpy as np
import pytest
import torch

from helpers import O, assert_f32_close

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("n,c,h,w,cpad", [(2, 3, 17, 9, 32), (1, 64, 8, 8, 64), (3, 40, 5, 7, 48), (1, 130, 3, 3, 160),
                                          (2, 32, 16, 16, 32), (1, 100, 8, 12, 128), (2, 256, 4, 8, 256),
                                          (3, 3, 16, 16, 32), (1, 128, 56, 56, 128)])
def test_layout_roundtrip(plb, ctx, n, c, h, w, cpad):
    rng = np.random.default_rng(c)
    x = rng.integers(-128, 128, (n, c, h, w), dtype=np.int8)
    y = ctx.nchw_to_nhwc_i8(dev(x), cpad)
    ctx.sync()
    got = y.cpu().numpy()
    assert np.array_equal(got[..., :c], x.transpose(0, 2, 3, 1))
    assert not got[..., c:].any()
    back = ctx.nhwc_to_nchw(y[..., :c].contiguous())
    assert np.array_equal(back.cpu().numpy(), x)
    f = rng.standard_normal((n, h, w, c)).astype(np.float32)
    assert np.array_equal(ctx.nhwc_to_nchw(dev(f)).cpu().numpy(), f.transpose(0, 3, 1, 2))


def test_calib(plb, ctx):
    rng = np.random.default_rng(0)
    x = (rng.standard_normal(100003) * 3).astype(np.float32)
    x[:8] = [-1000.0, -1.5, -0.5, 0.5, 1.5, 2.5, 126.6, 1000.0]
    scale = 0.0371
    q = ctx.calib_f32_to_i8(dev(x), scale).cpu().numpy()
    assert np.array_equal(q, O.calib_f32_to_i8(x, scale))
    y = ctx.calib_i8_to_f32(dev(q), scale).cpu().numpy()
    assert np.array_equal(y, O.calib_i8_to_f32(q, scale))
    img = rng.standard_normal((2, 3, 19, 23)).astype(np.float32)
    got = ctx.calib_nchw_f32_to_nhwc_i8(dev(img), 32, 0.03).cpu().numpy()
    ctx.sync()
    assert np.array_equal(got[..., :3], O.calib_f32_to_i8(img, 0.03).transpose(0, 2, 3, 1))
    assert not got[..., 3:].any()


def test_pooling(plb, ctx):
    rng = np.random.default_rng(1)
    x = rng.integers(-128, 128, (2, 64, 23, 23), dtype=np.int8)
    y = ctx.maxpool_nhwc_i8(dev(x.transpose(0, 2, 3, 1)), 3, 2, 1).cpu().numpy()
    assert np.array_equal(y.transpose(0, 3, 1, 2), O.maxpool_i8(x, 3, 2, 1))
    # other windows (generic kernel), stride 1, and a channel count that is not a multiple of 16
    for xs, k, s, p in ((x, 2, 2, 0), (x, 3, 1, 1), (x[:, :20], 3, 2, 1), (x, 5, 2, 2)):
        y = ctx.maxpool_nhwc_i8(dev(xs.transpose(0, 2, 3, 1)), k, s, p).cpu().numpy()
        assert np.array_equal(y.transpose(0, 3, 1, 2), O.maxpool_i8(np.ascontiguousarray(xs), k, s, p))
    f = rng.standard_normal((3, 7, 7, 96)).astype(np.float32)
    s = np.zeros((3, 96), dtype=np.float32)
    for p in range(49):
        s = s + f.reshape(3, 49, 96)[:, p]
    want = s / np.float32(49)
    avg, q = ctx.global_avgpool_nhwc_f32(dev(f), scale=0.01)
    ctx.sync()
    assert np.array_equal(avg.cpu().numpy(), want)
    assert np.array_equal(q.cpu().numpy(), O.calib_f32_to_i8(want, 0.01))


@pytest.mark.parametrize("rows,cols", [(128, 1000), (3, 7), (2, 5000), (0, 10)])
def test_softmax_rows(plb, ctx, rows, cols):
    """fp32 tolerance of the path: 1e-5 relative (largest output as floor) against the oracle's
    double-precision evaluation of the reference form."""
    rng = np.random.default_rng(rows * 31 + cols)
    x = (rng.standard_normal((rows, cols)) * 6).astype(np.float32)
    if rows > 1:
        x[1, 0] = 150.0
    y = ctx.softmax(torch.from_numpy(x).cuda()).cpu().numpy()
    ctx.sync()
    if rows == 0:
        return
    want = O.softmax(x)
    assert_f32_close(y, want, rel=1e-5, floor=float(want.max()))


def test_copies_follow_the_ctx_stream(plb, ctx):
    """io_copy pair: h2d is ordered before the kernels that follow it on the ctx stream, d2h
    returns with the data."""
    rng = np.random.default_rng(9)
    src = rng.standard_normal(100003).astype(np.float32)
    d = torch.empty(src.size, dtype=torch.float32, device="cuda")
    ctx.copy_h2d(d, src)
    q = ctx.calib_f32_to_i8(d, 0.05)
    back = np.empty(src.size, dtype=np.int8)
    ctx.copy_d2h(back, q)
    assert np.array_equal(back, O.calib_f32_to_i8(src, 0.05))
