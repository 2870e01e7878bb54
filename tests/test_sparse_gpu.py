"""sparse_conv2d (1x1) on the GPU over the reference's encoding, checked against the dense
convolution on the densified weights (int8: exact oracle; fp32: the ARM accumulation order)."""
import numpy as np
import pytest
import torch

from helpers import O, assert_f32_close

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def sparse_weights(seed, cout, cin, semi, keep=0.2):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((cout, cin)) * 0.05).astype(np.float32)
    if semi:
        mask = np.repeat(rng.random(((cout + 1) // 2, cin)) < keep, 2, axis=0)[:cout]
    else:
        mask = rng.random((cout, cin)) < keep
    return (w * mask).astype(np.float32)


# cin, cout, hw side, batch
SHAPES = [(32, 64, 12, 2), (128, 128, 14, 2), (256, 256, 7, 3), (109, 33, 5, 1), (512, 512, 7, 1),
          # images of more than 1024 pixels (several blocks of the shared-memory slab kernels, ragged last block),
          # channel counts on each side of the slab kernels' pixels-per-thread thresholds, odd pixel counts
          (24, 40, 36, 1), (48, 16, 34, 2), (100, 20, 33, 1), (150, 8, 36, 1),
          # fp32 pixel-tile kernel: 16 and 8 lanes per output channel (cin > 128, > 256), ragged last tile, cin > 512 (fallback)
          (200, 96, 16, 2), (512, 48, 12, 1), (130, 37, 30, 1), (520, 24, 8, 1)]


@pytest.mark.parametrize("impl", [1, 2, 0], ids=["walk", "densified", "auto"])
@pytest.mark.parametrize("semi", [False, True], ids=["unstructured", "semi"])
@pytest.mark.parametrize("cin,cout,side,batch", SHAPES)
def test_sparse_int8(plb, ctx, cin, cout, side, batch, semi, impl):
    wf = sparse_weights(cin + cout, cout, cin, semi)
    wq, ws = O.quantize_per_channel(wf)
    rng = np.random.default_rng(5)
    xq, in_s = O.quantize_per_tensor(rng.standard_normal((batch, cin, side, side)).astype(np.float32))
    bias = (rng.standard_normal(cout) * 0.1).astype(np.float32)
    enc = O.sparse_encode(wq, side * side, semi=semi)
    assert np.array_equal(O.sparse_decode(enc, cout, cin, side * side), wq)
    acc = O.conv_acc_i32(xq, wq[:, :, None, None])
    y_ref = O.epilogue(acc, ws, in_s, bias, O.ACT_RELU, 0.0)
    out_s = float(np.abs(y_ref).max() / 127)
    q_ref = O.epilogue(acc, ws, in_s, bias, O.ACT_RELU, 0.0, out_scale=out_s)
    args = (enc["nonzero_weights"], enc["oc_nonzeros"], enc["diffs"], enc["first_ic"], enc["flag_semi"])
    kw = dict(cin=cin, cout=cout, in_hw=(side, side), wscale=ws, in_scale=in_s, bias=bias, act=O.ACT_RELU,
              impl=impl)
    x = dev(xq)
    y = plb.SparseConv(ctx, *args, **kw).run(x).cpu().numpy()
    q = plb.SparseConv(ctx, *args, out_scale=out_s, **kw).run(x).cpu().numpy()
    ctx.sync()
    assert np.array_equal(y, y_ref)
    assert np.array_equal(q, q_ref)


@pytest.mark.parametrize("semi", [False, True], ids=["unstructured", "semi"])
@pytest.mark.parametrize("cin,cout,side,batch", SHAPES[:4] + SHAPES[5:])  # (512 x 512 takes the oracle too long)
def test_sparse_fp32(plb, ctx, cin, cout, side, batch, semi):
    wf = sparse_weights(cin * 3 + cout, cout, cin, semi)
    rng = np.random.default_rng(6)
    x = rng.standard_normal((batch, cin, side, side)).astype(np.float32)
    bias = (rng.standard_normal(cout) * 0.1).astype(np.float32)
    enc = O.sparse_encode(wf, side * side, semi=semi)
    y_ref = O.sparse_conv_f32(x, wf, bias, O.ACT_RELU)
    y64 = O.sparse_conv_f32(x, wf, bias, O.ACT_RELU, f64=True)
    sp = plb.SparseConv(ctx, enc["nonzero_weights"], enc["oc_nonzeros"], enc["diffs"], enc["first_ic"],
                        enc["flag_semi"], cin=cin, cout=cout, in_hw=(side, side), bias=bias, act=O.ACT_RELU)
    y = sp.run(dev(x)).cpu().numpy()
    ctx.sync()
    assert np.array_equal(y, y_ref), "fp32 sparse differs from the ordered fma oracle"
    # against fp64: 1e-5 of the output range (single fp32 sums of ~0.2*cin products carry ~1e-7)
    assert_f32_close(y, y64, rel=1e-5, floor=float(np.abs(y64).max()))


# the sparse_conv benchmark shapes: MobileNetV1 pointwise layers at batch 256, 80 % of the weights masked
CONFIG5 = [(32, 64, 112), (128, 128, 56), (256, 256, 28), (512, 512, 14), (1024, 1024, 7)]


@pytest.mark.parametrize("semi", [False, True], ids=["unstructured", "semi"])
@pytest.mark.parametrize("cin,cout,side", CONFIG5)
def test_sparse_int8_benchmark_size(plb, ctx, cin, cout, side, semi):
    """Full benchmark size (batch 256).  The oracle cannot run 2 GOP per case in seconds, so the whole output is
    checked through an exact integer identity and three images are checked element by element:
    * with unit scales, no bias and no activation the fp32 output IS the int32 accumulator (|acc| < 2^24), and
      sum over pixels of acc[n, oc, :] = sum_ic W[oc, ic] * (sum over pixels of x[n, ic, :])  -- exact in int64;
    * images 0, 100 and 255 of the int8-out layer (per-channel scales, bias, ReLU) equal the oracle bit for bit."""
    batch = 256
    hw = side * side
    wf = sparse_weights(7 * cin + cout, cout, cin, semi)
    wq, ws = O.quantize_per_channel(wf)
    enc = O.sparse_encode(wq, hw, semi=semi)
    args = (enc["nonzero_weights"], enc["oc_nonzeros"], enc["diffs"], enc["first_ic"], enc["flag_semi"])
    g = torch.Generator(device="cuda").manual_seed(cin + side)
    x = torch.randint(-127, 128, (batch, cin, side, side), dtype=torch.int8, device="cuda", generator=g)
    # 1. accumulators of the whole batch through the fp32-out kernel
    ident = plb.SparseConv(ctx, *args, cin=cin, cout=cout, in_hw=(side, side), wscale=np.ones(cout, np.float32),
                           in_scale=1.0)
    acc = ident.run(x)
    ctx.sync()
    got = acc.view(batch, cout, hw).to(torch.int64).sum(dim=2).cpu().numpy()
    xsum = x.view(batch, cin, hw).to(torch.int64).sum(dim=2).cpu().numpy()       # [batch, cin]
    want = xsum @ wq.astype(np.int64).T                                          # [batch, cout]
    assert np.array_equal(got, want), "pixel sums of the accumulators break the linear identity"
    del acc
    # 2. int8-out layer, three images against the oracle
    rng = np.random.default_rng(cin)
    bias = (rng.standard_normal(cout) * 0.1).astype(np.float32)
    in_s, out_s = 0.02, 0.06
    q = plb.SparseConv(ctx, *args, cin=cin, cout=cout, in_hw=(side, side), wscale=ws, in_scale=in_s, bias=bias,
                       act=O.ACT_RELU, out_scale=out_s).run(x)
    ctx.sync()
    for n in (0, 100, 255):
        xs = x[n:n + 1].cpu().numpy()
        a = O.conv_acc_i32(xs, wq[:, :, None, None])
        q_ref = O.epilogue(a, ws, in_s, bias, O.ACT_RELU, 0.0, out_scale=out_s)
        assert np.array_equal(q[n:n + 1].cpu().numpy(), q_ref), "image %d differs from the oracle" % n


def test_sparse_errors(plb, ctx):
    wq = np.zeros((4, 8), dtype=np.int8)
    wq[1, 3] = 5
    enc = O.sparse_encode(wq, 4)
    with pytest.raises(plb.PlbError):
        plb.SparseConv(ctx, enc["nonzero_weights"], enc["oc_nonzeros"], enc["diffs"], enc["first_ic"], 0,
                       cin=8, cout=4, in_hw=(2, 2), wscale=np.ones(3, np.float32), in_scale=1.0)
    bad = enc["diffs"].copy()
    bad[:] = 3  # not a multiple of the channel pitch
    with pytest.raises(plb.PlbError):
        plb.SparseConv(ctx, np.array([5, 6], np.int8), np.array([0, 2, 2, 2], np.uint32),
                       np.array([3, 3], np.int32), 3, 0, cin=8, cout=4, in_hw=(2, 2),
                       wscale=np.ones(4, np.float32), in_scale=1.0)
