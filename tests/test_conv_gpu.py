"""Parity of the CUDA conv2d / depthwise_conv2d kernels with the exact-integer oracle and the
reference golden vectors, called through the C ABI (plb_conv_*)."""
import numpy as np
import pytest
import torch

from helpers import O, assert_f32_close, assert_i8_close, conv_case, golden, golden_names

pytestmark = pytest.mark.gpu
DATA = golden()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def run_case(plb, ctx, xq, in_s, wq, ws, bias, *, stride=(1, 1), pads=(0, 0, 0, 0), dil=(1, 1), groups=1,
             act=0, alpha=0.0, impl=0, check_i8=True, leaky_compat=False):
    """Runs accumulators, fp32-out and int8-out through the ABI and checks all three against the oracle."""
    kw = dict(stride=stride, pads=pads, dil=dil, groups=groups)
    acc_ref = O.conv_acc_i32(xq, wq, **kw)
    y_ref = O.epilogue(acc_ref, ws, in_s, bias, act, alpha)
    x = dev(xq)
    conv = plb.Conv(ctx, wq, ws, in_s, bias, in_hw=xq.shape[2:], act=act, alpha=alpha, impl=impl, **kw)
    acc = conv.acc_i32(x)
    y = conv.run(x)
    ctx.sync()
    assert np.array_equal(acc.cpu().numpy(), acc_ref), "int32 accumulators differ (%d of %d)" % (
        int((acc.cpu().numpy() != acc_ref).sum()), acc_ref.size)
    assert np.array_equal(y.cpu().numpy(), y_ref), "fp32 outputs are not bit-identical to the oracle"
    if check_i8:
        out_s = float(max(np.abs(y_ref).max(), 1e-6) / 127.0)
        q_ref = O.epilogue(acc_ref, ws, in_s, bias, act, alpha, out_scale=out_s, leaky_compat=leaky_compat)
        conv8 = plb.Conv(ctx, wq, ws, in_s, bias, in_hw=xq.shape[2:], act=act, alpha=alpha, impl=impl,
                         out_scale=out_s, leaky_compat=leaky_compat, **kw)
        q = conv8.run(x)
        ctx.sync()
        assert np.array_equal(q.cpu().numpy(), q_ref), "int8 outputs are not bit-identical to the oracle"
    return y_ref


@pytest.mark.parametrize("impl", [1, 0], ids=["direct", "auto"])
@pytest.mark.parametrize("name", golden_names(DATA, "conv"))
def test_golden_vectors(plb, ctx, name, impl):
    """Outputs of the reference's own x86 objects (committed fixtures): fp32 within 1e-5 of the
    largest output, int8 within 1 LSB on at most 0.1 % of the elements."""
    g = {k.split("/")[1]: DATA[k] for k in DATA.files if k.startswith(name + "/")}
    n, cin, h, w, cout, k, s, p, groups, act = [int(v) for v in g["meta"]]
    kw = dict(stride=(s, s), pads=(p, p, p, p), groups=groups, act=act, alpha=float(g["alpha"]), impl=impl)
    x = dev(g["x"])
    conv = plb.Conv(ctx, g["w"], g["ws"], float(g["in_s"]), g["bias"], in_hw=(h, w), **kw)
    y = conv.run(x).cpu().numpy()
    conv8 = plb.Conv(ctx, g["w"], g["ws"], float(g["in_s"]), g["bias"], in_hw=(h, w),
                     out_scale=float(g["out_s"]), leaky_compat=True, **kw)
    q = conv8.run(x).cpu().numpy()
    ctx.sync()
    assert_f32_close(y, g["y_f32"], rel=1e-5, floor=float(np.abs(g["y_f32"]).max()))
    assert_i8_close(q, g["y_i8"])


# (n, cin, h, w, cout, k, stride, pad, act, alpha)
DENSE_CASES = [
    (1, 64, 56, 56, 64, 3, 1, 1, 1, 0.0),      # the single-layer benchmark config
    (2, 64, 14, 14, 256, 1, 1, 0, 1, 0.0),     # pointwise, flat GEMM path
    (3, 128, 28, 28, 128, 3, 2, 1, 1, 0.0),    # strided 3x3
    (2, 256, 14, 14, 512, 1, 2, 0, 0, 0.0),    # strided 1x1 (downsample)
    (2, 3, 32, 32, 32, 7, 2, 3, 1, 0.0),       # stem: 3 input channels, 7x7
    (1, 32, 9, 11, 48, 3, 1, 1, 2, 6.0),       # odd sizes, relu6, cout not a multiple of 32
    (5, 96, 7, 7, 24, 1, 1, 0, 3, 0.1),        # leaky, ragged tile tails
    (1, 512, 7, 7, 512, 3, 1, 1, 1, 0.0),      # long K
    (1, 40, 6, 6, 20, 3, 1, 0, 0, 0.0),        # cin, cout not multiples of 16/32
]


@pytest.mark.parametrize("impl", [1, 0], ids=["direct", "auto"])
@pytest.mark.parametrize("case", DENSE_CASES, ids=lambda c: "x".join(map(str, c[:8])))
def test_dense_conv_bit_exact(plb, ctx, case, impl):
    n, cin, h, w, cout, k, s, p, act, alpha = case
    xq, in_s, wq, ws, bias = conv_case(hash(case) % 10000, n, cin, h, w, cout, k)
    run_case(plb, ctx, xq, in_s, wq, ws, bias, stride=(s, s), pads=(p, p, p, p), act=act, alpha=alpha,
             impl=impl)


# (n, cin, h, w, cout, k, pads, dil, act)
WINDOW_CASES = [
    (2, 64, 56, 56, 64, 3, (1, 1, 1, 1), (1, 1), 1),      # the 3x3 layers of the first residual stage
    (3, 128, 14, 14, 32, 3, (1, 1, 1, 1), (1, 1), 1),     # 128-byte rows, image smaller than a tile
    (1, 96, 12, 19, 64, 3, (1, 1, 1, 1), (1, 1), 0),      # three 32-byte channel chunks, ragged tiles
    (2, 64, 20, 13, 32, (3, 2), (0, 1, 2, 0), (2, 1), 2),  # asymmetric padding, dilation, 3x2 filter
    (1, 32, 17, 23, 64, 5, (2, 2, 2, 2), (1, 1), 3),      # 5x5
    (1, 40, 9, 9, 32, 3, (0, 0, 0, 0), (1, 1), 0),        # no padding, channels padded to 64
]

# stride-1 filters that are too large to stay in shared memory (or need several channel tiles): im2col mode
LARGE_FILTER_CASES = [
    (2, 128, 28, 28, 128, 3, (1, 1, 1, 1), (1, 1), 1),
    (1, 256, 14, 14, 256, 3, (1, 1, 1, 1), (1, 1), 1),    # two channel chunks, 256-wide tile
    (1, 64, 20, 20, 320, 3, (1, 1, 1, 1), (1, 1), 2),     # ragged second channel tile (64 of 256)
    (1, 32, 12, 12, 320, (2, 3), (1, 0, 1, 1), (1, 1), 0),
    (24, 128, 28, 28, 128, 3, (1, 1, 1, 1), (1, 1), 1),   # 192 tiles on 148 CTAs
    (41, 64, 14, 14, 512, 3, (1, 1, 1, 1), (1, 1), 0),    # two channel tiles, odd tile counts per CTA
]


@pytest.mark.parametrize("case", WINDOW_CASES, ids=lambda c: "x".join(map(str, c[:5])))
def test_window_mode_bit_exact(plb, ctx, case, monkeypatch):
    """Stride-1 filters in window mode (one fetch of a tile's input window, taps addressed by
    shifted matrix descriptors), forced on for shapes the heuristic would leave to im2col."""
    monkeypatch.setenv("PLB_TC_SLAB", "1")
    monkeypatch.setenv("PLB_TC_BN", "256")  # one channel tile even though the problem is small
    n, cin, h, w, cout, k, pads, dil, act = case
    xq, in_s, wq, ws, bias = conv_case(hash(case[:5]) % 10000, n, cin, h, w, cout, k)
    before = ctx.window_launch_count()
    run_case(plb, ctx, xq, in_s, wq, ws, bias, pads=pads, dil=dil, act=act, alpha=6.0 if act == 2 else 0.1)
    assert ctx.window_launch_count() >= before + 3, "window mode was not taken"


@pytest.mark.parametrize("case", LARGE_FILTER_CASES, ids=lambda c: "x".join(map(str, c[:5])))
def test_large_filter_bit_exact(plb, ctx, case, monkeypatch):
    """The same kind of layer with a filter that cannot stay resident: streamed through the operand ring."""
    monkeypatch.setenv("PLB_TC_BN", "256")
    n, cin, h, w, cout, k, pads, dil, act = case
    xq, in_s, wq, ws, bias = conv_case(hash(case[:5]) % 10000, n, cin, h, w, cout, k)
    run_case(plb, ctx, xq, in_s, wq, ws, bias, pads=pads, dil=dil, act=act, alpha=6.0 if act == 2 else 0.1)


# (n, cin, h, w, cout, act): unpadded stride-1 1x1 layers whose images have a multiple of 16 pixels
NCHW_1X1_CASES = [
    (2, 32, 112, 112, 64, 1),     # first MobileNetV1 pointwise shape: one K step, 64 of 128 accumulator lanes used
    (3, 128, 28, 28, 128, 1),     # 784 pixels: three full 256-pixel tiles and a 16-pixel one
    (2, 256, 28, 28, 256, 2),     # two channel tiles, two K steps of 128
    (1, 40, 8, 8, 24, 0),         # input channels padded to 64, 64 pixels, ragged channels
    (2, 64, 20, 20, 200, 3),      # ragged second channel tile
    (5, 1024, 4, 4, 1024, 1),     # long K, 16 pixels per image
    (1, 96, 16, 24, 32, 1),       # three K steps of 32
    (150, 64, 16, 16, 64, 1),     # more tiles than SMs: filter resident in shared memory, several tiles per CTA
    (40, 512, 12, 12, 256, 1),    # streamed filter, several tiles per CTA
    # pixel counts that are not multiples of 16: TMA cannot address the rows
    (2, 512, 14, 14, 512, 1),     # 196 pixels (4-byte aligned rows)
    (3, 1024, 7, 7, 1024, 1),     # 49 pixels (rows at any byte alignment)
    (2, 64, 9, 9, 32, 2),         # 81 pixels
    (1, 40, 5, 7, 24, 3),         # 35 pixels, ragged channels
    (7, 32, 1, 1, 16, 0),         # one pixel per image
]
# more of those, for the kernel whose operand tiles are filled by gather warps (4-byte copies, or aligned loads + funnel
# shifts for rows of odd length)
NCHW_GATHER_CASES = [c for c in NCHW_1X1_CASES if (c[2] * c[3]) % 16] + [
    (300, 64, 6, 6, 64, 1),       # 36 pixels -> 48 columns, five images per tile, more tiles than SMs, filter resident,
                                  # duplicated accumulator rows
    (37, 128, 14, 14, 160, 2),    # one image per tile (208 columns), ragged second channel tile
    (9, 96, 10, 10, 128, 1),      # 100 pixels -> 112 columns, two images per tile, odd image count
    (3, 64, 17, 17, 96, 3),       # 289 pixels: two tiles per image, rows at every byte alignment
    (300, 64, 7, 7, 64, 1),       # 49 pixels -> 64 columns, four images per tile, duplicated accumulator rows
    (170, 1024, 7, 7, 256, 1),    # long K: two images per tile so that the pixel tile stays resident
    (2, 160, 18, 18, 64, 1),      # 324 pixels: two tiles per image
    (170, 1024, 6, 6, 256, 1),    # streamed filter, long K, several stages of copies in flight
    (5, 64, 6, 14, 96, 0),        # 84 pixels -> 96 columns, two images per tile, odd image count
    (330, 128, 10, 10, 256, 1),   # more pixel tiles than SMs: several resident pixel tiles per CTA, chunks handed back
                                  # only after the last channel-tile pass
]


@pytest.mark.parametrize("case", NCHW_1X1_CASES, ids=lambda c: "x".join(map(str, c[:5])))
def test_nchw_native_1x1(plb, ctx, case, monkeypatch):
    """1x1 layers through the NCHW entry point run on the NCHW tensors directly (output channels in the
    accumulator lanes, pixels in its columns); accumulators, fp32 and int8 outputs bit-identical to the oracle."""
    monkeypatch.setenv("PLB_TC_NCHW", "1")  # also for images of fewer than 100 pixels, which default to the staged path
    n, cin, h, w, cout, act = case
    xq, in_s, wq, ws, bias = conv_case(hash(case) % 10000, n, cin, h, w, cout, 1)
    before = ctx.nchw_launch_count()
    run_case(plb, ctx, xq, in_s, wq, ws, bias, act=act, alpha=6.0 if act == 2 else 0.1)
    assert ctx.nchw_launch_count() == before + 3, "the NCHW-native kernel was not taken"


@pytest.mark.parametrize("case", NCHW_GATHER_CASES, ids=lambda c: "x".join(map(str, c[:5])))
@pytest.mark.parametrize("gather", ["resident", "streamed", "0"])
def test_nchw_images_tma_cannot_address(plb, ctx, case, gather, monkeypatch):
    """Images whose pixel count is not a multiple of 16: gather warps fill the operand tiles and the epilogue writes the
    rows itself -- with a pixel tile kept in shared memory for all channel tiles ("resident", where it fits) or gathered
    per channel tile ("streamed") -- or the rows are re-pitched around the TMA kernel ("0"); all bit-identical to the oracle."""
    monkeypatch.setenv("PLB_TC_NCHW", "1")
    monkeypatch.setenv("PLB_TC_NCHW_BRES", "1" if gather == "resident" else "0")
    gather = "0" if gather == "0" else "1"
    monkeypatch.setenv("PLB_TC_NCHW_GATHER", gather)
    n, cin, h, w, cout, act = case
    xq, in_s, wq, ws, bias = conv_case(hash(case) % 10000 + 1, n, cin, h, w, cout, 1)
    before, before_g = ctx.nchw_launch_count(), ctx.nchw_gather_launch_count()
    run_case(plb, ctx, xq, in_s, wq, ws, bias, act=act, alpha=6.0 if act == 2 else 0.1)
    assert ctx.nchw_launch_count() == before + 3
    assert ctx.nchw_gather_launch_count() == before_g + (3 if gather == "1" else 0)


def test_nchw_native_switch_off(plb, ctx, monkeypatch):
    monkeypatch.setenv("PLB_TC_NCHW", "0")
    xq, in_s, wq, ws, bias = conv_case(3, 2, 64, 16, 16, 64, 1)
    before = ctx.nchw_launch_count()
    run_case(plb, ctx, xq, in_s, wq, ws, bias, act=1)
    assert ctx.nchw_launch_count() == before


# (n, cin, h, w, cout, k, stride, pad, act)
PAIR_CASES = [
    (4, 128, 28, 28, 128, 3, 1, 1, 1),    # 13 pair tiles of 256 pixels, the last one ragged
    (8, 256, 14, 14, 256, 3, 1, 1, 1),    # 256-wide channel tile: each CTA holds 128 filter rows
    (2, 512, 28, 28, 256, 1, 1, 0, 2),    # flat GEMM, four K steps of 128
    (5, 512, 7, 7, 512, 3, 1, 1, 0),      # 245 rows: the follower CTA of the only row tile has no valid row; two channel tiles
    (2, 64, 56, 56, 64, 3, 1, 1, 3),      # 64-channel tile (32 filter rows per CTA), K steps of 64
    (3, 128, 30, 30, 128, 3, 2, 1, 1),    # strided
    (150, 128, 8, 8, 320, 3, 1, 1, 1),    # more tiles than pairs: several tiles per pair, ragged second channel tile
    (1, 96, 20, 20, 64, 3, 1, 1, 1),      # three channel chunks of 32 per tap
]


@pytest.mark.parametrize("case", PAIR_CASES, ids=lambda c: "x".join(map(str, c[:7])))
def test_two_sm_tiles_bit_exact(plb, ctx, case, monkeypatch):
    """256 x N output tiles on pairs of SMs (tcgen05.mma.cta_group::2, each CTA holding its 128 rows of A and half of
    the filter tile), forced on for shapes of every kind: accumulators, fp32 and int8 outputs against the oracle."""
    monkeypatch.setenv("PLB_TC_PAIR", "1")
    monkeypatch.setenv("PLB_TC_NCHW", "0")  # 1x1 layers through the channels-last kernels, where the pair tiles live
    n, cin, h, w, cout, k, s, p, act = case
    xq, in_s, wq, ws, bias = conv_case(hash(case) % 10000, n, cin, h, w, cout, k)
    before = ctx.pair_launch_count()
    run_case(plb, ctx, xq, in_s, wq, ws, bias, stride=(s, s), pads=(p, p, p, p), act=act, alpha=6.0 if act == 2 else 0.1)
    assert ctx.pair_launch_count() == before + 3, "the two-SM kernel was not taken"
    ctx.sync()


def test_golden_config1_shape(plb, ctx):
    """The single-layer benchmark config (1 x 64 x 56 x 56 -> 64, 3x3, pad 1, ReLU) against the committed output of
    the reference objects, through the NCHW entry point; and bit-identical to the oracle."""
    from helpers import golden_bench_shapes, assert_matches_reference_f32
    g, _ = golden_bench_shapes()
    x = dev(g["x"])
    kw = dict(in_hw=(56, 56), pads=(1, 1, 1, 1), act=plb.ACT_RELU)
    y = plb.Conv(ctx, g["w"], g["ws"], g["in_s"], g["bias"], **kw).run(x).cpu().numpy()
    q = plb.Conv(ctx, g["w"], g["ws"], g["in_s"], g["bias"], out_scale=g["out_s"], **kw).run(x).cpu().numpy()
    ctx.sync()
    assert_matches_reference_f32(y, g["y_f32"], "config1 (CUDA)")
    assert_i8_close(q, g["y_i8"])
    assert np.array_equal(y, O.conv_int8(g["x"], g["w"], g["ws"], g["in_s"], g["bias"], O.ACT_RELU, pads=(1, 1, 1, 1)))


def test_plan_is_reused(plb, ctx):
    """A prepared layer stores the tile plan and tensor maps of the (batch, pointers) it has run on: the second run
    with the same buffers re-launches it (and gives the same bytes), other buffers or batches get plans of their own."""
    xq, in_s, wq, ws, bias = conv_case(99, 4, 64, 28, 28, 96, 3)
    conv = plb.Conv(ctx, wq, ws, in_s, bias, in_hw=(28, 28), pads=(1, 1, 1, 1), act=plb.ACT_RELU, out_scale=0.05)
    x = ctx.nchw_to_nhwc_i8(dev(xq))
    y = torch.empty((4, 28, 28, 96), dtype=torch.int8, device="cuda")
    conv.run_nhwc(x, out=y)
    first = y.clone()
    h0 = conv.plan_cache_hits()
    y.zero_()
    conv.run_nhwc(x, out=y)
    assert conv.plan_cache_hits() == h0 + 1
    assert torch.equal(y, first)
    y2 = torch.empty_like(y)
    conv.run_nhwc(x, out=y2)                 # another output buffer: a new plan, same result
    assert conv.plan_cache_hits() == h0 + 1
    assert torch.equal(y2, first)
    conv.run_nhwc(x[:2], out=y2[:2])         # another batch
    assert conv.plan_cache_hits() == h0 + 1
    for _ in range(12):                      # more distinct problems than the cache holds, then the first one again
        conv.run_nhwc(x, out=torch.empty_like(y))
    y.zero_()
    conv.run_nhwc(x, out=y)
    ctx.sync()
    assert torch.equal(y, first)
    want = O.conv_int8(xq, wq, ws, in_s, bias, O.ACT_RELU, pads=(1, 1, 1, 1), out_scale=0.05)
    assert np.array_equal(ctx.nhwc_to_nchw(y).cpu().numpy(), want)


def test_asymmetric_pad_dilation(plb, ctx):
    xq, in_s, wq, ws, bias = conv_case(77, 2, 32, 13, 10, 32, (3, 2))
    for impl in (1, 0):
        run_case(plb, ctx, xq, in_s, wq, ws, bias, stride=(2, 1), pads=(0, 1, 2, 0), dil=(1, 2), act=1,
                 impl=impl)


# (n, c, h, w, k, stride, pad, act, alpha)
DW_CASES = [
    (2, 32, 112, 112, 3, 1, 1, 1, 0.0),
    (2, 64, 56, 56, 3, 2, 1, 1, 0.0),
    (1, 512, 14, 14, 3, 1, 1, 2, 6.0),
    (3, 24, 9, 9, 3, 2, 1, 0, 0.0),   # channels not a multiple of 16
    (1, 1024, 7, 7, 3, 1, 1, 1, 0.0),
    (1, 16, 10, 10, 5, 1, 2, 3, 0.2),
]


@pytest.mark.parametrize("case", DW_CASES, ids=lambda c: "x".join(map(str, c[:7])))
def test_depthwise_bit_exact(plb, ctx, case):
    n, c, h, w, k, s, p, act, alpha = case
    xq, in_s, wq, ws, bias = conv_case(hash(case) % 10000, n, c, h, w, c, k, groups=c, w_std=0.3)
    run_case(plb, ctx, xq, in_s, wq, ws, bias, stride=(s, s), pads=(p, p, p, p), groups=c, act=act,
             alpha=alpha)


def test_grouped_conv(plb, ctx):
    xq, in_s, wq, ws, bias = conv_case(9, 2, 32, 12, 12, 48, 3, groups=4)
    run_case(plb, ctx, xq, in_s, wq, ws, bias, pads=(1, 1, 1, 1), groups=4, act=1)


def test_scalar_weight_scale_and_no_bias(plb, ctx):
    xq, in_s, wq, ws, _ = conv_case(10, 1, 32, 8, 8, 32, 1)
    run_case(plb, ctx, xq, in_s, wq, ws[:1], None, act=1)


def test_leaky_compat_switch(plb, ctx):
    xq, in_s, wq, ws, bias = conv_case(12, 1, 32, 8, 8, 32, 3)
    run_case(plb, ctx, xq, in_s, wq, ws, bias, pads=(1, 1, 1, 1), act=3, alpha=0.1, leaky_compat=True)
    run_case(plb, ctx, xq, in_s, wq, ws, bias, pads=(1, 1, 1, 1), act=3, alpha=0.1, leaky_compat=False)


def test_batch_zero_and_rerun(plb, ctx):
    xq, in_s, wq, ws, bias = conv_case(13, 4, 32, 8, 8, 32, 3)
    conv = plb.Conv(ctx, wq, ws, in_s, bias, in_hw=(8, 8), pads=(1, 1, 1, 1), act=1)
    empty = torch.empty((0, 32, 8, 8), dtype=torch.int8, device="cuda")
    assert conv.run(empty).shape[0] == 0
    want = O.conv_int8(xq, wq, ws, in_s, bias, O.ACT_RELU, pads=(1, 1, 1, 1))
    for nb in (4, 1, 3):  # batch changes between runs of one prepared layer
        y = conv.run(dev(xq[:nb])).cpu().numpy()
        assert np.array_equal(y, want[:nb])
    ctx.sync()


def test_prepare_errors(plb, ctx):
    xq, in_s, wq, ws, bias = conv_case(14, 1, 32, 8, 8, 32, 3)
    with pytest.raises(plb.PlbError) as e:  # conv_compute.cc:242-244
        plb.Conv(ctx, wq, ws[:5], in_s, bias, in_hw=(8, 8))
    assert e.value.code == plb.E_INVALID
    with pytest.raises(plb.PlbError):
        plb.Conv(ctx, wq, ws, in_s, bias, in_hw=(1, 1))  # empty output
    with pytest.raises(plb.PlbError):
        plb.Conv(ctx, wq, ws, in_s, bias, in_hw=(8, 8), act=7)
    with pytest.raises(plb.PlbError):
        plb.Conv(ctx, wq, ws, -1.0, bias, in_hw=(8, 8))


@pytest.mark.parametrize("prefetch", ["0", "1"])
def test_nhwc_entry_and_fused_add_relu(plb, ctx, prefetch, monkeypatch):
    """Channels-last entry points: same values as the NCHW path; the fused conv + add + relu +
    calib equals the unfused oracle sequence bit for bit, with the residual tiles fetched in
    step with the chunks or one chunk ahead."""
    monkeypatch.setenv("PLB_TC_RES_PREFETCH", prefetch)
    xq, in_s, wq, ws, bias = conv_case(15, 3, 64, 14, 14, 128, 1)
    acc = O.conv_acc_i32(xq, wq)
    y_ref = O.epilogue(acc, ws, in_s, bias, O.ACT_NONE, 0.0)
    rng = np.random.default_rng(3)
    res = rng.standard_normal(y_ref.shape).astype(np.float32)
    s_ref = np.maximum(y_ref + res, np.float32(0))
    next_s = float(np.abs(s_ref).max() / 127)
    q_ref = O.calib_f32_to_i8(s_ref, next_s)
    x_nhwc = dev(np.ascontiguousarray(xq.transpose(0, 2, 3, 1)))
    conv = plb.Conv(ctx, wq, ws, in_s, bias, in_hw=(14, 14))
    y = conv.run_nhwc(x_nhwc).cpu().numpy().transpose(0, 3, 1, 2)
    assert np.array_equal(y, y_ref)
    yf, yq = conv.run_nhwc_add_relu(x_nhwc, dev(np.ascontiguousarray(res.transpose(0, 2, 3, 1))), next_s)
    ctx.sync()
    assert np.array_equal(yf.cpu().numpy().transpose(0, 3, 1, 2), s_ref)
    assert np.array_equal(yq.cpu().numpy().transpose(0, 3, 1, 2), q_ref)


@pytest.mark.parametrize("n,cin_m,cin_s,hw,cout,stride", [(3, 64, 64, 14, 256, 1), (2, 128, 256, 28, 512, 2),
                                                         (5, 32, 96, 9, 64, 2), (1, 256, 512, 7, 320, 1)])
@pytest.mark.parametrize("generic_loops", ["0", "1"])
def test_block_add_relu_equals_the_unfused_sequence(plb, ctx, n, cin_m, cin_s, hw, cout, stride, generic_loops, monkeypatch):
    """Projection-block tail in one launch: relu(main 1x1 conv + strided 1x1 shortcut conv) and its
    calib, bit-identical to conv(fp32_out), conv(fp32_out), add, relu, calib through the oracle;
    through the short role loops and through the generic ones."""
    if generic_loops == "1":
        monkeypatch.setenv("PLB_TC_FAST_DUAL", "0")
    hs = hw * stride - (stride - 1) * (n % 2)  # shortcut input: even and odd sizes
    xm, in_m, wm, wsm, bm = conv_case(31 + cout, n, cin_m, hw, hw, cout, 1)
    xs, in_s, wsh, wss, bs = conv_case(32 + cout, n, cin_s, hs, hs, cout, 1)
    y_main = O.epilogue(O.conv_acc_i32(xm, wm), wsm, in_m, bm, O.ACT_NONE, 0.0)
    y_short = O.epilogue(O.conv_acc_i32(xs, wsh, stride=(stride, stride)), wss, in_s, bs, O.ACT_NONE, 0.0)
    assert y_short.shape == y_main.shape
    s_ref = np.maximum(y_main + y_short, np.float32(0))
    next_s = float(np.abs(s_ref).max() / 127)
    q_ref = O.calib_f32_to_i8(s_ref, next_s)
    main = plb.Conv(ctx, wm, wsm, in_m, bm, in_hw=(hw, hw))
    short = plb.Conv(ctx, wsh, wss, in_s, bs, in_hw=(hs, hs), stride=(stride, stride))
    nhwc = lambda a: dev(np.ascontiguousarray(a.transpose(0, 2, 3, 1)))  # noqa: E731
    yf, yq = main.run_nhwc_block_add_relu(nhwc(xm), short, nhwc(xs), next_s)
    ctx.sync()
    assert np.array_equal(yf.cpu().numpy().transpose(0, 3, 1, 2), s_ref)
    assert np.array_equal(yq.cpu().numpy().transpose(0, 3, 1, 2), q_ref)
    _, yq2 = main.run_nhwc_block_add_relu(nhwc(xm), short, nhwc(xs), next_s, want_f32=False)
    ctx.sync()
    assert np.array_equal(yq2.cpu().numpy().transpose(0, 3, 1, 2), q_ref)


def test_window_mode_fused_add_relu(plb, ctx, monkeypatch):
    """conv3x3 + residual add + relu + calib in window mode: residual tiles and both outputs move
    through the four-dimensional tensor maps."""
    monkeypatch.setenv("PLB_TC_SLAB", "1")
    monkeypatch.setenv("PLB_TC_BN", "256")
    xq, in_s, wq, ws, bias = conv_case(21, 2, 64, 21, 18, 64, 3)
    acc = O.conv_acc_i32(xq, wq, pads=(1, 1, 1, 1))
    y_ref = O.epilogue(acc, ws, in_s, bias, O.ACT_NONE, 0.0)
    rng = np.random.default_rng(4)
    res = rng.standard_normal(y_ref.shape).astype(np.float32)
    s_ref = np.maximum(y_ref + res, np.float32(0))
    next_s = float(np.abs(s_ref).max() / 127)
    q_ref = O.calib_f32_to_i8(s_ref, next_s)
    x_nhwc = dev(np.ascontiguousarray(xq.transpose(0, 2, 3, 1)))
    conv = plb.Conv(ctx, wq, ws, in_s, bias, in_hw=(21, 18), pads=(1, 1, 1, 1))
    before = ctx.window_launch_count()
    yf, yq = conv.run_nhwc_add_relu(x_nhwc, dev(np.ascontiguousarray(res.transpose(0, 2, 3, 1))), next_s)
    ctx.sync()
    assert ctx.window_launch_count() == before + 1
    assert np.array_equal(yf.cpu().numpy().transpose(0, 3, 1, 2), s_ref)
    assert np.array_equal(yq.cpu().numpy().transpose(0, 3, 1, 2), q_ref)


@pytest.mark.parametrize("cin,k,s,p,hw", [(3, 7, 2, 3, (37, 41)), (3, 3, 2, 1, (37, 41)), (4, 5, 1, 2, (37, 41)),
                                          (16, 3, 1, 1, (37, 41)), (3, 7, 2, 3, (64, 48)), (3, 3, 2, 1, (50, 32)),
                                          (3, 7, 2, 3, (224, 224))])
def test_image_entry(plb, ctx, cin, k, s, p, hw):
    """fp32 NCHW image -> calib -> first layer, channels-last output; stems with cin*kw <= 32 take
    the row-folded staging (pre-swizzled and fed by bulk copies when the output width is a
    multiple of 8, as in the last three cases), (16,3,1,1) the plain one."""
    rng = np.random.default_rng(cin * 10 + k)
    img = rng.standard_normal((3, cin) + hw).astype(np.float32)
    in_s = float(np.abs(img).max() / 127)
    wq, ws = O.quantize_per_channel((rng.standard_normal((64, cin, k, k)) * 0.1).astype(np.float32))
    bias = (rng.standard_normal(64) * 0.1).astype(np.float32)
    xq = O.calib_f32_to_i8(img, in_s)
    kw = dict(stride=(s, s), pads=(p, p, p, p))
    y_ref = O.conv_int8(xq, wq, ws, in_s, bias, O.ACT_RELU, **kw)
    out_s = float(np.abs(y_ref).max() / 127)
    q_ref = O.conv_int8(xq, wq, ws, in_s, bias, O.ACT_RELU, out_scale=out_s, **kw)
    conv = plb.Conv(ctx, wq, ws, in_s, bias, in_hw=hw, act=1, out_scale=out_s, **kw)
    got = conv.run_image_f32(dev(img)).cpu().numpy().transpose(0, 3, 1, 2)
    got_nchw = conv.run(dev(xq)).cpu().numpy()
    ctx.sync()
    assert np.array_equal(got, q_ref)
    assert np.array_equal(got_nchw, q_ref)


@pytest.mark.parametrize("k,s,p,cout,hw,n,act,alpha", [
    (7, 2, 3, 64, (224, 224), 3, 1, 0.0),    # the ResNet-50 stem
    (3, 2, 1, 32, (224, 224), 5, 1, 0.0),    # the MobileNetV1 stem
    (7, 2, 3, 64, (128, 256), 2, 2, 6.0),    # one output row = one tile
    (7, 2, 3, 32, (96, 64), 4, 0, 0.0),      # four output rows per item, 32-pixel rows
    (3, 2, 1, 64, (160, 224), 150, 3, 0.1),  # more work items than SMs: several items per CTA, ragged last round
    (4, 2, 1, 32, (64, 128), 3, 1, 0.0),     # 4x4: all four 16-byte windows of a pixel carry filter taps
    (3, 2, 1, 32, (96, 64), 4, 2, 6.0),      # 16-byte windows, four output rows per item
    (8, 2, 3, 64, (64, 128), 2, 1, 0.0),     # 8x8: all eight 32-byte windows carry filter taps
])
def test_one_launch_stem(plb, ctx, k, s, p, cout, hw, n, act, alpha, monkeypatch):
    """First layer from the fp32 image in one launch (calib, row folding and GEMM operand never reach memory):
    bit-identical to the oracle and to the staged path it replaces."""
    rng = np.random.default_rng(k * 100 + cout + hw[0])
    img = rng.standard_normal((n, 3) + hw).astype(np.float32)
    img[0, :, :3, :5] *= 40.0  # values far outside the quantiser's range saturate
    in_s = float(np.abs(img[1:]).max() / 127) if n > 1 else 0.03
    wq, ws = O.quantize_per_channel((rng.standard_normal((cout, 3, k, k)) * 0.1).astype(np.float32))
    bias = (rng.standard_normal(cout) * 0.1).astype(np.float32)
    kw = dict(stride=(s, s), pads=(p, p, p, p))
    small = slice(0, min(n, 3))
    xq = O.calib_f32_to_i8(img[small], in_s)
    y_ref = O.conv_int8(xq, wq, ws, in_s, bias, act, alpha, **kw)
    out_s = float(np.abs(y_ref).max() / 127)
    q_ref = O.conv_int8(xq, wq, ws, in_s, bias, act, alpha, out_scale=out_s, leaky_compat=True, **kw)
    conv = plb.Conv(ctx, wq, ws, in_s, bias, in_hw=hw, act=act, alpha=alpha, out_scale=out_s, leaky_compat=True, **kw)
    before = ctx.stem_launch_count()
    got = conv.run_image_f32(dev(img))
    ctx.sync()
    assert ctx.stem_launch_count() == before + 1
    assert np.array_equal(got[small].cpu().numpy().transpose(0, 3, 1, 2), q_ref)
    monkeypatch.setenv("PLB_STEM", "0")
    staged = plb.Conv(ctx, wq, ws, in_s, bias, in_hw=hw, act=act, alpha=alpha, out_scale=out_s, leaky_compat=True, **kw)
    want = staged.run_image_f32(dev(img))
    ctx.sync()
    assert ctx.stem_launch_count() == before + 1
    assert torch.equal(got, want)


def test_linearity_at_full_size(plb, ctx):
    """Size-independent property at benchmark scale (batch 32 of the 64->64 3x3 layer):
    accumulators are linear in the input, acc(x1) + acc(x2) == acc(x1 + x2) for inputs whose sum
    stays in int8 range."""
    rng = np.random.default_rng(21)
    x1 = rng.integers(-60, 61, (32, 64, 56, 56), dtype=np.int8)
    x2 = rng.integers(-60, 61, (32, 64, 56, 56), dtype=np.int8)
    wq = rng.integers(-127, 128, (64, 64, 3, 3), dtype=np.int8)
    conv = plb.Conv(ctx, wq, [0.01], 0.02, None, in_hw=(56, 56), pads=(1, 1, 1, 1))
    a1 = conv.acc_i32(dev(x1))
    a2 = conv.acc_i32(dev(x2))
    a3 = conv.acc_i32(dev((x1 + x2).astype(np.int8)))
    ctx.sync()
    assert torch.equal(a1 + a2, a3)
    # spot-check one image against the oracle
    assert np.array_equal(a3[5:6].cpu().numpy(), O.conv_acc_i32((x1 + x2)[5:6], wq, pads=(1, 1, 1, 1)))


def _random_cases(count, seed):
    rng = np.random.default_rng(seed)
    cases = []
    while len(cases) < count:
        k = (int(rng.choice([1, 1, 2, 3, 3, 5])), int(rng.choice([1, 1, 2, 3, 3, 5])))
        s = (int(rng.choice([1, 1, 2])), int(rng.choice([1, 1, 2])))
        dil = (int(rng.choice([1, 1, 2])), int(rng.choice([1, 1, 2])))
        pads = tuple(int(v) for v in rng.integers(0, 3, 4))
        n = int(rng.integers(1, 5))
        cin = int(rng.choice([3, 16, 32, 40, 64, 96, 128]))
        cout = int(rng.choice([8, 24, 32, 64, 72, 128, 160, 256]))
        h, w = int(rng.integers(5, 30)), int(rng.integers(5, 30))
        ho = (h + pads[0] + pads[1] - dil[0] * (k[0] - 1) - 1) // s[0] + 1
        wo = (w + pads[2] + pads[3] - dil[1] * (k[1] - 1) - 1) // s[1] + 1
        if ho < 1 or wo < 1:
            continue
        cases.append((n, cin, h, w, cout, k, s, pads, dil, int(rng.integers(0, 4))))
    return cases


@pytest.mark.parametrize("force_window", ["0", "1"])
@pytest.mark.parametrize("case", _random_cases(24, 2024), ids=lambda c: "n%dc%dh%dw%do%dk%dx%d" % (c[:5] + c[5]))
def test_random_geometries(plb, ctx, case, force_window, monkeypatch):
    """Seeded random geometries (filter size, stride, dilation, asymmetric padding, ragged channel
    counts, every activation) through accumulators, fp32-out and int8-out, once with the default
    choice of operand mode and once with window mode forced wherever it applies."""
    if force_window == "1":
        monkeypatch.setenv("PLB_TC_SLAB", "1")
    n, cin, h, w, cout, k, s, pads, dil, act = case
    xq, in_s, wq, ws, bias = conv_case(hash(case[:5]) % 10000, n, cin, h, w, cout, k)
    run_case(plb, ctx, xq, in_s, wq, ws, bias, stride=s, pads=pads, dil=dil, act=act,
             alpha=6.0 if act == 2 else 0.1)


def _random_dw(count, seed):
    rng = np.random.default_rng(seed)
    out = []
    for _ in range(count):
        k = int(rng.choice([3, 3, 3, 5]))
        out.append((int(rng.integers(1, 4)), int(rng.choice([4, 8, 24, 32, 64, 100, 128])), int(rng.integers(4, 40)),
                    int(rng.integers(4, 40)), k, int(rng.choice([1, 2])), int(rng.integers(0, k // 2 + 2)),
                    int(rng.integers(0, 4))))
    return out


@pytest.mark.parametrize("case", _random_dw(16, 5), ids=lambda c: "n%dc%dh%dw%dk%ds%dp%da%d" % c)
def test_random_depthwise(plb, ctx, case):
    n, c, h, w, k, s, p, act = case
    if (h + 2 * p - k) // s + 1 < 1 or (w + 2 * p - k) // s + 1 < 1:
        pytest.skip("empty output")
    xq, in_s, wq, ws, bias = conv_case(hash(case) % 10000, n, c, h, w, c, k, groups=c, w_std=0.3)
    run_case(plb, ctx, xq, in_s, wq, ws, bias, stride=(s, s), pads=(p, p, p, p), groups=c, act=act,
             alpha=6.0 if act == 2 else 0.1)


@pytest.mark.parametrize("strip", ["0", "1", "3", "4", "7", "32"])
@pytest.mark.parametrize("shape", [(2, 32, 13, 17, 1, 1, 1), (1, 64, 29, 9, 2, 1, 2), (3, 8, 7, 7, 1, 0, 3),
                                   (1, 128, 14, 14, 2, 1, 0), (1, 24, 5, 33, 1, 2, 1)],
                         ids=lambda s: "n%dc%dh%dw%ds%dp%da%d" % s)
def test_depthwise_strip_heights(plb, ctx, shape, strip, monkeypatch):
    """Depthwise 3x3 through the column-strip kernel with forced strip heights (ragged last strip,
    strips shorter than the filter, one strip for the whole image) and through the register-tiled
    kernel it replaced ("0"): all bit-identical to the oracle."""
    monkeypatch.setenv("PLB_DW_STRIP", strip)
    n, c, h, w, s, p, act = shape
    xq, in_s, wq, ws, bias = conv_case(4242 + h * w + c, n, c, h, w, c, 3, groups=c, w_std=0.3)
    run_case(plb, ctx, xq, in_s, wq, ws, bias, stride=(s, s), pads=(p, p, p, p), groups=c, act=act,
             alpha=6.0 if act == 2 else 0.1)


@pytest.mark.parametrize("act,alpha", [(0, 0.0), (1, 0.0), (2, 6.0), (2, 1e9), (2, -3.0), (3, 0.1), (3, -2.5)])
def test_requantiser_extremes(plb, ctx, act, alpha):
    """int8 outputs whose pre-clamp values leave the range in which the rounding add is exact
    (|v| up to 2^27 through a large scale), for every activation, odd ReLU6 bounds included; the
    tensor-core path (1x1, 64 channels: small-accumulator conversion) and the depthwise path."""
    rng = np.random.default_rng(17)
    for groups, cin, k in ((1, 64, 1), (64, 64, 3)):
        xq = rng.integers(-127, 128, (2, cin, 9, 11), dtype=np.int8)
        wq = rng.integers(-127, 128, (64, cin // groups, k, k), dtype=np.int8)
        ws = np.full(64, 1.0, np.float32)
        ws[::3] = 1e-4
        bias = rng.standard_normal(64).astype(np.float32) * 100
        kw = dict(stride=(1, 1), pads=(k // 2,) * 4, groups=groups)
        acc_ref = O.conv_acc_i32(xq, wq, **kw)
        for out_s in (1.0, 1e-3, 37.5):
            q_ref = O.epilogue(acc_ref, ws, 0.5, bias, act, alpha, out_scale=out_s)
            conv8 = plb.Conv(ctx, wq, ws, 0.5, bias, in_hw=xq.shape[2:], act=act, alpha=alpha, out_scale=out_s, **kw)
            q = conv8.run(dev(xq))
            ctx.sync()
            assert np.array_equal(q.cpu().numpy(), q_ref), "groups %d out_scale %g" % (groups, out_s)


_FLAT_CASES = {}


def _flat_case(cin, cout):
    """Inputs and oracle bytes of one shape, computed once for all switch settings."""
    if (cin, cout) not in _FLAT_CASES:
        xq, in_s, wq, ws, bias = conv_case(77 + cin + cout, 4, cin, 224, 224, cout, 1)
        acc_ref = O.conv_acc_i32(xq, wq)
        y_ref = O.epilogue(acc_ref, ws, in_s, bias, 1, 0.0)
        out_s = float(max(np.abs(y_ref).max(), 1e-6) / 127.0)
        _FLAT_CASES[(cin, cout)] = (xq, in_s, wq, ws, bias, out_s, O.epilogue(acc_ref, ws, in_s, bias, 1, 0.0, out_scale=out_s))
    return _FLAT_CASES[(cin, cout)]


@pytest.mark.parametrize("env", [{}, {"PLB_TC_FAST_FLAT": "0"}, {"PLB_TC_ACC_BUFS": "8"},
                                 {"PLB_TC_ACC_BUFS": "8", "PLB_TC_FAST_FLAT": "0"}, {"PLB_TC_SB_SMEM": "0", "PLB_TC_ACC_SMALL": "0"}],
                         ids=lambda e: ",".join("%s=%s" % kv for kv in e.items()) or "default")
@pytest.mark.parametrize("cin,cout", [(32, 64), (256, 64), (64, 32)])
def test_flat_tiles_many_per_cta(plb, ctx, cin, cout, env, monkeypatch):
    """1x1 convolutions with a resident filter and ten tiles per CTA, so that the operand ring wraps
    and every accumulator buffer is reused: the short role loops, the generic ones, eight
    accumulator buffers, and the epilogue without its shared-memory tables and without the
    small-accumulator conversion all give the oracle's bytes."""
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    xq, in_s, wq, ws, bias, out_s, q_ref = _flat_case(cin, cout)
    conv8 = plb.Conv(ctx, wq, ws, in_s, bias, in_hw=(224, 224), act=1, out_scale=out_s)
    q = conv8.run(dev(xq))
    ctx.sync()
    assert np.array_equal(q.cpu().numpy(), q_ref)


_IM2COL_CASE = {}


@pytest.mark.parametrize("env", [{}, {"PLB_TC_FAST_IM2COL": "0"}, {"PLB_TC_FAST_MMA": "0"},
                                 {"PLB_TC_FAST_IM2COL": "0", "PLB_TC_FAST_MMA": "0"}],
                         ids=lambda e: ",".join("%s=%s" % kv for kv in e.items()) or "default")
def test_im2col_role_loops_agree(plb, ctx, env, monkeypatch):
    """A strided 3x3 convolution (im2col tiles, streamed filter, two channel tiles, several tiles
    per CTA) through the lean and the generic producer / MMA loops: the oracle's bytes each time."""
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    monkeypatch.setenv("PLB_TC_BN", "64")
    if not _IM2COL_CASE:
        xq, in_s, wq, ws, bias = conv_case(4711, 8, 64, 112, 112, 128, 3)
        kw = dict(stride=(2, 2), pads=(1, 1, 1, 1))
        acc_ref = O.conv_acc_i32(xq, wq, **kw)
        y_ref = O.epilogue(acc_ref, ws, in_s, bias, 1, 0.0)
        out_s = float(max(np.abs(y_ref).max(), 1e-6) / 127.0)
        _IM2COL_CASE["c"] = (xq, in_s, wq, ws, bias, kw, out_s, O.epilogue(acc_ref, ws, in_s, bias, 1, 0.0, out_scale=out_s))
    xq, in_s, wq, ws, bias, kw, out_s, q_ref = _IM2COL_CASE["c"]
    conv8 = plb.Conv(ctx, wq, ws, in_s, bias, in_hw=(112, 112), act=1, out_scale=out_s, **kw)
    q = conv8.run(dev(xq))
    ctx.sync()
    assert np.array_equal(q.cpu().numpy(), q_ref)
