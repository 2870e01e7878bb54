"""The oracle against the reference: committed golden vectors (outputs of the reference's
own gemm_s8u8 + im2col objects) and, when they are built, the objects themselves."""
import numpy as np
import pytest

from helpers import (O, assert_f32_close, assert_i8_close, assert_matches_reference_f32, conv_case, fc_case, golden,
                     golden_bench_shapes, golden_names)

DATA = golden()


@pytest.mark.parametrize("name", golden_names(DATA, "conv"))
def test_oracle_matches_golden_conv(name):
    g = {k.split("/")[1]: DATA[k] for k in DATA.files if k.startswith(name + "/")}
    n, cin, h, w, cout, k, s, p, groups, act = [int(v) for v in g["meta"]]
    kw = dict(stride=(s, s), pads=(p, p, p, p), dil=(1, 1), groups=groups)
    y = O.conv_int8(g["x"], g["w"], g["ws"], float(g["in_s"]), g["bias"], act, float(g["alpha"]), **kw)
    # The reference adds a compensated bias (bias - 128*s*sum(A)) to float(acc + 128*sum(A))*s,
    # so its fp32 result carries rounding of values ~128*|sum A| times larger than y.
    assert_f32_close(y, g["y_f32"], rel=1e-5, floor=float(np.abs(g["y_f32"]).max()))
    assert_matches_reference_f32(y, g["y_f32"], name)
    q = O.conv_int8(g["x"], g["w"], g["ws"], float(g["in_s"]), g["bias"], act, float(g["alpha"]),
                    out_scale=float(g["out_s"]), leaky_compat=True, **kw)
    assert_i8_close(q, g["y_i8"])


@pytest.mark.parametrize("name", golden_names(DATA, "fc"))
def test_oracle_matches_golden_fc(name):
    g = {k.split("/")[1]: DATA[k] for k in DATA.files if k.startswith(name + "/")}
    m, k, n, act = [int(v) for v in g["meta"]]
    y = O.fc_int8(g["x"], g["w"], g["ws"], float(g["in_s"]), g["bias"], act, float(g["alpha"]))
    assert_f32_close(y, g["y_f32"], rel=1e-5, floor=float(np.abs(g["y_f32"]).max()))
    assert_matches_reference_f32(y, g["y_f32"], name)
    q = O.fc_int8(g["x"], g["w"], g["ws"], float(g["in_s"]), g["bias"], act, float(g["alpha"]),
                  out_scale=float(g["out_s"]))
    assert_i8_close(q, g["y_i8"])


def test_oracle_matches_golden_bench_shapes():
    """The single-layer benchmark config (1x64x56x56 -> 64, 3x3, pad 1, ReLU) and the (64, 2048, 1000) fc of
    the fc sweep against the committed outputs of the reference objects (weights within +-63)."""
    conv, fc = golden_bench_shapes()
    y = O.conv_int8(conv["x"], conv["w"], conv["ws"], conv["in_s"], conv["bias"], O.ACT_RELU, pads=(1, 1, 1, 1))
    assert_matches_reference_f32(y, conv["y_f32"], "config1")
    q = O.conv_int8(conv["x"], conv["w"], conv["ws"], conv["in_s"], conv["bias"], O.ACT_RELU, pads=(1, 1, 1, 1),
                    out_scale=conv["out_s"])
    assert_i8_close(q, conv["y_i8"])
    y = O.fc_int8(fc["x"], fc["w"], fc["ws"], fc["in_s"], fc["bias"], O.ACT_RELU6, 6.0)
    assert_matches_reference_f32(y, fc["y_f32"], "fc 64x2048x1000")
    q = O.fc_int8(fc["x"], fc["w"], fc["ws"], fc["in_s"], fc["bias"], O.ACT_RELU6, 6.0, out_scale=fc["out_s"])
    assert_i8_close(q, fc["y_i8"])


needs_ref = pytest.mark.skipif(not O.ref_available(), reason="reference objects not built")


@needs_ref
def test_oracle_vs_reference_config1():
    """The single-layer benchmark config (1x64x56x56, 3x3, pad 1, ReLU) with +-63 weights."""
    xq, in_s, wq, ws, bias = conv_case(1001, 1, 64, 56, 56, 64, 3, qmax=63)
    kw = dict(pads=(1, 1, 1, 1))
    y = O.conv_int8(xq, wq, ws, in_s, bias, O.ACT_RELU, **kw)
    yr = O.ref_conv_int8(xq, wq, ws, in_s, bias, O.ACT_RELU, **kw)
    assert_f32_close(y, yr, rel=1e-5, floor=float(np.abs(yr).max()))
    out_s = float(np.abs(y).max() / 127)
    q = O.conv_int8(xq, wq, ws, in_s, bias, O.ACT_RELU, out_scale=out_s, **kw)
    qr = O.ref_conv_int8(xq, wq, ws, in_s, bias, O.ACT_RELU, out_scale=out_s, **kw)
    assert_i8_close(q, qr)


@needs_ref
def test_reference_saturates_full_range_weights():
    """With +-127 weights the reference's vpmaddubsw pair sums saturate and it leaves exact
    arithmetic; this is why parity against it uses +-63 weights."""
    xq, in_s, wq, ws, bias = conv_case(1001, 1, 64, 56, 56, 64, 3, qmax=127)
    y = O.conv_int8(xq, wq, ws, in_s, bias, O.ACT_RELU, pads=(1, 1, 1, 1))
    yr = O.ref_conv_int8(xq, wq, ws, in_s, bias, O.ACT_RELU, pads=(1, 1, 1, 1))
    assert np.abs(y - yr).max() > 1e-2


@needs_ref
@pytest.mark.parametrize("kh,kw,stride,pads,dil", [
    (3, 3, (1, 1), (1, 1, 1, 1), (1, 1)),
    (3, 2, (2, 1), (0, 1, 2, 0), (1, 2)),
    (1, 1, (2, 2), (0, 0, 0, 0), (1, 1)),
    (5, 5, (2, 2), (2, 2, 2, 2), (1, 1)),
    (7, 7, (2, 2), (3, 3, 3, 3), (1, 1)),
])
def test_oracle_index_arithmetic_vs_reference_im2col(kh, kw, stride, pads, dil):
    rng = np.random.default_rng(7)
    x = rng.integers(-127, 128, (5, 13, 17), dtype=np.int8)
    w = rng.integers(-127, 128, (4, 5, kh, kw), dtype=np.int8)
    col = O.ref_im2col(x, kh, kw, stride, pads, dil)
    acc = O.conv_acc_i32(x[None], w, stride, pads, dil)
    want = (w.reshape(4, -1).astype(np.int64) @ col.astype(np.int64)).reshape(acc.shape[1:])
    assert np.array_equal(acc[0], want)


@needs_ref
def test_oracle_vs_reference_fc_and_depthwise():
    x, wq, ws, bias = fc_case(3, 17, 128, 40, qmax=63)
    y = O.fc_int8(x, wq, ws, 0.02, bias, O.ACT_RELU6, 6.0)
    yr = O.ref_fc_int8(x, wq, ws, 0.02, bias, O.ACT_RELU6, 6.0)
    assert_f32_close(y, yr, rel=1e-5, floor=float(np.abs(yr).max()))
    xq, in_s, wq, ws, bias = conv_case(5, 2, 24, 11, 11, 24, 3, groups=24, qmax=63)
    kw = dict(stride=(2, 2), pads=(1, 1, 1, 1), groups=24)
    y = O.conv_int8(xq, wq, ws, in_s, bias, O.ACT_RELU, **kw)
    yr = O.ref_conv_int8(xq, wq, ws, in_s, bias, O.ACT_RELU, **kw)
    assert_f32_close(y, yr, rel=1e-5, floor=float(np.abs(yr).max()))


def test_fc_acc_matches_numpy():
    x, wq, _, _ = fc_case(11, 9, 100, 30)
    assert np.array_equal(O.fc_acc_i32(x, wq), x.astype(np.int64) @ wq.astype(np.int64))


def test_epilogue_rounding_and_clamp():
    acc = np.array([[[-1000, -3, -1, 0, 1, 3, 5, 1000]]], dtype=np.int32).reshape(1, 1, 8)
    # scale 0.5: ties at +-0.5, +-1.5, 2.5 round to even; large values clamp to +-127
    q = O.epilogue(acc, [0.5], 1.0, None, O.ACT_NONE, 0.0, out_scale=1.0)
    assert q.reshape(-1).tolist() == [-127, -2, 0, 0, 0, 2, 2, 127]
    y = O.epilogue(acc, [0.5], 1.0, [1.0], O.ACT_RELU6, 6.0)
    assert y.reshape(-1).tolist() == [0.0, 0.0, 0.5, 1.0, 1.5, 2.5, 3.5, 6.0]


def test_calib_rounding():
    x = np.array([-1000.0, -1.5, -0.5, 0.5, 1.5, 2.5, 126.6, 1000.0], dtype=np.float32)
    assert O.calib_f32_to_i8(x, 1.0).tolist() == [-127, -2, 0, 0, 2, 2, 127, 127]


@pytest.mark.parametrize("dtype", [np.int8, np.float32])
@pytest.mark.parametrize("semi", [False, True])
@pytest.mark.parametrize("m,k", [(7, 12), (8, 16), (1, 5), (5, 1), (64, 109)])
def test_sparse_encode_decode_roundtrip(dtype, semi, m, k):
    """Encoders of sparse_conv_detect_pass.cc:35-301 walked with the ARM start-pointer rule give
    back the dense matrix, including empty channels and an odd channel count."""
    rng = np.random.default_rng(m * 100 + k)
    w = rng.integers(-5, 6, (m, k)).astype(dtype)
    w = (w * (rng.random((m, k)) < 0.3)).astype(dtype)
    if m > 3:
        w[3] = 0
    hw = 6
    enc = O.sparse_encode(w, hw, semi=semi)
    assert np.array_equal(O.sparse_decode(enc, m, k, hw), w)
    if not semi and dtype == np.int8:
        nnz = np.count_nonzero(w, axis=1)
        assert np.array_equal(enc["oc_nonzeros"], np.cumsum(nnz).astype(np.uint32))


def test_sparse_all_zero():
    w = np.zeros((4, 6), dtype=np.int8)
    enc = O.sparse_encode(w, 3)
    assert enc["nonzero_weights"].size == 0 and np.all(enc["oc_nonzeros"] == 0)
    assert np.array_equal(O.sparse_decode(enc, 4, 6, 3), w)


def test_semi_detection_rule():
    """flag_semi iff at least 90 % of the non-zeros sit in filled 2x1 blocks (pass :356)."""
    rng = np.random.default_rng(0)
    mask = rng.random((8, 32)) < 0.2
    w = (rng.integers(1, 5, (16, 32)) * np.repeat(mask, 2, axis=0)).astype(np.int8)
    assert O.sparse_zeros(w)["flag_semi"] == 1
    w2 = (rng.integers(1, 5, (16, 32)) * (rng.random((16, 32)) < 0.2)).astype(np.int8)
    assert O.sparse_zeros(w2)["flag_semi"] == 0


@pytest.mark.parametrize("dtype", [np.int8, np.float32])
@pytest.mark.parametrize("semi", [False, True])
@pytest.mark.parametrize("m,k", [(7, 12), (8, 16), (5, 1), (64, 109)])
def test_numpy_encoder_of_the_package_matches_the_oracle_encoder(dtype, semi, m, k):
    """paddle-lite_b200/sparse_format.py (numpy) and oracle/plb_oracle.c (C) restate the same pass
    independently; they must produce identical tensors."""
    import importlib
    S = importlib.import_module("paddle-lite_b200.sparse_format")
    rng = np.random.default_rng(m * 31 + k)
    w = (rng.integers(-5, 6, (m, k)) * (rng.random((m, k)) < 0.3)).astype(dtype)
    if m > 3:
        w[2] = 0
    a, b = S.encode(w, 6, semi=semi), O.sparse_encode(w, 6, semi=semi)
    assert a["first_ic"] == b["first_ic"] and a["flag_semi"] == b["flag_semi"]
    assert np.array_equal(a["nonzero_weights"], b["nonzero_weights"])
    assert np.array_equal(a["oc_nonzeros"], b["oc_nonzeros"])
    assert np.array_equal(a["diffs"], b["diffs"])


def test_softmax_oracle_matches_numpy():
    rng = np.random.default_rng(5)
    x = (rng.standard_normal((7, 1000)) * 8).astype(np.float32)
    x[3, 10] = 200.0  # everything else in that row is clipped at -64
    y = O.softmax(x)
    d = (x - x.max(axis=1, keepdims=True)).astype(np.float64)  # the shift is a float subtraction, as in the reference
    e = np.exp(np.maximum(d, -64.0))
    want = e / e.sum(axis=1, keepdims=True)
    assert np.allclose(y, want, rtol=1e-6, atol=0)
    assert np.allclose(y.sum(axis=1), 1.0, atol=1e-5)
