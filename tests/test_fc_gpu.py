"""Parity of the CUDA fc kernel (plb_fc_*) with the oracle and the reference golden vectors."""
import numpy as np
import pytest
import torch

from helpers import O, assert_f32_close, assert_i8_close, fc_case, golden, golden_names

pytestmark = pytest.mark.gpu
DATA = golden()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("name", golden_names(DATA, "fc"))
def test_golden_vectors(plb, ctx, name):
    g = {k.split("/")[1]: DATA[k] for k in DATA.files if k.startswith(name + "/")}
    m, k, n, act = [int(v) for v in g["meta"]]
    x = dev(g["x"])
    y = plb.Fc(ctx, g["w"], g["ws"], float(g["in_s"]), g["bias"], act, float(g["alpha"])).run(x).cpu().numpy()
    q = plb.Fc(ctx, g["w"], g["ws"], float(g["in_s"]), g["bias"], act, float(g["alpha"]),
               out_scale=float(g["out_s"])).run(x).cpu().numpy()
    ctx.sync()
    assert_f32_close(y, g["y_f32"], rel=1e-5, floor=float(np.abs(g["y_f32"]).max()))
    assert_i8_close(q, g["y_i8"])


# the fc sweep of the benchmark configs plus ragged shapes
@pytest.mark.parametrize("m,k,n", [(1, 1024, 1000), (64, 2048, 1000), (256, 4096, 4096), (7, 96, 17),
                                   (130, 160, 40), (3, 100, 12)])
def test_fc_bit_exact(plb, ctx, m, k, n):
    x, wq, ws, bias = fc_case(m * 7 + n, m, k, n)
    in_s = 0.02
    acc_ref = O.fc_acc_i32(x, wq)
    y_ref = O.epilogue(acc_ref, ws, in_s, bias, O.ACT_RELU6, 6.0)
    out_s = float(max(np.abs(y_ref).max(), 1e-6) / 127)
    q_ref = O.epilogue(acc_ref, ws, in_s, bias, O.ACT_RELU6, 6.0, out_scale=out_s)
    xd = dev(x)
    fc = plb.Fc(ctx, wq, ws, in_s, bias, O.ACT_RELU6, 6.0)
    fc8 = plb.Fc(ctx, wq, ws, in_s, bias, O.ACT_RELU6, 6.0, out_scale=out_s)
    acc = fc.acc_i32(xd).cpu().numpy()
    y = fc.run(xd).cpu().numpy()
    q = fc8.run(xd).cpu().numpy()
    ctx.sync()
    assert np.array_equal(acc, acc_ref)
    assert np.array_equal(y, y_ref)
    assert np.array_equal(q, q_ref)


def test_fc_4096_cubed_checksum(plb, ctx):
    """Largest sweep shape: the oracle would need minutes, so check the column sums instead:
    sum_m acc[m, :] == (sum_m x[m, :]) @ w, exact in int64."""
    x, wq, ws, bias = fc_case(99, 4096, 4096, 4096)
    fc = plb.Fc(ctx, wq, ws, 0.02, bias)
    acc = fc.acc_i32(dev(x))
    ctx.sync()
    got = acc.to(torch.int64).sum(dim=0).cpu().numpy()
    want = x.astype(np.int64).sum(axis=0) @ wq.astype(np.int64)
    assert np.array_equal(got, want)
    rows = [0, 1, 2047, 4095]
    assert np.array_equal(acc[rows].cpu().numpy(), O.fc_acc_i32(x[rows], wq))


def test_golden_fc_sweep_shape(plb, ctx):
    """(M, K, N) = (64, 2048, 1000) of the fc sweep, ReLU6, against the committed output of the reference objects."""
    from helpers import golden_bench_shapes, assert_matches_reference_f32, assert_i8_close
    _, g = golden_bench_shapes()
    x = dev(g["x"])
    y = plb.Fc(ctx, g["w"], g["ws"], g["in_s"], g["bias"], plb.ACT_RELU6, 6.0).run(x).cpu().numpy()
    q = plb.Fc(ctx, g["w"], g["ws"], g["in_s"], g["bias"], plb.ACT_RELU6, 6.0, out_scale=g["out_s"]).run(x).cpu().numpy()
    ctx.sync()
    assert_matches_reference_f32(y, g["y_f32"], "fc 64x2048x1000 (CUDA)")
    assert_i8_close(q, g["y_i8"])
    assert np.array_equal(y, O.fc_int8(g["x"], g["w"], g["ws"], g["in_s"], g["bias"], O.ACT_RELU6, 6.0))


@pytest.mark.parametrize("m,k,n", [(300, 1024, 1000), (64, 2048, 256), (515, 512, 128)])
def test_fc_two_sm_tiles(plb, ctx, m, k, n, monkeypatch):
    """fc as 256-row tiles on pairs of SMs (forced): ragged rows and a ragged last channel tile."""
    monkeypatch.setenv("PLB_TC_PAIR", "1")
    x, wq, ws, bias = fc_case(m + n, m, k, n)
    acc_ref = O.fc_acc_i32(x, wq)
    y_ref = O.epilogue(acc_ref, ws, 0.02, bias, O.ACT_RELU6, 6.0)
    out_s = float(max(np.abs(y_ref).max(), 1e-6) / 127)
    q_ref = O.epilogue(acc_ref, ws, 0.02, bias, O.ACT_RELU6, 6.0, out_scale=out_s)
    xd = dev(x)
    before = ctx.pair_launch_count()
    f32 = plb.Fc(ctx, wq, ws, 0.02, bias, O.ACT_RELU6, 6.0)
    acc = f32.acc_i32(xd).cpu().numpy()
    y = f32.run(xd).cpu().numpy()
    q = plb.Fc(ctx, wq, ws, 0.02, bias, O.ACT_RELU6, 6.0, out_scale=out_s).run(xd).cpu().numpy()
    ctx.sync()
    # (rows of 1000 int8 outputs are not 16-byte multiples: that layer keeps the one-SM kernel)
    assert ctx.pair_launch_count() == before + (3 if n % 16 == 0 else 2)
    assert np.array_equal(acc, acc_ref)
    assert np.array_equal(y, y_ref)
    assert np.array_equal(q, q_ref)


def test_fc_errors(plb, ctx):
    x, wq, ws, bias = fc_case(1, 4, 64, 8)
    with pytest.raises(plb.PlbError):
        plb.Fc(ctx, wq, ws[:3], 0.02, bias)
    fc = plb.Fc(ctx, wq, ws, 0.02, bias)
    assert fc.run(torch.empty((0, 64), dtype=torch.int8, device="cuda")).shape == (0, 8)


@pytest.mark.parametrize("k,below", [(256, True), (288, False)])
def test_extreme_accumulators(plb, ctx, k, below):
    """Largest possible accumulators, on both sides of 2^22 (where float spacing is still below 1)
    and beyond: all weights +-127, inputs -128 / 127.  k = 256: |acc| <= 4 161 536; k = 288: 4 681 728."""
    m, n = 64, 64
    w = np.where(np.arange(n)[None, :] % 2 == 0, 127, -127).astype(np.int8) * np.ones((k, 1), np.int8)
    x = np.where(np.arange(m)[:, None] % 2 == 0, -128, 127).astype(np.int8) * np.ones((1, k), np.int8)
    x[5, ::3] = 0
    ws = np.full(n, 1e-6, np.float32)
    bias = np.linspace(-1, 1, n).astype(np.float32)
    acc_ref = O.fc_acc_i32(x, w)
    assert (np.abs(acc_ref).max() < 2 ** 22) == below
    y_ref = O.epilogue(acc_ref, ws, 0.5, bias, O.ACT_NONE, 0.0)
    q_ref = O.epilogue(acc_ref, ws, 0.5, bias, O.ACT_NONE, 0.0, out_scale=0.02)
    xd = dev(x)
    y = plb.Fc(ctx, w, ws, 0.5, bias).run(xd).cpu().numpy()
    q = plb.Fc(ctx, w, ws, 0.5, bias, out_scale=0.02).run(xd).cpu().numpy()
    ctx.sync()
    assert np.array_equal(y, y_ref)
    assert np.array_equal(q, q_ref)


def _random_fc(count, seed):
    rng = np.random.default_rng(seed)
    return [(int(rng.integers(1, 300)), int(rng.choice([32, 64, 96, 100, 160, 256, 512, 1000])),
             int(rng.choice([8, 17, 40, 80, 96, 160, 250, 320, 1000]))) for _ in range(count)]


@pytest.mark.parametrize("m,k,n", _random_fc(16, 77))
def test_random_fc_shapes(plb, ctx, m, k, n):
    x, wq, ws, bias = fc_case(m + k + n, m, k, n)
    acc_ref = O.fc_acc_i32(x, wq)
    y_ref = O.epilogue(acc_ref, ws, 0.02, bias, O.ACT_RELU, 0.0)
    out_s = float(max(np.abs(y_ref).max(), 1e-6) / 127)
    q_ref = O.epilogue(acc_ref, ws, 0.02, bias, O.ACT_RELU, 0.0, out_scale=out_s)
    xd = dev(x)
    y = plb.Fc(ctx, wq, ws, 0.02, bias, O.ACT_RELU).run(xd).cpu().numpy()
    q = plb.Fc(ctx, wq, ws, 0.02, bias, O.ACT_RELU, out_scale=out_s).run(xd).cpu().numpy()
    ctx.sync()
    assert np.array_equal(y, y_ref)
    assert np.array_equal(q, q_ref)
