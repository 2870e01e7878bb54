"""Seeded synthetic inputs and comparison helpers shared by the tests."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402

GOLDEN = os.path.join(ROOT, "tests", "golden", "ref_x86_cases.npz")


def conv_case(seed, n, cin, h, w, cout, k, groups=1, qmax=127, w_std=0.05):
    """Inputs in the style of the benchmark configs: x ~ N(0,1) quantised per tensor,
    weights ~ N(0, w_std) quantised per output channel, bias ~ N(0, 0.1)."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, cin, h, w)).astype(np.float32)
    xq, in_s = O.quantize_per_tensor(x)
    kh, kw = (k, k) if isinstance(k, int) else k
    wf = (rng.standard_normal((cout, cin // groups, kh, kw)) * w_std).astype(np.float32)
    wq, ws = O.quantize_per_channel(wf, qmax=qmax)
    bias = (rng.standard_normal(cout) * 0.1).astype(np.float32)
    return xq, in_s, wq, ws, bias


def fc_case(seed, m, k, n, qmax=127):
    rng = np.random.default_rng(seed)
    x = rng.integers(-127, 128, (m, k), dtype=np.int8)
    wf = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    wq, ws = O.quantize_per_channel(wf, axis=1, qmax=qmax)
    bias = (rng.standard_normal(n) * 0.1).astype(np.float32)
    return x, wq, ws, bias


def assert_i8_close(got, want, max_frac=1e-3):
    """int8 parity rule of the path: no element off by more than 1 LSB and at most
    max_frac of the elements off by exactly 1."""
    d = np.abs(got.astype(np.int32) - want.astype(np.int32))
    assert d.max(initial=0) <= 1, "an int8 output differs by %d LSB" % d.max()
    frac = float((d == 1).mean()) if d.size else 0.0
    assert frac <= max_frac, "%.4f%% of int8 outputs are off by one (limit %.4f%%)" % (100 * frac, 100 * max_frac)


def assert_f32_close(got, want, rel=1e-5, floor=None):
    """fp32 parity rule: |d| <= rel * max(|want|, floor); floor defaults to the largest
    magnitude in `want` times 1e-3 so that cancellation near zero does not dominate."""
    want = np.asarray(want, dtype=np.float64)
    got = np.asarray(got, dtype=np.float64)
    if floor is None:
        floor = max(float(np.abs(want).max(initial=0.0)) * 1e-3, 1e-30)
    tol = rel * np.maximum(np.abs(want), floor)
    bad = np.abs(got - want) > tol
    assert not bad.any(), "%d of %d fp32 outputs outside rel %g (max abs diff %g)" % (
        int(bad.sum()), bad.size, rel, float(np.abs(got - want).max()))


def golden():
    return np.load(GOLDEN)


def golden_names(data, kind):
    names = sorted({k.split("/")[0] for k in data.files})
    return [n for n in names if n.startswith("fc") == (kind == "fc")]
