"""Generates tests/golden/ref_x86_cases.npz.

Run in a container that has the reference tree (so that oracle/_ref/libref_x86.so, the
reference's own gemm_s8u8 + im2col objects, can be built).  Every case stores seeded inputs
together with the OUTPUT OF THE REFERENCE OBJECTS on them; the tests then check the
exact-integer oracle, and through it the CUDA kernels, against these vectors.  Weights stay
within +-63 so that the reference's vpmaddubsw pair sums cannot saturate
(lite/tests/math/x86_gemm_s8u8_compute_test.cc:131 does the same).

A second file, ref_x86_bench_shapes.npz, holds two layers at benchmark size (the single-layer
config 1 x 64 x 56 x 56 -> 64, 3x3, ReLU, and the (64, 2048, 1000) fc of the fc sweep), drawn from
their own seed so that the small cases above keep their values.

Usage: python tests/golden/gen_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402

CASES = [
    # name, N, Cin, H, W, Cout, k, stride, pad, groups, act, alpha
    ("c3x3_relu", 2, 16, 12, 12, 16, 3, 1, 1, 1, O.ACT_RELU, 0.0),
    ("c1x1_none", 1, 32, 9, 9, 24, 1, 1, 0, 1, O.ACT_NONE, 0.0),
    ("c3x3_s2_relu6", 1, 8, 15, 15, 12, 3, 2, 1, 1, O.ACT_RELU6, 6.0),
    ("c1x1_s2_leaky", 2, 16, 10, 10, 8, 1, 2, 0, 1, O.ACT_LEAKY, 0.1),
    ("dw3x3_relu", 1, 16, 14, 14, 16, 3, 1, 1, 16, O.ACT_RELU, 0.0),
    ("dw3x3_s2_relu6", 2, 8, 13, 13, 8, 3, 2, 1, 8, O.ACT_RELU6, 6.0),
    ("g2_3x3", 1, 8, 8, 8, 8, 3, 1, 1, 2, O.ACT_NONE, 0.0),
]
FC_CASES = [("fc_relu", 5, 64, 40, O.ACT_RELU, 0.0), ("fc_relu6", 33, 96, 17, O.ACT_RELU6, 6.0)]


def main():
    if not O.ref_available():
        O.ensure_built(quiet=False)
    out = {}
    rng = np.random.default_rng(20240611)
    for name, n, cin, h, w, cout, k, s, p, g, act, alpha in CASES:
        x = rng.standard_normal((n, cin, h, w)).astype(np.float32)
        xq, in_s = O.quantize_per_tensor(x)
        wf = (rng.standard_normal((cout, cin // g, k, k)) * 0.05).astype(np.float32)
        wq, ws = O.quantize_per_channel(wf, qmax=63)
        bias = (rng.standard_normal(cout) * 0.1).astype(np.float32)
        kw = dict(stride=(s, s), pads=(p, p, p, p), dil=(1, 1), groups=g)
        y = O.ref_conv_int8(xq, wq, ws, in_s, bias, act, alpha, **kw)
        out_s = float(np.abs(y).max() / 127.0)
        q = O.ref_conv_int8(xq, wq, ws, in_s, bias, act, alpha, out_scale=out_s, **kw)
        for key, val in dict(x=xq, w=wq, ws=ws, bias=bias, in_s=np.float32(in_s), out_s=np.float32(out_s),
                             y_f32=y, y_i8=q,
                             meta=np.array([n, cin, h, w, cout, k, s, p, g, act], dtype=np.int32),
                             alpha=np.float32(alpha)).items():
            out["%s/%s" % (name, key)] = val
    for name, m, k, n, act, alpha in FC_CASES:
        xq = rng.integers(-127, 128, (m, k), dtype=np.int8)
        wf = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
        wq, ws = O.quantize_per_channel(wf, axis=1, qmax=63)
        bias = (rng.standard_normal(n) * 0.1).astype(np.float32)
        in_s = 0.02
        y = O.ref_fc_int8(xq, wq, ws, in_s, bias, act, alpha)
        out_s = float(np.abs(y).max() / 127.0)
        q = O.ref_fc_int8(xq, wq, ws, in_s, bias, act, alpha, out_scale=out_s)
        for key, val in dict(x=xq, w=wq, ws=ws, bias=bias, in_s=np.float32(in_s), out_s=np.float32(out_s),
                             y_f32=y, y_i8=q, meta=np.array([m, k, n, act], dtype=np.int32),
                             alpha=np.float32(alpha)).items():
            out["%s/%s" % (name, key)] = val
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_x86_cases.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")
    bench_shapes()


def bench_shapes():
    """Layers at benchmark size.  Inputs are NOT stored (they would be megabytes of noise): the tests
    redraw them with tests/helpers.py conv_case / fc_case from the stored seed and check a stored
    checksum of the inputs first, so a generator that drifted shows up as such."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from helpers import conv_case, fc_case
    out = {}
    seed = 1001
    xq, in_s, wq, ws, bias = conv_case(seed, 1, 64, 56, 56, 64, 3, qmax=63)
    kw = dict(pads=(1, 1, 1, 1))
    y = O.ref_conv_int8(xq, wq, ws, in_s, bias, O.ACT_RELU, 0.0, **kw)
    out_s = float(np.abs(y).max() / 127.0)
    q = O.ref_conv_int8(xq, wq, ws, in_s, bias, O.ACT_RELU, 0.0, out_scale=out_s, **kw)
    out.update({"config1/seed": np.int64(seed), "config1/in_sum": np.int64(xq.astype(np.int64).sum() * 31 + wq.astype(np.int64).sum()),
                "config1/out_s": np.float32(out_s), "config1/y_f32": y, "config1/y_i8": q})
    seed = 1002
    x, wq, ws, bias = fc_case(seed, 64, 2048, 1000, qmax=63)
    y = O.ref_fc_int8(x, wq, ws, 0.02, bias, O.ACT_RELU6, 6.0)
    out_s = float(np.abs(y).max() / 127.0)
    q = O.ref_fc_int8(x, wq, ws, 0.02, bias, O.ACT_RELU6, 6.0, out_scale=out_s)
    out.update({"fc64x2048x1000/seed": np.int64(seed),
                "fc64x2048x1000/in_sum": np.int64(x.astype(np.int64).sum() * 31 + wq.astype(np.int64).sum()),
                "fc64x2048x1000/out_s": np.float32(out_s), "fc64x2048x1000/y_f32": y, "fc64x2048x1000/y_i8": q})
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_x86_bench_shapes.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
