#!/usr/bin/env python
"""Per-layer timing of the library's kernels (one prepared layer, inputs resident in HBM).

    python paddle-lite_b200/layer_bench.py conv   --cin 64 --hw 56 --cout 64 --k 3 --pad 1 --batch 128 [--out i8|f32|addrelu]
    python paddle-lite_b200/layer_bench.py dw     --cin 32 --hw 112 --stride 1 --batch 128
    python paddle-lite_b200/layer_bench.py block  --cin 64 --cin2 64 --hw 56 --cout 256 --stride 1 --batch 128   # projection-block tail
    python paddle-lite_b200/layer_bench.py fc     --m 4096 --kdim 4096 --n 4096 [--out i8|f32]
    python paddle-lite_b200/layer_bench.py sparse --cin 128 --cout 128 --hw 56 --batch 256 [--fp32] [--semi] [--impl walk|dense]
    python paddle-lite_b200/layer_bench.py fc-sweep | sparse-sweep      # the shapes of the benchmark configs
    python paddle-lite_b200/layer_bench.py int8-peak                    # library int8 GEMM (cuBLASLt via torch._int_mm) as a measured denominator

Prints one JSON line per layer: microseconds per launch (CUDA events on the launching stream,
after a warm-up that also brings the clocks up), algorithmic bytes and operations, and the
achieved fractions of the measured HBM bandwidth and of the dense int8 tensor peak.  Used as
the target command of the ncu captures summarised under profiles/ (`--iters` keeps those short).
"""
import argparse
import importlib
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

INT8_PEAK_TOPS = 4500.0  # dense int8 datasheet figure (2 x bf16); not measured on this pool


def hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def time_launches(fn, iters, warm_seconds):
    import torch
    t0 = time.time()
    fn()
    torch.cuda.synchronize()
    while time.time() - t0 < warm_seconds:
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3


def report(name, us, nbytes, ops, extra=None):
    peak, kind = hbm_peak()
    line = {"layer": name, "us": round(us, 2), "bytes": int(nbytes), "ops": int(ops),
            "GBps": round(nbytes / us / 1e3, 1), "TOPS": round(ops / us / 1e6, 1),
            "hbm_frac": round(nbytes / us / 1e3 / peak, 3), "hbm_peak": "%s %.1f GB/s" % (kind, peak),
            "tensor_frac_of_4.5POPS": round(ops / us / 1e6 / INT8_PEAK_TOPS, 3)}
    if extra:
        line.update(extra)
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kind", choices=["conv", "dw", "block", "fc", "sparse", "fc-sweep", "sparse-sweep", "int8-peak"])
    ap.add_argument("--cin2", type=int, default=64, help="block: input channels of the shortcut conv")
    ap.add_argument("--cin", type=int, default=64)
    ap.add_argument("--cout", type=int, default=64)
    ap.add_argument("--hw", type=int, default=56)
    ap.add_argument("--k", type=int, default=1)
    ap.add_argument("--stride", type=int, default=1)
    ap.add_argument("--pad", type=int, default=0)
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--kdim", type=int, default=4096, help="K of the fc layer")
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--out", default="i8", choices=["i8", "f32", "addrelu"])
    ap.add_argument("--fp32", action="store_true")
    ap.add_argument("--semi", action="store_true")
    ap.add_argument("--impl", default="walk", choices=["walk", "dense"])
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--warm", type=float, default=0.3, help="seconds of warm-up launches")
    args = ap.parse_args()

    import torch
    plb = importlib.import_module("paddle-lite_b200")
    ctx = plb.Context(0)
    rng = np.random.default_rng(1)

    def conv_layer(cin, hw, cout, k, stride, pad, batch, out, groups=1):
        w = rng.integers(-127, 128, (cout, cin // groups, k, k), dtype=np.int8)
        x = torch.randint(-127, 128, (batch, hw, hw, cin), dtype=torch.int8, device="cuda")
        kw = dict(in_hw=(hw, hw), stride=(stride, stride), pads=(pad,) * 4, groups=groups)
        if out == "addrelu":
            conv = plb.Conv(ctx, w, [0.001], 0.02, None, **kw)
            shape = (batch, conv.ho, conv.wo, cout)
            res = torch.randn(shape, device="cuda")
            yf = torch.empty(shape, device="cuda")
            yq = torch.empty(shape, dtype=torch.int8, device="cuda")
            fn = lambda: conv.run_nhwc_add_relu(x, res, 0.05, out_f32=yf, out_i8=yq)  # noqa: E731
            out_bytes = yq.numel() * 9
        else:
            conv = plb.Conv(ctx, w, [0.001], 0.02, None, act=plb.ACT_RELU,
                            out_scale=0.05 if out == "i8" else None, **kw)
            y = torch.empty((batch, conv.ho, conv.wo, cout), dtype=torch.int8 if out == "i8" else torch.float32,
                            device="cuda")
            fn = lambda: conv.run_nhwc(x, out=y)  # noqa: E731
            out_bytes = y.numel() * y.element_size()
        us = time_launches(fn, args.iters, args.warm)
        ops = 2.0 * batch * conv.ho * conv.wo * cout * (cin // groups) * k * k
        name = "%s cin%d %dx%d cout%d k%d s%d b%d %s" % ("dw" if groups > 1 else "conv", cin, hw, hw, cout, k, stride,
                                                        batch, out)
        report(name, us, x.numel() + w.size + out_bytes, ops)
        ctx.sync()

    def fc_layer(m, k, n, out):
        w = rng.integers(-127, 128, (k, n), dtype=np.int8)
        x = torch.randint(-127, 128, (m, k), dtype=torch.int8, device="cuda")
        fc = plb.Fc(ctx, w, [0.0001], 0.02, np.zeros(n, np.float32), plb.ACT_RELU6, 6.0,
                    out_scale=0.05 if out == "i8" else None)
        y = torch.empty((m, n), dtype=torch.int8 if out == "i8" else torch.float32, device="cuda")
        us = time_launches(lambda: fc.run(x, out=y), args.iters, args.warm)
        report("fc m%d k%d n%d %s" % (m, k, n, out), us, m * k + k * n + y.numel() * y.element_size() + 8 * n,
               2.0 * m * k * n)
        ctx.sync()

    def sparse_layer(cin, cout, hw, batch, fp32, semi, impl):
        S = importlib.import_module("paddle-lite_b200.sparse_format")
        wf = (rng.standard_normal((cout, cin)) * 0.05).astype(np.float32)
        if semi:
            mask = np.repeat(rng.random(((cout + 1) // 2, cin)) < 0.2, 2, axis=0)[:cout]
        else:
            mask = rng.random((cout, cin)) < 0.2
        wf = (wf * mask).astype(np.float32)
        if fp32:
            enc = S.encode(wf, hw * hw, semi=semi)
            x = torch.randn((batch, cin, hw, hw), device="cuda")
            sp = plb.SparseConv(ctx, enc["nonzero_weights"], enc["oc_nonzeros"], enc["diffs"], enc["first_ic"],
                                enc["flag_semi"], cin=cin, cout=cout, in_hw=(hw, hw), act=plb.ACT_RELU)
            y = torch.empty((batch, cout, hw, hw), device="cuda")
            esz = 4
        else:
            wq, ws = S.quantize_per_channel(wf)
            enc = S.encode(wq, hw * hw, semi=semi)
            x = torch.randint(-127, 128, (batch, cin, hw, hw), dtype=torch.int8, device="cuda")
            sp = plb.SparseConv(ctx, enc["nonzero_weights"], enc["oc_nonzeros"], enc["diffs"], enc["first_ic"],
                                enc["flag_semi"], cin=cin, cout=cout, in_hw=(hw, hw), wscale=ws, in_scale=0.02,
                                act=plb.ACT_RELU, out_scale=0.05,
                                impl=plb.IMPL_TC if impl == "dense" else plb.IMPL_DIRECT)
            y = torch.empty((batch, cout, hw, hw), dtype=torch.int8, device="cuda")
            esz = 1
        nnz = int(np.count_nonzero(wf))
        us = time_launches(lambda: sp.run(x, out=y), args.iters, args.warm)
        nbytes = batch * hw * hw * (cin + cout) * esz + nnz * (esz + 4) + 4 * cout
        report("sparse %s %s cin%d cout%d %dx%d b%d %s" % ("fp32" if fp32 else "int8", "semi" if semi else "unstr", cin,
                                                           cout, hw, hw, batch, impl), us, nbytes,
               2.0 * nnz * hw * hw * batch, {"nnz": nnz})
        ctx.sync()

    if args.kind == "int8-peak":
        # not a kernel of this library: the vendor int8 GEMM on the same GPU, as a measured tensor-core denominator
        for n in (4096, 8192):
            a = torch.randint(-127, 128, (n, n), dtype=torch.int8, device="cuda")
            b = torch.randint(-127, 128, (n, n), dtype=torch.int8, device="cuda").t().contiguous().t()
            us = time_launches(lambda: torch._int_mm(a, b), args.iters, args.warm)
            report("cublaslt int8 gemm %d^3 (int32 out)" % n, us, 2 * n * n + 4 * n * n, 2.0 * n ** 3)
        return
    if args.kind == "block":
        # relu(1x1 conv(x) + strided 1x1 shortcut(x2)) + calib in one launch, fp32 and int8 outputs
        hw, s2 = args.hw, args.stride
        wm = rng.integers(-127, 128, (args.cout, args.cin, 1, 1), dtype=np.int8)
        wsh = rng.integers(-127, 128, (args.cout, args.cin2, 1, 1), dtype=np.int8)
        main = plb.Conv(ctx, wm, [0.001], 0.02, None, in_hw=(hw, hw))
        short = plb.Conv(ctx, wsh, [0.001], 0.02, None, in_hw=(hw * s2, hw * s2), stride=(s2, s2))
        xm = torch.randint(-127, 128, (args.batch, hw, hw, args.cin), dtype=torch.int8, device="cuda")
        xs = torch.randint(-127, 128, (args.batch, hw * s2, hw * s2, args.cin2), dtype=torch.int8, device="cuda")
        yf = torch.empty((args.batch, hw, hw, args.cout), device="cuda")
        yq = torch.empty((args.batch, hw, hw, args.cout), dtype=torch.int8, device="cuda")
        us = time_launches(lambda: main.run_nhwc_block_add_relu(xm, short, xs, 0.05, out_f32=yf, out_i8=yq),
                           args.iters, args.warm)
        pix = args.batch * hw * hw
        report("block %d->%d + %d->%d(s%d) %dx%d b%d" % (args.cin, args.cout, args.cin2, args.cout, s2, hw, hw, args.batch),
               us, pix * (args.cin + args.cin2 + 5 * args.cout) + args.cout * (args.cin + args.cin2),
               2.0 * pix * args.cout * (args.cin + args.cin2))
        ctx.sync()
        return
    if args.kind == "conv":
        conv_layer(args.cin, args.hw, args.cout, args.k, args.stride, args.pad, args.batch, args.out)
    elif args.kind == "dw":
        conv_layer(args.cin, args.hw, args.cin, 3, args.stride, 1, args.batch, args.out, groups=args.cin)
    elif args.kind == "fc":
        fc_layer(args.m, args.kdim, args.n, args.out)
    elif args.kind == "fc-sweep":
        for m, k, n in [(1, 1024, 1000), (64, 2048, 1000), (256, 4096, 4096), (4096, 4096, 4096)]:
            for out in ("f32", "i8"):
                fc_layer(m, k, n, out)
    elif args.kind == "sparse":
        sparse_layer(args.cin, args.cout, args.hw, args.batch, args.fp32, args.semi, args.impl)
    elif args.kind == "sparse-sweep":
        for cin, cout, hw in [(32, 64, 112), (128, 128, 56), (256, 256, 28), (512, 512, 14), (1024, 1024, 7)]:
            for semi in (False, True):
                sparse_layer(cin, cout, hw, args.batch if args.batch != 128 else 256, False, semi, "walk")
                sparse_layer(cin, cout, hw, args.batch if args.batch != 128 else 256, False, semi, "dense")
            sparse_layer(cin, cout, hw, args.batch if args.batch != 128 else 256, True, False, "walk")


if __name__ == "__main__":
    main()
