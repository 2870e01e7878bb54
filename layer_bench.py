#!/usr/bin/env python
"""Per-layer timing of the library's kernels (one prepared layer, inputs resident in HBM).

    python layer_bench.py conv   --cin 64 --hw 56 --cout 64 --k 3 --pad 1 --batch 128 [--out i8|f32|addrelu] [--nchw]
    python layer_bench.py dw     --cin 32 --hw 112 --stride 1 --batch 128
    python layer_bench.py dwpw   --cin 128 --cout 128 --hw 56 --stride 1 --batch 256            # depthwise 3x3 + 1x1 in one launch
    python layer_bench.py stem   --k 7 --cout 64 --batch 128                                   # first layer from the fp32 image
    python layer_bench.py block  --cin 64 --cin2 64 --hw 56 --cout 256 --stride 1 --batch 128   # projection-block tail
    python layer_bench.py fc     --m 4096 --kdim 4096 --n 4096 [--out i8|f32]
    python layer_bench.py sparse --cin 128 --cout 128 --hw 56 --batch 256 [--fp32] [--semi] [--impl walk|dense]
    python layer_bench.py fc-sweep | sparse-sweep      # the shapes of the benchmark configs
    python layer_bench.py int8-peak                    # library int8 GEMM (cuBLASLt via torch._int_mm) as a measured denominator

Prints one JSON line per layer: microseconds per launch (CUDA events on the launching stream,
after a warm-up that also brings the clocks up), algorithmic bytes and operations, and the
achieved fractions of the measured HBM bandwidth and of the dense int8 tensor peak.  The same
functions feed the per-layer table of bench.py; the command is also the target of the ncu
captures (`--iters` keeps those short).
"""
import argparse
import importlib
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

INT8_PEAK_TOPS = 4500.0   # dense int8 datasheet figure (2 x bf16)
HBM_NOMINAL_GBS = 8000.0  # the "about 8 TB/s" of the benchmark definition; the measured copy bandwidth is lower

FC_SWEEP = [(1, 1024, 1000), (64, 2048, 1000), (256, 4096, 4096), (4096, 4096, 4096)]
SPARSE_SWEEP = [(32, 64, 112), (128, 128, 56), (256, 256, 28), (512, 512, 14), (1024, 1024, 7)]


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


def report(name, us, nbytes, ops, extra=None, int8_measured_tops=None):
    peak, kind = hbm_peak()
    line = {"layer": name, "us": round(us, 2), "bytes": int(nbytes), "ops": int(ops),
            "GBps": round(nbytes / us / 1e3, 1), "TOPS": round(ops / us / 1e6, 1),
            "hbm_frac": round(nbytes / us / 1e3 / peak, 3), "hbm_peak": "%s %.1f GB/s" % (kind, peak),
            "hbm_frac_of_8TBs": round(nbytes / us / 1e3 / HBM_NOMINAL_GBS, 3),
            "tensor_frac_of_4.5POPS": round(ops / us / 1e6 / INT8_PEAK_TOPS, 3)}
    if int8_measured_tops:
        line["tensor_frac_of_vendor_gemm"] = round(ops / us / 1e6 / int8_measured_tops, 3)
    if extra:
        line.update(extra)
    return line


class Layers:
    """Builds one layer of a kind on seeded data and times its launches."""

    def __init__(self, plb, ctx, iters=50, warm=0.3, seed=1):
        self.plb, self.ctx, self.iters, self.warm = plb, ctx, iters, warm
        self.rng = np.random.default_rng(seed)

    def conv(self, cin, hw, cout, k, stride, pad, batch, out, groups=1, nchw=False):
        import torch
        plb, ctx, rng = self.plb, self.ctx, self.rng
        w = rng.integers(-127, 128, (cout, cin // groups, k, k), dtype=np.int8)
        shape = (batch, cin, hw, hw) if nchw else (batch, hw, hw, cin)
        x = torch.randint(-127, 128, shape, dtype=torch.int8, device="cuda")
        kw = dict(in_hw=(hw, hw), stride=(stride, stride), pads=(pad,) * 4, groups=groups)
        if out == "addrelu":
            conv = plb.Conv(ctx, w, [0.001], 0.02, None, **kw)
            oshape = (batch, conv.ho, conv.wo, cout)
            res = torch.randn(oshape, device="cuda")
            yf = torch.empty(oshape, device="cuda")
            yq = torch.empty(oshape, dtype=torch.int8, device="cuda")
            fn = lambda: conv.run_nhwc_add_relu(x, res, 0.05, out_f32=yf, out_i8=yq)  # noqa: E731
            out_bytes = yq.numel() * 9
        else:
            conv = plb.Conv(ctx, w, [0.001], 0.02, None, act=plb.ACT_RELU,
                            out_scale=0.05 if out == "i8" else None, **kw)
            oshape = (batch, cout, conv.ho, conv.wo) if nchw else (batch, conv.ho, conv.wo, cout)
            y = torch.empty(oshape, dtype=torch.int8 if out == "i8" else torch.float32, device="cuda")
            fn = (lambda: conv.run(x, out=y)) if nchw else (lambda: conv.run_nhwc(x, out=y))  # noqa: E731
            out_bytes = y.numel() * y.element_size()
        us = time_launches(fn, self.iters, self.warm)
        ops = 2.0 * batch * conv.ho * conv.wo * cout * (cin // groups) * k * k
        name = "%s cin%d %dx%d cout%d k%d s%d b%d %s%s" % ("dw" if groups > 1 else "conv", cin, hw, hw, cout, k, stride,
                                                          batch, out, " nchw" if nchw else "")
        ctx.sync()
        return report(name, us, x.numel() + w.size + out_bytes, ops)

    def fc(self, m, k, n, out, int8_measured_tops=None):
        import torch
        plb, ctx, rng = self.plb, self.ctx, self.rng
        w = rng.integers(-127, 128, (k, n), dtype=np.int8)
        x = torch.randint(-127, 128, (m, k), dtype=torch.int8, device="cuda")
        fc = plb.Fc(ctx, w, [0.0001], 0.02, np.zeros(n, np.float32), plb.ACT_RELU6, 6.0,
                    out_scale=0.05 if out == "i8" else None)
        y = torch.empty((m, n), dtype=torch.int8 if out == "i8" else torch.float32, device="cuda")
        us = time_launches(lambda: fc.run(x, out=y), self.iters, self.warm)
        ctx.sync()
        return report("fc m%d k%d n%d %s" % (m, k, n, out), us, m * k + k * n + y.numel() * y.element_size() + 8 * n,
                      2.0 * m * k * n, int8_measured_tops=int8_measured_tops)

    def sparse(self, cin, cout, hw, batch, fp32, semi, impl):
        import torch
        plb, ctx, rng = self.plb, self.ctx, self.rng
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
                                impl={"dense": plb.IMPL_TC, "walk": plb.IMPL_DIRECT, "auto": plb.IMPL_AUTO}[impl])
            y = torch.empty((batch, cout, hw, hw), dtype=torch.int8, device="cuda")
            esz = 1
        nnz = int(np.count_nonzero(wf))
        us = time_launches(lambda: sp.run(x, out=y), self.iters, self.warm)
        nbytes = batch * hw * hw * (cin + cout) * esz + nnz * (esz + 4) + 4 * cout
        ctx.sync()
        return report("sparse %s %s cin%d cout%d %dx%d b%d %s" % ("fp32" if fp32 else "int8", "semi" if semi else "unstr",
                                                                 cin, cout, hw, hw, batch, impl), us, nbytes,
                      2.0 * nnz * hw * hw * batch, {"nnz": nnz})

    def block(self, cin, cin2, hw, cout, s2, batch):
        """relu(1x1 conv(x) + strided 1x1 shortcut(x2)) + calib in one launch, fp32 and int8 outputs."""
        import torch
        plb, ctx, rng = self.plb, self.ctx, self.rng
        wm = rng.integers(-127, 128, (cout, cin, 1, 1), dtype=np.int8)
        wsh = rng.integers(-127, 128, (cout, cin2, 1, 1), dtype=np.int8)
        main = plb.Conv(ctx, wm, [0.001], 0.02, None, in_hw=(hw, hw))
        short = plb.Conv(ctx, wsh, [0.001], 0.02, None, in_hw=(hw * s2, hw * s2), stride=(s2, s2))
        xm = torch.randint(-127, 128, (batch, hw, hw, cin), dtype=torch.int8, device="cuda")
        xs = torch.randint(-127, 128, (batch, hw * s2, hw * s2, cin2), dtype=torch.int8, device="cuda")
        yf = torch.empty((batch, hw, hw, cout), device="cuda")
        yq = torch.empty((batch, hw, hw, cout), dtype=torch.int8, device="cuda")
        us = time_launches(lambda: main.run_nhwc_block_add_relu(xm, short, xs, 0.05, out_f32=yf, out_i8=yq),
                           self.iters, self.warm)
        pix = batch * hw * hw
        ctx.sync()
        return report("block %d->%d + %d->%d(s%d) %dx%d b%d" % (cin, cout, cin2, cout, s2, hw, hw, batch), us,
                      pix * (cin + cin2 + 5 * cout) + cout * (cin + cin2), 2.0 * pix * cout * (cin + cin2))

    def dwpw(self, cin, cout, hw, stride, batch):
        """Depthwise 3x3 + 1x1 convolution (a MobileNet block): one launch against the two launches it replaces."""
        import torch
        plb, ctx, rng = self.plb, self.ctx, self.rng
        wdw = rng.integers(-127, 128, (cin, 1, 3, 3), dtype=np.int8)
        wpw = rng.integers(-127, 128, (cout, cin, 1, 1), dtype=np.int8)
        dw = plb.Conv(ctx, wdw, [0.002], 0.02, None, in_hw=(hw, hw), stride=(stride, stride), pads=(1,) * 4, groups=cin,
                      act=plb.ACT_RELU, out_scale=0.05)
        pw = plb.Conv(ctx, wpw, [0.001], 0.05, None, in_hw=(dw.ho, dw.wo), act=plb.ACT_RELU, out_scale=0.05)
        x = torch.randint(-127, 128, (batch, hw, hw, cin), dtype=torch.int8, device="cuda")
        mid = torch.empty((batch, dw.ho, dw.wo, cin), dtype=torch.int8, device="cuda")
        y = torch.empty((batch, dw.ho, dw.wo, cout), dtype=torch.int8, device="cuda")

        def two():
            dw.run_nhwc(x, out=mid)
            pw.run_nhwc(mid, out=y)
        us2 = time_launches(two, self.iters, self.warm)
        pix = batch * dw.ho * dw.wo
        nbytes = x.numel() + y.numel() + 9 * cin + cin * cout
        ops = 2.0 * pix * cin * (cout + 9)
        extra = {"two_launches_us": round(us2, 2), "two_launches_bytes": int(nbytes + 2 * mid.numel())}
        name = "dw3x3+1x1 cin%d %dx%d s%d cout%d b%d" % (cin, hw, hw, stride, cout, batch)
        if not dw.dwpw_fusable(pw):
            ctx.sync()
            return report(name + " (two launches)", us2, nbytes + 2 * mid.numel(), ops, extra)
        us = time_launches(lambda: dw.run_nhwc_dwpw(pw, x, out=y), self.iters, self.warm)
        ctx.sync()
        return report(name, us, nbytes, ops, extra)

    def stem(self, k, cout, batch, hw=224):
        """First layer of a network from the fp32 NCHW image (calib + convolution), int8 channels-last out."""
        import torch
        plb, ctx, rng = self.plb, self.ctx, self.rng
        w = rng.integers(-127, 128, (cout, 3, k, k), dtype=np.int8)
        conv = plb.Conv(ctx, w, [0.001], 0.03, None, in_hw=(hw, hw), stride=(2, 2), pads=(k // 2,) * 4, act=plb.ACT_RELU,
                        out_scale=0.05)
        img = torch.randn((batch, 3, hw, hw), device="cuda")
        y = torch.empty((batch, conv.ho, conv.wo, cout), dtype=torch.int8, device="cuda")
        before = ctx.stem_launch_count()
        us = time_launches(lambda: conv.run_image_f32(img, out=y), self.iters, self.warm)
        one = ctx.stem_launch_count() > before
        ctx.sync()
        return report("stem k%d 3->%d %dx%d b%d %s" % (k, cout, hw, hw, batch, "one launch" if one else "staged"), us,
                      img.numel() * 4 + y.numel() + w.size, 2.0 * batch * conv.ho * conv.wo * cout * 3 * k * k)

    def int8_peak(self, n):
        """Not a kernel of this library: the vendor int8 GEMM on the same GPU, as a measured tensor-core denominator."""
        import torch
        a = torch.randint(-127, 128, (n, n), dtype=torch.int8, device="cuda")
        b = torch.randint(-127, 128, (n, n), dtype=torch.int8, device="cuda").t().contiguous().t()
        us = time_launches(lambda: torch._int_mm(a, b), self.iters, self.warm)
        return report("cublaslt int8 gemm %d^3 (int32 out)" % n, us, 2 * n * n + 4 * n * n, 2.0 * n ** 3)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kind", choices=["conv", "dw", "dwpw", "stem", "block", "fc", "sparse", "fc-sweep", "sparse-sweep", "int8-peak"])
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
    ap.add_argument("--nchw", action="store_true", help="conv: through the NCHW entry point (reference layout)")
    ap.add_argument("--fp32", action="store_true")
    ap.add_argument("--semi", action="store_true")
    ap.add_argument("--impl", default="walk", choices=["walk", "dense", "auto"])
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--warm", type=float, default=0.3, help="seconds of warm-up launches")
    args = ap.parse_args()

    plb = importlib.import_module("paddle-lite_b200")
    L = Layers(plb, plb.Context(0), args.iters, args.warm)
    show = lambda line: print(json.dumps(line), flush=True)  # noqa: E731
    if args.kind == "int8-peak":
        for n in (4096, 8192):
            show(L.int8_peak(n))
    elif args.kind == "block":
        show(L.block(args.cin, args.cin2, args.hw, args.cout, args.stride, args.batch))
    elif args.kind == "conv":
        show(L.conv(args.cin, args.hw, args.cout, args.k, args.stride, args.pad, args.batch, args.out, nchw=args.nchw))
    elif args.kind == "dw":
        show(L.conv(args.cin, args.hw, args.cin, 3, args.stride, 1, args.batch, args.out, groups=args.cin))
    elif args.kind == "stem":
        show(L.stem(args.k, args.cout, args.batch))
    elif args.kind == "dwpw":
        show(L.dwpw(args.cin, args.cout, args.hw, args.stride, args.batch))
    elif args.kind == "fc":
        show(L.fc(args.m, args.kdim, args.n, args.out))
    elif args.kind == "fc-sweep":
        for m, k, n in FC_SWEEP:
            for out in ("f32", "i8"):
                show(L.fc(m, k, n, out))
    elif args.kind == "sparse":
        show(L.sparse(args.cin, args.cout, args.hw, args.batch, args.fp32, args.semi, args.impl))
    elif args.kind == "sparse-sweep":
        batch = args.batch if args.batch != 128 else 256
        for cin, cout, hw in SPARSE_SWEEP:
            for semi in (False, True):
                show(L.sparse(cin, cout, hw, batch, False, semi, "walk"))
                show(L.sparse(cin, cout, hw, batch, False, semi, "dense"))
            show(L.sparse(cin, cout, hw, batch, True, False, "walk"))


if __name__ == "__main__":
    main()
