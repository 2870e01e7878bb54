"""The two whole networks the path is measured on, as chains of the int8 layers of this
library: ResNet-50 v1.5 and MobileNetV1 1.0 at 224x224, post-training quantised.

Graph semantics follow what the reference's optimiser produces for a quantised model
(lite/core/optimizer/optimizer.cc:128-294): conv + BN folded into an int8 conv with fp32 bias,
ReLU fused into the conv, a conv whose consumers are all int8 layers writes int8 (alias
int8_out), a conv feeding an fp32 op (elementwise_add, pool2d avg) writes fp32 (fp32_out),
`calib` converts fp32 -> int8 in front of the next int8 layer
(lite/core/optimizer/mir/static_kernel_pick_pass.cc:100-121, type_precision_cast_pass.cc:75-105).
Max pooling runs on the int8 tensor: max commutes with the monotonic quantiser, so it equals
fp32 pooling followed by calib at the same scale.

There are no model files: weights are seeded He-init, activation scales come from an fp32
calibration pass over seeded N(0,1) images (set-up work, done with torch ops; the timed path
is only the C-ABI library).
"""
import os

import numpy as np

ACT_NONE, ACT_RELU = 0, 1


# ----------------------------------------------------------------------------- specs
def resnet50_spec():
    """List of ops.  Tensor names: 'x' is the int8 image; every op names its inputs/outputs."""
    ops = [dict(op="conv", name="conv1", src="x", dst="c1", cin=3, cout=64, k=7, s=2, p=3, act=ACT_RELU, out="i8"),
           dict(op="maxpool", name="pool1", src="c1", dst="b0", k=3, s=2, p=1)]
    cin = 64
    prev = "b0"          # int8 block input
    prev_f32 = None      # fp32 block input (identity shortcut)
    for stage, (width, blocks, stride) in enumerate([(64, 3, 1), (128, 4, 2), (256, 6, 2), (512, 3, 2)], 1):
        for b in range(blocks):
            s = stride if b == 0 else 1
            pre = "s%db%d" % (stage, b)
            ops.append(dict(op="conv", name=pre + "a", src=prev, dst=pre + "a", cin=cin, cout=width, k=1, s=1,
                            p=0, act=ACT_RELU, out="i8"))
            ops.append(dict(op="conv", name=pre + "b", src=pre + "a", dst=pre + "b", cin=width, cout=width,
                            k=3, s=s, p=1, act=ACT_RELU, out="i8"))
            if b == 0:
                ops.append(dict(op="conv", name=pre + "ds", src=prev, dst=pre + "ds", cin=cin, cout=4 * width,
                                k=1, s=s, p=0, act=ACT_NONE, out="f32"))
                shortcut = pre + "ds"
            else:
                shortcut = prev_f32
            last = stage == 4 and b == blocks - 1
            next_needs_f32 = (b != blocks - 1) or last
            ops.append(dict(op="conv_add_relu", name=pre + "c", src=pre + "b", residual=shortcut,
                            dst_f32=(pre + "f") if next_needs_f32 else None,
                            dst_i8=None if last else pre + "q", cin=width, cout=4 * width, k=1, s=1, p=0))
            prev, prev_f32, cin = pre + "q", pre + "f", 4 * width
    ops.append(dict(op="avgpool_calib", name="pool5", src=prev_f32, dst="feat", c=2048))
    ops.append(dict(op="fc", name="fc", src="feat", dst="logits", k=2048, n=1000))
    return dict(name="resnet50_v1.5", ops=ops, image=(3, 224, 224))


def mobilenet_v1_spec():
    ops = [dict(op="conv", name="conv1", src="x", dst="c1", cin=3, cout=32, k=3, s=2, p=1, act=ACT_RELU, out="i8")]
    cfg = [(32, 64, 1), (64, 128, 2), (128, 128, 1), (128, 256, 2), (256, 256, 1), (256, 512, 2)] + \
          [(512, 512, 1)] * 5 + [(512, 1024, 2), (1024, 1024, 1)]
    prev = "c1"
    for i, (cin, cout, s) in enumerate(cfg, 1):
        ops.append(dict(op="conv", name="dw%d" % i, src=prev, dst="dw%d" % i, cin=cin, cout=cin, k=3, s=s, p=1,
                        groups=cin, act=ACT_RELU, out="i8"))
        last = i == len(cfg)
        ops.append(dict(op="conv", name="pw%d" % i, src="dw%d" % i, dst="pw%d" % i, cin=cin, cout=cout, k=1, s=1,
                        p=0, act=ACT_RELU, out="f32" if last else "i8"))
        prev = "pw%d" % i
    ops.append(dict(op="avgpool_calib", name="pool", src=prev, dst="feat", c=1024))
    ops.append(dict(op="fc", name="fc", src="feat", dst="logits", k=1024, n=1000))
    return dict(name="mobilenet_v1_1.0", ops=ops, image=(3, 224, 224))


SPECS = {"resnet50": resnet50_spec, "mobilenet_v1": mobilenet_v1_spec}


def conv_macs_per_image(spec):
    """Multiply-accumulates of the conv and fc layers for one image."""
    c, h, w = spec["image"]
    hw = {"x": (h, w)}
    macs = 0
    for op in spec["ops"]:
        if op["op"] in ("conv", "conv_add_relu"):
            ih, iw = hw[op["src"]]
            oh, ow = (ih + 2 * op["p"] - op["k"]) // op["s"] + 1, (iw + 2 * op["p"] - op["k"]) // op["s"] + 1
            macs += oh * ow * op["cout"] * (op["cin"] // op.get("groups", 1)) * op["k"] ** 2
            for key in ("dst", "dst_f32", "dst_i8"):
                if op.get(key):
                    hw[op[key]] = (oh, ow)
        elif op["op"] == "maxpool":
            ih, iw = hw[op["src"]]
            hw[op["dst"]] = ((ih + 2 * op["p"] - op["k"]) // op["s"] + 1, (iw + 2 * op["p"] - op["k"]) // op["s"] + 1)
        elif op["op"] == "fc":
            macs += op["k"] * op["n"]
    return macs


# ----------------------------------------------------------------------------- weights + calibration
def _quant_per_channel(w):
    red = tuple(range(1, w.ndim))
    amax = np.maximum(np.abs(w).max(axis=red, keepdims=True), 1e-12)
    scale = (amax / 127.0).astype(np.float32)
    return np.clip(np.rint(w / scale), -127, 127).astype(np.int8), scale.reshape(-1).astype(np.float32)


def build_quantized(spec, seed=1234, calib_images=16, device="cpu"):
    """He-init weights, per-channel int8 quantisation, activation scales from an fp32 pass over
    `calib_images` seeded N(0,1) images.  Returns a dict the runner and the test oracle share."""
    import torch
    import torch.nn.functional as F
    rng = np.random.default_rng(seed)
    params = {}
    for op in spec["ops"]:
        if op["op"] in ("conv", "conv_add_relu"):
            cig = op["cin"] // op.get("groups", 1)
            fan_in = cig * op["k"] ** 2
            w = (rng.standard_normal((op["cout"], cig, op["k"], op["k"])) * np.sqrt(2.0 / fan_in)).astype(np.float32)
            b = (rng.standard_normal(op["cout"]) * 0.1).astype(np.float32)
            params[op["name"]] = dict(w=w, b=b)
        elif op["op"] == "fc":
            w = (rng.standard_normal((op["k"], op["n"])) * np.sqrt(2.0 / op["k"])).astype(np.float32)
            b = (rng.standard_normal(op["n"]) * 0.1).astype(np.float32)
            params[op["name"]] = dict(w=w, b=b)
    # fp32 calibration pass: maxima of every tensor that will be stored as int8
    x = torch.from_numpy(rng.standard_normal((calib_images,) + spec["image"]).astype(np.float32)).to(device)
    t = {"x": x}
    amax = {"x": float(x.abs().max())}
    tt = lambda a: torch.from_numpy(a).to(device)  # noqa: E731
    for op in spec["ops"]:
        if op["op"] == "conv":
            p = params[op["name"]]
            y = F.conv2d(t[op["src"]], tt(p["w"]), tt(p["b"]), stride=op["s"], padding=op["p"],
                         groups=op.get("groups", 1))
            if op["act"] == ACT_RELU:
                y = F.relu(y)
            t[op["dst"]] = y
            amax[op["dst"]] = float(y.abs().max())
        elif op["op"] == "conv_add_relu":
            p = params[op["name"]]
            y = F.relu(F.conv2d(t[op["src"]], tt(p["w"]), tt(p["b"])) + t[op["residual"]])
            for key in ("dst_f32", "dst_i8"):
                if op.get(key):
                    t[op[key]] = y
                    amax[op[key]] = float(y.abs().max())
        elif op["op"] == "maxpool":
            y = F.max_pool2d(t[op["src"]], op["k"], op["s"], op["p"])
            t[op["dst"]] = y
            amax[op["dst"]] = amax[op["src"]]  # same scale as its input: pooling happens in int8
        elif op["op"] == "avgpool_calib":
            y = t[op["src"]].mean(dim=(2, 3))
            t[op["dst"]] = y
            amax[op["dst"]] = float(y.abs().max())
        elif op["op"] == "fc":
            p = params[op["name"]]
            t[op["dst"]] = t[op["src"]] @ tt(p["w"]) + tt(p["b"])
    scales = {k: np.float32(max(v, 1e-8) / 127.0) for k, v in amax.items()}
    layers = {}
    for op in spec["ops"]:
        if op["name"] in params:
            p = params[op["name"]]
            if op["op"] == "fc":
                wq_t, ws = _quant_per_channel(np.ascontiguousarray(p["w"].T))  # per output feature
                wq = np.ascontiguousarray(wq_t.T)
            else:
                wq, ws = _quant_per_channel(p["w"])
            layers[op["name"]] = dict(wq=wq, ws=ws, bias=p["b"])
    return dict(spec=spec, layers=layers, scales=scales)


# ----------------------------------------------------------------------------- GPU runner
def fusable_shortcuts(spec):
    """Projection shortcuts that can run inside the launch of the block's last convolution
    (plb_conv_run_nhwc_block_add_relu): an unpadded 1x1 conv with fp32 output and no activation
    whose only reader is the residual input of a conv_add_relu whose own conv is 1x1, stride 1.
    Returns {tensor name: shortcut op}."""
    readers = {}
    for op in spec["ops"]:
        for key in ("src", "residual"):
            if key in op:
                readers.setdefault(op[key], []).append((op, key))
    out = {}
    for op in spec["ops"]:
        if op["op"] != "conv" or op.get("out") != "f32" or op["k"] != 1 or op["p"] != 0 or op["act"] != ACT_NONE:
            continue
        if op.get("groups", 1) != 1 or op["cin"] % 32:
            continue
        r = readers.get(op["dst"], [])
        if len(r) == 1 and r[0][1] == "residual" and r[0][0]["op"] == "conv_add_relu":
            main = r[0][0]
            if main["k"] == 1 and main["s"] == 1 and main["p"] == 0 and main["cin"] % 32 == 0:
                out[op["dst"]] = op
    return out


class Runner:
    """Holds the prepared layers and all activation buffers for one batch size on one GPU and
    enqueues a whole forward pass on the context's stream (no allocation, no host sync).

    `micro_batch` (a divisor of `batch`) makes the step run depth-first over slices of that
    many images through the same set of activation buffers: every intermediate tensor of a
    slice is then small enough to stay in the 126 MB L2 between the layer that writes it and
    the layer that reads it, instead of making a round trip through HBM."""

    def __init__(self, plb, ctx, qnet, batch, micro_batch=None, fuse_blocks=True):
        import torch
        self.plb, self.ctx, self.q = plb, ctx, qnet
        self.full_batch = batch
        micro_batch = micro_batch or batch
        if batch % micro_batch:
            raise ValueError("micro_batch must divide batch")
        self.micro_batch = micro_batch
        full_batch, batch = batch, micro_batch
        spec, scales = qnet["spec"], qnet["scales"]
        dev = "cuda:%d" % ctx.device
        c, h, w = spec["image"]
        self.hw = {"x": (h, w)}
        self.buf = {}
        self.steps = []
        self.image_shape = (full_batch, c, h, w)
        if os.environ.get("PLB_FUSE_BLOCKS", "1") == "0":  # A/B switch for measurements
            fuse_blocks = False
        shortcuts = fusable_shortcuts(spec) if fuse_blocks else {}
        shortcut_convs = {}
        for op in spec["ops"]:
            kind = op["op"]
            if kind in ("conv", "conv_add_relu"):
                L = qnet["layers"][op["name"]]
                ih, iw = self.hw[op["src"]]
                wq = L["wq"]
                in_s = float(scales[op["src"]])
                if kind == "conv":
                    out_s = float(scales[op["dst"]]) if op["out"] == "i8" else None
                    groups = op.get("groups", 1)
                    conv = plb.Conv(ctx, wq, L["ws"], in_s, L["bias"], in_hw=(ih, iw), stride=(op["s"], op["s"]),
                                    pads=(op["p"],) * 4, groups=groups, act=op["act"], out_scale=out_s)
                    dt = torch.int8 if out_s is not None else torch.float32
                    self.buf[op["dst"]] = torch.empty((batch, conv.ho, conv.wo, op["cout"]), dtype=dt, device=dev)
                    self.hw[op["dst"]] = (conv.ho, conv.wo)
                    if op["dst"] in shortcuts:
                        # runs inside the launch of the block's last conv; its fp32 tensor is never written
                        shortcut_convs[op["dst"]] = (conv, op["src"])
                        del self.buf[op["dst"]]
                        continue
                    self.steps.append(("conv_image" if op["src"] == "x" else "conv", conv, op["src"], op["dst"]))
                else:
                    conv = plb.Conv(ctx, wq, L["ws"], in_s, L["bias"], in_hw=(ih, iw))
                    shape = (batch, conv.ho, conv.wo, op["cout"])
                    if op["dst_f32"]:
                        self.buf[op["dst_f32"]] = torch.empty(shape, dtype=torch.float32, device=dev)
                        self.hw[op["dst_f32"]] = (conv.ho, conv.wo)
                    if op["dst_i8"]:
                        self.buf[op["dst_i8"]] = torch.empty(shape, dtype=torch.int8, device=dev)
                        self.hw[op["dst_i8"]] = (conv.ho, conv.wo)
                    next_s = float(scales[op["dst_i8"]]) if op["dst_i8"] else None
                    if op["residual"] in shortcut_convs:
                        sc_conv, sc_src = shortcut_convs[op["residual"]]
                        self.steps.append(("block_add_relu", conv, op["src"], sc_conv, sc_src, op["dst_f32"],
                                           op["dst_i8"], next_s))
                    else:
                        self.steps.append(("conv_add_relu", conv, op["src"], op["residual"], op["dst_f32"],
                                           op["dst_i8"], next_s))
            elif kind == "maxpool":
                ih, iw = self.hw[op["src"]]
                oh, ow = (ih + 2 * op["p"] - op["k"]) // op["s"] + 1, (iw + 2 * op["p"] - op["k"]) // op["s"] + 1
                cch = self.buf[op["src"]].shape[3]
                self.buf[op["dst"]] = torch.empty((batch, oh, ow, cch), dtype=torch.int8, device=dev)
                self.hw[op["dst"]] = (oh, ow)
                self.steps.append(("maxpool", op["src"], op["dst"], op["k"], op["s"], op["p"]))
            elif kind == "avgpool_calib":
                self.buf[op["dst"]] = torch.empty((batch, op["c"]), dtype=torch.int8, device=dev)
                self.buf[op["dst"] + "_f32"] = torch.empty((batch, op["c"]), dtype=torch.float32, device=dev)
                self.steps.append(("avgpool_calib", op["src"], op["dst"], float(scales[op["dst"]])))
            elif kind == "fc":
                L = qnet["layers"][op["name"]]
                fc = plb.Fc(ctx, L["wq"], L["ws"], float(scales[op["src"]]), L["bias"])
                self.buf[op["dst"]] = torch.empty((batch, op["n"]), dtype=torch.float32, device=dev)
                self.steps.append(("fc", fc, op["src"], op["dst"]))
        self.in_scale = float(scales["x"])
        # Measured slower than the two launches it replaces (both roles are bound by instruction issue and latency, and
        # one CTA cannot hold as many warps of each as the two kernels do), so it is opt-in.
        if os.environ.get("PLB_DWPW", "0") == "1":
            self._fuse_depthwise_pairs()
        self.logits = torch.empty((full_batch, self.buf["logits"].shape[1]), dtype=torch.float32, device=dev)
        self.buf["logits"] = self.logits[:batch]

    def _fuse_depthwise_pairs(self):
        """A depthwise 3x3 layer whose only reader is the 1x1 layer after it runs in that layer's launch
        (plb_conv_run_nhwc_dwpw) where the pair qualifies; the tensor between them is then never written."""
        readers = {}
        for st in self.steps:
            for name in (st[2:3] if st[0] in ("conv", "conv_image") else ()):
                readers[name] = readers.get(name, 0) + 1
            if st[0] in ("conv_add_relu", "block_add_relu"):
                for name in (st[2], st[3] if st[0] == "conv_add_relu" else st[4]):
                    readers[name] = readers.get(name, 0) + 1
            if st[0] in ("maxpool", "avgpool_calib"):
                readers[st[1]] = readers.get(st[1], 0) + 1
        fused, i = [], 0
        while i < len(self.steps):
            a = self.steps[i]
            b = self.steps[i + 1] if i + 1 < len(self.steps) else None
            if (a[0] == "conv" and b is not None and b[0] == "conv" and b[2] == a[3] and readers.get(a[3], 0) == 1
                    and a[1].desc.groups > 1 and a[1].dwpw_fusable(b[1])):
                fused.append(("dwpw", a[1], b[1], a[2], b[3]))
                del self.buf[a[3]]
                i += 2
            else:
                fused.append(a)
                i += 1
        self.steps = fused

    def forward(self, image_f32_nchw):
        """image_f32_nchw: device float32 [batch,3,224,224].  Returns the fp32 logits [batch,1000]."""
        mb = self.micro_batch
        for i in range(0, self.full_batch, mb):
            self.buf["logits"] = self.logits[i:i + mb]
            self.forward_head(image_f32_nchw[i:i + mb])
            self.forward_body()
        self.buf["logits"] = self.logits[:mb]
        return self.logits

    def forward_head(self, image_f32_nchw):
        """First layer: calib + staging of the fp32 image and the stem convolution (the only
        reader of the input tensor)."""
        st = self.steps[0]
        assert st[0] == "conv_image"
        st[1].run_image_f32(image_f32_nchw, out=self.buf[st[3]])

    def forward_body(self):
        """Everything after the first layer; touches only preallocated buffers."""
        b, ctx = self.buf, self.ctx
        for st in self.steps[1:]:
            if st[0] == "conv":
                st[1].run_nhwc(b[st[2]], out=b[st[3]])
            elif st[0] == "dwpw":
                st[1].run_nhwc_dwpw(st[2], b[st[3]], out=b[st[4]])
            elif st[0] == "conv_add_relu":
                _, conv, src, res, df, dq, next_s = st
                conv.run_nhwc_add_relu(b[src], b[res], next_s, want_f32=df is not None,
                                       out_f32=b[df] if df else None, out_i8=b[dq] if dq else None)
            elif st[0] == "block_add_relu":
                _, conv, src, sc_conv, sc_src, df, dq, next_s = st
                conv.run_nhwc_block_add_relu(b[src], sc_conv, b[sc_src], next_s, want_f32=df is not None,
                                             out_f32=b[df] if df else None, out_i8=b[dq] if dq else None)
            elif st[0] == "maxpool":
                ctx.maxpool_nhwc_i8(b[st[1]], st[3], st[4], st[5], out=b[st[2]])
            elif st[0] == "avgpool_calib":
                ctx.global_avgpool_nhwc_f32(b[st[1]], scale=st[3], out_f32=b[st[2] + "_f32"], out_i8=b[st[2]])
            elif st[0] == "fc":
                st[1].run(b[st[2]], out=b[st[3]])
        return b["logits"]
