"""CPU forward pass of the quantised networks with the oracle functions (NCHW, the
reference's layout), op for op what paddle-lite_b200/networks.py enqueues on the GPU."""
import numpy as np

from helpers import O


def forward(qnet, images_f32):
    spec, layers, scales = qnet["spec"], qnet["layers"], qnet["scales"]
    t = {"x": O.calib_f32_to_i8(images_f32, float(scales["x"]))}
    for op in spec["ops"]:
        kind = op["op"]
        if kind == "conv":
            L = layers[op["name"]]
            out_s = float(scales[op["dst"]]) if op["out"] == "i8" else None
            t[op["dst"]] = O.conv_int8(t[op["src"]], L["wq"], L["ws"], float(scales[op["src"]]), L["bias"],
                                       op["act"], 0.0, out_scale=out_s, stride=(op["s"],) * 2,
                                       pads=(op["p"],) * 4, groups=op.get("groups", 1))
        elif kind == "conv_add_relu":
            L = layers[op["name"]]
            y = O.conv_int8(t[op["src"]], L["wq"], L["ws"], float(scales[op["src"]]), L["bias"], O.ACT_NONE)
            s = np.maximum(y + t[op["residual"]], np.float32(0)).astype(np.float32)
            if op["dst_f32"]:
                t[op["dst_f32"]] = s
            if op["dst_i8"]:
                t[op["dst_i8"]] = O.calib_f32_to_i8(s, float(scales[op["dst_i8"]]))
        elif kind == "maxpool":
            t[op["dst"]] = O.maxpool_i8(t[op["src"]], op["k"], op["s"], op["p"])
        elif kind == "avgpool_calib":
            x = t[op["src"]]
            n, c, h, w = x.shape
            flat = x.reshape(n, c, h * w)
            s = np.zeros((n, c), dtype=np.float32)
            for p in range(h * w):  # ascending pixel order, fp32, as the GPU kernel sums
                s = s + flat[:, :, p]
            avg = s / np.float32(h * w)
            t[op["dst"] + "_f32"] = avg
            t[op["dst"]] = O.calib_f32_to_i8(avg, float(scales[op["dst"]]))
        elif kind == "fc":
            L = layers[op["name"]]
            t[op["dst"]] = O.fc_int8(t[op["src"]], L["wq"], L["ws"], float(scales[op["src"]]), L["bias"])
    return t
