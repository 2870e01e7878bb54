"""ctypes bindings for the CPU checkers under ``oracle/``.

TEST INFRASTRUCTURE ONLY.  Only the tests, the smoke check and the CPU-baseline /
reference legs of ``bench.py`` import this module; the library itself never does.

``liboracle.so``       exact-integer restatement of the reference arithmetic (plb_oracle.c)
``_ref/libref_x86.so`` the reference's own gemm_s8u8 + im2col objects (ref_x86_shim.cc),
                       present when it was built from the reference tree

Both are built by ``make -C oracle`` (``ensure_built`` does that on first use).
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_ORACLE_SO = os.path.join(_HERE, "liboracle.so")
_REF_SO = os.path.join(_HERE, "_ref", "libref_x86.so")

ACT_NONE, ACT_RELU, ACT_RELU6, ACT_LEAKY = 0, 1, 2, 3

_lib = None
_ref = None


def ensure_built(quiet=True):
    """Build liboracle.so (and libref_x86.so when the reference tree is present)."""
    need = not os.path.exists(_ORACLE_SO) or os.path.getmtime(_ORACLE_SO) < os.path.getmtime(
        os.path.join(_HERE, "plb_oracle.c"))
    if need or (os.path.isdir("/root/reference") and not os.path.exists(_REF_SO)):
        subprocess.run(["make", "-C", _HERE, "-j8"], check=True,
                       stdout=subprocess.DEVNULL if quiet else None)


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t)) if a is not None else None


def lib():
    global _lib
    if _lib is None:
        ensure_built()
        _lib = C.CDLL(_ORACLE_SO)
    return _lib


def ref_available():
    return os.path.exists(_REF_SO)


def ref():
    """The reference's own x86 objects; raises if they were not built."""
    global _ref
    if _ref is None:
        ensure_built()
        if not os.path.exists(_REF_SO):
            raise RuntimeError("oracle/_ref/libref_x86.so is not built (reference tree absent)")
        _ref = C.CDLL(_REF_SO)
    return _ref


# --------------------------------------------------------------------------- conv / fc

def conv_out_hw(h, w, kh, kw, stride, pads, dil):
    sh, sw = stride
    pt, pb, pl, pr = pads
    dh, dw = dil
    ho = (h + pt + pb - (dh * (kh - 1) + 1)) // sh + 1
    wo = (w + pl + pr - (dw * (kw - 1) + 1)) // sw + 1
    return ho, wo


def conv_acc_i32(x, w, stride=(1, 1), pads=(0, 0, 0, 0), dil=(1, 1), groups=1):
    """Exact int32 accumulators.  x [N,Cin,H,W] int8, w [Cout,Cin/g,kh,kw] int8."""
    x = np.ascontiguousarray(x, dtype=np.int8)
    w = np.ascontiguousarray(w, dtype=np.int8)
    n, cin, h, wd = x.shape
    cout, _, kh, kw = w.shape
    ho, wo = conv_out_hw(h, wd, kh, kw, stride, pads, dil)
    acc = np.empty((n, cout, ho, wo), dtype=np.int32)
    rc = lib().orc_conv_acc_i32(_p(x, C.c_int8), _p(w, C.c_int8), _p(acc, C.c_int32), n, cin, h, wd,
                                cout, kh, kw, stride[0], stride[1], pads[0], pads[1], pads[2],
                                pads[3], dil[0], dil[1], groups)
    if rc:
        raise ValueError("orc_conv_acc_i32 rejected the shape")
    return acc


def fc_acc_i32(x, w):
    """x [M,K] int8, w [K,N] int8 -> [M,N] int32."""
    x = np.ascontiguousarray(x, dtype=np.int8)
    w = np.ascontiguousarray(w, dtype=np.int8)
    m, k = x.shape
    n = w.shape[1]
    acc = np.empty((m, n), dtype=np.int32)
    lib().orc_fc_acc_i32(_p(x, C.c_int8), _p(w, C.c_int8), _p(acc, C.c_int32), m, k, n)
    return acc


def epilogue(acc, wscale, in_scale, bias=None, act=ACT_NONE, alpha=0.0, out_scale=None,
             leaky_compat=False, channel_axis=1):
    """Dequantise / requantise accumulators.  out_scale None -> fp32 out, else int8 out."""
    acc = np.ascontiguousarray(acc, dtype=np.int32)
    c = acc.shape[channel_axis]
    outer = int(np.prod(acc.shape[:channel_axis], dtype=np.int64))
    inner = int(np.prod(acc.shape[channel_axis + 1:], dtype=np.int64))
    wscale = np.ascontiguousarray(np.atleast_1d(wscale), dtype=np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    is_i8 = out_scale is not None
    out = np.empty(acc.shape, dtype=np.int8 if is_i8 else np.float32)
    rc = lib().orc_epilogue(_p(acc, C.c_int32), out.ctypes.data_as(C.c_void_p), C.c_long(outer), c,
                            C.c_long(inner), _p(wscale, C.c_float), int(wscale.size),
                            C.c_float(in_scale), C.c_float(out_scale if is_i8 else 1.0),
                            _p(b, C.c_float), act, C.c_float(alpha), int(is_i8),
                            int(bool(leaky_compat)))
    if rc:
        raise ValueError("weight scale size must be 1 or the channel count")
    return out


def epilogue_f64(acc, wscale, in_scale, bias=None, act=ACT_NONE, alpha=0.0, channel_axis=1):
    acc = np.ascontiguousarray(acc, dtype=np.int32)
    c = acc.shape[channel_axis]
    outer = int(np.prod(acc.shape[:channel_axis], dtype=np.int64))
    inner = int(np.prod(acc.shape[channel_axis + 1:], dtype=np.int64))
    wscale = np.ascontiguousarray(np.atleast_1d(wscale), dtype=np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    out = np.empty(acc.shape, dtype=np.float64)
    lib().orc_epilogue_f64(_p(acc, C.c_int32), _p(out, C.c_double), C.c_long(outer), c,
                           C.c_long(inner), _p(wscale, C.c_float), int(wscale.size),
                           C.c_float(in_scale), _p(b, C.c_float), act, C.c_float(alpha))
    return out


def conv_int8(x, w, wscale, in_scale, bias=None, act=ACT_NONE, alpha=0.0, out_scale=None,
              stride=(1, 1), pads=(0, 0, 0, 0), dil=(1, 1), groups=1, leaky_compat=False):
    acc = conv_acc_i32(x, w, stride, pads, dil, groups)
    return epilogue(acc, wscale, in_scale, bias, act, alpha, out_scale, leaky_compat)


def fc_int8(x, w, wscale, in_scale, bias=None, act=ACT_NONE, alpha=0.0, out_scale=None):
    return epilogue(fc_acc_i32(x, w), wscale, in_scale, bias, act, alpha, out_scale)


# --------------------------------------------------------------------------- calib

def calib_f32_to_i8(x, scale):
    x = np.ascontiguousarray(x, dtype=np.float32)
    q = np.empty(x.shape, dtype=np.int8)
    lib().orc_calib_f32_to_i8(_p(x, C.c_float), _p(q, C.c_int8), C.c_long(x.size), C.c_float(scale))
    return q


def calib_i8_to_f32(q, scale):
    q = np.ascontiguousarray(q, dtype=np.int8)
    y = np.empty(q.shape, dtype=np.float32)
    lib().orc_calib_i8_to_f32(_p(q, C.c_int8), _p(y, C.c_float), C.c_long(q.size), C.c_float(scale))
    return y


def softmax(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = x.shape
    y = np.empty_like(x)
    lib().orc_softmax_f32(_p(x, C.c_float), _p(y, C.c_float), rows, cols)
    return y


def maxpool_i8(x, k=3, s=2, p=1):
    x = np.ascontiguousarray(x, dtype=np.int8)
    n, c, h, w = x.shape
    ho, wo = (h + 2 * p - k) // s + 1, (w + 2 * p - k) // s + 1
    y = np.empty((n, c, ho, wo), dtype=np.int8)
    lib().orc_maxpool_i8(_p(x, C.c_int8), _p(y, C.c_int8), n, c, h, w, k, s, p)
    return y


# --------------------------------------------------------------------------- sparse

def sparse_zeros(w):
    """ComputeSemiSparseZeros: returns dict(zeros, count_nonzeroes, count_channels, count_blocks, flag_semi)."""
    w = np.ascontiguousarray(w)
    m, k = w.shape
    vals = [C.c_int(0) for _ in range(4)]
    if w.dtype == np.int8:
        fn, t = lib().orc_sparse_zeros_i8, C.c_int8
    else:
        w = w.astype(np.float32)
        fn, t = lib().orc_sparse_zeros_f32, C.c_float
    zeros = fn(_p(w, t), m, k, *[C.byref(v) for v in vals])
    return dict(zeros=zeros, count_nonzeroes=vals[0].value, count_channels=vals[1].value,
                count_blocks=vals[2].value, flag_semi=vals[3].value)


def sparse_encode(w, hw, semi=False, pad4=None):
    """Encode a dense [M,K] weight matrix the way sparse_conv_detect_pass does.

    int8 weights use the unpadded unstructured encoder, fp32 weights the pad-to-4 one
    (pad4 overrides), semi=True the 2x1 semi-structured encoder.
    Returns dict(nonzero_weights, oc_nonzeros [M] uint32, diffs int32, first_ic, flag_semi).
    """
    w = np.ascontiguousarray(w)
    m, k = w.shape
    is_i8 = w.dtype == np.int8
    if not is_i8:
        w = np.ascontiguousarray(w, dtype=np.float32)
    t = C.c_int8 if is_i8 else C.c_float
    if pad4 is None:
        pad4 = (not is_i8) and not semi
    nnz = int(np.count_nonzero(w))
    cum = np.zeros(m, dtype=np.uint32)
    if semi:
        info = sparse_zeros(w)
        # The semi encoder itself does not need flag_semi to be 1; sizes follow count_* of a
        # forced 2x1 blocking.
        pairs = m // 2
        blk = 0
        for p in range(pairs):
            blk += int(np.count_nonzero((w[2 * p] != 0) | (w[2 * p + 1] != 0)))
        rem = int(np.count_nonzero(w[2 * pairs:])) if m % 2 else 0
        n_vals, n_blocks = 2 * blk + rem, blk + rem
        nz = np.zeros(max(n_vals, 1), dtype=w.dtype)
        diffs = np.zeros(max(n_blocks, 1), dtype=np.int32)
        fn = lib().orc_sparse_encode_semi_i8 if is_i8 else lib().orc_sparse_encode_semi_f32
        first_ic = fn(_p(w, t), m, k, hw, _p(nz, t), _p(cum, C.c_uint32), _p(diffs, C.c_int32))
        return dict(nonzero_weights=nz[:n_vals], oc_nonzeros=cum, diffs=diffs[:n_blocks],
                    first_ic=first_ic, flag_semi=1, would_pick_semi=info["flag_semi"])
    if pad4:
        per = np.count_nonzero(w, axis=1)
        stored = int(np.sum((per + 3) // 4 * 4))
        nz = np.zeros(max(stored, 1), dtype=np.float32)
        diffs = np.zeros(max(stored, 1), dtype=np.int32)
        n_stored = C.c_int(0)
        first_ic = lib().orc_sparse_encode_pad4_f32(_p(w, C.c_float), m, k, hw, _p(nz, C.c_float),
                                                    _p(cum, C.c_uint32), _p(diffs, C.c_int32),
                                                    C.byref(n_stored))
        assert n_stored.value == stored
        return dict(nonzero_weights=nz[:stored], oc_nonzeros=cum, diffs=diffs[:stored],
                    first_ic=first_ic, flag_semi=0, pad4=1)
    nz = np.zeros(max(nnz, 1), dtype=w.dtype)
    diffs = np.zeros(max(nnz, 1), dtype=np.int32)
    fn = lib().orc_sparse_encode_i8 if is_i8 else lib().orc_sparse_encode_unpadded_f32
    first_ic = fn(_p(w, t), m, k, hw, _p(nz, t), _p(cum, C.c_uint32), _p(diffs, C.c_int32))
    return dict(nonzero_weights=nz[:nnz], oc_nonzeros=cum, diffs=diffs[:nnz], first_ic=first_ic,
                flag_semi=0)


def sparse_decode(enc, m, k, hw):
    nz = np.ascontiguousarray(enc["nonzero_weights"])
    is_i8 = nz.dtype == np.int8
    t = C.c_int8 if is_i8 else C.c_float
    dense = np.zeros((m, k), dtype=nz.dtype)
    cum = np.ascontiguousarray(enc["oc_nonzeros"], dtype=np.uint32)
    diffs = np.ascontiguousarray(enc["diffs"], dtype=np.int32)
    if nz.size == 0:
        return dense
    fn = lib().orc_sparse_decode_i8 if is_i8 else lib().orc_sparse_decode_f32
    rc = fn(_p(nz, t), _p(cum, C.c_uint32), _p(diffs, C.c_int32), m, k, hw, int(enc["first_ic"]),
            int(enc["flag_semi"]), int(enc.get("pad4", 0)), _p(dense, t))
    if rc:
        raise ValueError("sparse encoding walks outside the input channels")
    return dense


def sparse_conv_f32(x, dense, bias=None, act=ACT_NONE, alpha=0.0, f64=False):
    """fp32 1x1 conv in the ARM kernel's accumulation order.  x [N,K,H,W] fp32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    dense = np.ascontiguousarray(dense, dtype=np.float32)
    n, k, h, w = x.shape
    m = dense.shape[0]
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    if f64:
        y = np.empty((n, m, h, w), dtype=np.float64)
        lib().orc_sparse_conv_f64(_p(x, C.c_float), _p(dense, C.c_float), _p(b, C.c_float),
                                  _p(y, C.c_double), n, m, k, h * w, act, C.c_float(alpha))
    else:
        y = np.empty((n, m, h, w), dtype=np.float32)
        lib().orc_sparse_conv_f32(_p(x, C.c_float), _p(dense, C.c_float), _p(b, C.c_float),
                                  _p(y, C.c_float), n, m, k, h * w, act, C.c_float(alpha))
    return y


# --------------------------------------------------------------------------- reference objects

def ref_conv_int8(x, w, wscale, in_scale, bias=None, act=ACT_NONE, alpha=0.0, out_scale=None,
                  stride=(1, 1), pads=(0, 0, 0, 0), dil=(1, 1), groups=1, threads=1, out=None):
    """The reference's im2col + gemm_s8u8 path (conv_compute.cc:216-472).

    For int8 out the relu6 bound and the leaky slope are divided by out_scale exactly as
    conv_compute.cc:386-396 does.
    """
    x = np.ascontiguousarray(x, dtype=np.int8)
    w = np.ascontiguousarray(w, dtype=np.int8)
    n, cin, h, wd = x.shape
    cout, _, kh, kw = w.shape
    ho, wo = conv_out_hw(h, wd, kh, kw, stride, pads, dil)
    ws = np.ascontiguousarray(np.broadcast_to(np.atleast_1d(wscale), (cout,)), dtype=np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    is_i8 = out_scale is not None
    if out is None:
        out = np.empty((n, cout, ho, wo), dtype=np.int8 if is_i8 else np.float32)
    a = alpha
    if is_i8 and act in (ACT_RELU6, ACT_LEAKY):
        a = np.float32(alpha) / np.float32(out_scale)
    rc = ref().ref_x86_conv_int8(_p(x, C.c_int8), _p(w, C.c_int8), _p(b, C.c_float),
                                 out.ctypes.data_as(C.c_void_p), int(is_i8), n, cin, h, wd, cout,
                                 kh, kw, stride[0], stride[1], pads[0], pads[1], pads[2], pads[3],
                                 dil[0], dil[1], groups, _p(ws, C.c_float), C.c_float(in_scale),
                                 C.c_float(out_scale if is_i8 else 1.0), act, C.c_float(a),
                                 threads)
    if rc:
        raise ValueError("ref_x86_conv_int8 rejected the shape")
    return out


class RefConv:
    """A layer prepared once on the reference objects (= PrepareForRun) and run many times (= Run): what the
    timed CPU arm uses, so that packing the filter is not inside the timed region."""

    def __init__(self, w, wscale, in_scale, bias=None, act=ACT_NONE, alpha=0.0, out_scale=None, *, in_hw,
                 stride=(1, 1), pads=(0, 0, 0, 0), dil=(1, 1), groups=1, threads=1):
        w = np.ascontiguousarray(w, dtype=np.int8)
        cout, cig, kh, kw = w.shape
        self.cin, self.cout, (self.h, self.wd) = cig * groups, cout, in_hw
        self.ho, self.wo = conv_out_hw(self.h, self.wd, kh, kw, stride, pads, dil)
        ws = np.ascontiguousarray(np.broadcast_to(np.atleast_1d(wscale), (cout,)), dtype=np.float32)
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        self.is_i8 = out_scale is not None
        a = alpha
        if self.is_i8 and act in (ACT_RELU6, ACT_LEAKY):
            a = np.float32(alpha) / np.float32(out_scale)
        lib = ref()
        lib.ref_x86_conv_prepare.restype = C.c_void_p
        self.handle = C.c_void_p(lib.ref_x86_conv_prepare(
            _p(w, C.c_int8), _p(b, C.c_float), int(self.is_i8), self.cin, self.h, self.wd, cout, kh, kw,
            stride[0], stride[1], pads[0], pads[1], pads[2], pads[3], dil[0], dil[1], groups, _p(ws, C.c_float),
            C.c_float(in_scale), C.c_float(out_scale if self.is_i8 else 1.0), act, C.c_float(a), threads))
        if not self.handle:
            raise ValueError("ref_x86_conv_prepare rejected the shape")

    def run(self, x):
        x = np.ascontiguousarray(x, dtype=np.int8)
        n = x.shape[0]
        out = np.empty((n, self.cout, self.ho, self.wo), dtype=np.int8 if self.is_i8 else np.float32)
        lib = ref()
        lib.ref_x86_conv_run.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        rc = lib.ref_x86_conv_run(self.handle, x.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p), n)
        if rc:
            raise ValueError("ref_x86_conv_run failed")
        return out

    def __del__(self):
        try:
            lib = ref()
            lib.ref_x86_conv_destroy.argtypes = [C.c_void_p]
            lib.ref_x86_conv_destroy(self.handle)
        except Exception:
            pass


def ref_fc_int8(x, w, wscale, in_scale, bias=None, act=ACT_NONE, alpha=0.0, out_scale=None):
    """fc through the reference GEMM in the conv orientation.  x [M,K], w [K,N] -> [M,N]."""
    x = np.ascontiguousarray(x, dtype=np.int8)
    w = np.ascontiguousarray(w, dtype=np.int8)
    m, k = x.shape
    n = w.shape[1]
    xt = np.ascontiguousarray(x.T)
    wt = np.ascontiguousarray(w.T)
    ws = np.ascontiguousarray(np.broadcast_to(np.atleast_1d(wscale), (n,)), dtype=np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    is_i8 = out_scale is not None
    out = np.empty((n, m), dtype=np.int8 if is_i8 else np.float32)
    a = alpha
    if is_i8 and act in (ACT_RELU6, ACT_LEAKY):
        a = np.float32(alpha) / np.float32(out_scale)
    ref().ref_x86_fc_int8_t(_p(xt, C.c_int8), _p(wt, C.c_int8), _p(b, C.c_float),
                            out.ctypes.data_as(C.c_void_p), int(is_i8), m, k, n, _p(ws, C.c_float),
                            C.c_float(in_scale), C.c_float(out_scale if is_i8 else 1.0), act,
                            C.c_float(a))
    return np.ascontiguousarray(out.T)


def ref_im2col(x, kh, kw, stride, pads, dil):
    x = np.ascontiguousarray(x, dtype=np.int8)
    c, h, w = x.shape
    ho, wo = conv_out_hw(h, w, kh, kw, stride, pads, dil)
    col = np.empty((c * kh * kw, ho * wo), dtype=np.int8)
    ref().ref_x86_im2col_int8(_p(x, C.c_int8), c, h, w, kh, kw, pads[0], pads[1], pads[2], pads[3],
                              stride[0], stride[1], dil[0], dil[1], _p(col, C.c_int8))
    return col


# --------------------------------------------------------------------------- quantisers

def quantize_per_tensor(x):
    """scale = max|x|/127, q = clip(rint(x/scale), -127, 127)."""
    scale = np.float32(max(float(np.max(np.abs(x))), 1e-12) / 127.0)
    q = np.clip(np.rint(x / scale), -127, 127).astype(np.int8)
    return q, float(scale)


def quantize_per_channel(w, axis=0, qmax=127):
    """Per-output-channel symmetric int8 (quant_dequant_op_fuser.cc:57-73): scale = max|w|/127."""
    red = tuple(i for i in range(w.ndim) if i != axis)
    amax = np.maximum(np.max(np.abs(w), axis=red, keepdims=True), 1e-12)
    scale = (amax / 127.0).astype(np.float32)
    q = np.clip(np.rint(w / scale), -qmax, qmax).astype(np.int8)
    return q, scale.reshape(-1).astype(np.float32)
