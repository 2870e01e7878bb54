"""paddle-lite_b200: Python binding of the plb200 C ABI (include/plb200.h).

The package is a thin ctypes layer: torch supplies device memory and the CUDA stream, every
computation goes through ``libplb200.so``.  There is no CPU or eager fallback: if the shared
object is missing or the device is not an sm_100 GPU, calls raise.

The directory name contains a hyphen, so import it with
``importlib.import_module("paddle-lite_b200")``.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# PLB200_LIBRARY selects another build of the same library (e.g. one compiled with extra diagnostics)
LIB_PATH = os.environ.get("PLB200_LIBRARY") or os.path.join(HERE, "libplb200.so")

OK, E_INVALID, E_UNSUPPORTED, E_CUDA, E_DEVICE, E_NOMEM = range(6)
ACT_NONE, ACT_RELU, ACT_RELU6, ACT_LEAKY = 0, 1, 2, 3
OUT_F32, OUT_I8 = 0, 1
IMPL_AUTO, IMPL_DIRECT, IMPL_TC = 0, 1, 2


class PlbError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("plb200 error %d: %s" % (code, msg))
        self.code = code


class ConvDesc(C.Structure):
    _fields_ = [("cin", C.c_int), ("h", C.c_int), ("w", C.c_int),
                ("cout", C.c_int), ("kh", C.c_int), ("kw", C.c_int),
                ("stride_h", C.c_int), ("stride_w", C.c_int),
                ("pad_top", C.c_int), ("pad_bottom", C.c_int), ("pad_left", C.c_int), ("pad_right", C.c_int),
                ("dil_h", C.c_int), ("dil_w", C.c_int),
                ("groups", C.c_int), ("act", C.c_int), ("act_alpha", C.c_float),
                ("in_scale", C.c_float), ("out_scale", C.c_float),
                ("out_dtype", C.c_int), ("leaky_compat", C.c_int), ("impl", C.c_int)]


class SparseDesc(C.Structure):
    _fields_ = [("cin", C.c_int), ("cout", C.c_int), ("h", C.c_int), ("w", C.c_int),
                ("is_int8", C.c_int), ("out_dtype", C.c_int),
                ("flag_semi", C.c_int), ("first_ic", C.c_int),
                ("act", C.c_int), ("act_alpha", C.c_float),
                ("in_scale", C.c_float), ("out_scale", C.c_float),
                ("leaky_compat", C.c_int), ("impl", C.c_int)]


# name -> (restype, argtypes); every symbol include/plb200.h declares
_P = C.c_void_p
SYMBOLS = {
    "plb_ctx_create": (C.c_int, [C.c_int, _P, C.POINTER(_P)]),
    "plb_ctx_destroy": (None, [_P]),
    "plb_ctx_sync": (C.c_int, [_P]),
    "plb_ctx_set_workspace": (C.c_int, [_P, _P, C.c_size_t]),
    "plb_conv_workspace_bytes": (C.c_size_t, [_P, C.c_int]),
    "plb_last_error": (C.c_char_p, []),
    "plb_ctx_launch_count": (C.c_long, [_P]),
    "plb_ctx_window_launch_count": (C.c_long, [_P]),
    "plb_ctx_nchw_launch_count": (C.c_long, [_P]),
    "plb_ctx_pair_launch_count": (C.c_long, [_P]),
    "plb_ctx_dwpw_launch_count": (C.c_long, [_P]),
    "plb_ctx_stem_launch_count": (C.c_long, [_P]),
    "plb_ctx_nchw_gather_launch_count": (C.c_long, [_P]),
    "plb_conv_dwpw_fusable": (C.c_int, [_P, _P]),
    "plb_conv_run_nhwc_dwpw": (C.c_int, [_P, _P, _P, _P, C.c_int]),
    "plb_ctx_workspace_size": (C.c_size_t, [_P]),
    "plb_conv_plan_cache_hits": (C.c_long, [_P]),
    "plb_conv_prepare": (C.c_int, [_P, C.POINTER(ConvDesc), _P, _P, C.c_int, _P, C.POINTER(_P)]),
    "plb_conv_run": (C.c_int, [_P, _P, _P, C.c_int]),
    "plb_conv_run_nhwc": (C.c_int, [_P, _P, _P, C.c_int]),
    "plb_conv_acc_i32": (C.c_int, [_P, _P, _P, C.c_int]),
    "plb_conv_run_static": (C.c_int, [_P, _P, _P, C.c_int]),
    "plb_conv_run_image_f32": (C.c_int, [_P, _P, _P, C.c_int]),
    "plb_conv_run_nhwc_add_relu": (C.c_int, [_P, _P, _P, _P, _P, C.c_float, C.c_int]),
    "plb_conv_run_nhwc_block_add_relu": (C.c_int, [_P, _P, _P, _P, _P, _P, C.c_float, C.c_int]),
    "plb_conv_out_dims": (C.c_int, [_P, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "plb_conv_destroy": (None, [_P]),
    "plb_fc_prepare": (C.c_int, [_P, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float, C.c_float, C.c_int,
                                 _P, _P, C.c_int, _P, C.POINTER(_P)]),
    "plb_fc_run": (C.c_int, [_P, _P, _P, C.c_int]),
    "plb_fc_acc_i32": (C.c_int, [_P, _P, _P, C.c_int]),
    "plb_fc_destroy": (None, [_P]),
    "plb_sparse_prepare": (C.c_int, [_P, C.POINTER(SparseDesc), _P, C.c_int, _P, _P, C.c_int, _P, C.c_int,
                                     _P, C.POINTER(_P)]),
    "plb_sparse_run": (C.c_int, [_P, _P, _P, C.c_int]),
    "plb_sparse_destroy": (None, [_P]),
    "plb_calib_f32_to_i8": (C.c_int, [_P, _P, _P, C.c_size_t, C.c_float]),
    "plb_softmax_f32": (C.c_int, [_P, _P, _P, C.c_int, C.c_int]),
    "plb_copy_h2d": (C.c_int, [_P, _P, _P, C.c_size_t]),
    "plb_copy_d2h": (C.c_int, [_P, _P, _P, C.c_size_t]),
    "plb_calib_i8_to_f32": (C.c_int, [_P, _P, _P, C.c_size_t, C.c_float]),
    "plb_nchw_to_nhwc_i8": (C.c_int, [_P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "plb_nhwc_to_nchw": (C.c_int, [_P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "plb_calib_nchw_f32_to_nhwc_i8": (C.c_int, [_P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                                C.c_float]),
    "plb_maxpool_nhwc_i8": (C.c_int, [_P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                      C.c_int]),
    "plb_global_avgpool_nhwc_f32": (C.c_int, [_P, _P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_float]),
}

_lib = None


def lib():
    """The loaded C-ABI library.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError("%s is missing: run `python paddle-lite_b200/build.py` "
                               "(there is no fallback path)" % LIB_PATH)
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def _check(rc):
    if rc != OK:
        raise PlbError(rc, lib().plb_last_error().decode("utf-8", "replace"))


def _np_ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _dev_ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


class Context:
    """One device + one CUDA stream (the reference keeps these in Context<TARGET>,
    lite/core/context.h:430-484)."""

    def __init__(self, device=0, stream=None):
        import torch
        import weakref
        self.device = device
        self._stream = stream if stream is not None else torch.cuda.current_stream(device)
        self._children = weakref.WeakSet()  # prepared layers; they must be destroyed before the ctx
        self.handle = _P()
        _check(lib().plb_ctx_create(device, C.c_void_p(self._stream.cuda_stream), C.byref(self.handle)))

    def sync(self):
        _check(lib().plb_ctx_sync(self.handle))

    def launch_count(self):
        return lib().plb_ctx_launch_count(self.handle)

    def window_launch_count(self):
        return lib().plb_ctx_window_launch_count(self.handle)

    def nchw_launch_count(self):
        return lib().plb_ctx_nchw_launch_count(self.handle)

    def pair_launch_count(self):
        return lib().plb_ctx_pair_launch_count(self.handle)

    def nchw_gather_launch_count(self):
        return lib().plb_ctx_nchw_gather_launch_count(self.handle)

    def stem_launch_count(self):
        return lib().plb_ctx_stem_launch_count(self.handle)

    def dwpw_launch_count(self):
        return lib().plb_ctx_dwpw_launch_count(self.handle)

    def workspace_size(self):
        return lib().plb_ctx_workspace_size(self.handle)

    def set_workspace(self, tensor):
        self._ws = tensor
        _check(lib().plb_ctx_set_workspace(self.handle, _dev_ptr(tensor),
                                           0 if tensor is None else tensor.numel() * tensor.element_size()))

    def close(self):
        if self.handle:
            for child in list(self._children):
                child.close()
            lib().plb_ctx_destroy(self.handle)
            self.handle = _P()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # glue ------------------------------------------------------------
    def calib_f32_to_i8(self, x, scale):
        import torch
        q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
        _check(lib().plb_calib_f32_to_i8(self.handle, _dev_ptr(x), _dev_ptr(q), x.numel(), scale))
        return q

    def calib_i8_to_f32(self, q, scale):
        import torch
        y = torch.empty(q.shape, dtype=torch.float32, device=q.device)
        _check(lib().plb_calib_i8_to_f32(self.handle, _dev_ptr(q), _dev_ptr(y), q.numel(), scale))
        return y

    def nchw_to_nhwc_i8(self, x, cpad=None):
        import torch
        n, c, h, w = x.shape
        cpad = cpad or c
        y = torch.empty((n, h, w, cpad), dtype=torch.int8, device=x.device)
        _check(lib().plb_nchw_to_nhwc_i8(self.handle, _dev_ptr(x), _dev_ptr(y), n, c, h, w, cpad))
        return y

    def nhwc_to_nchw(self, x):
        import torch
        n, h, w, c = x.shape
        y = torch.empty((n, c, h, w), dtype=x.dtype, device=x.device)
        _check(lib().plb_nhwc_to_nchw(self.handle, _dev_ptr(x), _dev_ptr(y), n, c, h, w, x.element_size()))
        return y

    def calib_nchw_f32_to_nhwc_i8(self, x, cpad, scale, out=None):
        import torch
        n, c, h, w = x.shape
        y = out if out is not None else torch.empty((n, h, w, cpad), dtype=torch.int8, device=x.device)
        _check(lib().plb_calib_nchw_f32_to_nhwc_i8(self.handle, _dev_ptr(x), _dev_ptr(y), n, c, h, w, cpad,
                                                   scale))
        return y

    def maxpool_nhwc_i8(self, x, k, stride, pad, out=None):
        import torch
        n, h, w, c = x.shape
        ho, wo = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
        y = out if out is not None else torch.empty((n, ho, wo, c), dtype=torch.int8, device=x.device)
        _check(lib().plb_maxpool_nhwc_i8(self.handle, _dev_ptr(x), _dev_ptr(y), n, c, h, w, k, stride, pad))
        return y

    def copy_h2d(self, dst, src_host):
        """Enqueue a host -> device copy of a C-contiguous numpy array into `dst` on the ctx stream."""
        _check(lib().plb_copy_h2d(self.handle, _dev_ptr(dst), C.c_void_p(src_host.ctypes.data), src_host.nbytes))

    def copy_d2h(self, dst_host, src):
        """Device -> host copy into a C-contiguous numpy array; returns when the bytes have arrived."""
        _check(lib().plb_copy_d2h(self.handle, C.c_void_p(dst_host.ctypes.data), _dev_ptr(src), dst_host.nbytes))

    def softmax(self, x, out=None):
        """Row softmax of a [rows, cols] fp32 tensor (reference form: shift by the row max, clip at -64)."""
        import torch
        rows, cols = x.shape
        y = out if out is not None else torch.empty_like(x)
        _check(lib().plb_softmax_f32(self.handle, _dev_ptr(x), _dev_ptr(y), rows, cols))
        return y

    def global_avgpool_nhwc_f32(self, x, scale=None, out_f32=None, out_i8=None):
        import torch
        n, h, w, c = x.shape
        y = out_f32 if out_f32 is not None else torch.empty((n, c), dtype=torch.float32, device=x.device)
        q = out_i8
        if scale is not None and q is None:
            q = torch.empty((n, c), dtype=torch.int8, device=x.device)
        _check(lib().plb_global_avgpool_nhwc_f32(self.handle, _dev_ptr(x), _dev_ptr(y), _dev_ptr(q), n, h * w,
                                                 c, scale if scale is not None else 1.0))
        return y, q


class Conv:
    """A prepared int8 conv2d / depthwise_conv2d layer (= one reference kernel instance after
    PrepareForRun, lite/kernels/x86/conv_compute.cc:216-289, :344-420)."""

    def __init__(self, ctx, filter_oihw, wscale, in_scale, bias=None, *, in_hw, stride=(1, 1),
                 pads=(0, 0, 0, 0), dil=(1, 1), groups=1, act=ACT_NONE, alpha=0.0, out_scale=None,
                 leaky_compat=False, impl=IMPL_AUTO):
        import numpy as np
        self.ctx = ctx
        f = np.ascontiguousarray(filter_oihw, dtype=np.int8)
        cout, cig, kh, kw = f.shape
        ws = np.ascontiguousarray(np.atleast_1d(wscale), dtype=np.float32)
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        d = ConvDesc(cin=cig * groups, h=in_hw[0], w=in_hw[1], cout=cout, kh=kh, kw=kw,
                     stride_h=stride[0], stride_w=stride[1], pad_top=pads[0], pad_bottom=pads[1],
                     pad_left=pads[2], pad_right=pads[3], dil_h=dil[0], dil_w=dil[1], groups=groups,
                     act=act, act_alpha=alpha, in_scale=in_scale,
                     out_scale=out_scale if out_scale is not None else 1.0,
                     out_dtype=OUT_I8 if out_scale is not None else OUT_F32,
                     leaky_compat=int(bool(leaky_compat)), impl=impl)
        self.desc = d
        self.out_is_i8 = out_scale is not None
        self.handle = _P()
        _check(lib().plb_conv_prepare(ctx.handle, C.byref(d), _np_ptr(f), _np_ptr(ws), int(ws.size),
                                      _np_ptr(b), C.byref(self.handle)))
        ctx._children.add(self)
        ho, wo = C.c_int(), C.c_int()
        _check(lib().plb_conv_out_dims(self.handle, C.byref(ho), C.byref(wo)))
        self.ho, self.wo = ho.value, wo.value

    def workspace_bytes(self, batch):
        return lib().plb_conv_workspace_bytes(self.handle, batch)

    def plan_cache_hits(self):
        return lib().plb_conv_plan_cache_hits(self.handle)

    def run(self, x, out=None):
        """x [N,Cin,H,W] int8 cuda -> [N,Cout,Ho,Wo] int8 or float32 (NCHW, reference layout)."""
        import torch
        n = x.shape[0]
        y = out if out is not None else torch.empty(
            (n, self.desc.cout, self.ho, self.wo), dtype=torch.int8 if self.out_is_i8 else torch.float32,
            device=x.device)
        _check(lib().plb_conv_run(self.handle, _dev_ptr(x), _dev_ptr(y), n))
        return y

    def acc_i32(self, x):
        import torch
        n = x.shape[0]
        y = torch.empty((n, self.desc.cout, self.ho, self.wo), dtype=torch.int32, device=x.device)
        _check(lib().plb_conv_acc_i32(self.handle, _dev_ptr(x), _dev_ptr(y), n))
        return y

    def run_static(self, x, out):
        """plb_conv_run_static: like run(), staged in the library's built-in 8 MiB scratch, no
        device allocation by the library.  `out` must be supplied by the caller."""
        _check(lib().plb_conv_run_static(self.handle, _dev_ptr(x), _dev_ptr(out), x.shape[0]))
        return out

    def run_nhwc(self, x, out=None):
        """x [N,H,W,Cin] int8 -> [N,Ho,Wo,Cout]."""
        import torch
        n = x.shape[0]
        y = out if out is not None else torch.empty(
            (n, self.ho, self.wo, self.desc.cout), dtype=torch.int8 if self.out_is_i8 else torch.float32,
            device=x.device)
        _check(lib().plb_conv_run_nhwc(self.handle, _dev_ptr(x), _dev_ptr(y), n))
        return y

    def run_image_f32(self, x, out=None):
        """x [N,Cin,H,W] float32 (NCHW image) -> [N,Ho,Wo,Cout]; calib + staging + layer."""
        import torch
        n = x.shape[0]
        y = out if out is not None else torch.empty(
            (n, self.ho, self.wo, self.desc.cout), dtype=torch.int8 if self.out_is_i8 else torch.float32,
            device=x.device)
        _check(lib().plb_conv_run_image_f32(self.handle, _dev_ptr(x), _dev_ptr(y), n))
        return y

    def run_nhwc_add_relu(self, x, residual=None, next_scale=None, want_f32=True, out_f32=None, out_i8=None):
        import torch
        n = x.shape[0]
        shape = (n, self.ho, self.wo, self.desc.cout)
        yf = out_f32 if out_f32 is not None else (
            torch.empty(shape, dtype=torch.float32, device=x.device) if want_f32 else None)
        yq = out_i8 if out_i8 is not None else (
            torch.empty(shape, dtype=torch.int8, device=x.device) if next_scale is not None else None)
        _check(lib().plb_conv_run_nhwc_add_relu(self.handle, _dev_ptr(x), _dev_ptr(residual), _dev_ptr(yf),
                                                _dev_ptr(yq), next_scale if next_scale is not None else 1.0,
                                                n))
        return yf, yq

    def run_nhwc_block_add_relu(self, x, shortcut, x_shortcut, next_scale=None, want_f32=True, out_f32=None,
                                out_i8=None):
        """relu(self(x) + shortcut(x_shortcut)) in one launch (both unpadded 1x1 fp32-out layers without
        activation); returns (fp32 tensor or None, int8 calib(next_scale) tensor or None)."""
        import torch
        n = x.shape[0]
        shape = (n, self.ho, self.wo, self.desc.cout)
        yf = out_f32 if out_f32 is not None else (
            torch.empty(shape, dtype=torch.float32, device=x.device) if want_f32 else None)
        yq = out_i8 if out_i8 is not None else (
            torch.empty(shape, dtype=torch.int8, device=x.device) if next_scale is not None else None)
        _check(lib().plb_conv_run_nhwc_block_add_relu(self.handle, _dev_ptr(x), shortcut.handle, _dev_ptr(x_shortcut),
                                                      _dev_ptr(yf), _dev_ptr(yq),
                                                      next_scale if next_scale is not None else 1.0, n))
        return yf, yq

    def dwpw_fusable(self, pointwise):
        """Whether this depthwise 3x3 layer and the 1x1 layer `pointwise` can run as one launch."""
        return bool(lib().plb_conv_dwpw_fusable(self.handle, pointwise.handle))

    def run_nhwc_dwpw(self, pointwise, x, out=None):
        """pointwise(self(x)) in one launch: self a depthwise 3x3 layer, `pointwise` the 1x1 layer on its output,
        both int8-out; the tensor between them is never written.  x [n,h,w,c] int8 channels-last."""
        import torch
        n = x.shape[0]
        y = out if out is not None else torch.empty((n, pointwise.ho, pointwise.wo, pointwise.desc.cout),
                                                    dtype=torch.int8, device=x.device)
        _check(lib().plb_conv_run_nhwc_dwpw(self.handle, pointwise.handle, _dev_ptr(x), _dev_ptr(y), n))
        return y

    def close(self):
        if self.handle:
            lib().plb_conv_destroy(self.handle)
            self.handle = _P()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Fc:
    """A prepared int8 fc layer (lite/kernels/x86/fc_compute.cc:176-269; scale and bias per
    output feature as lite/kernels/arm/fc_compute.cc:207-260)."""

    def __init__(self, ctx, w_kn, wscale, in_scale, bias=None, act=ACT_NONE, alpha=0.0, out_scale=None):
        import numpy as np
        self.ctx = ctx
        w = np.ascontiguousarray(w_kn, dtype=np.int8)
        self.k, self.n = w.shape
        ws = np.ascontiguousarray(np.atleast_1d(wscale), dtype=np.float32)
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        self.out_is_i8 = out_scale is not None
        self.handle = _P()
        _check(lib().plb_fc_prepare(ctx.handle, self.k, self.n, act, alpha, in_scale,
                                    out_scale if out_scale is not None else 1.0,
                                    OUT_I8 if self.out_is_i8 else OUT_F32, _np_ptr(w), _np_ptr(ws),
                                    int(ws.size), _np_ptr(b), C.byref(self.handle)))
        ctx._children.add(self)

    def run(self, x, out=None):
        import torch
        m = x.shape[0]
        y = out if out is not None else torch.empty(
            (m, self.n), dtype=torch.int8 if self.out_is_i8 else torch.float32, device=x.device)
        _check(lib().plb_fc_run(self.handle, _dev_ptr(x), _dev_ptr(y), m))
        return y

    def acc_i32(self, x):
        import torch
        m = x.shape[0]
        y = torch.empty((m, self.n), dtype=torch.int32, device=x.device)
        _check(lib().plb_fc_acc_i32(self.handle, _dev_ptr(x), _dev_ptr(y), m))
        return y

    def close(self):
        if self.handle:
            lib().plb_fc_destroy(self.handle)
            self.handle = _P()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class SparseConv:
    """A prepared sparse_conv2d (1x1) layer over the reference's encoding
    (lite/kernels/arm/sparse_conv_compute.cc:33-267)."""

    def __init__(self, ctx, nonzero_weights, oc_nonzeros, diffs, first_ic, flag_semi, *, cin, cout, in_hw,
                 wscale=None, in_scale=1.0, bias=None, act=ACT_NONE, alpha=0.0, out_scale=None,
                 leaky_compat=False, impl=IMPL_AUTO):
        import numpy as np
        self.ctx = ctx
        nz = np.ascontiguousarray(nonzero_weights)
        is_i8 = nz.dtype == np.int8
        if not is_i8:
            nz = np.ascontiguousarray(nz, dtype=np.float32)
        cum = np.ascontiguousarray(oc_nonzeros, dtype=np.uint32)
        df = np.ascontiguousarray(diffs, dtype=np.int32)
        ws = None if wscale is None else np.ascontiguousarray(np.atleast_1d(wscale), dtype=np.float32)
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        self.out_is_i8 = out_scale is not None
        self.is_i8 = is_i8
        d = SparseDesc(cin=cin, cout=cout, h=in_hw[0], w=in_hw[1], is_int8=int(is_i8),
                       out_dtype=OUT_I8 if self.out_is_i8 else OUT_F32, flag_semi=int(flag_semi),
                       first_ic=int(first_ic), act=act, act_alpha=alpha, in_scale=in_scale,
                       out_scale=out_scale if out_scale is not None else 1.0,
                       leaky_compat=int(bool(leaky_compat)), impl=impl)
        self.desc = d
        self.handle = _P()
        _check(lib().plb_sparse_prepare(ctx.handle, C.byref(d), _np_ptr(nz), int(nz.size), _np_ptr(cum),
                                        _np_ptr(df), int(df.size), _np_ptr(ws),
                                        0 if ws is None else int(ws.size), _np_ptr(b), C.byref(self.handle)))
        ctx._children.add(self)

    def run(self, x, out=None):
        import torch
        n = x.shape[0]
        y = out if out is not None else torch.empty(
            (n, self.desc.cout, self.desc.h, self.desc.w),
            dtype=torch.int8 if self.out_is_i8 else torch.float32, device=x.device)
        _check(lib().plb_sparse_run(self.handle, _dev_ptr(x), _dev_ptr(y), n))
        return y

    def close(self):
        if self.handle:
            lib().plb_sparse_destroy(self.handle)
            self.handle = _P()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
