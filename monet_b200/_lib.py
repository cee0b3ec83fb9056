"""ctypes binding of ``libmonet_b200.so`` (the C ABI declared in ``include/monet_b200.h``).

There is no fallback: if the shared library is missing, ``lib()`` raises, and every
operator that needs a kernel raises with it.  A non-zero status from an entry point
becomes a ``RuntimeError`` carrying ``mb_last_error()``, which is what the reference's
``try/except`` retry in conv.py:279-283 and the profiler's failure handling in
meminfo.py:52-55 expect from a native op.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libmonet_b200.so"

MB_NCHW, MB_NHWC = 0, 1

c_f = C.c_void_p      # device pointers travel as integers
c_sz = C.c_size_t


class PoolDesc(C.Structure):
    _fields_ = [(n, C.c_int) for n in
                ("N", "C", "H", "W", "P", "Q", "kh", "kw", "sh", "sw", "ph", "pw", "dh", "dw",
                 "layout")]


class BnDesc(C.Structure):
    _fields_ = [("N", C.c_int), ("C", C.c_int), ("HW", C.c_int), ("layout", C.c_int),
                ("eps", C.c_float), ("momentum", C.c_float)]


class ConvDesc(C.Structure):
    _fields_ = [(n, C.c_int) for n in
                ("N", "C", "H", "W", "K", "R", "S", "P", "Q", "stride_h", "stride_w", "pad_h",
                 "pad_w", "dil_h", "dil_w", "groups")]


MB_CONV_FPROP, MB_CONV_DGRAD, MB_CONV_WGRAD = 0, 1, 2
MB_CAT_MAX_PIECES = 8


# name -> (restype, argtypes); every symbol of include/monet_b200.h
PROTOTYPES = {
    "mb_last_error": (C.c_char_p, []),
    "mb_abi_version": (C.c_int, []),
    "mb_launch_count": (C.c_ulonglong, []),
    "mb_relu_fwd": (C.c_int, [c_f, c_f, c_sz, c_f]),
    "mb_relu_fwd_mask": (C.c_int, [c_f, c_f, c_f, c_sz, c_f]),
    "mb_relu_bwd_mask": (C.c_int, [c_f, c_f, c_f, c_sz, c_f]),
    "mb_relu_bwd_act": (C.c_int, [c_f, c_f, C.c_float, c_f, c_sz, c_f]),
    "mb_relu_bwd_act2": (C.c_int, [c_f, c_f, c_f, C.c_float, c_f, c_sz, c_f]),
    "mb_pack_bits": (C.c_int, [c_f, c_f, c_sz, c_f]),
    "mb_unpack_bits": (C.c_int, [c_f, c_f, c_sz, c_f]),
    "mb_unpack_multiply": (C.c_int, [c_f, c_f, c_f, c_sz, c_f]),
    "mb_pack_nibbles": (C.c_int, [c_f, c_f, c_sz, c_f]),
    "mb_unpack_nibbles": (C.c_int, [c_f, c_f, c_sz, c_f]),
    "mb_hardtanh_fwd": (C.c_int, [c_f, c_f, C.c_float, C.c_float, c_sz, c_f]),
    "mb_hardtanh_bwd": (C.c_int, [c_f, c_f, C.c_float, C.c_float, c_f, c_sz, c_f]),
    "mb_add_fwd": (C.c_int, [c_f, c_f, C.c_float, c_f, c_sz, c_f]),
    "mb_add_relu_fwd": (C.c_int, [c_f, c_f, C.c_float, c_f, c_sz, c_f]),
    "mb_scale": (C.c_int, [c_f, C.c_float, c_f, c_sz, c_f]),
    "mb_pool_out_size": (C.c_int, [C.c_int] * 6),
    "mb_maxpool2d_fwd": (C.c_int, [c_f, c_f, c_f, C.POINTER(PoolDesc), c_f]),
    "mb_maxpool2d_bwd": (C.c_int, [c_f, c_f, c_f, C.POINTER(PoolDesc), c_f]),
    "mb_bn_workspace_bytes": (c_sz, [C.POINTER(BnDesc)]),
    "mb_bn_fwd_train": (C.c_int, [c_f] * 8 + [C.POINTER(BnDesc), c_f, c_sz, c_f]),
    "mb_bn_fwd_train_noalloc": (C.c_int, [c_f] * 8 + [C.POINTER(BnDesc), c_f]),
    "mb_bn_fwd_apply": (C.c_int, [c_f] * 6 + [C.POINTER(BnDesc), c_f]),
    "mb_bn_bwd_from_output": (C.c_int, [c_f] * 8 + [C.POINTER(BnDesc), c_f, c_sz, c_f]),
    "mb_bn_bwd_from_input": (C.c_int, [c_f] * 8 + [C.POINTER(BnDesc), c_f, c_sz, c_f]),
    "mb_bn_act_fwd_train": (C.c_int, [c_f, c_f, C.c_int] + [c_f] * 7 + [C.POINTER(BnDesc), c_f, c_sz, c_f]),
    "mb_bn_act_fwd_apply": (C.c_int, [c_f, c_f, C.c_int] + [c_f] * 5 + [C.POINTER(BnDesc), c_f]),
    "mb_bn_act_fwd_train_partials": (C.c_int, [c_f, c_f, C.c_int] + [c_f] * 7 + [C.POINTER(BnDesc), c_f, C.c_int, c_f, c_f]),
    "mb_bn_add_relu_bwd": (C.c_int, [c_f] * 11 + [C.POINTER(BnDesc), c_f, c_sz, c_f]),
    "mb_bn_act_bwd_from_input": (C.c_int, [c_f] * 6 + [C.c_int] + [c_f] * 3 + [C.POINTER(BnDesc), c_f, c_sz, c_f]),
    "mb_bn_relu_bwd_from_input": (C.c_int, [c_f] * 9 + [C.POINTER(BnDesc), c_f, c_sz, c_f]),
    "mb_softmax_fwd": (C.c_int, [c_f, c_f, c_sz, C.c_int, c_sz, C.c_int, c_f]),
    "mb_softmax_bwd": (C.c_int, [c_f, c_f, c_f, c_sz, C.c_int, c_sz, C.c_int, c_f]),
    "mb_softmax_ce_fwd_bwd": (C.c_int, [c_f, c_f, c_f, c_f, c_sz, C.c_int, c_sz, C.c_float, c_f]),
    "mb_nchw_to_nhwc": (C.c_int, [c_f, c_f, C.c_int, C.c_int, C.c_int, C.c_int, c_f]),
    "mb_nhwc_to_nchw": (C.c_int, [c_f, c_f, C.c_int, C.c_int, C.c_int, C.c_int, c_f]),
    "mb_nchw_to_nhwc_pad": (C.c_int, [c_f, c_f, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, c_f]),
    "mb_conv_num_variants": (C.c_int, [C.c_int]),
    "mb_conv_workspace_bytes": (c_sz, [C.c_int, C.c_int, C.POINTER(ConvDesc)]),
    "mb_conv2d_fprop": (C.c_int, [c_f, c_f, c_f, c_f, C.POINTER(ConvDesc), C.c_int, c_f, c_sz, c_f]),
    "mb_conv_bnstats_bytes": (c_sz, [C.POINTER(ConvDesc)]),
    "mb_conv2d_fprop_bnstats": (C.c_int, [c_f, c_f, c_f, c_f, C.POINTER(ConvDesc), C.c_int, c_f, c_sz,
                                           c_f, c_f, c_sz, C.POINTER(C.c_int), c_f]),
    "mb_conv2d_dgrad": (C.c_int, [c_f, c_f, c_f, C.POINTER(ConvDesc), C.c_int, c_f, c_sz, c_f]),
    "mb_conv2d_wgrad": (C.c_int, [c_f, c_f, c_f, c_f, C.POINTER(ConvDesc), C.c_int, c_f, c_sz, c_f]),
    "mb_depthwise_fprop": (C.c_int, [c_f, c_f, c_f, c_f, C.POINTER(ConvDesc), c_f]),
    "mb_depthwise_dgrad": (C.c_int, [c_f, c_f, c_f, C.POINTER(ConvDesc), c_f]),
    "mb_depthwise_wgrad": (C.c_int, [c_f, c_f, c_f, c_f, C.POINTER(ConvDesc), c_f]),
    "mb_conv_device_status": (C.c_int, [C.c_int]),
    "mb_conv_debug_counters": (C.c_int, [c_f]),
    "mb_conv_smallc_geometry": (C.c_int, [C.POINTER(ConvDesc), C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "mb_conv_smallc_pack_input": (C.c_int, [c_f, c_f, C.POINTER(ConvDesc), c_f]),
    "mb_conv2d_fprop_smallc": (C.c_int, [c_f, c_f, c_f, c_f, C.POINTER(ConvDesc), c_f]),
    "mb_conv_smallc2_geometry": (C.c_int, [C.POINTER(ConvDesc), C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "mb_conv_smallc2_pack_input": (C.c_int, [c_f, c_f, C.POINTER(ConvDesc), c_f]),
    "mb_conv2d_fprop_smallc2": (C.c_int, [c_f, c_f, c_f, c_f, C.POINTER(ConvDesc), c_f]),
    "mb_conv_smallc_wgrad_workspace_bytes": (c_sz, [C.POINTER(ConvDesc), C.c_int]),
    "mb_conv2d_wgrad_smallc": (C.c_int, [c_f, c_f, c_f, c_f, C.POINTER(ConvDesc), C.c_int, c_f, c_sz, c_f]),
    "mb_cat_rows": (C.c_int, [c_f, C.POINTER(C.c_void_p), C.POINTER(C.c_int), C.c_int, c_sz, C.c_int, c_f]),
    "mb_global_avgpool_fwd": (C.c_int, [c_f, c_f, C.c_int, C.c_int, C.c_int, C.c_int, c_f]),
    "mb_global_avgpool_bwd": (C.c_int, [c_f, c_f, C.c_int, C.c_int, C.c_int, C.c_int, c_f]),
}

_lib = None
_probe = None     # optional (before, after) callables invoked around every C-ABI call


def set_probe(before=None, after=None) -> None:
    """Install hooks called as before(name) / after(name) around each entry point; used by
    bench.py to bracket launches with CUDA events.  set_probe() removes them."""
    global _probe
    _probe = (before, after) if before is not None and after is not None else None


class _Api:
    """Typed entry points as attributes; routes through the probe hooks when set."""

    def __init__(self, handle):
        self._handle = handle
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(handle, name)     # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
            setattr(self, name, self._wrap(name, fn))

    @staticmethod
    def _wrap(name, fn):
        def call(*a):
            probe = _probe
            if probe is None:
                return fn(*a)
            probe[0](name)
            try:
                return fn(*a)
            finally:
                probe[1](name)
        call.__name__ = name
        return call


def lib() -> "_Api":
    """The loaded library with typed entry points; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m monet_b200.build` "
                "(there is no fallback path)")
        _lib = _Api(C.CDLL(str(LIB_PATH)))
    return _lib


def last_error() -> str:
    return lib().mb_last_error().decode("utf-8", "replace")


def check(status: int, what: str = "") -> None:
    """Raise RuntimeError for a non-zero status of a C-ABI call."""
    if status != 0:
        raise RuntimeError(f"libmonet_b200 {what} failed (status {status}): {last_error()}")
