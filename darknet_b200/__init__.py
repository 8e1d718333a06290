"""darknet_b200: ctypes binding of libdarknet_b200.so, the sm_100a implementation
of Darknet's convolutional forward path.

The Python layer is plumbing only (argument marshalling, device memory through
torch): every computation happens in the CUDA library behind the C ABI declared
in include/darknet_b200.h.  There is no CPU or PyTorch fallback: if the shared
library is missing, or a compute call is made without a CUDA device, an error
is raised.

The module mirrors the reference's own Python binding (python/darknet.py:47-115,
ctypes over libdarknet.so): ``load_network`` / ``network_predict`` keep their
names and argument meaning.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libdarknet_b200.so")

OK, EINVAL, EUNSUPPORTED, ECUDA, EIO, ETIMEOUT, ENOMEM = range(7)
MODE_TF32, MODE_BF16, MODE_FP32 = 0, 1, 2
NCHW, NHWC = 0, 1
F32, BF16 = 0, 1
ACTIVATIONS = {"logistic": 0, "relu": 1, "relie": 2, "linear": 3, "ramp": 4, "tanh": 5, "plse": 6,
               "leaky": 7, "elu": 8, "loggy": 9, "stair": 10, "hardtan": 11, "lhtan": 12, "selu": 13}


class DarknetB200Error(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"[status {status}] {message}")
        self.status = status


class Tensor(C.Structure):
    """struct dnb_tensor."""
    _fields_ = [("data", C.c_void_p), ("layout", C.c_int), ("dtype", C.c_int), ("n", C.c_int), ("c", C.c_int),
                ("h", C.c_int), ("w", C.c_int), ("cpitch", C.c_int)]


class ConvDesc(C.Structure):
    """struct dnb_conv_desc."""
    _fields_ = [(k, C.c_int) for k in ("batch", "h", "w", "c", "n", "groups", "size", "stride", "pad",
                                       "batch_normalize", "activation", "xnor")]


# name -> (restype, argtypes); every symbol include/darknet_b200.h declares
_P, _I, _F = C.c_void_p, C.c_int, C.c_float
_TP = C.POINTER(Tensor)
SIGNATURES = {
    "dnb_last_error": (C.c_char_p, []),
    "dnb_version": (_I, []),
    "dnb_set_device": (_I, [_I]),
    "dnb_device_count": (_I, [C.POINTER(_I)]),
    "dnb_cpitch": (_I, [_I]),
    "dnb_conv_plan_create": (_I, [C.POINTER(ConvDesc), _I, C.POINTER(_P)]),
    "dnb_conv_plan_destroy": (None, [_P]),
    "dnb_conv_plan_set_params": (_I, [_P, _P, _P, _P, _P, _P]),
    "dnb_conv_forward": (_I, [_P, _TP, _TP, _TP, _P]),
    "dnb_conv_xnor_accumulate": (_I, [_P, _TP, _P, _P]),
    "dnb_conv_shortcut_forward": (_I, [_P, _TP, _TP, _TP, _F, _F, _I, _P]),
    "dnb_conv_yolo_forward": (_I, [_P, _TP, _TP, _I, _I, _P]),
    "dnb_conv_plan_check_status": (_I, [_P]),
    "dnb_conv_xnor_forward_static": (_I, [C.POINTER(ConvDesc), _TP, _P, _P, _P, _P, _TP, _P]),
    "dnb_conv_plan_set_diagnostics": (_I, [_P, C.c_longlong, _I]),
    "dnb_conv_plan_kernel": (C.c_char_p, [_P]),
    "dnb_conv_plan_describe": (_I, [_P, C.c_char_p, _I]),
    "dnb_network_layer_describe": (_I, [_P, _I, C.c_char_p, _I]),
    "dnb_maxpool_forward": (_I, [_TP, _TP, _I, _I, _I, _P]),
    "dnb_upsample_forward": (_I, [_TP, _TP, _I, _F, _P]),
    "dnb_shortcut_forward": (_I, [_TP, _TP, _TP, _F, _F, _I, _P]),
    "dnb_route_forward": (_I, [C.POINTER(_TP), _I, _TP, _P]),
    "dnb_convert": (_I, [_TP, _TP, _I, _P]),
    "dnb_yolo_forward": (_I, [_TP, _TP, _I, _I, _P]),
    "dnb_avgpool_forward": (_I, [_TP, _TP, _P]),
    "dnb_softmax_forward": (_I, [_TP, _TP, _I, _F, _P]),
    "dnb_parse_network_cfg": (_I, [C.c_char_p, _I, _I, C.POINTER(_P)]),
    "dnb_parse_network_cfg_text": (_I, [C.c_char_p, _I, _I, C.POINTER(_P)]),
    "dnb_load_weights": (_I, [_P, C.c_char_p]),
    "dnb_load_weights_packed": (_I, [_P, C.c_char_p]),
    "dnb_free_network": (None, [_P]),
    "dnb_network_predict": (_I, [_P, _P, C.POINTER(C.POINTER(_F))]),
    "dnb_network_set_conv_params": (_I, [_P, _I, _P, _P, _P, _P, _P]),
    "dnb_network_export_layer": (_I, [_P, _I, _P, _P]),
    "dnb_network_enable_graph": (_I, [_P, _I]),
    "dnb_network_submit": (_I, [_P, _P]),
    "dnb_network_collect": (_I, [_P, C.POINTER(C.POINTER(_F))]),
    "dnb_network_forward": (_I, [_P, _P, _P]),
    "dnb_network_num_layers": (_I, [_P]),
    "dnb_network_batch": (_I, [_P]),
    "dnb_network_inputs": (_I, [_P]),
    "dnb_network_outputs": (_I, [_P]),
    "dnb_network_layer_shape": (_I, [_P, _I, C.POINTER(_I), C.POINTER(_I), C.POINTER(_I)]),
    "dnb_network_layer_type": (C.c_char_p, [_P, _I]),
    "dnb_network_layer_kernel": (C.c_char_p, [_P, _I]),
    "dnb_network_layer_output": (_I, [_P, _I, _P]),
    "dnb_network_layer_output_images": (_I, [_P, _I, _I, _I, _P]),
    "dnb_network_check_status": (_I, [_P]),
    "dnb_network_set_diagnostics": (_I, [_P, _I, C.c_longlong, _I]),
    "dnb_network_yolo_output": (_I, [_P, _I, C.POINTER(C.POINTER(_F))]),
    "dnb_network_flops": (C.c_double, [_P]),
    "dnb_network_launches": (_I, [_P]),
    "dnb_network_profile": (_I, [_P, _P, _P]),
    "dnb_network_forward_timed": (_I, [_P, _P, _P, _I]),
    "dnb_network_timed_ms": (_I, [_P, _I, _P]),
}

_lib = None


def lib() -> C.CDLL:
    """The loaded shared library.  Raises if it has not been built: there is no
    fallback implementation."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `make -C {os.path.join(HERE, 'csrc')}` "
                              "(or __graft_entry__.build()); darknet_b200 has no fallback path")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError if the library does not export a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(status: int) -> None:
    if status != OK:
        raise DarknetB200Error(status, lib().dnb_last_error().decode())


from .api import (ConvPlan, Network, as_tensor, avgpool, convert, load_network, maxpool, network_predict,  # noqa: E402
                  route, shortcut, softmax, upsample, yolo)

__all__ = ["lib", "check", "Tensor", "ConvDesc", "ConvPlan", "Network", "load_network", "network_predict", "as_tensor",
           "maxpool", "upsample", "shortcut", "route", "convert", "yolo", "avgpool", "softmax", "DarknetB200Error"]
