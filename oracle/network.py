"""Whole-network CPU forward built on the C restatement (liboracle.so).

TEST INFRASTRUCTURE ONLY: the checker the CUDA path is compared with.  Only the
test-suite, the smoke check and the benchmark's CPU-baseline leg import this
module; the shipped library never does.

It follows the reference's ``parse_network_cfg`` (src/parser.c:742-889) for the
layer geometry and ``forward_network`` (src/network.c:188-211) for the loop:
each layer reads the previous layer's output (or, for shortcut/route, the
outputs of the layers it names) and every layer's output is kept.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ACT = {"logistic": 0, "relu": 1, "relie": 2, "linear": 3, "ramp": 4, "tanh": 5, "plse": 6,
       "leaky": 7, "elu": 8, "loggy": 9, "stair": 10, "hardtan": 11, "lhtan": 12, "selu": 13}

_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")


class ConvDesc(C.Structure):
    _fields_ = [(k, C.c_int) for k in ("batch", "h", "w", "c", "n", "groups", "size", "stride", "pad",
                                       "batch_normalize", "activation", "xnor")]


def build(ref: bool = False) -> None:
    """Compile liboracle.so (and, with ``ref``, the unmodified reference under
    oracle/_ref when its sources are present)."""
    targets = ["all"] + (["ref"] if ref else [])
    subprocess.run(["make", "-s", "-C", HERE] + targets, check=True,
                   stdout=subprocess.DEVNULL, stderr=subprocess.PIPE)


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        path = os.path.join(HERE, "liboracle.so")
        if not os.path.exists(path):
            build()
        L = C.CDLL(path)
        L.orc_conv_forward.argtypes = [C.POINTER(ConvDesc)] + [C.c_void_p] * 8
        L.orc_xnor_accumulate.argtypes = [C.POINTER(ConvDesc)] + [C.c_void_p] * 4
        L.orc_conv_workspace_bytes.argtypes = [C.POINTER(ConvDesc)]
        L.orc_conv_workspace_bytes.restype = C.c_size_t
        L.orc_maxpool_forward.argtypes = [C.c_void_p] + [C.c_int] * 7 + [C.c_void_p, C.c_void_p]
        L.orc_upsample_forward.argtypes = [C.c_void_p] + [C.c_int] * 5 + [C.c_float, C.c_void_p]
        L.orc_shortcut_forward.argtypes = [C.c_void_p, C.c_void_p] + [C.c_int] * 7 + [C.c_float, C.c_float, C.c_int, C.c_void_p]
        L.orc_route_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        L.orc_yolo_forward.argtypes = [C.c_void_p] + [C.c_int] * 5 + [C.c_void_p]
        L.orc_avgpool_forward.argtypes = [C.c_void_p] + [C.c_int] * 4 + [C.c_void_p]
        L.orc_softmax_forward.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_void_p]
        L.orc_connected_forward.argtypes = [C.c_int] * 5 + [C.c_void_p] * 7
        L.orc_im2col.argtypes = [C.c_void_p] + [C.c_int] * 6 + [C.c_void_p]
        L.orc_gemm_nn.argtypes = [C.c_int] * 3 + [C.c_float, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_int]
        L.orc_activate_array.argtypes = [C.c_void_p, C.c_long, C.c_int]
        _lib = L
    return _lib


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


# ------------------------------------------------------------------ single layers


def conv_forward(x, weights, biases, scales=None, mean=None, var=None, *, stride=1, pad=0, groups=1,
                 activation="linear", xnor=False):
    """x [B,C,H,W], weights [N,C/groups,k,k]; ``pad`` is the padding in pixels."""
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(weights, np.float32)
    B, Cc, H, W = x.shape
    d = ConvDesc(B, H, W, Cc, w.shape[0], groups, w.shape[2], stride, pad, int(scales is not None),
                 ACT[activation], int(xnor))
    oh, ow = (H + 2 * pad - d.size) // stride + 1, (W + 2 * pad - d.size) // stride + 1
    out = np.empty((B, d.n, oh, ow), np.float32)
    ws = np.empty(lib().orc_conv_workspace_bytes(C.byref(d)) // 4 + 1, np.float32)
    args = [np.ascontiguousarray(a, np.float32) if a is not None else None for a in (biases, scales, mean, var)]
    lib().orc_conv_forward(C.byref(d), _p(x), _p(w), _p(args[0]), _p(args[1]), _p(args[2]), _p(args[3]), _p(out), _p(ws))
    return out


def xnor_accumulate(x, weights, *, stride=1, pad=0):
    """Integer accumulators (as exact fp32) of the sign(w) x sign(x) convolution."""
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(weights, np.float32)
    B, Cc, H, W = x.shape
    d = ConvDesc(B, H, W, Cc, w.shape[0], 1, w.shape[2], stride, pad, 0, ACT["linear"], 1)
    oh, ow = (H + 2 * pad - d.size) // stride + 1, (W + 2 * pad - d.size) // stride + 1
    out = np.empty((B, d.n, oh, ow), np.float32)
    ws = np.empty(lib().orc_conv_workspace_bytes(C.byref(d)) // 4 + 1, np.float32)
    lib().orc_xnor_accumulate(C.byref(d), _p(x), _p(w), _p(out), _p(ws))
    return out


def maxpool_forward(x, size, stride, pad=None):
    x = np.ascontiguousarray(x, np.float32)
    B, Cc, H, W = x.shape
    pad = size - 1 if pad is None else pad
    oh, ow = (H + pad - size) // stride + 1, (W + pad - size) // stride + 1
    out = np.empty((B, Cc, oh, ow), np.float32)
    lib().orc_maxpool_forward(_p(x), B, Cc, H, W, size, stride, pad, _p(out), None)
    return out


def upsample_forward(x, stride=2, scale=1.0):
    x = np.ascontiguousarray(x, np.float32)
    B, Cc, H, W = x.shape
    out = np.empty((B, Cc, H * stride, W * stride), np.float32)
    lib().orc_upsample_forward(_p(x), B, Cc, H, W, stride, scale, _p(out))
    return out


def shortcut_forward(x, add, alpha=1.0, beta=1.0, activation="linear"):
    """x [B,c2,h2,w2] is the layer's input, add [B,c1,h1,w1] the earlier output."""
    x = np.ascontiguousarray(x, np.float32)
    add = np.ascontiguousarray(add, np.float32)
    B, c2, h2, w2 = x.shape
    _, c1, h1, w1 = add.shape
    out = np.empty_like(x)
    lib().orc_shortcut_forward(_p(x), _p(add), B, w1, h1, c1, w2, h2, c2, alpha, beta, ACT[activation], _p(out))
    return out


def route_forward(inputs):
    inputs = [np.ascontiguousarray(a, np.float32) for a in inputs]
    B = inputs[0].shape[0]
    sizes = np.array([a[0].size for a in inputs], np.int32)
    ptrs = (C.c_void_p * len(inputs))(*[a.ctypes.data for a in inputs])
    same = all(a.shape[2:] == inputs[0].shape[2:] for a in inputs)
    shape = (B, sum(a.shape[1] for a in inputs)) + inputs[0].shape[2:] if same else (B, int(sizes.sum()))
    out = np.empty(shape, np.float32)
    lib().orc_route_forward(ptrs, _p(sizes), len(inputs), B, _p(out))
    return out


def yolo_forward(x, n, classes):
    x = np.ascontiguousarray(x, np.float32)
    B, Cc, H, W = x.shape
    out = np.empty_like(x)
    lib().orc_yolo_forward(_p(x), B, n, classes, H, W, _p(out))
    return out


def avgpool_forward(x):
    x = np.ascontiguousarray(x, np.float32)
    B, Cc, H, W = x.shape
    out = np.empty((B, Cc, 1, 1), np.float32)
    lib().orc_avgpool_forward(_p(x), B, Cc, H, W, _p(out))
    return out


def connected_forward(x, weights, biases, scales=None, mean=None, var=None, *, activation="linear"):
    """x [B, ...] flattened per image in the reference's order, weights [outputs, inputs]; returns [B, outputs, 1, 1]."""
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(weights, np.float32)
    B = x.shape[0]
    outputs, inputs = w.shape
    assert x[0].size == inputs
    out = np.empty((B, outputs, 1, 1), np.float32)
    args = [np.ascontiguousarray(a, np.float32) if a is not None else None for a in (biases, scales, mean, var)]
    lib().orc_connected_forward(B, inputs, outputs, int(scales is not None), ACT[activation], _p(x), _p(w),
                                _p(args[0]), _p(args[1]), _p(args[2]), _p(args[3]), _p(out))
    return out


def softmax_forward(x, groups=1, temperature=1.0):
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty_like(x)
    lib().orc_softmax_forward(_p(x), x.shape[0], x[0].size, groups, temperature, _p(out))
    return out


# ------------------------------------------------------------------ whole network


def forward_network(cfg_text: str, params, x: np.ndarray, upto: int | None = None) -> list[np.ndarray]:
    """Run the cfg on input x [B,C,H,W]; returns every layer's output (NCHW).

    ``params`` is the list of per-convolution parameter records in file order
    (objects with weights, biases, scales, rolling_mean, rolling_variance)."""
    from darknet_b200.synth import parse_cfg  # text splitting only

    sections = parse_cfg(cfg_text)[1:]
    outs: list[np.ndarray] = []
    cur = np.ascontiguousarray(x, np.float32)
    pi = 0
    for idx, (kind, opt) in enumerate(sections):
        if upto is not None and idx >= upto:
            break
        if kind == "convolutional":
            p = params[pi]
            pi += 1
            size = int(opt.get("size", 1))
            # src/parser.c:184-187: "pad=1" means padding = size/2
            padding = size // 2 if int(opt.get("pad", 0)) else int(opt.get("padding", 0))
            cur = conv_forward(cur, p.weights, p.biases, p.scales, p.rolling_mean, p.rolling_variance,
                               stride=int(opt.get("stride", 1)), pad=padding, groups=int(opt.get("groups", 1)),
                               activation=opt.get("activation", "logistic"), xnor=bool(int(opt.get("xnor", 0))))
        elif kind == "connected":
            p = params[pi]
            pi += 1
            cur = connected_forward(cur, p.weights, p.biases, p.scales, p.rolling_mean, p.rolling_variance,
                                    activation=opt.get("activation", "logistic"))
        elif kind == "maxpool":
            stride = int(opt.get("stride", 1))
            size = int(opt.get("size", stride))
            cur = maxpool_forward(cur, size, stride, int(opt.get("padding", size - 1)))
        elif kind == "upsample":
            cur = upsample_forward(cur, int(opt.get("stride", 2)), float(opt.get("scale", 1)))
        elif kind == "shortcut":
            frm = int(opt["from"])
            frm = frm if frm >= 0 else idx + frm
            cur = shortcut_forward(cur, outs[frm], float(opt.get("alpha", 1)), float(opt.get("beta", 1)),
                                   opt.get("activation", "linear"))
        elif kind == "route":
            ids = [int(t) for t in opt["layers"].split(",")]
            cur = route_forward([outs[i if i >= 0 else idx + i] for i in ids])
        elif kind == "yolo":
            n = len(opt["mask"].split(",")) if "mask" in opt else int(opt.get("num", 1))
            cur = yolo_forward(cur, n, int(opt.get("classes", 20)))
        elif kind == "avgpool":
            cur = avgpool_forward(cur)
        elif kind == "softmax":
            cur = softmax_forward(cur, int(opt.get("groups", 1)), float(opt.get("temperature", 1)))
        else:
            raise NotImplementedError(f"layer type [{kind}] is outside the convolutional forward path")
        outs.append(cur)
    return outs


# ------------------------------------------------------------------ the unmodified reference


class Reference:
    """ctypes view of oracle/_ref/libdarknet_ref.so (the unmodified reference,
    CPU build, behind ref_harness.c).  Exists only where that library was built."""

    path = os.path.join(HERE, "_ref", "libdarknet_ref.so")

    @classmethod
    def available(cls) -> bool:
        return os.path.exists(cls.path)

    def __init__(self):
        L = C.CDLL(self.path)
        L.ref_load_network.restype = C.c_void_p
        L.ref_load_network.argtypes = [C.c_char_p, C.c_char_p]
        L.ref_free_network.argtypes = [C.c_void_p]
        for f in ("ref_num_layers", "ref_batch", "ref_inputs", "ref_outputs"):
            getattr(L, f).argtypes = [C.c_void_p]
        L.ref_layer_info.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_int)]
        L.ref_layer_output.restype = C.POINTER(C.c_float)
        L.ref_layer_output.argtypes = [C.c_void_p, C.c_int]
        L.ref_network_predict.restype = C.POINTER(C.c_float)
        L.ref_network_predict.argtypes = [C.c_void_p, C.c_void_p]
        L.ref_time_predict.restype = C.c_double
        L.ref_time_predict.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.ref_im2col.argtypes = [C.c_void_p] + [C.c_int] * 6 + [C.c_void_p]
        L.ref_gemm_nn.argtypes = [C.c_int] * 3 + [C.c_void_p] * 3
        if hasattr(L, "ref_save_weights"):
            L.ref_save_weights.argtypes = [C.c_void_p, C.c_char_p]
        if hasattr(L, "ref_save_conv_binary"):
            L.ref_save_conv_binary.argtypes = [C.c_void_p, C.c_int, C.c_char_p]
            L.ref_load_conv_binary.argtypes = [C.c_void_p, C.c_int, C.c_char_p]
            L.ref_layer_weights.restype = C.POINTER(C.c_float)
            L.ref_layer_weights.argtypes = [C.c_void_p, C.c_int]
        self.L = L

    def load(self, cfg_path: str, weights_path: str | None):
        return self.L.ref_load_network(cfg_path.encode(), (weights_path or "").encode())

    def save_weights(self, net, path: str) -> None:
        """The reference's own save_weights (src/parser.c:1080-1083) on the loaded network."""
        self.L.ref_save_weights(net, path.encode())

    def predict_all(self, net, x: np.ndarray) -> list[np.ndarray]:
        """network_predict, then a copy of every layer's output buffer."""
        x = np.ascontiguousarray(x, np.float32)
        self.L.ref_network_predict(net, _p(x))
        outs = []
        info = (C.c_int * 8)()
        for i in range(self.L.ref_num_layers(net)):
            self.L.ref_layer_info(net, i, info)
            _, oc, oh, ow, outputs, batch = list(info)[:6]
            buf = np.ctypeslib.as_array(self.L.ref_layer_output(net, i), shape=(batch * outputs,)).copy()
            shape = (batch, oc, oh, ow) if oc * oh * ow == outputs and outputs > 0 else (batch, outputs)
            outs.append(buf.reshape(shape))
        return outs


class ReferenceGpu(Reference):
    """ctypes view of oracle/_ref/libdarknet_ref_gpu.so: the unmodified reference's own CUDA build
    (-DGPU: im2col + cuBLAS + separate bias / batchnorm / activation kernels), recompiled for sm_100a,
    linked with the attach shim (darknet_b200/shim/b200_attach.c).  Needs a GPU at load time.  The
    reference exits the process on any error, so callers that must survive one run it in a child."""

    path = os.path.join(HERE, "_ref", "libdarknet_ref_gpu.so")

    def __init__(self):
        super().__init__()
        self.L.ref_attach_b200.argtypes = [C.c_void_p, C.c_int]
        self.L.ref_detach_b200.argtypes = [C.c_void_p]
        self.L.ref_attach_network_b200.argtypes = [C.c_void_p, C.c_int]

    def attach(self, net, mode: int) -> int:
        """b200_attach: re-point forward_gpu of the covered layers at libdarknet_b200."""
        return self.L.ref_attach_b200(net, mode)

    def attach_network(self, net, mode: int) -> int:
        """b200_attach_network: the whole forward pass through the library's own network object."""
        return self.L.ref_attach_network_b200(net, mode)

    def detach(self, net) -> None:
        self.L.ref_detach_b200(net)

    def time_predict(self, net, x: np.ndarray, reps: int) -> float:
        x = np.ascontiguousarray(x, np.float32)
        return float(self.L.ref_time_predict(net, _p(x), reps))
