"""Python mirror of the C ABI: thin classes over opaque handles.

torch is used only to own device memory and streams; tensors are handed to the
library as raw pointers inside ``struct dnb_tensor``.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import (ACTIVATIONS, BF16, F32, MODE_TF32, NCHW, NHWC, ConvDesc, Tensor, check, lib)


def _stream(stream=None) -> C.c_void_p:
    if stream is not None:
        return C.c_void_p(int(stream))
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def as_tensor(t, layout: int = NCHW, c: int | None = None) -> Tensor:
    """Describe a contiguous CUDA torch tensor to the library.

    NCHW: ``t`` is [n, c, h, w] float32.  NHWC: ``t`` is [n, h, w, cpitch]
    float32 or bfloat16 and ``c`` (default cpitch) is the logical channel count."""
    import torch
    if not t.is_cuda or not t.is_contiguous():
        raise ValueError("as_tensor needs a contiguous CUDA tensor")
    dtype = {torch.float32: F32, torch.bfloat16: BF16}[t.dtype]
    if layout == NCHW:
        n, ch, h, w = t.shape
        return Tensor(t.data_ptr(), NCHW, dtype, n, ch, h, w, 0)
    n, h, w, cp = t.shape
    return Tensor(t.data_ptr(), NHWC, dtype, n, c if c is not None else cp, h, w, cp)


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class ConvPlan:
    """dnb_conv_plan: one convolutional layer (make_convolutional_layer +
    forward_convolutional_layer_gpu of the reference)."""

    def __init__(self, batch, c, h, w, n, size, stride=1, pad=0, groups=1, batch_normalize=False,
                 activation="linear", xnor=False, mode=MODE_TF32):
        self.desc = ConvDesc(batch, h, w, c, n, groups, size, stride, pad, int(batch_normalize),
                             ACTIVATIONS[activation] if isinstance(activation, str) else int(activation), int(xnor))
        self.handle = C.c_void_p()
        check(lib().dnb_conv_plan_create(C.byref(self.desc), mode, C.byref(self.handle)))
        self.out_h = (h + 2 * pad - size) // stride + 1
        self.out_w = (w + 2 * pad - size) // stride + 1

    def set_params(self, weights, biases, scales=None, rolling_mean=None, rolling_variance=None):
        arrs = [_f32(a) for a in (weights, biases, scales, rolling_mean, rolling_variance)]
        d = self.desc
        assert arrs[0].size == d.n * (d.c // d.groups) * d.size * d.size and arrs[1].size == d.n
        check(lib().dnb_conv_plan_set_params(self.handle, *[_ptr(a) for a in arrs]))
        return self

    @property
    def kernel(self) -> str:
        return lib().dnb_conv_plan_kernel(self.handle).decode()

    def describe(self) -> str:
        """Kernel and tiling of the plan as one line (tiling fields are known after the first forward)."""
        buf = C.create_string_buffer(256)
        check(lib().dnb_conv_plan_describe(self.handle, buf, 256))
        return buf.value.decode()

    def forward(self, x: Tensor, y: Tensor, y2: Tensor | None = None, stream=None):
        check(lib().dnb_conv_forward(self.handle, C.byref(x), C.byref(y), C.byref(y2) if y2 is not None else None, _stream(stream)))

    def xnor_accumulate(self, x: Tensor, acc, stream=None):
        """acc: int32 CUDA torch tensor [batch, n, out_h, out_w]."""
        check(lib().dnb_conv_xnor_accumulate(self.handle, C.byref(x), C.c_void_p(acc.data_ptr()), _stream(stream)))

    def check_status(self):
        check(lib().dnb_conv_plan_check_status(self.handle))

    def set_diagnostics(self, wait_limit_cycles: int = 0, debug_bits: int = 0):
        """Bound of the device-side waits in SM cycles (0: default) and diagnostic bits (32: withhold a load)."""
        check(lib().dnb_conv_plan_set_diagnostics(self.handle, wait_limit_cycles, debug_bits))

    def close(self):
        if self.handle:
            lib().dnb_conv_plan_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def maxpool(x: Tensor, y: Tensor, size: int, stride: int, padding: int | None = None, stream=None):
    check(lib().dnb_maxpool_forward(C.byref(x), C.byref(y), size, stride, size - 1 if padding is None else padding, _stream(stream)))


def upsample(x: Tensor, y: Tensor, stride: int = 2, scale: float = 1.0, stream=None):
    check(lib().dnb_upsample_forward(C.byref(x), C.byref(y), stride, scale, _stream(stream)))


def shortcut(x: Tensor, add: Tensor, y: Tensor, alpha=1.0, beta=1.0, activation="linear", stream=None):
    check(lib().dnb_shortcut_forward(C.byref(x), C.byref(add), C.byref(y), alpha, beta, ACTIVATIONS[activation], _stream(stream)))


def route(inputs: list[Tensor], y: Tensor, stream=None):
    arr = (C.POINTER(Tensor) * len(inputs))(*[C.pointer(t) for t in inputs])
    check(lib().dnb_route_forward(arr, len(inputs), C.byref(y), _stream(stream)))


def convert(x: Tensor, y: Tensor, round_tf32: bool = False, stream=None):
    check(lib().dnb_convert(C.byref(x), C.byref(y), int(round_tf32), _stream(stream)))


def yolo(x: Tensor, y: Tensor, anchors: int, classes: int, stream=None):
    check(lib().dnb_yolo_forward(C.byref(x), C.byref(y), anchors, classes, _stream(stream)))


def avgpool(x: Tensor, y: Tensor, stream=None):
    check(lib().dnb_avgpool_forward(C.byref(x), C.byref(y), _stream(stream)))


def softmax(x: Tensor, y: Tensor, groups: int = 1, temperature: float = 1.0, stream=None):
    check(lib().dnb_softmax_forward(C.byref(x), C.byref(y), groups, temperature, _stream(stream)))


class Network:
    """dnb_network: parse_network_cfg + load_weights + network_predict."""

    def __init__(self, cfg: str, weights: str | None = None, mode: int = MODE_TF32, batch: int = 0, text: bool = False):
        self.handle = C.c_void_p()
        fn = lib().dnb_parse_network_cfg_text if text else lib().dnb_parse_network_cfg
        check(fn(cfg.encode(), mode, batch, C.byref(self.handle)))
        if weights:
            self.load_weights(weights)

    def load_weights(self, path: str, packed: bool = False):
        """load_weights; ``packed``: the file stores its xnor convolutions in the packed-binary layer format."""
        fn = lib().dnb_load_weights_packed if packed else lib().dnb_load_weights
        check(fn(self.handle, path.encode()))

    n = property(lambda self: lib().dnb_network_num_layers(self.handle))
    batch = property(lambda self: lib().dnb_network_batch(self.handle))
    inputs = property(lambda self: lib().dnb_network_inputs(self.handle))
    outputs = property(lambda self: lib().dnb_network_outputs(self.handle))
    flops = property(lambda self: lib().dnb_network_flops(self.handle))
    launches = property(lambda self: lib().dnb_network_launches(self.handle))

    def layer_shape(self, i: int) -> tuple[int, int, int]:
        c, h, w = C.c_int(), C.c_int(), C.c_int()
        check(lib().dnb_network_layer_shape(self.handle, i, C.byref(c), C.byref(h), C.byref(w)))
        return c.value, h.value, w.value

    def layer_type(self, i: int) -> str:
        return lib().dnb_network_layer_type(self.handle, i).decode()

    def layer_kernel(self, i: int) -> str:
        return lib().dnb_network_layer_kernel(self.handle, i).decode()

    def layer_describe(self, i: int) -> str:
        buf = C.create_string_buffer(256)
        check(lib().dnb_network_layer_describe(self.handle, i, buf, 256))
        return buf.value.decode()

    def predict_ptr(self, host_ptr: int) -> np.ndarray:
        """network_predict on a raw host pointer to batch*inputs floats."""
        out = C.POINTER(C.c_float)()
        check(lib().dnb_network_predict(self.handle, C.c_void_p(host_ptr), C.byref(out)))
        return np.ctypeslib.as_array(out, shape=(self.batch, self.outputs))

    def predict(self, x) -> np.ndarray:
        """network_predict: x is a host array (numpy, or a CPU torch tensor, pinned
        or not) of batch*inputs floats in NCHW order.  The returned array aliases
        host memory owned by the network."""
        if hasattr(x, "data_ptr"):
            assert x.device.type == "cpu" and x.is_contiguous() and x.numel() == self.batch * self.inputs
            return self.predict_ptr(x.data_ptr())
        x = _f32(x)
        assert x.size == self.batch * self.inputs
        return self.predict_ptr(x.ctypes.data)

    def submit(self, x) -> None:
        """First half of a pipelined network_predict: enqueue upload, forward and result
        copies of one step.  x (numpy or CPU torch tensor, ideally pinned) must stay
        untouched until the step is collected; at most two steps may be in flight."""
        if hasattr(x, "data_ptr"):
            assert x.device.type == "cpu" and x.is_contiguous() and x.numel() == self.batch * self.inputs
            ptr = x.data_ptr()
        else:
            assert x.dtype == np.float32 and x.flags.c_contiguous and x.size == self.batch * self.inputs
            ptr = x.ctypes.data
        check(lib().dnb_network_submit(self.handle, C.c_void_p(ptr)))

    def collect(self) -> np.ndarray:
        """Second half: wait for the oldest submitted step; returns its output as predict does."""
        out = C.POINTER(C.c_float)()
        check(lib().dnb_network_collect(self.handle, C.byref(out)))
        return np.ctypeslib.as_array(out, shape=(self.batch, self.outputs))

    def enable_graph(self, on: bool = True) -> None:
        """Replay forward() as a CUDA graph from the third call with the same tensor and (non-default) stream."""
        check(lib().dnb_network_enable_graph(self.handle, int(on)))

    def forward(self, x_dev, stream=None):
        """Device-resident forward: x_dev is a CUDA float32 tensor [batch, c, h, w]."""
        assert x_dev.is_cuda and x_dev.is_contiguous() and x_dev.numel() == self.batch * self.inputs
        check(lib().dnb_network_forward(self.handle, C.c_void_p(x_dev.data_ptr()), _stream(stream)))

    def layer_output(self, i: int) -> np.ndarray:
        c, h, w = self.layer_shape(i)
        out = np.empty((self.batch, c, h, w), np.float32)
        check(lib().dnb_network_layer_output(self.handle, i, _ptr(out)))
        return out

    def layer_output_images(self, i: int, first: int, count: int = 1) -> np.ndarray:
        """Images first .. first+count-1 of layer i's output, NCHW f32."""
        c, h, w = self.layer_shape(i)
        out = np.empty((count, c, h, w), np.float32)
        check(lib().dnb_network_layer_output_images(self.handle, i, first, count, _ptr(out)))
        return out

    def check_status(self):
        check(lib().dnb_network_check_status(self.handle))

    def set_diagnostics(self, layer: int, wait_limit_cycles: int = 0, debug_bits: int = 0):
        check(lib().dnb_network_set_diagnostics(self.handle, layer, wait_limit_cycles, debug_bits))

    def yolo_output(self, i: int) -> np.ndarray:
        c, h, w = self.layer_shape(i)
        out = C.POINTER(C.c_float)()
        check(lib().dnb_network_yolo_output(self.handle, i, C.byref(out)))
        return np.ctypeslib.as_array(out, shape=(self.batch, c, h, w))

    def profile(self, x_dev) -> np.ndarray:
        ms = np.zeros(self.n, np.float32)
        check(lib().dnb_network_profile(self.handle, C.c_void_p(x_dev.data_ptr()), _ptr(ms)))
        return ms

    def forward_timed(self, x_dev, slot: int = 0, stream=None):
        check(lib().dnb_network_forward_timed(self.handle, C.c_void_p(x_dev.data_ptr()), _stream(stream), slot))

    def timed_ms(self, slot: int = 0) -> np.ndarray:
        ms = np.zeros(self.n, np.float32)
        check(lib().dnb_network_timed_ms(self.handle, slot, _ptr(ms)))
        return ms

    def close(self):
        if self.handle:
            lib().dnb_free_network(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def load_network(cfg: str, weights: str | None = None, clear: int = 0, mode: int = MODE_TF32, batch: int = 0) -> Network:
    """load_network(cfg, weights, clear) of the reference (src/network.c:53-61,
    python/darknet.py:79-80).  ``clear`` only resets the training counter there
    and is accepted and ignored."""
    return Network(cfg, weights, mode, batch)


def network_predict(net: Network, data) -> np.ndarray:
    """network_predict(net, input) of the reference (src/network.c:497-508)."""
    return net.predict(data)
