"""The allocation-free xnor entry point against the plan-based one.

Runs last (pytest collects files alphabetically): if it fails, a run that stops at
the first failure has already exercised every other test.

dnb_conv_xnor_forward_static exists for callers that cannot call cudaMalloc while
they run (fixed-arena serving loops, plug-ins in processes that forbid allocation
after start-up): its scratch is a fixed array inside the library image.  The test
hands it device buffers it owns (torch is only the allocator of the test's own
inputs and outputs), calls it twice in a row, and checks both results against
dnb_conv_forward on an xnor plan and against the CPU checker's xnor convolution,
within the tolerance of the xnor tests (1e-5 of the layer maximum: the CPU adds
+-mean one product at a time, the GPU multiplies the integer sum by the mean).
The plan path runs the same kernels; the checker also validates the host-side
packing of sign bits, filter means and folded batchnorm that a caller of this
entry point has to do itself.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import darknet_b200 as dn
from conftest import parity
from gpu_util import dev_nchw, dev_nhwc, empty_nchw, empty_nhwc, host_from_nhwc
from oracle import network as orc

pytestmark = pytest.mark.gpu


def pack_params(w, scales, mean, var, biases):
    """Host-side packing the caller of the static entry point is responsible for."""
    n, c, k, _ = w.shape
    cwords = (c + 31) // 32
    bits = np.zeros((n, k * k, cwords), np.uint32)
    pos = (w > 0).transpose(0, 2, 3, 1).reshape(n, k * k, c)          # [n][tap][c]
    for ch in range(c):
        bits[:, :, ch // 32] |= pos[:, :, ch].astype(np.uint32) << np.uint32(ch % 32)
    wmean = np.zeros(n, np.float32)
    flat = np.abs(w.reshape(n, -1)).astype(np.float32)
    for i in range(flat.shape[1]):                                      # float running sum in index order
        wmean += flat[:, i]
    wmean = (wmean / np.float32(flat.shape[1])).astype(np.float32)
    s = (scales.astype(np.float64) / (np.sqrt(var.astype(np.float64)) + np.float64(np.float32(1e-6)))).astype(np.float32)
    sh = (biases.astype(np.float64) - mean.astype(np.float64) * (scales.astype(np.float64) / (np.sqrt(var.astype(np.float64)) + np.float64(np.float32(1e-6))))).astype(np.float32)
    return bits, wmean, s, sh


@pytest.mark.parametrize("layout", ["nchw", "nhwc"])
def test_static_xnor_matches_plan(layout):
    g = np.random.Generator(np.random.Philox(key=[2024, 5]))
    b, c, h, w_, n, k = 2, 72, 13, 11, 40, 3
    x = g.standard_normal((b, c, h, w_), dtype=np.float32)
    w = g.standard_normal((n, c, k, k), dtype=np.float32) * np.float32(0.05)
    biases = g.standard_normal(n, dtype=np.float32) * np.float32(0.1)
    scales = g.uniform(0.9, 1.1, n).astype(np.float32)
    mean = g.standard_normal(n, dtype=np.float32) * np.float32(0.3)
    var = g.uniform(0.5, 1.5, n).astype(np.float32)

    plan = dn.ConvPlan(b, c, h, w_, n, k, 1, 1, 1, True, "leaky", True, dn.MODE_TF32).set_params(w, biases, scales, mean, var)
    xt, xd = dev_nchw(x) if layout == "nchw" else dev_nhwc(x)
    rt, rd = empty_nchw(b, n, h, w_) if layout == "nchw" else empty_nhwc(b, n, h, w_)
    plan.forward(xd, rd)
    torch.cuda.synchronize()
    want = rt.cpu().numpy() if layout == "nchw" else host_from_nhwc(rt, n)
    want_cpu = orc.conv_forward(x, w, biases, scales, mean, var, stride=1, pad=1, groups=1, activation="leaky", xnor=True)
    want_cpu_neg = orc.conv_forward(-x, w, biases, scales, mean, var, stride=1, pad=1, groups=1, activation="leaky", xnor=True)

    bits, wmean, s, sh = pack_params(w, scales, mean, var, biases)
    dev = [torch.from_numpy(a).cuda() for a in (bits.view(np.int32), wmean, s, sh)]
    desc = dn.ConvDesc(b, h, w_, c, n, 1, k, 1, 1, 1, dn.ACTIVATIONS["leaky"], 1)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call in range(2):   # the second call finds the first call's bits in the shared scratch
        yt, yd = empty_nchw(b, n, h, w_) if layout == "nchw" else empty_nhwc(b, n, h, w_)
        if layout == "nhwc":
            yt.zero_()
        dn.check(dn.lib().dnb_conv_xnor_forward_static(C.byref(desc), C.byref(xd), C.c_void_p(dev[0].data_ptr()),
                                                       C.c_void_p(dev[1].data_ptr()), C.c_void_p(dev[2].data_ptr()),
                                                       C.c_void_p(dev[3].data_ptr()), C.byref(yd), stream))
        torch.cuda.synchronize()
        got = yt.cpu().numpy() if layout == "nchw" else host_from_nhwc(yt, n)
        parity(got, want, 1e-5, f"call {call} against the plan path")
        parity(got, want_cpu, 1e-5, f"call {call} against the CPU checker")
        # a different input between the calls, so that stale scratch would show
        if call == 0:
            x2 = -x
            x2t, x2d = dev_nchw(x2) if layout == "nchw" else dev_nhwc(x2)
            tt, td = empty_nchw(b, n, h, w_) if layout == "nchw" else empty_nhwc(b, n, h, w_)
            dn.check(dn.lib().dnb_conv_xnor_forward_static(C.byref(desc), C.byref(x2d), C.c_void_p(dev[0].data_ptr()),
                                                           C.c_void_p(dev[1].data_ptr()), C.c_void_p(dev[2].data_ptr()),
                                                           C.c_void_p(dev[3].data_ptr()), C.byref(td), stream))
            torch.cuda.synchronize()
            got_neg = tt.cpu().numpy() if layout == "nchw" else host_from_nhwc(tt, n)
            parity(got_neg, want_cpu_neg, 1e-5, "negated input against the CPU checker")


def test_static_xnor_rejects_oversized_layer():
    # 64 x 1024 channels x 32 x 32 needs 2^21 words of packed input: twice the built-in scratch
    desc = dn.ConvDesc(64, 32, 32, 1024, 8, 1, 3, 1, 1, 0, dn.ACTIVATIONS["linear"], 1)
    xt = torch.zeros(8, device="cuda")
    x = dn.Tensor(xt.data_ptr(), dn.NCHW, dn.F32, 64, 1024, 32, 32, 0)
    y = dn.Tensor(xt.data_ptr(), dn.NCHW, dn.F32, 64, 8, 32, 32, 0)
    p = C.c_void_p(xt.data_ptr())
    st = dn.lib().dnb_conv_xnor_forward_static(C.byref(desc), C.byref(x), p, p, p, p, C.byref(y), None)
    assert st == dn.EINVAL and b"scratch" in dn.lib().dnb_last_error()
