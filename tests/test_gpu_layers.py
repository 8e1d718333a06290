"""Per-layer parity on the GPU: every kernel, called through the C ABI on device
buffers, against the CPU checker (oracle/) on identical seeded inputs.

Tolerances (max |gpu - cpu| / max |cpu| per layer output):
  integer / copy / compare kernels (maxpool, upsample, route, layout, xnor
  accumulators): bit-exact;
  fp32 CUDA-core kernels: 2e-6 (fused multiply-add and fp32 vs double constants);
  TF32 tensor-core convolution: 1e-2;  BF16: 3e-2.
"""
import numpy as np
import pytest
import torch

import darknet_b200 as dn
from conftest import parity, rel_to_max
from gpu_util import bf16_round, dev_nchw, dev_nhwc, empty_nchw, empty_nhwc, host_from_nhwc, padding_is_zero
from oracle import network as orc

pytestmark = pytest.mark.gpu

TOL_FP32 = 2e-6
TOL_TF32 = 1e-2
TOL_BF16 = 3e-2


def rng(seed):
    return np.random.Generator(np.random.Philox(key=[seed, 77]))


# ------------------------------------------------------------------ memory-bound layers
@pytest.mark.parametrize("shape,size,stride,padding", [
    ((2, 16, 16, 16), 2, 2, 1), ((2, 24, 13, 13), 2, 1, 1), ((1, 8, 15, 17), 3, 2, 2),
    ((3, 40, 7, 9), 2, 2, 1), ((1, 64, 112, 112), 2, 2, 1), ((2, 5, 9, 9), 3, 1, 2)])
@pytest.mark.parametrize("layout", ["nhwc", "nchw", "nhwc_bf16"])
def test_maxpool(shape, size, stride, padding, layout):
    x = rng(1).standard_normal(shape, dtype=np.float32)
    if layout == "nhwc_bf16":
        x = bf16_round(x)
    want = orc.maxpool_forward(x, size, stride, padding)
    n, c, oh, ow = want.shape
    if layout == "nchw":
        xt, xd = dev_nchw(x)
        yt, yd = empty_nchw(n, c, oh, ow)
        dn.maxpool(xd, yd, size, stride, padding)
        got = yt.cpu().numpy()
    else:
        dt = torch.bfloat16 if layout == "nhwc_bf16" else torch.float32
        xt, xd = dev_nhwc(x, dt)
        yt, yd = empty_nhwc(n, c, oh, ow, dt)
        dn.maxpool(xd, yd, size, stride, padding)
        got = host_from_nhwc(yt, c)
        assert padding_is_zero(yt, c)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("shape,stride", [((2, 128, 13, 13), 2), ((1, 256, 19, 19), 2), ((2, 12, 5, 7), 3)])
@pytest.mark.parametrize("layout", ["nhwc", "nchw", "nhwc_bf16"])
def test_upsample(shape, stride, layout):
    x = rng(2).standard_normal(shape, dtype=np.float32)
    if layout == "nhwc_bf16":
        x = bf16_round(x)
    want = orc.upsample_forward(x, stride)
    n, c, oh, ow = want.shape
    if layout == "nchw":
        xt, xd = dev_nchw(x)
        yt, yd = empty_nchw(n, c, oh, ow)
        dn.upsample(xd, yd, stride)
        got = yt.cpu().numpy()
    else:
        dt = torch.bfloat16 if layout == "nhwc_bf16" else torch.float32
        xt, xd = dev_nhwc(x, dt)
        yt, yd = empty_nhwc(n, c, oh, ow, dt)
        dn.upsample(xd, yd, stride)
        got = host_from_nhwc(yt, c)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_producers_write_into_a_channel_range_of_a_wider_tensor(dtype):
    """What the zero-copy [route] relies on: upsample and the tensor-core convolution write a tensor that is a channel
    range of a wider channels-last tensor (own channel count, the wider tensor's pitch) without touching its
    neighbours, and route skips an input that already is its range of the output."""
    g = rng(40)
    b, h, w = 2, 9, 11
    x = g.standard_normal((b, 64, h, w), dtype=np.float32)
    other = g.standard_normal((b, 64, 2 * h, 2 * w), dtype=np.float32)
    if dtype == torch.bfloat16:
        x, other = bf16_round(x), bf16_round(other)
    es = 2 if dtype == torch.bfloat16 else 4
    wide = torch.full((b, 2 * h, 2 * w, 128), 7.0, dtype=dtype, device="cuda")    # [upsampled 64 | other 64]; ranges start on 128-byte boundaries
    up_view = dn.Tensor(wide.data_ptr(), dn.NHWC, dn.BF16 if dtype == torch.bfloat16 else dn.F32, b, 64, 2 * h, 2 * w, 128)
    ot_view = dn.Tensor(wide.data_ptr() + 64 * es, dn.NHWC, up_view.dtype, b, 64, 2 * h, 2 * w, 128)
    xt, xd = dev_nhwc(x, dtype)
    dn.upsample(xd, up_view, 2)
    torch.cuda.synchronize()
    assert np.array_equal(wide[..., :64].permute(0, 3, 1, 2).float().cpu().numpy(), orc.upsample_forward(x, 2))
    assert bool((wide[..., 64:] == 7.0).all().item())                             # the neighbour's channels are untouched
    # a convolution writes the other range
    case = conv_case(41, b=b, c=16, h=2 * h, w=2 * w, n=64, size=3)
    mode = dn.MODE_BF16 if dtype == torch.bfloat16 else dn.MODE_TF32
    plan = dn.ConvPlan(b, 16, 2 * h, 2 * w, 64, 3, 1, 1, 1, True, "leaky", False, mode)
    plan.set_params(case["w"], case["biases"], case["scales"], case["mean"], case["var"])
    ct, cd = dev_nhwc(case["x"], dtype)
    plan.forward(cd, ot_view)
    torch.cuda.synchronize()
    plan.check_status()
    conv_out = wide[..., 64:].permute(0, 3, 1, 2).float().cpu().numpy()
    parity(conv_out, oracle_conv(case), TOL_BF16 if dtype == torch.bfloat16 else TOL_TF32, "convolution into a channel range")
    assert np.array_equal(wide[..., :64].permute(0, 3, 1, 2).float().cpu().numpy(), orc.upsample_forward(x, 2))
    # route over the two ranges of its own output copies nothing and leaves the tensor as it is
    before = wide.clone()
    y_all = dn.Tensor(wide.data_ptr(), dn.NHWC, up_view.dtype, b, 128, 2 * h, 2 * w, 128)
    dn.route([up_view, ot_view], y_all)
    torch.cuda.synchronize()
    assert torch.equal(wide, before)
    # and the same route into a separate tensor copies both ranges
    yt, yd = empty_nhwc(b, 128, 2 * h, 2 * w, dtype)
    dn.route([up_view, ot_view], yd)
    torch.cuda.synchronize()
    assert torch.equal(yt, wide)


@pytest.mark.parametrize("xs,adds,act", [
    ((2, 64, 19, 19), (2, 64, 19, 19), "linear"),     # YOLOv3 residual
    ((2, 256, 14, 14), (2, 64, 14, 14), "leaky"),     # ResNet: add has fewer channels
    ((2, 128, 7, 7), (2, 64, 14, 14), "leaky"),       # ResNet: add is twice as large, sampled with stride 2
    ((1, 16, 8, 8), (1, 16, 4, 4), "linear"),         # add is smaller: scattered with `sample`
    ((2, 20, 5, 5), (2, 20, 5, 5), "logistic")])
@pytest.mark.parametrize("layout", ["nhwc", "nchw"])
def test_shortcut(xs, adds, act, layout):
    g = rng(3)
    x = g.standard_normal(xs, dtype=np.float32)
    add = g.standard_normal(adds, dtype=np.float32)
    want = orc.shortcut_forward(x, add, 1.0, 1.0, act)
    n, c, h, w = xs
    if layout == "nchw":
        xt, xd = dev_nchw(x)
        at, ad = dev_nchw(add)
        yt, yd = empty_nchw(n, c, h, w)
        dn.shortcut(xd, ad, yd, 1.0, 1.0, act)
        got = yt.cpu().numpy()
    else:
        xt, xd = dev_nhwc(x)
        at, ad = dev_nhwc(add)
        yt, yd = empty_nhwc(n, c, h, w)
        yt.zero_()
        dn.shortcut(xd, ad, yd, 1.0, 1.0, act)
        got = host_from_nhwc(yt, c)
        assert padding_is_zero(yt, c)
    parity(got, want, TOL_FP32)


def test_shortcut_bf16_storage():
    g = rng(4)
    x = bf16_round(g.standard_normal((2, 64, 10, 10), dtype=np.float32))
    add = bf16_round(g.standard_normal((2, 64, 10, 10), dtype=np.float32))
    want = orc.shortcut_forward(x, add, 1.0, 1.0, "linear")
    xt, xd = dev_nhwc(x, torch.bfloat16)
    at, ad = dev_nhwc(add, torch.bfloat16)
    yt, yd = empty_nhwc(2, 64, 10, 10, torch.bfloat16)
    dn.shortcut(xd, ad, yd)
    parity(host_from_nhwc(yt, 64), want, 2 ** -8)


@pytest.mark.parametrize("chans,hw", [((256, 512), (19, 19)), ((128, 256, 3), (13, 11)), ((255,), (7, 7)), ((12, 20), (5, 5))])
@pytest.mark.parametrize("layout", ["nhwc", "nchw"])
def test_route(chans, hw, layout):
    g = rng(5)
    ins = [g.standard_normal((2, c) + hw, dtype=np.float32) for c in chans]
    want = orc.route_forward(ins)
    ctot = sum(chans)
    if layout == "nchw":
        held = [dev_nchw(a) for a in ins]
        yt, yd = empty_nchw(2, ctot, *hw)
        dn.route([d for _, d in held], yd)
        got = yt.cpu().numpy()
    else:
        held = [dev_nhwc(a) for a in ins]
        yt, yd = empty_nhwc(2, ctot, *hw)
        yt.zero_()
        dn.route([d for _, d in held], yd)
        got = host_from_nhwc(yt, ctot)
        assert padding_is_zero(yt, ctot)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("shape", [(2, 3, 17, 19), (1, 255, 13, 13), (2, 64, 8, 8), (1, 33, 5, 70)])
def test_layout_round_trip(shape):
    x = rng(6).standard_normal(shape, dtype=np.float32)
    xt, xd = dev_nchw(x)
    mt, md = empty_nhwc(*shape)
    dn.convert(xd, md)
    assert np.array_equal(host_from_nhwc(mt, shape[1]), x) and padding_is_zero(mt, shape[1])
    yt, yd = empty_nchw(*shape)
    dn.convert(md, yd)
    assert np.array_equal(yt.cpu().numpy(), x)
    # bf16 storage and TF32 rounding
    bt, bd = empty_nhwc(*shape, dtype=torch.bfloat16)
    dn.convert(xd, bd)
    assert np.array_equal(host_from_nhwc(bt, shape[1]), bf16_round(x))
    rt, rd = empty_nhwc(*shape)
    dn.convert(xd, rd, round_tf32=True)
    r = host_from_nhwc(rt, shape[1])
    assert (r.view(np.uint32) & 0x1fff).max() == 0 and rel_to_max(r, x) < 2 ** -10


@pytest.mark.parametrize("layout", ["nhwc", "nchw"])
def test_yolo_head(layout):
    x = rng(7).standard_normal((2, 255, 13, 13), dtype=np.float32)
    want = orc.yolo_forward(x, 3, 80)
    xt, xd = dev_nhwc(x) if layout == "nhwc" else dev_nchw(x)
    yt, yd = empty_nchw(2, 255, 13, 13)
    dn.yolo(xd, yd, 3, 80)
    parity(yt.cpu().numpy(), want, TOL_FP32)


@pytest.mark.parametrize("layout", ["nhwc", "nchw"])
def test_avgpool_softmax(layout):
    x = rng(8).standard_normal((3, 1000, 7, 7), dtype=np.float32)
    want_a = orc.avgpool_forward(x)
    want_s = orc.softmax_forward(want_a)
    if layout == "nchw":
        xt, xd = dev_nchw(x)
        at, ad = empty_nchw(3, 1000, 1, 1)
        st, sd = empty_nchw(3, 1000, 1, 1)
    else:
        xt, xd = dev_nhwc(x)
        at, ad = empty_nhwc(3, 1000, 1, 1)
        st, sd = empty_nhwc(3, 1000, 1, 1)
    dn.avgpool(xd, ad)
    dn.softmax(ad, sd)
    got_a = at.cpu().numpy() if layout == "nchw" else host_from_nhwc(at, 1000)
    got_s = st.cpu().numpy() if layout == "nchw" else host_from_nhwc(st, 1000)
    parity(got_a, want_a, 1e-5)
    parity(got_s, want_s, 1e-5)


# ------------------------------------------------------------------ convolution
def conv_case(seed, b, c, h, w, n, size, stride=1, pad=None, groups=1, bn=True, act="leaky", dist="normal"):
    g = rng(seed)
    pad = size // 2 if pad is None else pad
    x = g.standard_normal((b, c, h, w), dtype=np.float32) if dist == "normal" else g.random((b, c, h, w), dtype=np.float32)
    fan = size * size * c // groups
    wts = g.standard_normal((n, c // groups, size, size), dtype=np.float32) * np.float32(np.sqrt(2.0 / fan))
    biases = g.standard_normal(n, dtype=np.float32) * np.float32(0.1)
    if bn:
        scales = g.uniform(0.9, 1.1, n).astype(np.float32)
        mean = g.standard_normal(n, dtype=np.float32) * np.float32(0.3)
        var = g.uniform(0.5, 1.5, n).astype(np.float32)
    else:
        scales = mean = var = None
    return dict(x=x, w=wts, biases=biases, scales=scales, mean=mean, var=var, stride=stride, pad=pad, groups=groups, act=act)


def run_conv(case, mode, in_layout="nchw", out_layout="nchw", xnor=False, both=False):
    x, w = case["x"], case["w"]
    b, c, h, wd = x.shape
    n, size = w.shape[0], w.shape[2]
    plan = dn.ConvPlan(b, c, h, wd, n, size, case["stride"], case["pad"], case["groups"], case["scales"] is not None,
                       case["act"], xnor, mode)
    plan.set_params(w, case["biases"], case["scales"], case["mean"], case["var"])
    store = torch.bfloat16 if mode == dn.MODE_BF16 else torch.float32
    xt, xd = dev_nchw(x) if in_layout == "nchw" else dev_nhwc(x, store)
    if out_layout == "nchw":
        yt, yd = empty_nchw(b, n, plan.out_h, plan.out_w)
    else:
        yt, yd = empty_nhwc(b, n, plan.out_h, plan.out_w, store)
    y2t = y2d = None
    if both:
        y2t, y2d = empty_nhwc(b, n, plan.out_h, plan.out_w, store) if out_layout == "nchw" else empty_nchw(b, n, plan.out_h, plan.out_w)
    plan.forward(xd, yd, y2d)
    torch.cuda.synchronize()
    plan.check_status()
    got = yt.cpu().numpy() if out_layout == "nchw" else host_from_nhwc(yt, n)
    if out_layout == "nhwc":
        assert padding_is_zero(yt, n)
    got2 = None
    if both:
        got2 = host_from_nhwc(y2t, n) if out_layout == "nchw" else y2t.cpu().numpy()
    return plan, got, got2


def oracle_conv(case, xnor=False, x=None):
    return orc.conv_forward(case["x"] if x is None else x, case["w"], case["biases"], case["scales"], case["mean"], case["var"],
                            stride=case["stride"], pad=case["pad"], groups=case["groups"], activation=case["act"], xnor=xnor)


DIRECT_CASES = {
    "stem3x3_c3": dict(b=2, c=3, h=32, w=32, n=32, size=3, dist="uniform"),
    "stem7x7_s2_c3": dict(b=2, c=3, h=30, w=30, n=64, size=7, stride=2, dist="uniform"),
    "groups2": dict(b=2, c=8, h=10, w=10, n=12, size=3, groups=2),
    "groups4_1x1": dict(b=1, c=16, h=6, w=6, n=40, size=1, groups=4),
    "k5_nopad": dict(b=1, c=8, h=11, w=11, n=8, size=5, pad=0),
    "wide_k": dict(b=1, c=96, h=6, w=6, n=20, size=3, act="linear", bn=False),
}


@pytest.mark.parametrize("name", list(DIRECT_CASES))
@pytest.mark.parametrize("layouts", [("nchw", "nchw"), ("nchw", "nhwc"), ("nhwc", "nhwc")])
def test_conv_direct_fp32(name, layouts):
    case = conv_case(100, **DIRECT_CASES[name])
    plan, got, _ = run_conv(case, dn.MODE_FP32, layouts[0], layouts[1])
    assert plan.kernel == "direct_fp32"
    parity(got, oracle_conv(case), 1e-5)


STEM_CASES = {
    "rgb_n32": dict(b=3, c=3, h=37, w=29, n=32, size=3, dist="uniform"),
    "rgb_n16": dict(b=2, c=3, h=32, w=32, n=16, size=3, dist="uniform"),
    "rgb_n64_s2": dict(b=2, c=3, h=31, w=45, n=64, size=3, stride=2, dist="uniform"),
    "rgb_n48_nopad_linear": dict(b=1, c=3, h=20, w=20, n=48, size=3, pad=0, bn=False, act="linear"),
    "gray_n32_logistic": dict(b=2, c=1, h=24, w=24, n=32, size=3, act="logistic"),
    "two_channels": dict(b=1, c=2, h=16, w=130, n=32, size=3),
    "many_tiles": dict(b=4, c=3, h=160, w=160, n=32, size=3, dist="uniform"),
    "rgb7x7_s2_n64": dict(b=2, c=3, h=46, w=46, n=64, size=7, stride=2, dist="uniform"),
    "rgb7x7_n16_ragged": dict(b=3, c=3, h=37, w=29, n=16, size=7, dist="uniform"),
    "rgb5x5_n32_logistic": dict(b=2, c=3, h=24, w=40, n=32, size=5, act="logistic"),
    "rgb7x7_many_tiles": dict(b=4, c=3, h=112, w=112, n=64, size=7, stride=2, dist="uniform"),
}


@pytest.mark.parametrize("name", list(STEM_CASES))
@pytest.mark.parametrize("mode", [dn.MODE_TF32, dn.MODE_BF16])
def test_conv_stem_tensor_core(name, mode):
    """First-layer kernel (im2col rows built by the threads, TF32 products): f32 input in Darknet's
    layout or channels-last, channels-last output in the mode's storage type.  Asked for Darknet's
    layout on the output side, the same plan falls back to the FP32 kernel."""
    case = conv_case(150, **STEM_CASES[name])
    want = oracle_conv(case)
    tol = TOL_TF32 if mode == dn.MODE_TF32 else TOL_BF16
    plan, got, _ = run_conv(case, mode, "nchw", "nhwc")
    assert plan.kernel == "stem_tc_tf32"
    parity(got, want, tol, name)
    if mode == dn.MODE_TF32:
        _, got2, _ = run_conv(case, mode, "nhwc", "nhwc")     # channels-last f32 input through the same strides
        assert np.array_equal(got, got2)
        _, got3, _ = run_conv(case, mode, "nchw", "nchw")     # fallback: exact FP32 arithmetic
        parity(got3, want, 1e-5)


TC_CASES = {
    "1x1_c32_onetile": dict(b=1, c=32, h=8, w=16, n=16, size=1, bn=False, act="linear"),
    "1x1_c64": dict(b=2, c=64, h=9, w=9, n=40, size=1),
    "1x1_c8_sw32": dict(b=1, c=8, h=8, w=8, n=16, size=1),
    "1x1_c16_sw64": dict(b=1, c=16, h=12, w=12, n=32, size=1),
    "1x1_c24_ragged_k": dict(b=1, c=24, h=7, w=7, n=16, size=1),
    "1x1_c48_ragged_k": dict(b=1, c=48, h=7, w=7, n=16, size=1),
    "3x3_c32": dict(b=1, c=32, h=8, w=16, n=32, size=3),
    "3x3_c16": dict(b=2, c=16, h=13, w=13, n=32, size=3),
    "3x3_s2": dict(b=2, c=32, h=16, w=16, n=64, size=3, stride=2),
    "3x3_s2_odd": dict(b=2, c=16, h=13, w=11, n=24, size=3, stride=2),
    "3x3_nopad": dict(b=2, c=8, h=9, w=9, n=16, size=3, pad=0),
    "5x5": dict(b=1, c=8, h=11, w=11, n=8, size=5),
    "7x7_s2": dict(b=1, c=8, h=20, w=20, n=16, size=7, stride=2),
    "heads_255": dict(b=2, c=64, h=13, w=13, n=255, size=1, bn=False, act="linear"),
    "n512_two_ntiles": dict(b=1, c=64, h=13, w=13, n=512, size=3),
    "n1000_logistic": dict(b=2, c=128, h=3, w=3, n=1000, size=1, bn=False, act="logistic"),
    "darknet53_mid": dict(b=1, c=256, h=13, w=13, n=512, size=3),
    "many_tiles": dict(b=4, c=64, h=64, w=64, n=64, size=3),
    "map19_batch_folded": dict(b=8, c=128, h=19, w=19, n=256, size=3),
    "k4608": dict(b=2, c=512, h=7, w=7, n=64, size=3),
}


@pytest.mark.parametrize("name", list(TC_CASES))
def test_conv_tc_tf32(name):
    case = conv_case(200, **TC_CASES[name])
    want = oracle_conv(case)
    plan, got, got2 = run_conv(case, dn.MODE_TF32, "nchw", "nchw", both=True)
    assert plan.kernel == "tc_tf32"
    parity(got, want, TOL_TF32, name)
    assert np.array_equal(got, got2), "NCHW and NHWC copies of one launch differ"
    # channels-last in, channels-last out (the layout used between layers)
    _, got3, _ = run_conv(case, dn.MODE_TF32, "nhwc", "nhwc")
    parity(got3, want, TOL_TF32)


@pytest.mark.parametrize("name", list(TC_CASES))
def test_conv_tc_bf16(name):
    case = conv_case(300, **TC_CASES[name])
    want = oracle_conv(case)
    plan, got, _ = run_conv(case, dn.MODE_BF16, "nchw", "nchw")
    assert plan.kernel == "tc_bf16"
    parity(got, want, TOL_BF16, name)
    _, got3, _ = run_conv(case, dn.MODE_BF16, "nhwc", "nhwc")
    parity(got3, want, TOL_BF16)


HALO_CASES = {
    "c32_n64": dict(b=2, c=32, h=32, w=24, n=64, size=3),
    "c64_n128_two_blocks": dict(b=1, c=64, h=48, w=40, n=128, size=3),
    "ragged_19x21": dict(b=3, c=32, h=21, w=19, n=32, size=3),
    "c40_ragged_k": dict(b=1, c=40, h=16, w=8, n=16, size=3),
    "c128_n256_forced": dict(b=1, c=128, h=32, w=16, n=256, size=3),
    "n512_two_ntiles_forced": dict(b=1, c=64, h=16, w=16, n=512, size=3),
}


@pytest.mark.parametrize("name", list(HALO_CASES))
@pytest.mark.parametrize("mode,tol", [(dn.MODE_TF32, TOL_TF32), (dn.MODE_BF16, TOL_BF16)])
def test_conv_tc_halo_mode(name, mode, tol, monkeypatch):
    """3x3 stride-1 layers in halo mode (one activation box per channel block serves all nine taps through
    shifted A descriptors), forced on wherever the geometry allows, against the ordinary rings and the checker."""
    case = conv_case(250, **HALO_CASES[name])
    want = oracle_conv(case)
    monkeypatch.setenv("DNB_TC_HALO", "2")
    _, got, _ = run_conv(case, mode, "nhwc", "nhwc")
    monkeypatch.setenv("DNB_TC_HALO", "0")
    _, plain, _ = run_conv(case, mode, "nhwc", "nhwc")
    parity(got, want, tol, name)
    # same products in another summation order: a few results land on the neighbouring TF32 (bf16) value when rounded for storage
    parity(got, plain, (2e-3 if mode == dn.MODE_TF32 else 1e-2))
    monkeypatch.setenv("DNB_TC_HALO", "2")
    _, got_nchw, got_nhwc = run_conv(case, mode, "nchw", "nchw", both=True)
    assert np.array_equal(got_nchw, got_nhwc)
    parity(got_nchw, want, tol)


PAIR_CASES = {
    # shapes with enough tiles of 256 filters for the CTA-pair kernel: (pixel tiles + 1) / 2 * (filters / 256) >= 74
    "c128_38x38_n512_odd_pixel_tiles": dict(b=8, c=128, h=38, w=38, n=512, size=3),          # 95 pixel tiles: the last pair is half empty
    "c64_19x19_n1024_batch9": dict(b=9, c=64, h=19, w=19, n=1024, size=3),                    # 45 pixel tiles of 32 x 4 x 1
    "s2_76_to_38_n512": dict(b=8, c=64, h=76, w=76, n=512, size=3, stride=2),
    "c64_76x76_n256_one_filter_tile": dict(b=4, c=64, h=76, w=76, n=256, size=3),
    "logistic_nobn_n256": dict(b=16, c=64, h=40, w=40, n=256, size=3, bn=False, act="logistic"),
}


@pytest.mark.parametrize("name", list(PAIR_CASES))
@pytest.mark.parametrize("mode,tol", [(dn.MODE_TF32, TOL_TF32), (dn.MODE_BF16, TOL_BF16)])
def test_conv_tc_cta_pairs(name, mode, tol, monkeypatch):
    """Layers large enough for the CTA-pair kernel (clusters of two CTAs sharing every MMA, half a weight tile
    each): against the checker, against the single-CTA kernel, and with Darknet's layout written beside."""
    case = conv_case(260, **PAIR_CASES[name])
    want = oracle_conv(case)
    monkeypatch.setenv("DNB_TC_SPLITK", "0")   # the pair kernel by itself; split-K has its own tests below
    monkeypatch.setenv("DNB_TC_PAIR", "1")
    plan, got, _ = run_conv(case, mode, "nhwc", "nhwc")
    assert "pair=1" in plan.describe(), plan.describe()
    parity(got, want, tol, name)
    monkeypatch.setenv("DNB_TC_PAIR", "0")
    plan0, single, _ = run_conv(case, mode, "nhwc", "nhwc")
    assert "pair=0" in plan0.describe()
    parity(got, single, (2e-3 if mode == dn.MODE_TF32 else 1e-2), "pair against single CTA")
    monkeypatch.setenv("DNB_TC_PAIR", "1")
    _, got_nchw, got_nhwc = run_conv(case, mode, "nchw", "nchw", both=True)   # Darknet's layout in and out, channels-last beside
    assert np.array_equal(got_nchw, got_nhwc)
    parity(got_nchw, want, tol, name)


def test_conv_tc_cta_pairs_1x1_when_forced(monkeypatch):
    case = conv_case(261, b=32, c=512, h=19, w=19, n=512, size=1)
    monkeypatch.setenv("DNB_TC_PAIR", "2")
    plan, got, _ = run_conv(case, dn.MODE_TF32, "nhwc", "nhwc")
    assert "pair=1" in plan.describe(), plan.describe()
    parity(got, oracle_conv(case), TOL_TF32, "1x1 in pair mode")


@pytest.mark.parametrize("mode,tol", [(dn.MODE_TF32, TOL_TF32), (dn.MODE_BF16, TOL_BF16)])
def test_conv_tc_cta_pairs_with_fused_shortcut(mode, tol, monkeypatch):
    import ctypes as C
    monkeypatch.setenv("DNB_TC_PAIR", "1")
    monkeypatch.setenv("DNB_TC_SPLITK", "0")
    case = conv_case(262, b=8, c=128, h=38, w=38, n=512, size=3)
    x, w = case["x"], case["w"]
    b, c, h, wd = x.shape
    n = w.shape[0]
    add = rng(263).standard_normal((b, n, h, wd), dtype=np.float32)
    store = torch.bfloat16 if mode == dn.MODE_BF16 else torch.float32
    if mode == dn.MODE_BF16:
        add = bf16_round(add)
    want = orc.shortcut_forward(oracle_conv(case), add, 1.0, 1.0, "linear")
    plan = dn.ConvPlan(b, c, h, wd, n, 3, 1, 1, 1, True, case["act"], False, mode)
    plan.set_params(w, case["biases"], case["scales"], case["mean"], case["var"])
    xt, xd = dev_nhwc(x, store)
    at, ad = dev_nhwc(add, store)
    yt, yd = empty_nhwc(b, n, h, wd, store)
    dn.check(dn.lib().dnb_conv_shortcut_forward(plan.handle, C.byref(xd), C.byref(ad), C.byref(yd), 1.0, 1.0, dn.ACTIVATIONS["linear"],
                                                C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    plan.check_status()
    assert "pair=1" in plan.describe(), plan.describe()
    parity(host_from_nhwc(yt, n), want, tol, "pair mode with fused shortcut")
    assert padding_is_zero(yt, n)


@pytest.mark.parametrize("mode,tol", [(dn.MODE_TF32, TOL_TF32), (dn.MODE_BF16, TOL_BF16)])
@pytest.mark.parametrize("shape", [dict(b=2, c=256, h=19, w=19, anchors=3, classes=80),      # YOLOv3's heads: 255 filters
                                   dict(b=3, c=64, h=13, w=11, anchors=2, classes=1),        # 12 filters, ragged tiles
                                   dict(b=1, c=128, h=8, w=8, anchors=5, classes=20)])       # 125 filters
def test_conv_with_fused_yolo_head(shape, mode, tol):
    """Convolution + the [yolo] layer after it in one launch against the checker's convolution followed by its
    yolo layer (src/yolo_layer.c:347-357: logistic on every entry but w and h of each anchor)."""
    import ctypes as C
    anchors, classes = shape["anchors"], shape["classes"]
    n = anchors * (classes + 5)
    case = conv_case(270 + n, b=shape["b"], c=shape["c"], h=shape["h"], w=shape["w"], n=n, size=1, bn=False, act="linear")
    x = case["x"]
    b, c, h, wd = x.shape
    store = torch.bfloat16 if mode == dn.MODE_BF16 else torch.float32
    want = orc.yolo_forward(oracle_conv(case), anchors, classes)
    plan = dn.ConvPlan(b, c, h, wd, n, 1, 1, 0, 1, False, "linear", False, mode)
    plan.set_params(case["w"], case["biases"], None, None, None)
    xt, xd = dev_nhwc(x, store)
    yt, yd = empty_nchw(b, n, h, wd)
    yt.fill_(float("nan"))
    dn.check(dn.lib().dnb_conv_yolo_forward(plan.handle, C.byref(xd), C.byref(yd), anchors, classes,
                                            C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    plan.check_status()
    got = yt.cpu().numpy()
    assert np.isfinite(got).all()
    parity(got, want, tol, f"fused yolo head, {n} filters")
    # the w and h entries are the raw predictions, everything else went through the logistic
    raw = got.reshape(b, anchors, classes + 5, h, wd)
    assert ((raw[:, :, [0, 1]] > 0) & (raw[:, :, [0, 1]] < 1)).all() and ((raw[:, :, 4:] > 0) & (raw[:, :, 4:] < 1)).all()
    assert (raw[:, :, 2:4] < 0).any()
    # wrong anchor count for the plan's filters
    with pytest.raises(dn.DarknetB200Error) as e:
        dn.check(dn.lib().dnb_conv_yolo_forward(plan.handle, C.byref(xd), C.byref(yd), anchors + 1, classes, None))
    assert e.value.status == dn.EINVAL


SPLIT_CASES = {
    # (case, forced ranges or None for the plan's own choice, expects pair mode)
    "single_19x19_c256_n128_forced3": (dict(b=2, c=256, h=19, w=19, n=128, size=3), "3", False),
    "single_1x1_c512_n64_forced2": (dict(b=1, c=512, h=13, w=13, n=64, size=1), "2", False),
    "single_s2_c128_n128_forced8": (dict(b=1, c=128, h=38, w=38, n=128, size=3, stride=2), "8", False),
    "pair_19x19_c1024_n512_batch4_auto": (dict(b=4, c=1024, h=19, w=19, n=512, size=3), None, True),       # YOLOv3's 19x19 shape at 8 images per GPU
    "pair_19x19_c1024_n1024_batch1_auto": (dict(b=1, c=1024, h=19, w=19, n=1024, size=3), None, True),    # one image of YOLOv3's last stage: 8 pair tiles
    "pair_19x19_c512_n256_batch3_forced5": (dict(b=3, c=512, h=19, w=19, n=256, size=3, act="linear", bn=False), "5", True),  # odd pixel tiles: a phantom tile delivers ranges too
}


@pytest.mark.parametrize("name", list(SPLIT_CASES))
@pytest.mark.parametrize("mode,tol", [(dn.MODE_TF32, TOL_TF32), (dn.MODE_BF16, TOL_BF16)])
def test_conv_tc_split_k(name, mode, tol, monkeypatch):
    """Split-K: every tile's K loop cut into ranges that run on different CTAs and meet through L2.  Against the
    checker, against the unsplit kernel, and three launches in a row (the counters reset themselves)."""
    shape, forced, pair = SPLIT_CASES[name]
    case = conv_case(280, **shape)
    want = oracle_conv(case)
    if forced:
        monkeypatch.setenv("DNB_TC_SPLITK", forced)
    else:
        monkeypatch.delenv("DNB_TC_SPLITK", raising=False)
    x, w = case["x"], case["w"]
    b, c, h, wd = x.shape
    n, size = w.shape[0], w.shape[2]
    plan = dn.ConvPlan(b, c, h, wd, n, size, case["stride"], case["pad"], 1, case["scales"] is not None, case["act"], False, mode)
    plan.set_params(w, case["biases"], case["scales"], case["mean"], case["var"])
    store = torch.bfloat16 if mode == dn.MODE_BF16 else torch.float32
    xt, xd = dev_nhwc(x, store)
    yt, yd = empty_nhwc(b, n, plan.out_h, plan.out_w, store)
    outs = []
    for _ in range(3):
        yt.zero_()
        plan.forward(xd, yd)
        torch.cuda.synchronize()
        plan.check_status()
        outs.append(host_from_nhwc(yt, n))
    d = plan.describe()
    assert f"pair={int(pair)}" in d, d
    splits = int(d.split("splits=")[1].split()[0])
    assert splits > 1 and (not forced or splits == int(forced)), d
    parity(outs[0], want, tol, name)
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])   # fixed order of the ranges: bit-reproducible
    assert padding_is_zero(yt, n)
    monkeypatch.setenv("DNB_TC_SPLITK", "0")
    plan0, whole, _ = run_conv(case, mode, "nhwc", "nhwc")
    assert "splits=1" in plan0.describe()
    parity(outs[0], whole, (2e-3 if mode == dn.MODE_TF32 else 1e-2), "split against unsplit")


@pytest.mark.parametrize("mode,tol", [(dn.MODE_TF32, TOL_TF32), (dn.MODE_BF16, TOL_BF16)])
def test_conv_tc_split_k_with_fused_shortcut(mode, tol, monkeypatch):
    """A residual block of YOLOv3's 19x19 stage at 2 images: CTA pairs, split-K chosen by the plan, residual added by
    the CTA that finishes each tile."""
    import ctypes as C
    monkeypatch.delenv("DNB_TC_SPLITK", raising=False)
    case = conv_case(281, b=2, c=1024, h=19, w=19, n=1024, size=3)
    x, w = case["x"], case["w"]
    b, c, h, wd = x.shape
    n = w.shape[0]
    add = rng(282).standard_normal((b, n, h, wd), dtype=np.float32)
    store = torch.bfloat16 if mode == dn.MODE_BF16 else torch.float32
    if mode == dn.MODE_BF16:
        add = bf16_round(add)
    want = orc.shortcut_forward(oracle_conv(case), add, 1.0, 1.0, "linear")
    plan = dn.ConvPlan(b, c, h, wd, n, 3, 1, 1, 1, True, case["act"], False, mode)
    plan.set_params(w, case["biases"], case["scales"], case["mean"], case["var"])
    xt, xd = dev_nhwc(x, store)
    at, ad = dev_nhwc(add, store)
    yt, yd = empty_nhwc(b, n, h, wd, store)
    for _ in range(2):
        yt.zero_()
        dn.check(dn.lib().dnb_conv_shortcut_forward(plan.handle, C.byref(xd), C.byref(ad), C.byref(yd), 1.0, 1.0, dn.ACTIVATIONS["linear"],
                                                    C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        torch.cuda.synchronize()
        plan.check_status()
        d = plan.describe()
        assert "pair=1" in d and "splits=1" not in d, d
        parity(host_from_nhwc(yt, n), want, tol, "split-K pair with fused shortcut")


@pytest.mark.parametrize("act", list(dn.ACTIVATIONS))
@pytest.mark.parametrize("kernel", ["tc_tf32", "tc_bf16", "direct_fp32", "shortcut"])
def test_every_activation(act, kernel):
    """All fourteen activations of src/activations.h:35-86 through every epilogue that applies one: the tensor-core
    convolution (compiled in: linear, leaky; the others through the run-time switch), the CUDA-core convolution and
    the shortcut kernel.  `stair` is a step function: values a rounding error away from a step land on the other side
    of it, so it is compared element by element with a small share of misses allowed."""
    mode, tol = {"tc_tf32": (dn.MODE_TF32, TOL_TF32), "tc_bf16": (dn.MODE_BF16, TOL_BF16), "direct_fp32": (dn.MODE_FP32, TOL_FP32),
                 "shortcut": (dn.MODE_FP32, TOL_FP32)}[kernel]
    if kernel == "shortcut":
        g = rng(301)
        x = g.standard_normal((2, 24, 9, 10), dtype=np.float32) * 2
        add = g.standard_normal((2, 24, 9, 10), dtype=np.float32) * 2
        want = orc.shortcut_forward(x, add, 1.0, 1.0, act)
        xt, xd = dev_nhwc(x)
        at, ad = dev_nhwc(add)
        yt, yd = empty_nhwc(2, 24, 9, 10)
        dn.shortcut(xd, ad, yd, 1.0, 1.0, act)
        torch.cuda.synchronize()
        got = host_from_nhwc(yt, 24)
    else:
        case = conv_case(300, b=2, c=16, h=12, w=12, n=24, size=3, act=act)
        plan, got, _ = run_conv(case, mode, "nhwc" if kernel.startswith("tc_") else "nchw", "nhwc" if kernel.startswith("tc_") else "nchw")
        assert plan.kernel == kernel
        want = oracle_conv(case)
    if act == "stair":
        close = np.abs(got - want) <= tol * np.abs(want).max()
        assert close.mean() > 0.99, f"{kernel} stair: {100 * (1 - close.mean()):.2f} % of the values on the other side of a step"
    else:
        parity(got, want, tol, f"{kernel} activation {act}")


@pytest.mark.parametrize("name", ["c128_38x38_n512_odd_pixel_tiles", "c64_76x76_n256_one_filter_tile"])
@pytest.mark.parametrize("mode,tol", [(dn.MODE_TF32, TOL_TF32), (dn.MODE_BF16, TOL_BF16)])
def test_conv_tc_per_warp_stores(name, mode, tol, monkeypatch):
    """The experimental epilogue in which every warp stores its own 32 rows (DNB_TC_WARP_STORES=1): pairs and single
    CTAs, against the checker and bit-equal to the default epilogue."""
    case = conv_case(290, **PAIR_CASES[name])
    want = oracle_conv(case)
    outs = {}
    for pair in ("1", "0"):
        monkeypatch.setenv("DNB_TC_PAIR", pair)
        for ws in ("0", "1"):
            monkeypatch.setenv("DNB_TC_WARP_STORES", ws)
            _, got, _ = run_conv(case, mode, "nhwc", "nhwc")
            outs[(pair, ws)] = got
        assert np.array_equal(outs[(pair, "0")], outs[(pair, "1")])
        parity(outs[(pair, "1")], want, tol, f"{name} per-warp stores, pair={pair}")


DUAL_CASES = {
    # Darknet's layout written beside the channels-last tensor (what the per-layer attach asks of every convolution),
    # in the kernel variants the plain cases do not reach
    "1x1_c512_n256_38x38_b16_pair_flat": (dict(b=16, c=512, h=38, w=38, n=256, size=1), "pair=1"),     # pairs over a plane treated as one row of pixels
    "3x3_c1024_n1024_19x19_b1_pair_split": (dict(b=1, c=1024, h=19, w=19, n=1024, size=3), "pair=1"),  # split-K finishing CTA writes both layouts
    "1x1_c256_n255_76x76_b2_flat": (dict(b=2, c=256, h=76, w=76, n=255, size=1, bn=False, act="linear"), "pair=0"),
    "3x3_s2_c64_n128_76_b4": (dict(b=4, c=64, h=76, w=76, n=128, size=3, stride=2), "pair=0"),
}


@pytest.mark.parametrize("name", list(DUAL_CASES))
@pytest.mark.parametrize("mode,tol", [(dn.MODE_TF32, TOL_TF32), (dn.MODE_BF16, TOL_BF16)])
def test_conv_tc_both_layouts(name, mode, tol, monkeypatch):
    monkeypatch.delenv("DNB_TC_SPLITK", raising=False)
    monkeypatch.delenv("DNB_TC_PAIR", raising=False)
    shape, expect = DUAL_CASES[name]
    case = conv_case(295, **shape)
    want = oracle_conv(case)
    plan, got_nchw, got_nhwc = run_conv(case, mode, "nhwc", "nchw", both=True)
    if mode == dn.MODE_TF32:
        assert expect in plan.describe(), plan.describe()
    assert np.array_equal(got_nchw, got_nhwc)
    parity(got_nchw, want, tol, name)
    _, only_nchw, _ = run_conv(case, mode, "nchw", "nchw")          # Darknet's layout in and out, nothing else
    parity(only_nchw, want, tol, name + " (NCHW only)")


def test_conv_tc_all_ones_counts_taps():
    # analytic known answer: ones everywhere -> in-image taps x channels, exact in TF32 and BF16
    C, H, W, N = 16, 9, 10, 16
    case = dict(x=np.ones((2, C, H, W), np.float32), w=np.ones((N, C, 3, 3), np.float32), biases=np.zeros(N, np.float32),
                scales=None, mean=None, var=None, stride=1, pad=1, groups=1, act="linear")
    ys, xs = np.arange(H), np.arange(W)
    ny = np.minimum(ys + 1, H - 1) - np.maximum(ys - 1, 0) + 1
    nx = np.minimum(xs + 1, W - 1) - np.maximum(xs - 1, 0) + 1
    want = np.broadcast_to((ny[:, None] * nx[None, :] * C).astype(np.float32), (2, N, H, W))
    for mode in (dn.MODE_TF32, dn.MODE_BF16, dn.MODE_FP32):
        _, got, _ = run_conv(case, mode)
        assert np.array_equal(got, want)


XNOR_CASES = {
    "3x3_c64": dict(b=2, c=64, h=10, w=10, n=32, size=3),
    "3x3_c32_one_mma_per_tap": dict(b=3, c=32, h=20, w=20, n=64, size=3),
    "3x3_c512_n1024_pairs": dict(b=16, c=512, h=7, w=7, n=1024, size=3),       # K = 4608; enough tiles for CTA pairs
    "1x1_c1024_n512": dict(b=8, c=1024, h=7, w=7, n=512, size=1),
    "3x3_c40_ragged_word": dict(b=2, c=40, h=6, w=7, n=9, size=3),
    "1x1_c128": dict(b=2, c=128, h=7, w=7, n=64, size=1),
    "3x3_c1024": dict(b=1, c=1024, h=7, w=7, n=70, size=3),
    "3x3_s2": dict(b=1, c=32, h=9, w=9, n=16, size=3, stride=2),
}


@pytest.mark.parametrize("name", list(XNOR_CASES))
@pytest.mark.parametrize("in_layout", ["nchw", "nhwc"])
@pytest.mark.parametrize("kernel", ["xnor_tc", "xnor_popc"])
def test_conv_xnor(name, in_layout, kernel, monkeypatch):
    """Both xnor kernels, the int8 tensor-core one (default) and the bit-packed popcount one (DNB_XNOR_TC=0): integer
    sums bit for bit against the checker, layer outputs within 1e-5."""
    monkeypatch.setenv("DNB_XNOR_TC", "1" if kernel == "xnor_tc" else "0")
    case = conv_case(400, **XNOR_CASES[name])
    x, w = case["x"], case["w"]
    x.reshape(-1)[::7] = 0.0   # exact zeros binarise to -1 (the CPU reference tests x > 0)
    b, c, h, wd = x.shape
    n = w.shape[0]
    plan = dn.ConvPlan(b, c, h, wd, n, w.shape[2], case["stride"], case["pad"], 1, True, case["act"], True, dn.MODE_TF32)
    plan.set_params(w, case["biases"], case["scales"], case["mean"], case["var"])
    assert plan.kernel == (kernel if case["stride"] <= 2 else "xnor_popc")
    xt, xd = dev_nchw(x) if in_layout == "nchw" else dev_nhwc(x)
    acc = torch.full((b, n, plan.out_h, plan.out_w), -12345, dtype=torch.int32, device="cuda")
    plan.xnor_accumulate(xd, acc)
    want_acc = orc.xnor_accumulate(x, w, stride=case["stride"], pad=case["pad"])
    assert np.array_equal(acc.cpu().numpy(), want_acc.astype(np.int32)), "popcount accumulators must be bit-exact"
    yt, yd = empty_nchw(b, n, plan.out_h, plan.out_w)
    y2t, y2d = empty_nhwc(b, n, plan.out_h, plan.out_w)
    plan.forward(xd, yd, y2d)
    want = oracle_conv(case, xnor=True)
    # the CPU adds +-mean one product at a time in fp32; mean * integer differs from that sum in the last bits
    parity(yt.cpu().numpy(), want, 1e-5)
    assert np.array_equal(host_from_nhwc(y2t, n), yt.cpu().numpy()) and padding_is_zero(y2t, n)


def test_conv_xnor_power_of_two_mean_is_bit_exact():
    # with |w| = 2^-3 everywhere the per-filter mean is a power of two, every partial sum on the CPU is
    # exact, and the whole layer output (bias only, linear) must match bit for bit
    g = rng(500)
    x = g.standard_normal((2, 64, 8, 8), dtype=np.float32)
    w = np.where(g.random((16, 64, 3, 3)) > 0.5, 0.125, -0.125).astype(np.float32)
    case = dict(x=x, w=w, biases=np.zeros(16, np.float32), scales=None, mean=None, var=None, stride=1, pad=1, groups=1, act="linear")
    plan = dn.ConvPlan(2, 64, 8, 8, 16, 3, 1, 1, 1, False, "linear", True, dn.MODE_TF32).set_params(w, case["biases"])
    xt, xd = dev_nchw(x)
    yt, yd = empty_nchw(2, 16, 8, 8)
    plan.forward(xd, yd)
    assert np.array_equal(yt.cpu().numpy(), oracle_conv(case, xnor=True))


def test_conv_rejects_mismatched_tensors():
    plan = dn.ConvPlan(1, 8, 8, 8, 16, 3, 1, 1).set_params(np.zeros((16, 8, 3, 3), np.float32), np.zeros(16, np.float32))
    xt, xd = dev_nchw(np.zeros((1, 8, 8, 8), np.float32))
    yt, yd = empty_nchw(1, 16, 7, 8)
    with pytest.raises(dn.DarknetB200Error):
        plan.forward(xd, yd)
    bt, bd = dev_nhwc(np.zeros((1, 8, 8, 8), np.float32), torch.bfloat16)
    gt, gd = empty_nchw(1, 16, 8, 8)
    with pytest.raises(dn.DarknetB200Error):
        plan.forward(bd, gd)   # bf16 input to a TF32 plan


@pytest.mark.parametrize("mode,tol", [(dn.MODE_TF32, TOL_TF32), (dn.MODE_BF16, TOL_BF16)])
@pytest.mark.parametrize("act2", ["linear", "leaky"])
@pytest.mark.parametrize("shape", [dict(b=2, c=64, h=13, w=13, n=64, size=3), dict(b=3, c=32, h=19, w=19, n=320, size=1),
                                   dict(b=1, c=16, h=9, w=10, n=24, size=3)])
def test_conv_with_fused_shortcut(mode, tol, act2, shape):
    import ctypes as C
    case = conv_case(600, **shape)
    x, w = case["x"], case["w"]
    b, c, h, wd = x.shape
    n = w.shape[0]
    add = rng(601).standard_normal((b, n, h, wd), dtype=np.float32)
    store = torch.bfloat16 if mode == dn.MODE_BF16 else torch.float32
    if mode == dn.MODE_BF16:
        add = bf16_round(add)
    want = orc.shortcut_forward(oracle_conv(case), add, 1.0, 1.0, act2)
    plan = dn.ConvPlan(b, c, h, wd, n, w.shape[2], 1, case["pad"], 1, True, case["act"], False, mode)
    plan.set_params(w, case["biases"], case["scales"], case["mean"], case["var"])
    xt, xd = dev_nhwc(x, store)
    at, ad = dev_nhwc(add, store)
    yt, yd = empty_nhwc(b, n, h, wd, store)
    dn.check(dn.lib().dnb_conv_shortcut_forward(plan.handle, C.byref(xd), C.byref(ad), C.byref(yd), 1.0, 1.0, dn.ACTIVATIONS[act2],
                                                C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    plan.check_status()
    parity(host_from_nhwc(yt, n), want, tol)
    assert padding_is_zero(yt, n)
