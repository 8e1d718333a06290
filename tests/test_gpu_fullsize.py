"""Parity at the benchmark's full sizes, where the CPU checker cannot redo every image in seconds.

* The isolated darknet-53 mid-stage layers (batch 64, 256 -> 512 3x3 and 512 -> 256 1x1 at 52x52): two
  of the 64 images are recomputed by the checker; the rest is held by properties that do not depend on
  the size: images are independent (a permuted batch gives the permuted output, bit for bit) and a
  bias-free linear layer is homogeneous (scaling the input by a power of two scales the output exactly).
* YOLOv3 at 608x608: one image through all 107 layers against the checker, per layer, plus image
  independence on a batch of two.

Tolerance: max |gpu - cpu| / max |cpu| per layer output, TF32 1e-2.
"""
import numpy as np
import pytest
import torch

import darknet_b200 as dn
from conftest import parity, rel_to_max
from darknet_b200 import synth
from gpu_util import dev_nhwc, empty_nhwc, host_from_nhwc
from oracle import network as orc

pytestmark = pytest.mark.gpu
TOL_TF32 = 1e-2


def philox(seed):
    return np.random.Generator(np.random.Philox(key=[seed, 99]))


def conv_full(b, c, n, size, seed, bn=True, act="leaky"):
    g = philox(seed)
    x = g.standard_normal((b, c, 52, 52), dtype=np.float32)
    w = g.standard_normal((n, c, size, size), dtype=np.float32) * np.float32(np.sqrt(2.0 / (size * size * c)))
    if bn:
        p = dict(biases=g.standard_normal(n, dtype=np.float32) * np.float32(0.1), scales=g.uniform(0.9, 1.1, n).astype(np.float32),
                 mean=g.standard_normal(n, dtype=np.float32) * np.float32(0.1), var=g.uniform(0.5, 1.5, n).astype(np.float32))
    else:
        p = dict(biases=np.zeros(n, np.float32), scales=None, mean=None, var=None)
    return x, w, p, act


def gpu_conv(x, w, p, act, size):
    b, c, h, wd = x.shape
    n = w.shape[0]
    plan = dn.ConvPlan(b, c, h, wd, n, size, 1, size // 2, 1, p["scales"] is not None, act, False, dn.MODE_TF32)
    plan.set_params(w, p["biases"], p["scales"], p["mean"], p["var"])
    xt, xd = dev_nhwc(x)
    yt, yd = empty_nhwc(b, n, plan.out_h, plan.out_w)
    plan.forward(xd, yd, None)
    torch.cuda.synchronize()
    plan.check_status()
    return host_from_nhwc(yt, n)


@pytest.mark.parametrize("c,n,size", [(256, 512, 3), (512, 256, 1)])
def test_isolated_layer_at_full_size(c, n, size):
    x, w, p, act = conv_full(64, c, n, size, seed=7)
    got = gpu_conv(x, w, p, act, size)
    for img in (0, 63):   # the checker redoes two images (6.4 GFLOP each for the 3x3 layer)
        want = orc.conv_forward(x[img:img + 1], w, p["biases"], p["scales"], p["mean"], p["var"], stride=1, pad=size // 2,
                                groups=1, activation=act)
        parity(got[img:img + 1], want, TOL_TF32, f"image {img}")
    # images are independent: the reversed batch gives the reversed output, bit for bit
    got_rev = gpu_conv(x[::-1].copy(), w, p, act, size)
    assert np.array_equal(got_rev[::-1], got)


@pytest.mark.parametrize("c,n,size", [(256, 512, 3), (512, 256, 1)])
def test_linear_layer_is_homogeneous_at_full_size(c, n, size):
    x, w, p, act = conv_full(64, c, n, size, seed=8, bn=False, act="linear")
    y1 = gpu_conv(x, w, p, act, size)
    y4 = gpu_conv(x * np.float32(4.0), w, p, act, size)
    assert np.array_equal(y4, y1 * np.float32(4.0))
    assert np.abs(y1).max() > 0.5


def test_yolov3_608_one_image_every_layer(tmp_path):
    cfg = synth.yolov3_cfg(batch=1, size=608)
    params = synth.seeded_params(cfg, 3)
    x = synth.seeded_input(cfg, 3, "uniform")
    wpath = str(tmp_path / "y.weights")
    synth.write_weights(wpath, params)
    want = orc.forward_network(cfg, params, x)            # 140.7 GFLOP on the host cores
    net = dn.Network(cfg, wpath, dn.MODE_TF32, text=True)
    net.predict(x)
    worst, checked = 0.0, 0
    for i, wnt in enumerate(want):
        try:
            got = net.layer_output(i)
        except dn.DarknetB200Error:
            continue                                        # a convolution fused with the shortcut or yolo layer after it has no output of its own
        e = parity(got, wnt, TOL_TF32, f"layer {i}")
        worst = max(worst, e)
        checked += 1
    assert checked >= 107 - 23 - 3
    print(f"yolov3-608: {checked} layer outputs checked, worst rel error {worst:.3g}")
    # a batch of two: each image's heads equal the single-image run, bit for bit
    cfg2 = synth.yolov3_cfg(batch=2, size=608)
    x2 = np.concatenate([synth.seeded_input(cfg, 4, "uniform"), x], 0)
    net2 = dn.Network(cfg2, wpath, dn.MODE_TF32, text=True)
    out2 = net2.predict(x2).copy()
    out1 = net.predict(x).copy()
    assert np.array_equal(out2[1], out1[0])


@pytest.mark.parametrize("name,gen,batch,seed", [
    ("yolov3-tiny-416 batch 1 (the reference's own CPU-runnable case)", lambda b: synth.yolov3_tiny_cfg(batch=b, size=416), 1, 5),
    ("resnet50-224 batch 2", lambda b: synth.resnet50_cfg(batch=b, size=224), 2, 6),
])
def test_other_benchmark_networks_at_full_resolution(name, gen, batch, seed, tmp_path):
    cfg = gen(batch)
    params = synth.seeded_params(cfg, seed)
    x = synth.seeded_input(cfg, seed, "uniform")
    wpath = str(tmp_path / "n.weights")
    synth.write_weights(wpath, params)
    want = orc.forward_network(cfg, params, x)
    net = dn.Network(cfg, wpath, dn.MODE_TF32, text=True)
    out = net.predict(x).copy()
    worst, checked = 0.0, 0
    for i, wnt in enumerate(want):
        try:
            got = net.layer_output(i)
        except dn.DarknetB200Error:
            continue
        e = parity(got, wnt, TOL_TF32, f"{name}, layer {i}")
        worst = max(worst, e)
        checked += 1
    parity(out.reshape(want[-1].shape), want[-1], TOL_TF32)
    print(f"{name}: {checked} layer outputs checked, worst rel error {worst:.3g}")


@pytest.mark.parametrize("size", [320, 416])
@pytest.mark.parametrize("mode,tol", [(dn.MODE_TF32, 1e-2), (dn.MODE_BF16, 6e-2)])
def test_yolov3_other_input_sizes(size, mode, tol, tmp_path):
    """The other customary YOLOv3 resolutions (10/20/40 and 13/26/52 maps instead of 19/38/76): pixel tiles,
    batch folding and tile counts all differ from the benchmark's.  One image, the three heads against the checker
    (BF16 end to end through 75 convolutions: 6e-2, as in test_gpu_network.py)."""
    cfg = synth.yolov3_cfg(batch=1, size=size)
    params = synth.seeded_params(cfg, 7)
    x = synth.seeded_input(cfg, 7, "uniform")
    wpath = str(tmp_path / "y.weights")
    synth.write_weights(wpath, params)
    want = orc.forward_network(cfg, params, x)
    net = dn.Network(cfg, wpath, mode, text=True)
    net.predict(x)
    heads = [i for i in range(net.n) if net.layer_type(i) == "yolo"]
    assert len(heads) == 3
    for i in heads:
        parity(net.yolo_output(i), want[i], tol, f"size {size}, head {i}")
