"""Parity at the benchmark configurations' own batch sizes.

The plan of every convolution depends on the batch (the batch is folded into the 128-pixel tile, and
filter-tile width, ring depth, CTAs per SM and tile counts follow), so a batch of one or two does not
cover the batch the benchmark runs.  Each test runs the whole batch on the GPU and lets the CPU checker
redo three of its images (first, middle, last) at batch 1: inference is independent per image
(src/convolutional_layer.c:461-475 loops over the batch, batchnorm uses the rolling statistics).

* YOLOv3-608, batch 64, TF32 and BF16: every layer output of the three images.
* ResNet-50-224, batch 256, TF32: every layer output of the three images.
* xnor Darknet-19-224, batch 128: binarisation turns last-bit differences into sign flips, so the xnor
  layers are checked teacher-forced, each at batch 128 on inputs the checker produced: integer
  accumulators bit for bit (the 112x112 one-word-per-pixel layer and the 7x7 layers with K = 4608,
  the longest sums of the network, among them), layer outputs within 1e-5; the whole network at batch 128 must give, bit for bit, what a
  batch of three gives.

Tolerance per layer output, max |gpu - cpu| / max |cpu|: TF32 1e-2, BF16 6e-2 end to end through 75
layers (3e-2 per layer is checked teacher-forced in test_gpu_layers.py).  The element-wise figure
(conftest.rel_elementwise) is recorded next to it for the end-of-run table.
"""
import numpy as np
import pytest
import torch

import darknet_b200 as dn
from conftest import parity, rel_to_max
from darknet_b200 import synth
from gpu_util import dev_nchw, empty_nchw
from oracle import network as orc

pytestmark = pytest.mark.gpu


def three_images(batch):
    return [0, batch // 2, batch - 1]


def checker_outputs(gen, params, x, images):
    """Every layer's output of the chosen images, recomputed by the CPU checker one image at a time."""
    cfg1 = gen(1)
    return {img: orc.forward_network(cfg1, params, x[img:img + 1]) for img in images}


def compare_layers(net, want_by_image, tol, name):
    checked = 0
    for img, want in want_by_image.items():
        for i, wnt in enumerate(want):
            try:
                got = net.layer_output_images(i, img, 1)
            except dn.DarknetB200Error as e:
                assert e.status == dn.EUNSUPPORTED   # a convolution fused with the shortcut or yolo layer after it has no output of its own
                continue
            parity(got, wnt.reshape(got.shape), tol, f"{name} image {img} layer {i} ({net.layer_kernel(i)})")
            checked += 1
    return checked


@pytest.fixture(scope="module")
def yolov3_b64(tmp_path_factory):
    gen = lambda b: synth.yolov3_cfg(batch=b, size=608)   # noqa: E731
    cfg = gen(64)
    params = synth.seeded_params(cfg, 21)
    x = synth.seeded_input(cfg, 21, "uniform")
    wpath = str(tmp_path_factory.mktemp("y64") / "y.weights")
    synth.write_weights(wpath, params)
    want = checker_outputs(gen, params, x, three_images(64))   # 3 x 140.7 GFLOP on the host cores
    return cfg, wpath, x, want


@pytest.mark.parametrize("mode,tol", [(dn.MODE_TF32, 1e-2), (dn.MODE_BF16, 6e-2)])
def test_yolov3_608_batch_64(yolov3_b64, mode, tol):
    cfg, wpath, x, want = yolov3_b64
    net = dn.Network(cfg, wpath, mode, text=True)
    out = net.predict(x)
    checked = compare_layers(net, want, tol, f"yolov3-608 b64 mode {mode}")
    assert checked >= 3 * (107 - 23 - 3)
    heads = [i for i in range(net.n) if net.layer_type(i) == "yolo"]
    for img, w in want.items():
        for i in heads:
            parity(net.yolo_output(i)[img], w[i][0], tol, f"yolov3-608 b64 mode {mode} image {img} head {i} (host copy)")
        parity(out[img], w[-1].reshape(-1), tol, f"yolov3-608 b64 mode {mode} image {img} network output")
    net.close()


def test_resnet50_224_batch_256(tmp_path):
    gen = lambda b: synth.resnet50_cfg(batch=b, size=224)   # noqa: E731
    cfg = gen(256)
    params = synth.seeded_params(cfg, 22)
    x = synth.seeded_input(cfg, 22, "uniform")
    wpath = str(tmp_path / "r.weights")
    synth.write_weights(wpath, params)
    want = checker_outputs(gen, params, x, three_images(256))
    net = dn.Network(cfg, wpath, dn.MODE_TF32, text=True)
    out = net.predict(x)
    checked = compare_layers(net, want, 1e-2, "resnet50-224 b256")
    assert checked >= 3 * 50
    for img, w in want.items():
        parity(out[img], w[-1].reshape(-1), 1e-2, f"resnet50-224 b256 image {img} network output")
    net.close()


@pytest.mark.parametrize("kernel", ["xnor_tc", "xnor_popc"])
def test_xnor_darknet19_224_batch_128(kernel, tmp_path, monkeypatch):
    monkeypatch.setenv("DNB_XNOR_TC", "1" if kernel == "xnor_tc" else "0")
    B = 128
    gen = lambda b: synth.darknet19_cfg(batch=b, size=224, xnor=True)   # noqa: E731
    cfg = gen(B)
    params = synth.seeded_params(cfg, 23)
    x = synth.seeded_input(cfg, 23, "uniform")
    src = three_images(B)
    want = checker_outputs(gen, params, x, src)
    sections = synth.parse_cfg(cfg)[1:]
    pi, xnor_layers, exact = 0, 0, []
    for i, (kind, opt) in enumerate(sections):
        if kind != "convolutional":
            continue
        p = params[pi]
        pi += 1
        if not int(opt.get("xnor", 0)):
            continue
        xnor_layers += 1
        # batch 128 of checker-produced inputs: image j is the checker's input of source image j % 3
        ins = [want[s][i - 1] for s in src]
        xin = np.concatenate([ins[j % 3] for j in range(B)], 0)
        _, c, h, w = xin.shape
        n, size, stride = int(opt["filters"]), int(opt["size"]), int(opt["stride"])
        plan = dn.ConvPlan(B, c, h, w, n, size, stride, size // 2, 1, True, opt["activation"], True)
        plan.set_params(p.weights, p.biases, p.scales, p.rolling_mean, p.rolling_variance)
        assert plan.kernel == kernel
        xt, xd = dev_nchw(xin)
        acc = torch.full((B, n, plan.out_h, plan.out_w), -12345, dtype=torch.int32, device="cuda")
        plan.xnor_accumulate(xd, acc)
        yt, yd = empty_nchw(B, n, plan.out_h, plan.out_w)
        plan.forward(xd, yd)
        torch.cuda.synchronize()
        for j in (0, 1, 2, B - 3, B - 2, B - 1):
            s = src[j % 3]
            want_acc = orc.xnor_accumulate(want[s][i - 1], p.weights, stride=stride, pad=size // 2)
            assert np.array_equal(acc[j:j + 1].cpu().numpy(), want_acc.astype(np.int32)), f"layer {i} image {j}: accumulators must be bit-exact"
            parity(yt[j:j + 1].cpu().numpy(), want[s][i], 1e-5, f"xnor darknet19-224 b128 layer {i} image {j} (teacher-forced)")
        exact.append((i, c, h, n, size))
        del xt, acc, yt
        plan.close()
    assert xnor_layers == 17
    assert any(c == 32 and h == 112 and n == 64 for _, c, h, n, _ in exact)          # one word per pixel
    assert any(c == 512 and h == 7 and size == 3 for _, c, h, _, size in exact)       # K = 4608: the network's longest sums

    # the whole network at batch 128 against a batch of three of the same images: integer accumulators and a
    # fixed order of floating-point operations per output element make the two bit-identical
    wpath = str(tmp_path / "d.weights")
    synth.write_weights(wpath, params)
    net = dn.Network(cfg, wpath, dn.MODE_TF32, text=True)
    out = net.predict(x).copy()
    assert sum(net.layer_kernel(i).startswith("xnor_") for i in range(net.n)) == 17
    first = net.layer_output_images(0, src[1], 1)
    parity(first, want[src[1]][0], 1e-3, "xnor darknet19-224 b128 first layer (TF32 stem)")
    net.close()
    net3 = dn.Network(gen(3), wpath, dn.MODE_TF32, text=True)
    out3 = net3.predict(np.ascontiguousarray(x[src])).copy()
    net3.close()
    assert np.array_equal(out[src], out3)
    assert np.isfinite(out).all() and abs(float(out[0].sum()) - 1.0) < 1e-3           # softmax rows
