"""Whole-network parity on the GPU: parse_network_cfg + load_weights +
network_predict through the C ABI, every layer's output against the CPU checker
and against the golden vectors the unmodified reference produced.

Per-layer tolerance, max |gpu - cpu| / max |cpu|: FP32 mode 1e-4, TF32 1e-2,
BF16 3e-2 (BF16 end-to-end through 75 layers is reported, and bounded at 6e-2;
the per-layer bound is checked teacher-forced in test_gpu_layers.py).
"""
import os
import sys

import numpy as np
import pytest
import torch

import darknet_b200 as dn
from conftest import parity, rel_to_max
from darknet_b200 import synth
from oracle import network as orc

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import make_golden  # noqa: E402

pytestmark = pytest.mark.gpu
CASES = make_golden.cases()
TOL = {dn.MODE_FP32: 1e-4, dn.MODE_TF32: 1e-2, dn.MODE_BF16: 6e-2}


def build(cfg, params, tmp_path, mode):
    wpath = str(tmp_path / "n.weights")
    cpath = str(tmp_path / "n.cfg")
    synth.write_weights(wpath, params)
    open(cpath, "w").write(cfg)
    return dn.load_network(cpath, wpath, 0, mode=mode)


@pytest.mark.parametrize("name", ["tiny64", "tiny96_b2", "yolov3_64", "resnet50_32", "resnet50_64_b2", "darknet19_64"])
@pytest.mark.parametrize("mode", [dn.MODE_FP32, dn.MODE_TF32, dn.MODE_BF16])
@pytest.mark.parametrize("fuse", [0, 1])
def test_network_matches_oracle_and_golden(name, mode, fuse, tmp_path, golden, monkeypatch):
    # fuse=0: every layer separate, every layer's output checked; fuse=1 (the default): convolutions absorb the
    # shortcut or yolo layer after them, their own outputs do not exist and are skipped
    monkeypatch.setenv("DNB_FUSE_SHORTCUT", str(fuse))
    monkeypatch.setenv("DNB_FUSE_YOLO", str(fuse))
    cfg, pseed, iseed, dist = CASES[name]
    params = synth.seeded_params(cfg, pseed)
    x = synth.seeded_input(cfg, iseed, dist)
    net = build(cfg, params, tmp_path, mode)
    out = net.predict(x).copy()
    want = orc.forward_network(cfg, params, x)
    assert net.n == len(want)
    kinds = [k for k, _ in synth.parse_cfg(cfg)[1:]]
    worst = 0.0
    skipped = 0
    for i, w in enumerate(want):
        try:
            got = net.layer_output(i)
        except dn.DarknetB200Error as e:
            assert fuse and e.status == dn.EUNSUPPORTED and kinds[i] == "convolutional" and kinds[i + 1] in ("shortcut", "yolo")
            skipped += 1
            continue
        assert got.shape == w.shape or got.size == w.size
        err = parity(got, w, TOL[mode], f"{name} layer {i} ({kinds[i]}, {net.layer_kernel(i)})")
        worst = max(worst, err)
        # golden sample straight from the unmodified reference
        sample = golden[f"{name}/{i}/sample"]
        g = got.reshape(-1)[make_golden.sample_index(got.size)]
        assert np.abs(g - sample).max() / max(np.abs(w).max(), 1e-30) < TOL[mode]
    # network_predict returns the last layer, yolo heads are pulled to the host as well
    parity(out.reshape(-1), want[-1].reshape(-1), TOL[mode])
    for i, k in enumerate(kinds):
        if k == "yolo":
            parity(net.yolo_output(i), want[i], TOL[mode])
    if fuse and mode != dn.MODE_FP32 and ("shortcut" in kinds or "yolo" in kinds):
        assert skipped > 0, "no convolution was fused with the shortcut or yolo layer after it"
    if not fuse:
        assert skipped == 0
    print(f"{name} mode {mode} fuse {fuse}: worst per-layer rel error {worst:.3g}, {skipped} fused layers")


def test_network_device_forward_equals_predict(tmp_path):
    cfg, pseed, iseed, dist = CASES["tiny64"]
    params = synth.seeded_params(cfg, pseed)
    x = synth.seeded_input(cfg, iseed, dist)
    net = build(cfg, params, tmp_path, dn.MODE_TF32)
    a = net.predict(x).copy()
    xd = torch.from_numpy(x).cuda()
    net.forward(xd)
    torch.cuda.synchronize()
    b = net.layer_output(net.n - 1).reshape(a.shape)
    assert np.array_equal(a, b)
    ms = net.profile(xd)
    assert ms.shape == (net.n,) and (ms >= 0).all()
    assert 0 < net.launches <= net.n + 1 and net.flops > 0   # a route whose inputs sit in place launches nothing


@pytest.mark.parametrize("name", ["tiny64", "resnet50_32"])
def test_network_submit_collect_equals_predict(name, tmp_path):
    """Two steps in flight give, step for step, the bytes the blocking call gives (yolo heads and
    the output layer), and the in-flight limit is enforced."""
    cfg, pseed, iseed, dist = CASES[name]
    params = synth.seeded_params(cfg, pseed)
    net = build(cfg, params, tmp_path, dn.MODE_TF32)
    xs = [torch.from_numpy(synth.seeded_input(cfg, iseed + k, dist)).pin_memory() for k in range(5)]
    yolos = [i for i in range(net.n) if net.layer_type(i) == "yolo"]
    want = []
    for x in xs:
        out = net.predict(x).copy()
        want.append((out, [net.yolo_output(i).copy() for i in yolos]))
    got = []
    net.submit(xs[0])
    for k in range(1, len(xs)):
        net.submit(xs[k])
        if k == 1:
            with pytest.raises(dn.DarknetB200Error) as e:
                net.submit(xs[k])          # a third step in flight
            assert e.value.status == dn.EINVAL
            with pytest.raises(dn.DarknetB200Error):
                net.predict(xs[k])         # the blocking call refuses while steps are in flight
        out = net.collect().copy()
        got.append((out, [net.yolo_output(i).copy() for i in yolos]))
    out = net.collect().copy()
    got.append((out, [net.yolo_output(i).copy() for i in yolos]))
    with pytest.raises(dn.DarknetB200Error):
        net.collect()                      # nothing left
    for (wo, wy), (go, gy) in zip(want, got):
        assert np.array_equal(wo, go)
        for a, b in zip(wy, gy):
            assert np.array_equal(a, b)
    assert not np.array_equal(want[0][0], want[1][0])


@pytest.mark.parametrize("name", ["tiny64", "yolov3_64", "resnet50_32", "darknet19_xnor_32"])
def test_network_graph_replay_equals_eager(name, tmp_path):
    """dnb_network_enable_graph: the captured forward gives the bytes the eager one gives, reads the input
    tensor's current contents on every replay, and is captured again for another tensor."""
    cfg, pseed, iseed, dist = CASES[name]
    params = synth.seeded_params(cfg, pseed)
    net = build(cfg, params, tmp_path, dn.MODE_TF32)
    x1 = synth.seeded_input(cfg, iseed, dist)
    x2 = synth.seeded_input(cfg, iseed + 1, dist)
    s = torch.cuda.Stream()
    xd = torch.from_numpy(x1).cuda()
    torch.cuda.synchronize()

    def run(t):
        net.forward(t, stream=s.cuda_stream)
        s.synchronize()
        return net.layer_output(net.n - 1).copy()

    want1 = run(xd)                    # eager, graphs off
    xd.copy_(torch.from_numpy(x2).cuda())
    want2 = run(xd)
    assert not np.array_equal(want1, want2)
    net.enable_graph(True)
    xd.copy_(torch.from_numpy(x1).cuda()); torch.cuda.synchronize()
    for k in range(4):                 # eager, captured, replayed, replayed
        assert np.array_equal(run(xd), want1), f"forward {k} with graphs on differs"
    xd.copy_(torch.from_numpy(x2).cuda()); torch.cuda.synchronize()
    assert np.array_equal(run(xd), want2)          # same pointer, new contents: the replay reads them
    other = torch.from_numpy(x1).cuda()            # another pointer: eager again, then a new capture
    torch.cuda.synchronize()
    for k in range(3):
        assert np.array_equal(run(other), want1)
    net.enable_graph(False)
    assert np.array_equal(run(xd), want2)
    assert np.array_equal(net.predict(x1).reshape(want1.shape), want1)   # the host-buffer path is untouched


@pytest.mark.parametrize("mode", [dn.MODE_FP32, dn.MODE_TF32, dn.MODE_BF16])
def test_network_of_memory_layers_only(mode, tmp_path):
    """A network without a convolution (maxpool, upsample, padded maxpool, shortcut, route, maxpool): the
    channels-last copy of the input feeds a maxpool, every layer against the checker.  Copies and compares are
    exact in f32 storage; BF16 storage rounds the input once."""
    cfg = synth.memory_layers_cfg(batch=3, c=24, size=20)
    x = synth.seeded_input(cfg, 9, "normal")
    want = orc.forward_network(cfg, [], x)
    net = build(cfg, [], tmp_path, mode)
    out = net.predict(x).copy()
    for i, w in enumerate(want):
        got = net.layer_output(i)
        if mode == dn.MODE_BF16:
            parity(got, w, 2e-2)
        elif mode == dn.MODE_TF32:
            parity(got, w, 1e-3)     # the input copy is rounded to TF32 once
        else:
            assert np.array_equal(got, w), f"layer {i}"
    assert out.shape == (3, net.outputs)


def test_network_batch_override_and_errors(tmp_path):
    cfg = synth.yolov3_tiny_cfg(batch=1, size=64)
    params = synth.seeded_params(cfg, 1)
    wpath = str(tmp_path / "n.weights")
    synth.write_weights(wpath, params)
    net = dn.Network(cfg, wpath, dn.MODE_TF32, batch=3, text=True)
    assert net.batch == 3
    x1 = synth.seeded_input(cfg, 1)
    x3 = np.concatenate([x1, x1 * 0.5, x1], 0)
    out = net.predict(x3).copy()
    assert np.array_equal(out[0], out[2]) and not np.array_equal(out[0], out[1])   # images are independent
    with pytest.raises(dn.DarknetB200Error) as e:
        dn.Network("[net]\nbatch=1\nwidth=8\nheight=8\nchannels=3\n[lstm]\noutput=4\n", None, text=True)
    assert e.value.status == dn.EUNSUPPORTED
    with pytest.raises(dn.DarknetB200Error) as e:
        dn.load_network(str(tmp_path / "missing.cfg"), None)
    assert e.value.status == dn.EIO
    short = str(tmp_path / "short.weights")
    open(short, "wb").write(open(wpath, "rb").read()[:1000])
    with pytest.raises(dn.DarknetB200Error) as e:
        dn.Network(cfg, short, text=True)
    assert e.value.status == dn.EIO


def test_xnor_network_teacher_forced(tmp_path):
    # Binarisation turns tiny differences of the previous layer into sign flips, so an xnor network is
    # checked layer by layer, each layer fed the CPU checker's own input: accumulators bit-exact (see
    # test_gpu_layers), outputs within 1e-5; and end to end in exact FP32 mode for the non-xnor layers.
    from gpu_util import dev_nchw, empty_nchw
    cfg, pseed, iseed, dist = CASES["darknet19_xnor_32"]
    params = synth.seeded_params(cfg, pseed)
    x = synth.seeded_input(cfg, iseed, dist)
    want = orc.forward_network(cfg, params, x)
    sections = synth.parse_cfg(cfg)[1:]
    pi = 0
    for i, (kind, opt) in enumerate(sections):
        if kind != "convolutional":
            continue
        p = params[pi]
        pi += 1
        if not int(opt.get("xnor", 0)):
            continue
        xin = want[i - 1]
        b, c, h, w = xin.shape
        size = int(opt["size"])
        plan = dn.ConvPlan(b, c, h, w, int(opt["filters"]), size, int(opt["stride"]), size // 2, 1, True, opt["activation"], True)
        plan.set_params(p.weights, p.biases, p.scales, p.rolling_mean, p.rolling_variance)
        xt, xd = dev_nchw(xin)
        yt, yd = empty_nchw(*want[i].shape)
        plan.forward(xd, yd)
        parity(yt.cpu().numpy(), want[i], 1e-5, f"layer {i}")
    net = build(cfg, params, tmp_path, dn.MODE_TF32)
    net.predict(x)
    assert sum(net.layer_kernel(i).startswith("xnor_") for i in range(net.n)) == 17
    parity(net.layer_output(0), want[0], 1e-3)   # fp32 stem, stored rounded to TF32 for the next layer


@pytest.mark.parametrize("size,batch", [(64, 3), (224, 2)])
def test_xnor_layers_in_a_row_share_their_signs(size, batch, tmp_path, monkeypatch):
    """Where one tensor-core xnor layer feeds the next, the first writes the second's int8 operand from its epilogue
    and the second runs no sign pass.  The signs are those of the stored f32 values, so every layer output must be
    bit-identical to the network that computes them with the separate pass (DNB_XNOR_SIGNS=0), and fewer kernels run."""
    cfg = synth.darknet19_cfg(batch=batch, size=size, xnor=True)
    params = synth.seeded_params(cfg, 31)
    x = synth.seeded_input(cfg, 31, "uniform")
    outs, launches = {}, {}
    for knob in ("0", "1"):
        monkeypatch.setenv("DNB_XNOR_SIGNS", knob)
        net = build(cfg, params, tmp_path, dn.MODE_TF32)
        out = net.predict(x).copy()
        layers = [net.layer_output(i).copy() for i in range(net.n)]
        assert sum(net.layer_kernel(i) == "xnor_tc" for i in range(net.n)) == 17
        outs[knob] = (out, layers)
        net.close()
    for i, (a, b) in enumerate(zip(outs["0"][1], outs["1"][1])):
        assert np.array_equal(a, b), f"layer {i} differs when the signs come from the previous layer's epilogue"
    assert np.array_equal(outs["0"][0], outs["1"][0])
    assert np.isfinite(outs["1"][0]).all()
