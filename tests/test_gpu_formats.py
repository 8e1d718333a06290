"""Connected layers and the weight-file variants of the reference's loader, on the GPU.

* [connected] (src/connected_layer.c:151-167, 288-306): a small classifier whose tail is two connected layers, one
  with batchnorm, every layer against the CPU checker in all three modes; and against the unmodified reference
  where oracle/_ref is present.
* load_weights variants (src/parser.c:1218-1306): the 32-bit `seen` header of versions before 0.2, files whose
  version (major or minor above 1000) marks connected matrices stored [inputs][outputs], convolutions declared
  flipped=1 (matrix stored [c*size*size][n]); a file written by the reference's own save_weights is read back.
  Each variant must give the network of the plain file, bit for bit.
"""
import os

import numpy as np
import pytest

import darknet_b200 as dn
from conftest import parity
from darknet_b200 import synth
from oracle import network as orc

pytestmark = pytest.mark.gpu
TOL = {dn.MODE_FP32: 1e-4, dn.MODE_TF32: 1e-2, dn.MODE_BF16: 6e-2}


def build(cfg, wpath, mode):
    return dn.Network(cfg, wpath, mode, text=True)


@pytest.mark.parametrize("mode", [dn.MODE_FP32, dn.MODE_TF32, dn.MODE_BF16])
@pytest.mark.parametrize("bn", [True, False])
def test_connected_layers_match_the_checker(mode, bn, tmp_path):
    cfg = synth.connected_cfg(batch=5, size=12, hidden=48, classes=10, bn=bn)
    params = synth.seeded_params(cfg, 51)
    x = synth.seeded_input(cfg, 51)
    wpath = str(tmp_path / "c.weights")
    synth.write_weights(wpath, params)
    want = orc.forward_network(cfg, params, x)
    net = build(cfg, wpath, mode)
    out = net.predict(x).copy()
    assert [net.layer_type(i) for i in range(net.n)].count("connected") == 2
    for i, w in enumerate(want):
        parity(net.layer_output(i).reshape(w.shape), w, TOL[mode], f"layer {i} ({net.layer_type(i)}, {net.layer_kernel(i)})")
    parity(out.reshape(want[-1].shape), want[-1], TOL[mode], "network output")
    assert abs(float(out[0].sum()) - 1.0) < 1e-3
    assert net.flops > 0


def test_connected_first_layer_and_large_batch(tmp_path):
    # a connected layer straight on the input image (the flattening order c, h, w matters), batch above one pixel tile
    cfg = ("[net]\nbatch=150\nsubdivisions=1\nwidth=6\nheight=5\nchannels=3\n"
           "\n[connected]\noutput=70\nactivation=leaky\n\n[connected]\nbatch_normalize=1\noutput=33\nactivation=logistic\n")
    params = synth.seeded_params(cfg, 52)
    x = synth.seeded_input(cfg, 52, "normal")
    wpath = str(tmp_path / "c.weights")
    synth.write_weights(wpath, params)
    want = orc.forward_network(cfg, params, x)
    net = build(cfg, wpath, dn.MODE_TF32)
    out = net.predict(x).copy()
    for i, w in enumerate(want):
        parity(net.layer_output(i).reshape(w.shape), w, 1e-2, f"layer {i}")
    parity(out.reshape(want[-1].shape), want[-1], 1e-2, "network output")


def test_weight_file_variants_load_the_same_network(tmp_path):
    cfg = synth.connected_cfg(batch=3, size=12, hidden=40, classes=9, bn=True)
    flipped_cfg = cfg.replace("filters=24\n", "filters=24\nflipped=1\n")
    params = synth.seeded_params(cfg, 53)
    x = synth.seeded_input(cfg, 53)
    plain = str(tmp_path / "plain.weights")
    synth.write_weights(plain, params, seen=7)

    def run(c, w):
        net = build(c, w, dn.MODE_TF32)       # predict() returns memory the network owns: copy before the network goes
        out = net.predict(x).copy()
        net.close()
        return out

    base = run(cfg, plain)
    # version 0.1: a 32-bit `seen`
    old = str(tmp_path / "old.weights")
    synth.write_weights(old, params, seen=7, version=(0, 1, 0))
    assert os.path.getsize(old) == os.path.getsize(plain) - 4
    assert np.array_equal(run(cfg, old), base)
    # a version above 1000: connected matrices transposed on disk (and a 32-bit seen)
    tr = str(tmp_path / "transposed.weights")
    synth.write_weights(tr, params, seen=7, version=(0, 1001, 0))
    assert open(tr, "rb").read() != open(old, "rb").read()
    assert np.array_equal(run(cfg, tr), base)
    # flipped=1 on the second convolution: its matrix is transposed on disk
    fl = str(tmp_path / "flipped.weights")
    synth.write_weights(fl, params, seen=7, flipped={1})
    assert open(fl, "rb").read() != open(plain, "rb").read()
    assert np.array_equal(run(flipped_cfg, fl), base)
    # the checker agrees with all of them
    parity(base.reshape(-1), orc.forward_network(cfg, params, x)[-1].reshape(-1), 1e-2, "against the checker")


@pytest.mark.skipif(not orc.Reference.available(), reason="oracle/_ref (the compiled reference) is not built here")
def test_reads_what_the_reference_saves_and_matches_its_outputs(tmp_path):
    """The reference loads a transposed-version file and a flipped convolution, runs the network, and writes the
    weights back with its own save_weights; this library reads the reference's file and reproduces its outputs."""
    import contextlib
    cfg = synth.connected_cfg(batch=2, size=12, hidden=32, classes=6, bn=True).replace("filters=24\n", "filters=24\nflipped=1\n")
    params = synth.seeded_params(cfg, 54)
    x = synth.seeded_input(cfg, 54)
    src = str(tmp_path / "src.weights")
    synth.write_weights(src, params, version=(0, 1001, 0), flipped={1})
    cpath = str(tmp_path / "n.cfg")
    open(cpath, "w").write(cfg)
    R = orc.Reference()
    devnull = os.open(os.devnull, os.O_WRONLY)
    saved = os.dup(2)
    os.dup2(devnull, 2)          # the reference prints its layer table to stderr
    try:
        rnet = R.load(cpath, src)
        ref_out = R.predict_all(rnet, x)
        back = str(tmp_path / "back.weights")
        R.save_weights(rnet, back)
    finally:
        os.dup2(saved, 2)
        os.close(devnull)
    mine = build(cfg, src, dn.MODE_TF32)
    out = mine.predict(x).copy()
    for i, w in enumerate(ref_out):
        parity(mine.layer_output(i).reshape(-1), w.reshape(-1), 1e-2, f"layer {i} against the reference")
    # save_weights writes version 0.2 with untransposed connected matrices; the flipped convolution is written as it
    # sits in memory (already transposed back by the loader), so the file is read with flipped=0
    plain_cfg = cfg.replace("flipped=1\n", "")
    net2 = build(plain_cfg, back, dn.MODE_TF32)
    again = net2.predict(x).copy()
    assert np.array_equal(again, out)


def test_packed_binary_weights_load_the_same_xnor_network(tmp_path):
    """dnb_load_weights_packed: every xnor convolution stored as mean |w| + sign bits (32 times smaller) gives, bit for
    bit, the network that the ordinary file with those layers' weights replaced by +-mean gives."""
    cfg = synth.darknet19_cfg(batch=2, size=64, xnor=True)
    params = synth.seeded_params(cfg, 55)
    x = synth.seeded_input(cfg, 55)
    xnor_pos = {i for i, (k, o) in enumerate([s for s in synth.parse_cfg(cfg)[1:] if s[0] == "convolutional"]) if int(o.get("xnor", 0))}
    assert len(xnor_pos) == 17
    packed = str(tmp_path / "packed.weights")
    synth.write_weights(packed, params, packed=xnor_pos)
    expanded = []
    for i, p in enumerate(params):
        if i in xnor_pos:
            flat = p.weights.reshape(p.weights.shape[0], -1)
            rec = 4 + flat.shape[1] // 8
            raw = synth.packed_filter_bytes(p.weights)
            means = np.frombuffer(b"".join(raw[f * rec: f * rec + 4] for f in range(flat.shape[0])), np.float32)
            w = np.where(flat > 0, means[:, None], -means[:, None]).astype(np.float32).reshape(p.weights.shape)
            expanded.append(synth.ConvParams(w, p.biases, p.scales, p.rolling_mean, p.rolling_variance))
        else:
            expanded.append(p)
    plain = str(tmp_path / "plain.weights")
    synth.write_weights(plain, expanded)
    assert os.path.getsize(packed) < os.path.getsize(plain) / 8
    a = dn.Network(cfg, None, dn.MODE_TF32, text=True)
    a.load_weights(packed, packed=True)
    b = build(cfg, plain, dn.MODE_TF32)
    out_a, out_b = a.predict(x).copy(), b.predict(x).copy()
    assert np.array_equal(out_a, out_b)
    for i in range(a.n):
        assert np.array_equal(a.layer_output(i), b.layer_output(i)), f"layer {i}"
    # a layer whose filters are not whole bytes of bits is refused, as the reference's size/8 would drop its tail
    odd = synth.single_conv_cfg(1, 3, 8, 8, 8, 3, xnor=True)
    op = synth.seeded_params(odd, 56)
    bad = str(tmp_path / "odd.weights")
    synth.write_weights(bad, op, packed={0})
    n = dn.Network(odd, None, dn.MODE_TF32, text=True)
    with pytest.raises(dn.DarknetB200Error) as e:
        n.load_weights(bad, packed=True)
    assert e.value.status == dn.EUNSUPPORTED
