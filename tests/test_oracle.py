"""The CPU checker against the reference: golden vectors produced by the
unmodified reference (tests/golden/make_golden.py), analytic known answers, and,
where oracle/_ref was built, the reference itself on fresh seeds."""
import hashlib
import os
import sys
import tempfile

import numpy as np
import pytest

from conftest import rel_to_max
from darknet_b200 import synth
from oracle import network as orc

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import make_golden  # noqa: E402

CASES = make_golden.cases()
# Layers downstream of an xnor convolution differ from the stock reference build in the last
# bits: its -Ofast vectorises the mean|w| sum (src/convolutional_layer.c:33-36), the checker
# adds in index order.  Everything else must match bit for bit.
XNOR_TOL = 2e-5


@pytest.mark.parametrize("name", list(CASES))
def test_oracle_matches_reference_golden(name, golden):
    cfg, pseed, iseed, dist = CASES[name]
    params = synth.seeded_params(cfg, pseed)
    x = synth.seeded_input(cfg, iseed, dist)
    assert hashlib.sha256(x.tobytes()).digest() == golden[f"{name}/input_sha"].tobytes(), "seeded input generator drifted"
    with tempfile.TemporaryDirectory() as d:
        synth.write_weights(d + "/n.weights", params)
        assert hashlib.sha256(open(d + "/n.weights", "rb").read()).digest() == golden[f"{name}/weights_sha"].tobytes()
    outs = orc.forward_network(cfg, params, x)
    assert len(outs) == int(golden[f"{name}/nlayers"])
    has_xnor = "xnor=1" in cfg
    kinds = [k for k, _ in synth.parse_cfg(cfg)[1:]]
    # avgpool, softmax and the connected layer's dot products (gemm_nt sums in a register, src/gemm.c:91-106) are
    # float reductions / divisions that the stock -Ofast build may reassociate or turn into reciprocal
    # multiplies: last-bit differences are expected there
    loose_from = min([i for i, k in enumerate(kinds) if k in ("avgpool", "softmax", "connected")], default=len(kinds))
    for i, o in enumerate(outs):
        flat = o.reshape(-1)
        assert list(o.shape) == list(golden[f"{name}/{i}/shape"]) or flat.size == int(np.prod(golden[f"{name}/{i}/shape"]))
        want = golden[f"{name}/{i}/sample"]
        got = flat[make_golden.sample_index(flat.size)]
        if has_xnor or i >= loose_from:
            assert rel_to_max(got, want) < XNOR_TOL, f"layer {i}"
        else:
            assert np.array_equal(got, want), f"layer {i}: sample differs from the reference"
            s = golden[f"{name}/{i}/sum"]
            assert flat.astype(np.float64).sum() == s[0] and np.abs(flat.astype(np.float64)).sum() == s[1], f"layer {i}: checksum"
            key = f"{name}/{i}/full"
            if key in golden.files:
                assert np.array_equal(flat, golden[key].reshape(-1)), f"layer {i}: full output"


def test_all_ones_counts_taps():
    # all-ones input and weights, no batchnorm, zero bias, linear: every output equals the number of
    # in-image taps times the channel count (the idea of the reference's own, commented-out
    # test_convolutional_layer, src/convolutional_layer.c:345-368)
    C, H, W, N = 3, 5, 6, 4
    x = np.ones((1, C, H, W), np.float32)
    w = np.ones((N, C, 3, 3), np.float32)
    out = orc.conv_forward(x, w, np.zeros(N, np.float32), stride=1, pad=1, activation="linear")
    ys, xs = np.arange(H), np.arange(W)
    ny = np.minimum(ys + 1, H - 1) - np.maximum(ys - 1, 0) + 1
    nx = np.minimum(xs + 1, W - 1) - np.maximum(xs - 1, 0) + 1
    want = (ny[:, None] * nx[None, :] * C).astype(np.float32)
    assert np.array_equal(out, np.broadcast_to(want, out.shape))


def test_xnor_accumulators_are_integers():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((2, 40, 6, 7)).astype(np.float32)
    w = rng.standard_normal((9, 40, 3, 3)).astype(np.float32)
    acc = orc.xnor_accumulate(x, w, stride=1, pad=1)
    assert np.array_equal(acc, np.round(acc)) and np.abs(acc).max() <= 40 * 9
    # same numbers from plain integer arithmetic
    sx = np.where(x > 0, 1, -1).astype(np.int64)
    sw = np.where(w > 0, 1, -1).astype(np.int64)
    xp = np.pad(sx, ((0, 0), (0, 0), (1, 1), (1, 1)))
    want = np.zeros(acc.shape, np.int64)
    for kh in range(3):
        for kw in range(3):
            want += np.einsum("bchw,nc->bnhw", xp[:, :, kh:kh + 6, kw:kw + 7], sw[:, :, kh, kw])
    assert np.array_equal(acc.astype(np.int64), want)


def test_maxpool_stride1_overhang():
    # yolov3-tiny's 2x2 stride-1 pool: padding 1, window origin -1/2 = 0, overhang right/bottom skipped
    x = np.arange(2 * 3 * 3, dtype=np.float32).reshape(1, 2, 3, 3)
    out = orc.maxpool_forward(x, 2, 1)
    assert out.shape == (1, 2, 3, 3)
    assert out[0, 0].tolist() == [[4, 5, 5], [7, 8, 8], [7, 8, 8]]


def test_shortcut_mismatched_shapes():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((2, 8, 4, 4)).astype(np.float32)
    add = rng.standard_normal((2, 4, 8, 8)).astype(np.float32)   # fewer channels, twice the size: stride-2 sampled add
    out = orc.shortcut_forward(x, add, activation="leaky")
    want = x.copy()
    want[:, :4] += add[:, :, ::2, ::2]
    want = np.where(want > 0, want, (0.1 * want.astype(np.float64)).astype(np.float32))
    assert np.array_equal(out, want)


@pytest.mark.skipif(not orc.Reference.available(), reason="oracle/_ref (the compiled reference) is not built here")
@pytest.mark.parametrize("seed", [101, 102])
def test_oracle_matches_reference_live(seed):
    R = orc.Reference()
    cfg = synth.yolov3_tiny_cfg(batch=2, size=64 + 32 * (seed % 2))
    params = synth.seeded_params(cfg, seed)
    x = synth.seeded_input(cfg, seed)
    with tempfile.TemporaryDirectory() as d:
        open(d + "/n.cfg", "w").write(cfg)
        synth.write_weights(d + "/n.weights", params)
        ref = R.predict_all(R.load(d + "/n.cfg", d + "/n.weights"), x)
    mine = orc.forward_network(cfg, params, x)
    for i, (a, b) in enumerate(zip(ref, mine)):
        assert np.array_equal(a.reshape(-1), b.reshape(-1)), f"layer {i}"
    # the two primitives on their own: im2col_cpu and gemm_nn
    rng = np.random.default_rng(seed)
    im = rng.standard_normal((5, 9, 8)).astype(np.float32)
    col_r = np.zeros((5 * 9, 5 * 4), np.float32)
    col_m = np.zeros_like(col_r)
    R.L.ref_im2col(im.ctypes.data, 5, 9, 8, 3, 2, 1, col_r.ctypes.data)
    orc.lib().orc_im2col(im.ctypes.data, 5, 9, 8, 3, 2, 1, col_m.ctypes.data)
    assert np.array_equal(col_r, col_m)
    A = rng.standard_normal((7, 45)).astype(np.float32)
    Cr = np.zeros((7, 20), np.float32)
    Cm = np.zeros_like(Cr)
    R.L.ref_gemm_nn(7, 20, 45, A.ctypes.data, col_r.ctypes.data, Cr.ctypes.data)
    orc.lib().orc_gemm_nn(7, 20, 45, 1.0, A.ctypes.data, 45, col_m.ctypes.data, 20, Cm.ctypes.data, 20)
    assert np.array_equal(Cr, Cm)


@pytest.mark.skipif(not orc.Reference.available() or not hasattr(orc.Reference().L, "ref_save_conv_binary"),
                    reason="oracle/_ref (the compiled reference) is not built here")
def test_packed_binary_layer_format_matches_the_reference(tmp_path):
    """The reference's dormant packed-binary layer format (src/parser.c:926-956, 1134-1162), driven through its own
    writer and reader: the writer of darknet_b200.synth produces the reference's bytes (sign bits exactly; the
    per-filter mean to the last bits, the stock -Ofast build vectorises that sum), and the reference's reader
    expands a file written here into the +-mean weights the loader of the CUDA library builds."""
    import ctypes as C
    import contextlib
    cfg = synth.single_conv_cfg(2, 16, 6, 6, 12, 3, xnor=True)
    params = synth.seeded_params(cfg, 77)
    p = params[0]
    d = str(tmp_path)
    open(d + "/n.cfg", "w").write(cfg)
    synth.write_weights(d + "/n.weights", params)
    R = orc.Reference()
    devnull = os.open(os.devnull, os.O_WRONLY)
    saved = os.dup(2)
    os.dup2(devnull, 2)
    try:
        net = R.load(d + "/n.cfg", d + "/n.weights")
    finally:
        os.dup2(saved, 2)
        os.close(devnull)
    assert R.L.ref_save_conv_binary(net, 0, (d + "/layer.bin").encode()) == 0
    ref_bytes = open(d + "/layer.bin", "rb").read()
    n, per = 12, 16 * 9
    head = b"".join(np.ascontiguousarray(a, np.float32).tobytes() for a in (p.biases, p.scales, p.rolling_mean, p.rolling_variance))
    mine = head + synth.packed_filter_bytes(p.weights)
    assert len(ref_bytes) == len(mine) == len(head) + n * (4 + per // 8)
    assert ref_bytes[:len(head)] == mine[:len(head)]
    rec = 4 + per // 8
    for f in range(n):
        a = ref_bytes[len(head) + f * rec: len(head) + (f + 1) * rec]
        b = mine[len(head) + f * rec: len(head) + (f + 1) * rec]
        assert a[4:] == b[4:], f"filter {f}: sign bits"
        ma, mb = np.frombuffer(a[:4], np.float32)[0], np.frombuffer(b[:4], np.float32)[0]
        assert abs(ma - mb) <= 1e-6 * abs(mb), f"filter {f}: mean"   # a few units in the last place: the reference build reassociates the sum
    # the reference's reader on the bytes written here
    open(d + "/mine.bin", "wb").write(mine)
    assert R.L.ref_load_conv_binary(net, 0, (d + "/mine.bin").encode()) == 0
    got = np.ctypeslib.as_array(R.L.ref_layer_weights(net, 0), shape=(n, per)).copy()
    flat = p.weights.reshape(n, per)
    means = np.frombuffer(b"".join(mine[len(head) + f * rec: len(head) + f * rec + 4] for f in range(n)), np.float32)
    want = np.where(flat > 0, means[:, None], -means[:, None]).astype(np.float32)
    assert np.array_equal(got, want)
