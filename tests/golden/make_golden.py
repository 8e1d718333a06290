"""Generate tests/golden/golden.npz from the UNMODIFIED reference.

Run in a container where the reference sources are mounted and
``make -C oracle ref`` has produced oracle/_ref/libdarknet_ref.so:

    python tests/golden/make_golden.py

Every case is (cfg text, parameter seed, input seed, input distribution).  Inputs
and parameters are regenerated from the seeds by darknet_b200.synth at test
time; the fixture stores what the reference computed: for every layer its shape,
float64 sum and sum of absolute values, a fixed strided sample of 256 values,
and the complete output when it has at most 2048 elements.  A checksum of the
seeded input and of the weights file guards against a drifting generator.
"""
from __future__ import annotations

import hashlib
import os
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from darknet_b200 import synth  # noqa: E402
from oracle import network as orc  # noqa: E402


def cases() -> dict[str, tuple[str, int, int, str]]:
    s = synth.single_conv_cfg
    return {
        "tiny64": (synth.yolov3_tiny_cfg(batch=1, size=64), 1, 1, "uniform"),
        "tiny96_b2": (synth.yolov3_tiny_cfg(batch=2, size=96), 2, 2, "uniform"),
        "yolov3_64": (synth.yolov3_cfg(batch=1, size=64), 3, 3, "uniform"),
        "resnet50_32": (synth.resnet50_cfg(batch=1, size=32), 4, 4, "uniform"),
        "resnet50_64_b2": (synth.resnet50_cfg(batch=2, size=64), 5, 5, "uniform"),
        "darknet19_xnor_32": (synth.darknet19_cfg(batch=1, size=32, xnor=True), 6, 6, "uniform"),
        "darknet19_64": (synth.darknet19_cfg(batch=2, size=64, xnor=False), 7, 7, "uniform"),
        "conv3x3_bn_leaky": (s(2, 8, 12, 12, 16, 3), 10, 10, "normal"),
        "conv3x3_s2": (s(2, 16, 13, 11, 24, 3, stride=2), 11, 11, "normal"),
        "conv1x1": (s(3, 32, 9, 9, 40, 1), 12, 12, "normal"),
        "conv7x7_s2_c3": (s(2, 3, 30, 30, 16, 7, stride=2), 13, 13, "uniform"),
        "conv3x3_groups2": (s(2, 8, 10, 10, 12, 3, groups=2), 14, 14, "normal"),
        "conv3x3_bias_linear": (s(2, 16, 8, 8, 255, 3, bn=False, act="linear"), 15, 15, "normal"),
        "conv1x1_logistic": (s(1, 64, 7, 7, 30, 1, bn=False, act="logistic"), 16, 16, "normal"),
        "conv3x3_nopad": (s(2, 8, 9, 9, 16, 3, pad=0), 17, 17, "normal"),
        "conv3x3_xnor": (s(2, 64, 10, 10, 32, 3, xnor=True), 18, 18, "normal"),
        "conv3x3_c256_k512": (s(1, 256, 13, 13, 512, 3), 19, 19, "normal"),
        "conv5x5": (s(1, 8, 11, 11, 8, 5), 20, 20, "normal"),
        "connected_bn": (synth.connected_cfg(batch=4, size=12, bn=True), 21, 21, "uniform"),
        "connected_bias": (synth.connected_cfg(batch=3, size=10, hidden=40, classes=7, bn=False), 22, 22, "uniform"),
    }


def sample_index(n: int) -> np.ndarray:
    return (np.arange(256, dtype=np.int64) * 2654435761 % max(n, 1)).astype(np.int64)


def main() -> None:
    assert orc.Reference.available(), "build oracle/_ref first: make -C oracle ref"
    R = orc.Reference()
    out: dict[str, np.ndarray] = {}
    for name, (cfg, pseed, iseed, dist) in cases().items():
        params = synth.seeded_params(cfg, pseed)
        x = synth.seeded_input(cfg, iseed, dist)
        with tempfile.TemporaryDirectory() as d:
            with open(d + "/n.cfg", "w") as f:
                f.write(cfg)
            synth.write_weights(d + "/n.weights", params)
            wsum = hashlib.sha256(open(d + "/n.weights", "rb").read()).hexdigest()
            net = R.load(d + "/n.cfg", d + "/n.weights")
            outs = R.predict_all(net, x)
        out[f"{name}/input_sha"] = np.frombuffer(hashlib.sha256(x.tobytes()).digest(), np.uint8)
        out[f"{name}/weights_sha"] = np.frombuffer(bytes.fromhex(wsum), np.uint8)
        out[f"{name}/nlayers"] = np.array(len(outs))
        for i, o in enumerate(outs):
            flat = o.reshape(-1)
            out[f"{name}/{i}/shape"] = np.array(o.shape)
            out[f"{name}/{i}/sum"] = np.array([flat.astype(np.float64).sum(), np.abs(flat.astype(np.float64)).sum()])
            out[f"{name}/{i}/sample"] = flat[sample_index(flat.size)]
            if flat.size <= 2048:
                out[f"{name}/{i}/full"] = o
        print(f"{name}: {len(outs)} layers")
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.npz"), **out)


if __name__ == "__main__":
    main()
