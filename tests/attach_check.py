"""Child process of test_gpu_attach.py: drives an UNMODIFIED Darknet GPU build (the reference's own
CUDA path, recompiled for sm_100a) through parse_network_cfg / load_weights / network_predict, then
calls b200_attach on the same `network` and predicts again.  Prints one JSON line with, per stage,
the worst per-layer error against the CPU checker.  Runs in a child because the reference calls
exit() on any error."""
import json
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.join(HERE, "golden"))

import make_golden  # noqa: E402
from darknet_b200 import synth  # noqa: E402
from oracle import network as orc  # noqa: E402


def rel_to_max(a, b):
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def main():
    name, mode = sys.argv[1], int(sys.argv[2])
    cfg, pseed, iseed, dist = make_golden.cases()[name]
    params = synth.seeded_params(cfg, pseed)
    x = synth.seeded_input(cfg, iseed, dist)
    want = orc.forward_network(cfg, params, x)
    d = tempfile.mkdtemp()
    cpath, wpath = os.path.join(d, "n.cfg"), os.path.join(d, "n.weights")
    open(cpath, "w").write(cfg)
    synth.write_weights(wpath, params)
    ref = orc.ReferenceGpu()
    net = ref.load(cpath, wpath)
    kinds = [k for k, _ in synth.parse_cfg(cfg)[1:]]

    def worst(outs):
        w = 0.0
        for i, (a, b) in enumerate(zip(outs, want)):
            if a.size != b.size:
                continue
            w = max(w, rel_to_max(a, b))
        return w

    stock = ref.predict_all(net, x)
    res = {"layers": len(kinds), "stock_vs_cpu": worst(stock)}
    res["attached"] = ref.attach(net, mode)
    res["coverable"] = sum(k in ("convolutional", "maxpool", "upsample", "shortcut", "route", "yolo") for k in kinds)
    ours = ref.predict_all(net, x)
    res["attached_vs_cpu"] = worst(ours)
    res["attached_vs_stock_last"] = rel_to_max(ours[-1], stock[-1])
    again = ref.predict_all(net, x * 0.5)
    res["second_input_differs"] = bool(not np.array_equal(again[-1], ours[-1]))
    ref.detach(net)
    back = ref.predict_all(net, x)
    res["detached_equals_stock"] = bool(all(np.array_equal(a, b) for a, b in zip(back, stock)))
    # the whole-network form: only the [yolo] layers and the last layer are written to Darknet's buffers
    res["whole_attached"] = ref.attach_network(net, mode)
    whole = ref.predict_all(net, x)
    watched = [i for i, k in enumerate(kinds) if k == "yolo" or i == len(kinds) - 1]
    res["whole_vs_cpu"] = max(rel_to_max(whole[i], want[i]) for i in watched)
    whole2 = ref.predict_all(net, x * 0.5)
    res["whole_second_input_differs"] = bool(not np.array_equal(whole2[-1], whole[-1]))
    ref.detach(net)
    back = ref.predict_all(net, x)
    res["whole_detached_equals_stock"] = bool(all(np.array_equal(a, b) for a, b in zip(back, stock)))
    print("ATTACH_RESULT " + json.dumps(res))


if __name__ == "__main__":
    main()
