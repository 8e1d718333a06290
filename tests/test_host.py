"""Host-side checks that need no GPU: the C ABI library loads and exports every
symbol the public headers declare, argument validation rejects bad geometry
before anything is launched, the cfg generators reproduce the reference's
network definitions, and the .weights writer follows the on-disk format."""
import ctypes as C
import glob
import os
import re
import struct

import numpy as np
import pytest

import darknet_b200 as dn
from darknet_b200 import synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_CFG = os.path.join(os.environ.get("DARKNET_ROOT", os.path.join(os.sep, "root", "reference")), "cfg")   # the reference tree, where it is mounted


def declared_symbols():
    names = set()
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = re.sub(r"/\*.*?\*/", "", open(h).read(), flags=re.S)
        names |= set(re.findall(r"\b(dnb_[a-z0-9_]+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    L = dn.lib()
    decl = declared_symbols()
    assert len(decl) >= 35
    for name in sorted(decl):
        assert hasattr(L, name), f"{name} is declared in include/ but not exported"
    # and the Python binding knows every one of them
    missing = {n for n in decl if n not in dn.SIGNATURES and not n.startswith("dnb_attach")}
    assert not missing, missing
    assert L.dnb_version() >= 100
    assert L.dnb_cpitch(255) == 256 and L.dnb_cpitch(3) == 8


def test_attach_shim_exports_its_header():
    """include/b200_attach.h is implemented by darknet_b200/shim/b200_attach.c, which is compiled inside a
    Darknet GPU tree; where the reference's CUDA build was made here, its library carries both symbols."""
    import ctypes
    text = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "b200_attach.h")).read(), flags=re.S)
    names = set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text))
    assert names == {"b200_attach", "b200_attach_network", "b200_detach"}
    src = open(os.path.join(ROOT, "darknet_b200", "shim", "b200_attach.c")).read()
    for n in names:
        assert re.search(r"^(int|void) %s\(" % n, src, flags=re.M), n
    lib = os.path.join(ROOT, "oracle", "_ref", "libdarknet_ref_gpu.so")
    if not os.path.exists(lib):
        pytest.skip("the reference's CUDA build was not made here (make -C oracle refgpu)")
    try:
        L = ctypes.CDLL(lib)
    except OSError as e:
        pytest.skip(f"cannot load the reference's CUDA build here: {e}")
    for n in names:
        assert hasattr(L, n)


def test_plan_validation_needs_no_device():
    L = dn.lib()
    h = C.c_void_p()
    bad = dn.ConvDesc(1, 8, 8, 6, 8, 4, 3, 1, 1, 0, 3, 0)     # groups 4 does not divide c 6
    assert L.dnb_conv_plan_create(C.byref(bad), dn.MODE_TF32, C.byref(h)) == dn.EINVAL
    assert b"groups" in L.dnb_last_error()
    empty = dn.ConvDesc(1, 2, 2, 8, 8, 1, 5, 1, 0, 0, 3, 0)   # 5x5 kernel on a 2x2 image, no padding
    assert L.dnb_conv_plan_create(C.byref(empty), dn.MODE_TF32, C.byref(h)) == dn.EINVAL
    quirk = dn.ConvDesc(1, 8, 8, 8, 8, 1, 1, 2, 0, 0, 3, 0)   # 1x1 stride 2: the reference's size-1 shortcut
    assert L.dnb_conv_plan_create(C.byref(quirk), dn.MODE_TF32, C.byref(h)) == dn.EUNSUPPORTED
    assert L.dnb_conv_plan_create(C.byref(bad), 7, C.byref(h)) == dn.EINVAL
    with pytest.raises(dn.DarknetB200Error):
        dn.check(L.dnb_conv_plan_create(None, 0, C.byref(h)))


def test_wide_strides_fall_back_to_the_cuda_core_kernel():
    """The tensor-core kernel carries input maps for strides 1 and 2; a wider stride is decided when the plan is
    made (the CUDA-core kernel takes it), not at the first forward."""
    L = dn.lib()
    for mode in (dn.MODE_TF32, dn.MODE_BF16):
        h = C.c_void_p()
        d = dn.ConvDesc(1, 16, 16, 16, 16, 1, 3, 3, 1, 0, 3, 0)
        assert L.dnb_conv_plan_create(C.byref(d), mode, C.byref(h)) == dn.OK
        assert L.dnb_conv_plan_kernel(h) == b"direct_fp32"
        L.dnb_conv_plan_destroy(h)
        d2 = dn.ConvDesc(1, 16, 16, 16, 16, 1, 3, 2, 1, 0, 3, 0)
        assert L.dnb_conv_plan_create(C.byref(d2), mode, C.byref(h)) == dn.OK
        assert L.dnb_conv_plan_kernel(h).startswith(b"tc_")
        L.dnb_conv_plan_destroy(h)


def test_degenerate_geometry_is_refused():
    """Empty batches, empty images, no filters, zero stride or size, negative padding, unknown activation:
    refused with a message, nothing is launched (the reference would divide by zero or abort)."""
    L = dn.lib()
    h = C.c_void_p()
    cases = [dn.ConvDesc(0, 8, 8, 8, 8, 1, 3, 1, 1, 0, 3, 0), dn.ConvDesc(1, 8, 8, 0, 8, 1, 3, 1, 1, 0, 3, 0),
             dn.ConvDesc(1, 8, 8, 8, 0, 1, 3, 1, 1, 0, 3, 0), dn.ConvDesc(1, 8, 8, 8, 8, 1, 3, 0, 1, 0, 3, 0),
             dn.ConvDesc(1, 8, 8, 8, 8, 1, 0, 1, 1, 0, 3, 0), dn.ConvDesc(1, 8, 8, 8, 8, 1, 3, 1, -1, 0, 3, 0),
             dn.ConvDesc(1, 8, 8, 8, 8, 1, 3, 1, 1, 0, 99, 0)]
    for d in cases:
        assert L.dnb_conv_plan_create(C.byref(d), dn.MODE_TF32, C.byref(h)) == dn.EINVAL
        assert len(L.dnb_last_error()) > 10
    t = dn.Tensor(256, dn.NHWC, dn.F32, 0, 8, 4, 4, 8)      # empty batch
    assert L.dnb_maxpool_forward(C.byref(t), C.byref(t), 2, 2, 1, None) == dn.EINVAL


def test_tensor_validation():
    L = dn.lib()
    t = dn.Tensor(0, dn.NHWC, dn.F32, 1, 8, 4, 4, 8)
    assert L.dnb_maxpool_forward(C.byref(t), C.byref(t), 2, 2, 1, None) == dn.EINVAL   # null data
    t2 = dn.Tensor(256, dn.NHWC, dn.F32, 1, 10, 4, 4, 12)                               # cpitch not a multiple of 8
    assert L.dnb_upsample_forward(C.byref(t2), C.byref(t2), 2, 1.0, None) == dn.EINVAL
    assert b"cpitch" in L.dnb_last_error()


@pytest.mark.skipif(not os.path.isdir(REF_CFG), reason="reference cfg files are not mounted here")
@pytest.mark.parametrize("name,gen", [("yolov3.cfg", synth.yolov3_cfg), ("yolov3-tiny.cfg", synth.yolov3_tiny_cfg),
                                      ("resnet50.cfg", synth.resnet50_cfg),
                                      ("darknet19.cfg", lambda: synth.darknet19_cfg(xnor=False))])
def test_generated_cfg_equals_reference_cfg(name, gen):
    def layers(text):
        return [(k, {a: b.replace(" ", "") for a, b in o.items()}) for k, o in synth.parse_cfg(text)[1:]]
    assert layers(open(os.path.join(REF_CFG, name)).read()) == layers(gen())


def test_generated_cfg_shapes():
    # layer counts and parameter totals of the published architectures
    y = synth.conv_shapes(synth.yolov3_cfg())
    assert len(y) == 75 and len(synth.parse_cfg(synth.yolov3_cfg())) == 108
    nparams = sum(s.n * (s.c // s.groups) * s.size ** 2 + s.n * (4 if s.batch_normalize else 1) for s in y)
    assert nparams == 62_001_757   # the published yolov3.weights is 20 header bytes + 4 bytes x this count
    assert len(synth.conv_shapes(synth.yolov3_tiny_cfg())) == 13
    assert len(synth.conv_shapes(synth.resnet50_cfg())) == 50
    d = synth.parse_cfg(synth.darknet19_cfg(xnor=True))[1:]
    convs = [o for k, o in d if k == "convolutional"]
    assert len(convs) == 19 and "xnor" not in convs[0] and "xnor" not in convs[-1] and all(o.get("xnor") == "1" for o in convs[1:-1])


def test_weights_file_format(tmp_path):
    cfg = synth.single_conv_cfg(1, 4, 5, 5, 6, 3) + synth._conv(3, 1, bn=False, act="linear")
    params = synth.seeded_params(cfg, 9)
    p = tmp_path / "w.weights"
    synth.write_weights(str(p), params, seen=1234)
    raw = p.read_bytes()
    assert struct.unpack("<iiiQ", raw[:20]) == (0, 2, 0, 1234)
    body = np.frombuffer(raw[20:], np.float32)
    n0 = 6 + 3 * 6 + 6 * 4 * 9
    assert body.size == n0 + 3 + 3 * 6
    assert np.array_equal(body[:6], params[0].biases) and np.array_equal(body[6:12], params[0].scales)
    assert np.array_equal(body[24:n0], params[0].weights.reshape(-1))
    assert np.array_equal(body[n0:n0 + 3], params[1].biases)


def test_bench_workloads_are_well_formed():
    """Every workload bench.py can name parses, has the layer mix it advertises, and the byte / FLOP accounting
    the roofline uses matches the published totals (YOLOv3-608: 140.69 GFLOP per image)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    kinds = {}
    for name, size in [("yolov3", 608), ("yolov3-tiny", 416), ("resnet50", 224), ("darknet19-xnor", 224), ("conv3x3", 224),
                       ("conv1x1", 224), ("memlayers", 152)]:
        cfg, metric, desc = bench.workload_cfg(name, 2, size)
        secs = synth.parse_cfg(cfg)
        assert secs[0][0] == "net" and int(secs[0][1]["batch"]) == 2 and metric.endswith("images_per_s") and desc
        kinds[name] = [k for k, _ in secs[1:]]
    assert kinds["yolov3"].count("convolutional") == 75 and kinds["yolov3"].count("shortcut") == 23 and kinds["yolov3"].count("yolo") == 3
    assert kinds["yolov3-tiny"].count("maxpool") == 6
    assert kinds["memlayers"] == ["maxpool", "upsample", "maxpool", "shortcut", "route", "maxpool"]
    assert kinds["conv3x3"] == ["convolutional"] and kinds["conv1x1"] == ["convolutional"]
    # FLOPs as examples/darknet.c:87-88 counts them
    cfg = synth.yolov3_cfg(1, 608)
    h = w = 608
    total, dims = 0.0, []
    shapes = {s.index: s for s in synth.conv_shapes(cfg)}
    for i, (k, o) in enumerate(synth.parse_cfg(cfg)[1:]):
        if k == "convolutional":
            st = int(o.get("stride", 1))
            h, w = (h - 1) // st + 1, (w - 1) // st + 1
            s_ = shapes[i]
            total += 2.0 * s_.n * s_.size * s_.size * s_.c * h * w
        elif k == "upsample":
            h, w = h * 2, w * 2
        elif k == "route":
            ids = [int(t) for t in o["layers"].split(",")]
            h, w = dims[ids[0] if ids[0] >= 0 else i + ids[0]]
        dims.append((h, w))
    assert abs(total - 140_691_900_416.0) < 1.0
    peaks = bench.load_peaks()
    assert peaks["hbm_gbs"] > 1000 and peaks["bf16_tflops"] >= peaks["bf16_sustained"] > 100
