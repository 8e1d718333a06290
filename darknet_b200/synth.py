"""Synthetic networks and parameters for tests and benchmarks.

Nothing here is on the hot path.  It produces (a) Darknet ``.cfg`` text for the
network families the benchmark configurations name, built from their published
architecture (stage counts and widths), (b) seeded random parameters with the
distributions the benchmark configurations prescribe, and (c) ``.weights`` files
in the on-disk format Darknet's ``load_weights`` reads (src/parser.c:1218-1306:
three int32 ``major, minor, revision``, a ``size_t seen``, then per
convolutional layer ``biases[n]``, and if batch-normalised ``scales[n]``,
``rolling_mean[n]``, ``rolling_variance[n]``, then ``weights[n*c/groups*size*size]``,
src/parser.c:1164-1215; per connected layer ``biases[outputs]``,
``weights[outputs*inputs]``, then the batchnorm vectors, src/parser.c:1098-1120).

The same file is read by the unmodified reference (the checker) and by this
library's loader, so both sides always see identical parameters.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field

import numpy as np

# --------------------------------------------------------------------------- cfg text


def parse_cfg(text: str) -> list[tuple[str, dict[str, str]]]:
    """Split cfg text into ``(section_name, options)`` pairs.

    Same rules as the reference's ``read_cfg`` (src/parser.c:891-924): a line
    starting with ``[`` opens a section; blank lines and lines starting with
    ``#`` or ``;`` are skipped; other lines are ``key=value`` with surrounding
    whitespace dropped."""
    sections: list[tuple[str, dict[str, str]]] = []
    for raw in text.splitlines():
        line = raw.strip()
        if not line or line[0] in "#;":
            continue
        if line[0] == "[":
            sections.append((line.strip("[]").strip(), {}))
            continue
        if "=" not in line or not sections:
            raise ValueError(f"cfg line not understood: {raw!r}")
        key, val = line.split("=", 1)
        sections[-1][1][key.strip()] = val.strip()
    return sections


def _net(batch: int, width: int, height: int, channels: int = 3) -> str:
    return f"[net]\nbatch={batch}\nsubdivisions=1\nwidth={width}\nheight={height}\nchannels={channels}\n"


def _conv(filters: int, size: int, stride: int = 1, bn: bool = True, act: str = "leaky",
          xnor: bool = False, groups: int = 1, pad: int = 1) -> str:
    s = "\n[convolutional]\n"
    if bn:
        s += "batch_normalize=1\n"
    s += f"filters={filters}\nsize={size}\nstride={stride}\npad={pad}\n"
    if groups != 1:
        s += f"groups={groups}\n"
    if xnor:
        s += "xnor=1\n"
    s += f"activation={act}\n"
    return s


def _shortcut(frm: int, act: str = "linear") -> str:
    return f"\n[shortcut]\nfrom={frm}\nactivation={act}\n"


def _yolo(mask: str, anchors: str, num: int, classes: int = 80) -> str:
    return (f"\n[yolo]\nmask = {mask}\nanchors = {anchors}\nclasses={classes}\nnum={num}\n"
            "jitter=.3\nignore_thresh = .7\ntruth_thresh = 1\nrandom=1\n")


_YOLOV3_ANCHORS = "10,13,  16,30,  33,23,  30,61,  62,45,  59,119,  116,90,  156,198,  373,326"
_TINY_ANCHORS = "10,14,  23,27,  37,58,  81,82,  135,169,  344,319"


def yolov3_cfg(batch: int = 64, size: int = 608) -> str:
    """YOLOv3: Darknet-53 backbone (residual stages of 1, 2, 8, 8, 4 blocks at
    widths 64..1024), three detection heads with an upsample+route feature
    pyramid.  Same layer sequence as the reference's cfg/yolov3.cfg (107 layers)."""
    s = _net(batch, size, size)
    s += _conv(32, 3)
    width = 32
    for blocks in (1, 2, 8, 8, 4):
        width *= 2
        s += _conv(width, 3, stride=2)
        for _ in range(blocks):
            s += _conv(width // 2, 1) + _conv(width, 3) + _shortcut(-3)
    heads = (("6,7,8", 512, None), ("3,4,5", 256, 61), ("0,1,2", 128, 36))
    for mask, w, lateral in heads:
        if lateral is not None:
            s += "\n[route]\nlayers = -4\n" + _conv(w, 1) + "\n[upsample]\nstride=2\n"
            s += f"\n[route]\nlayers = -1, {lateral}\n"
        for _ in range(3):
            s += _conv(w, 1) + _conv(2 * w, 3)
        s += _conv(255, 1, bn=False, act="linear") + _yolo(mask, _YOLOV3_ANCHORS, 9)
    return s


def yolov3_tiny_cfg(batch: int = 1, size: int = 416) -> str:
    """YOLOv3-tiny: 13 convolutions, six 2x2 maxpools (the last with stride 1),
    two heads.  Same layer sequence as the reference's cfg/yolov3-tiny.cfg."""
    s = _net(batch, size, size)
    for i, w in enumerate((16, 32, 64, 128, 256, 512)):
        s += _conv(w, 3) + f"\n[maxpool]\nsize=2\nstride={1 if i == 5 else 2}\n"
    s += _conv(1024, 3) + _conv(256, 1) + _conv(512, 3)
    s += _conv(255, 1, bn=False, act="linear") + _yolo("3,4,5", _TINY_ANCHORS, 6)
    s += "\n[route]\nlayers = -4\n" + _conv(128, 1) + "\n[upsample]\nstride=2\n"
    s += "\n[route]\nlayers = -1, 8\n" + _conv(256, 3)
    s += _conv(255, 1, bn=False, act="linear") + _yolo("0,1,2", _TINY_ANCHORS, 6)
    return s


def resnet50_cfg(batch: int = 256, size: int = 224) -> str:
    """ResNet-50 as Darknet expresses it (cfg/resnet50.cfg): 7x7/2 stem, 2x2/2
    maxpool, bottleneck stages of 3, 4, 6, 3 blocks (the stride-2 sits on the 3x3
    of each stage's first block), leaky shortcuts ``from=-4``, global average
    pool, 1x1 convolution to 1000 classes, softmax."""
    s = _net(batch, size, size)
    s += _conv(64, 7, stride=2) + "\n[maxpool]\nsize=2\nstride=2\n"
    for stage, (blocks, w) in enumerate(((3, 64), (4, 128), (6, 256), (3, 512))):
        for b in range(blocks):
            stride = 2 if (stage > 0 and b == 0) else 1
            s += _conv(w, 1) + _conv(w, 3, stride=stride) + _conv(4 * w, 1, act="linear")
            s += _shortcut(-4, act="leaky")
    s += "\n[avgpool]\n" + _conv(1000, 1, bn=False, act="linear") + "\n[softmax]\ngroups=1\n"
    return s


def darknet19_cfg(batch: int = 128, size: int = 224, xnor: bool = True) -> str:
    """Darknet-19 classifier (cfg/darknet19.cfg) with ``xnor=1`` on every
    convolution except the first and the last when ``xnor`` is set."""
    s = _net(batch, size, size)
    plan = [(32,), "M", (64,), "M", (128, 64, 128), "M", (256, 128, 256), "M",
            (512, 256, 512, 256, 512), "M", (1024, 512, 1024, 512, 1024)]
    first = True
    for item in plan:
        if item == "M":
            s += "\n[maxpool]\nsize=2\nstride=2\n"
            continue
        for i, w in enumerate(item):
            s += _conv(w, 3 if i % 2 == 0 else 1, xnor=(xnor and not first))
            first = False
    s += _conv(1000, 1, bn=False, act="linear") + "\n[avgpool]\n\n[softmax]\ngroups=1\n"
    return s


def connected_cfg(batch: int = 4, size: int = 12, hidden: int = 48, classes: int = 10, bn: bool = True) -> str:
    """A small classifier that ends in connected layers, in the style of the reference's older cfgs
    (cfg/darknet.cfg's tail, cfg/alexnet.cfg): convolution, maxpool, a connected layer over the whole
    feature map (its input is the map flattened channel by channel), a second connected layer, softmax."""
    s = _net(batch, size, size)
    s += _conv(16, 3) + "\n[maxpool]\nsize=2\nstride=2\n" + _conv(24, 3)
    s += f"\n[connected]\n{'batch_normalize=1' if bn else ''}\noutput={hidden}\nactivation=leaky\n"
    s += f"\n[connected]\noutput={classes}\nactivation=linear\n\n[softmax]\ngroups=1\n"
    return s


def single_conv_cfg(batch: int, c: int, h: int, w: int, filters: int, size: int, stride: int = 1,
                    pad: int = 1, bn: bool = True, act: str = "leaky", xnor: bool = False,
                    groups: int = 1) -> str:
    """One convolutional layer as a whole network (isolated-layer configurations)."""
    return _net(batch, w, h, c) + _conv(filters, size, stride, bn, act, xnor, groups, pad)


def memory_layers_cfg(batch: int = 64, c: int = 128, size: int = 152) -> str:
    """The memory-bound layer types of the path chained into one network without a convolution: maxpool 2x2/2,
    upsample x2, maxpool 2x2/1 (the padded form of yolov3-tiny), shortcut, route, maxpool; the shapes are
    those of YOLOv3's 152x152 stage.  For measuring those kernels against the HBM copy rate."""
    return (_net(batch, size, size, c) +
            "[maxpool]\nsize=2\nstride=2\n\n[upsample]\nstride=2\n\n[maxpool]\nsize=2\nstride=1\n\n"
            "[shortcut]\nfrom=-2\nactivation=linear\n\n[route]\nlayers=-1,-3\n\n[maxpool]\nsize=2\nstride=2\n\n")


# --------------------------------------------------------------------------- parameters


@dataclass
class ConvParams:
    """Host parameters of one convolutional or connected layer, in Darknet's layouts."""
    weights: np.ndarray            # [n, c/groups, size, size] fp32; connected: [outputs, inputs]
    biases: np.ndarray             # [n]
    scales: np.ndarray | None      # [n] (batchnorm gamma) or None
    rolling_mean: np.ndarray | None
    rolling_variance: np.ndarray | None
    kind: str = "convolutional"    # or "connected" (the two differ in the order of their arrays on disk)


@dataclass
class ConvShape:
    index: int
    c: int
    n: int
    size: int
    groups: int
    batch_normalize: bool
    kind: str = "convolutional"    # "connected": c is the number of inputs (channels x height x width), size 1


def param_shapes(cfg_text: str) -> list[ConvShape]:
    """Walk the cfg and return the parameter shape of every layer that has parameters (convolutional and
    connected), in file order, tracking channels and map size through the other layers the way
    parse_network_cfg does (src/parser.c:742-889)."""
    sections = parse_cfg(cfg_text)
    net = sections[0][1]
    c, h, w = int(net.get("channels", 3)), int(net.get("height", 0)), int(net.get("width", 0))
    dims: list[tuple[int, int, int]] = []
    shapes: list[ConvShape] = []
    for idx, (kind, opt) in enumerate(sections[1:]):
        if kind == "convolutional":
            n, size, stride = int(opt.get("filters", 1)), int(opt.get("size", 1)), int(opt.get("stride", 1))
            pad = size // 2 if int(opt.get("pad", 0)) else int(opt.get("padding", 0))
            shapes.append(ConvShape(idx, c, n, size, int(opt.get("groups", 1)), bool(int(opt.get("batch_normalize", 0)))))
            c, h, w = n, (h + 2 * pad - size) // stride + 1, (w + 2 * pad - size) // stride + 1
        elif kind == "connected":
            n = int(opt.get("output", 1))
            shapes.append(ConvShape(idx, c * h * w, n, 1, 1, bool(int(opt.get("batch_normalize", 0))), "connected"))
            c, h, w = n, 1, 1
        elif kind == "maxpool":
            stride = int(opt.get("stride", 1))
            size = int(opt.get("size", stride))
            pad = int(opt.get("padding", size - 1))
            h, w = (h + pad - size) // stride + 1, (w + pad - size) // stride + 1
        elif kind == "upsample":
            st = int(opt.get("stride", 2))
            h, w = h * st, w * st
        elif kind == "route":
            ids = [int(t) for t in opt["layers"].split(",")]
            ids = [i if i >= 0 else idx + i for i in ids]
            c = sum(dims[i][0] for i in ids)
            h, w = dims[ids[0]][1], dims[ids[0]][2]
        elif kind == "avgpool":
            h = w = 1
        # shortcut, yolo, softmax keep the shape
        dims.append((c, h, w))
    return shapes


def conv_shapes(cfg_text: str) -> list[ConvShape]:
    """The convolutional layers of param_shapes."""
    return [s for s in param_shapes(cfg_text) if s.kind == "convolutional"]


def seeded_params(cfg_text: str, seed: int = 0, pow2_mean_xnor: bool = False) -> list[ConvParams]:
    """Random parameters for every convolutional and connected layer from a counter-based PRNG
    (Philox), one independent stream per layer: weights He-normal
    N(0, 2/(size^2 * c/groups)), biases N(0, 0.01), batchnorm gamma U(0.9, 1.1),
    rolling_mean N(0, 0.1), rolling_variance U(0.5, 1.5) (second argument of N is
    the variance)."""
    out = []
    for shp in param_shapes(cfg_text):
        rng = np.random.Generator(np.random.Philox(key=[seed, shp.index]))
        fan = shp.size * shp.size * (shp.c // shp.groups)
        if shp.kind == "connected":
            w = rng.standard_normal((shp.n, shp.c), dtype=np.float32)
        else:
            w = rng.standard_normal((shp.n, shp.c // shp.groups, shp.size, shp.size), dtype=np.float32)
        w *= np.float32(np.sqrt(2.0 / fan))
        b = (rng.standard_normal(shp.n, dtype=np.float32) * np.float32(0.1))
        if shp.batch_normalize:
            g = rng.uniform(0.9, 1.1, shp.n).astype(np.float32)
            m = (rng.standard_normal(shp.n, dtype=np.float32) * np.float32(np.sqrt(0.1)))
            v = rng.uniform(0.5, 1.5, shp.n).astype(np.float32)
            out.append(ConvParams(w, b, g, m, v, shp.kind))
        else:
            out.append(ConvParams(w, b, None, None, None, shp.kind))
    return out


def packed_filter_bytes(w: np.ndarray) -> bytes:
    """One convolution's weights [n, ...] in the reference's packed-binary form (save_convolutional_weights_binary,
    src/parser.c:926-956): per filter the mean |w| (summed in a float in index order, src/convolutional_layer.c:28-41)
    and size/8 bytes of sign bits, lowest bit first, set where w > 0."""
    n = w.shape[0]
    flat = np.ascontiguousarray(w, np.float32).reshape(n, -1)
    size = flat.shape[1]
    mean = np.zeros(n, np.float32)
    for k in range(size):
        mean += np.abs(flat[:, k])
    mean = (mean / np.float32(size)).astype(np.float32)
    bits = np.packbits((flat[:, :size // 8 * 8] > 0).astype(np.uint8), axis=1, bitorder="little")
    return b"".join(mean[i].tobytes() + bits[i].tobytes() for i in range(n))


def write_weights(path: str, params: list[ConvParams], seen: int = 0, version: tuple[int, int, int] = (0, 2, 0),
                  flipped: set[int] | frozenset = frozenset(), packed: set[int] | frozenset = frozenset()) -> None:
    """Write a ``.weights`` file: header major, minor, revision and ``seen`` (64-bit from version 0.2 on,
    32-bit before; src/parser.c:1018-1024, 1234-1241), then each layer's arrays in load order.
    A major or minor version above 1000 marks a file whose connected-layer matrices are stored
    [inputs][outputs] (src/parser.c:1244, 1098-1104); ``flipped`` names the positions in ``params`` of
    convolutions whose cfg section says ``flipped=1`` and whose matrix is stored [c*size*size][n]
    (src/parser.c:1206-1208)."""
    major, minor, revision = version
    transposed = major > 1000 or minor > 1000
    with open(path, "wb") as f:
        f.write(struct.pack("<iii", major, minor, revision))
        f.write(struct.pack("<Q", seen) if (major * 10 + minor) >= 2 and major < 1000 and minor < 1000 else struct.pack("<i", seen))
        for i, p in enumerate(params):
            f.write(np.ascontiguousarray(p.biases, dtype=np.float32).tobytes())
            w = np.ascontiguousarray(p.weights, dtype=np.float32)
            bn = [] if p.scales is None else [p.scales, p.rolling_mean, p.rolling_variance]
            if p.kind == "connected":
                if transposed:
                    w = np.ascontiguousarray(w.T)      # the loader transposes [inputs][outputs] back
                f.write(w.tobytes())
                for a in bn:
                    f.write(np.ascontiguousarray(a, dtype=np.float32).tobytes())
            else:
                for a in bn:
                    f.write(np.ascontiguousarray(a, dtype=np.float32).tobytes())
                if i in packed:       # positions in ``params`` of convolutions stored in the packed-binary form
                    f.write(packed_filter_bytes(w))
                    continue
                if i in flipped:
                    w = np.ascontiguousarray(w.reshape(w.shape[0], -1).T)
                f.write(w.tobytes())


def seeded_input(cfg_text: str, seed: int = 0, dist: str = "uniform") -> np.ndarray:
    """Seeded input batch [batch, channels, height, width]: U[0,1) or N(0,1)."""
    net = parse_cfg(cfg_text)[0][1]
    shape = (int(net["batch"]) // int(net.get("subdivisions", 1)), int(net.get("channels", 3)),
             int(net["height"]), int(net["width"]))
    rng = np.random.Generator(np.random.Philox(key=[seed, 1 << 20]))
    if dist == "uniform":
        return rng.random(shape, dtype=np.float32)
    return rng.standard_normal(shape, dtype=np.float32)
