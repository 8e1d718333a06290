"""The drop-in boundary on an unmodified Darknet: the reference's own GPU build (its CUDA sources
recompiled for sm_100a, cuBLAS) parses the cfg, loads the weights and predicts; b200_attach then
re-points the forward_gpu pointers of the same `network` at libdarknet_b200 and network_predict is
called again.  Every layer's output (read back from Darknet's own l.output_gpu buffers) is compared
with the CPU checker: FP32 plans 1e-4, TF32 plans 1e-2, BF16 plans 6e-2 of the layer's largest value."""
import json
import os
import subprocess
import sys

import pytest

import darknet_b200 as dn
from oracle import network as orc

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(not orc.ReferenceGpu.available(), reason="oracle/_ref/libdarknet_ref_gpu.so was not built (make -C oracle refgpu)")
@pytest.mark.parametrize("name", ["tiny96_b2", "yolov3_64", "resnet50_32"])
@pytest.mark.parametrize("mode", [dn.MODE_FP32, dn.MODE_TF32, dn.MODE_BF16])
def test_attach_to_unmodified_darknet(name, mode):
    p = subprocess.run([sys.executable, os.path.join(HERE, "attach_check.py"), name, str(mode)],
                       capture_output=True, text=True, timeout=600)
    lines = [ln for ln in p.stdout.splitlines() if ln.startswith("ATTACH_RESULT ")]
    assert p.returncode == 0 and lines, f"child failed ({p.returncode}):\n{p.stdout[-2000:]}\n{p.stderr[-3000:]}"
    r = json.loads(lines[-1][len("ATTACH_RESULT "):])
    print(name, mode, r)
    # the reference's GPU path against its CPU path: they differ by design in the batchnorm
    # denominator (sqrtf(var + 1e-5f), src/blas_kernels.cu:200, against sqrt(var) + 1e-6f, src/blas.c:154)
    assert r["stock_vs_cpu"] < 2e-3
    assert r["attached"] == r["coverable"] > 0           # every layer of the five covered types was re-pointed
    tol = {dn.MODE_FP32: 1e-4, dn.MODE_TF32: 1e-2, dn.MODE_BF16: 6e-2}[mode]
    assert r["attached_vs_cpu"] < tol
    assert r["second_input_differs"]
    assert r["detached_equals_stock"]
    # b200_attach_network: the whole forward pass behind the same network_predict
    assert r["whole_attached"] == r["layers"]
    assert r["whole_vs_cpu"] < tol
    assert r["whole_second_input_differs"]
    assert r["whole_detached_equals_stock"]
