"""The failure paths of the GPU library, exercised without faulting, trapping or hanging the device.

* A bounded device-side wait that runs out: a diagnostic bit makes every CTA of the tensor-core
  convolution withhold one operand load, and the wait bound is shortened to about two milliseconds for
  that plan.  A wait expires (the MMA role's for the operands, code 102, or the epilogue's for the
  accumulator, code 104, whichever began first), the CTA raises its abort flag, drains, frees its TMEM and
  returns; the host reads DNB_ETIMEOUT with the code of the wait, the status word is cleared, and
  the next ordinary launch of the same plan is correct.  The same through the network object, blocking
  and with two steps in flight, where each step has its own status word.
* Parameters set a second time: the cached tensor map over the weights and a captured CUDA graph are
  rebuilt, and the next forward uses the new weights.
* A plan or network used with another CUDA device current is refused before anything is launched
  (needs two devices; skipped otherwise).
* A convolution with a stride the tensor-core kernel has no lattice maps for runs on the CUDA-core kernel.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import darknet_b200 as dn
from conftest import parity
from darknet_b200 import synth
from gpu_util import dev_nhwc, empty_nhwc, host_from_nhwc
from oracle import network as orc

pytestmark = pytest.mark.gpu
SHORT_WAIT = 4_000_000   # cycles: about 2 ms at 1.9 GHz
WITHHOLD = 32


def rng(seed):
    return np.random.Generator(np.random.Philox(key=[seed, 7]))


def make_conv(seed, b, c, h, w, n, size, stride=1):
    g = rng(seed)
    x = g.standard_normal((b, c, h, w), dtype=np.float32)
    wt = g.standard_normal((n, c, size, size), dtype=np.float32) * np.float32(np.sqrt(2.0 / (size * size * c)))
    p = dict(biases=g.standard_normal(n, dtype=np.float32) * np.float32(0.1), scales=g.uniform(0.9, 1.1, n).astype(np.float32),
             mean=g.standard_normal(n, dtype=np.float32) * np.float32(0.1), var=g.uniform(0.5, 1.5, n).astype(np.float32))
    return x, wt, p


def oracle(x, wt, p, size, stride=1):
    return orc.conv_forward(x, wt, p["biases"], p["scales"], p["mean"], p["var"], stride=stride, pad=size // 2, groups=1, activation="leaky")


@pytest.mark.parametrize("mode,store,tol", [(dn.MODE_TF32, torch.float32, 1e-2), (dn.MODE_BF16, torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("shape", [dict(b=2, c=64, h=13, w=13, n=64, size=3), dict(b=4, c=128, h=19, w=19, n=512, size=1),
                                   dict(b=1, c=32, h=40, w=40, n=320, size=3),
                                   dict(b=8, c=64, h=38, w=38, n=512, size=3),     # runs as CTA pairs
                                   dict(b=1, c=1024, h=19, w=19, n=1024, size=3)])  # pairs with split-K: the tile counters a timed-out launch leaves part-way are zeroed
def test_wait_expiry_is_reported_and_the_plan_recovers(mode, store, tol, shape):
    size = shape["size"]
    x, wt, p = make_conv(70, **shape)
    want = oracle(x, wt, p, size)
    b, c, h, w = x.shape
    n = wt.shape[0]
    plan = dn.ConvPlan(b, c, h, w, n, size, 1, size // 2, 1, True, "leaky", False, mode)
    plan.set_params(wt, p["biases"], p["scales"], p["mean"], p["var"])
    assert plan.kernel.startswith("tc_")
    xt, xd = dev_nhwc(x, store)

    def run():
        yt, yd = empty_nhwc(b, n, h, w, store)
        plan.forward(xd, yd)
        torch.cuda.synchronize()
        return host_from_nhwc(yt, n)

    got = run()
    plan.check_status()
    parity(got, want, tol, "before the injected time-out")
    plan.set_diagnostics(SHORT_WAIT, WITHHOLD)
    run()                                              # returns: the kernel gave up instead of hanging
    with pytest.raises(dn.DarknetB200Error) as e:
        plan.check_status()
    assert e.value.status == dn.ETIMEOUT and ("code 102" in str(e.value) or "code 104" in str(e.value)), str(e.value)
    plan.check_status()                                # the word was cleared by the read
    plan.set_diagnostics(0, 0)
    got = run()
    plan.check_status()
    parity(got, want, tol, "after the injected time-out")


def test_wait_expiry_with_a_fused_residual():
    x, wt, p = make_conv(71, 2, 64, 26, 26, 128, 3)
    add = rng(72).standard_normal((2, 128, 26, 26), dtype=np.float32)
    want = orc.shortcut_forward(oracle(x, wt, p, 3), add, 1.0, 1.0, "linear")
    plan = dn.ConvPlan(2, 64, 26, 26, 128, 3, 1, 1, 1, True, "leaky", False, dn.MODE_TF32)
    plan.set_params(wt, p["biases"], p["scales"], p["mean"], p["var"])
    xt, xd = dev_nhwc(x)
    at, ad = dev_nhwc(add)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def run():
        yt, yd = empty_nhwc(2, 128, 26, 26)
        dn.check(dn.lib().dnb_conv_shortcut_forward(plan.handle, C.byref(xd), C.byref(ad), C.byref(yd), 1.0, 1.0, dn.ACTIVATIONS["linear"], stream))
        torch.cuda.synchronize()
        return host_from_nhwc(yt, 128)

    parity(run(), want, 1e-2, "fused residual before")
    plan.set_diagnostics(SHORT_WAIT, WITHHOLD)
    run()
    with pytest.raises(dn.DarknetB200Error) as e:
        plan.check_status()
    assert e.value.status == dn.ETIMEOUT
    plan.set_diagnostics(0, 0)
    parity(run(), want, 1e-2, "fused residual after")
    plan.check_status()


def small_net(tmp_path, mode=dn.MODE_TF32, seed=31):
    cfg = synth.yolov3_tiny_cfg(batch=2, size=64)
    params = synth.seeded_params(cfg, seed)
    wpath = str(tmp_path / f"n{seed}.weights")
    synth.write_weights(wpath, params)
    return cfg, params, dn.Network(cfg, wpath, mode, text=True)


def test_network_predict_reports_a_wait_expiry_and_recovers(tmp_path):
    cfg, params, net = small_net(tmp_path)
    x = synth.seeded_input(cfg, 31)
    good = net.predict(x).copy()
    victim = next(i for i in range(net.n) if net.layer_kernel(i).startswith("tc_"))
    net.set_diagnostics(victim, SHORT_WAIT, WITHHOLD)
    with pytest.raises(dn.DarknetB200Error) as e:
        net.predict(x)
    assert e.value.status == dn.ETIMEOUT and ("code 102" in str(e.value) or "code 104" in str(e.value)), str(e.value)
    net.set_diagnostics(victim, 0, 0)
    assert np.array_equal(net.predict(x), good)        # the word was cleared, the context is intact
    # the device-resident forward reports through dnb_network_check_status
    xd = torch.from_numpy(x).cuda()
    net.set_diagnostics(victim, SHORT_WAIT, WITHHOLD)
    net.forward(xd)
    with pytest.raises(dn.DarknetB200Error) as e:
        net.check_status()
    assert e.value.status == dn.ETIMEOUT
    net.check_status()
    net.set_diagnostics(victim, 0, 0)
    net.forward(xd)
    net.check_status()
    assert np.array_equal(net.layer_output(net.n - 1).reshape(good.shape), good)


def test_each_step_in_flight_has_its_own_status_word(tmp_path):
    cfg, params, net = small_net(tmp_path)
    xs = [torch.from_numpy(synth.seeded_input(cfg, 40 + k)).pin_memory() for k in range(3)]
    good = [net.predict(x).copy() for x in xs]
    victim = next(i for i in range(net.n) if net.layer_kernel(i).startswith("tc_"))
    net.submit(xs[0])                                  # step 0: sound
    net.set_diagnostics(victim, SHORT_WAIT, WITHHOLD)
    net.submit(xs[1])                                  # step 1: will time out
    net.set_diagnostics(victim, 0, 0)
    assert np.array_equal(net.collect(), good[0])      # step 0 is not blamed for step 1
    net.submit(xs[2])                                  # step 2 reuses step 0's slot
    with pytest.raises(dn.DarknetB200Error) as e:
        net.collect()                                  # step 1
    assert e.value.status == dn.ETIMEOUT
    assert np.array_equal(net.collect(), good[2])      # and step 2 is sound again
    assert np.array_equal(net.predict(xs[1]), good[1])


@pytest.mark.parametrize("mode,store,tol", [(dn.MODE_TF32, torch.float32, 1e-2), (dn.MODE_BF16, torch.bfloat16, 3e-2)])
def test_parameters_set_twice_reach_the_kernel(mode, store, tol):
    x, w1, p1 = make_conv(80, 2, 64, 20, 20, 96, 3)
    _, w2, p2 = make_conv(81, 2, 64, 20, 20, 96, 3)
    plan = dn.ConvPlan(2, 64, 20, 20, 96, 3, 1, 1, 1, True, "leaky", False, mode)
    xt, xd = dev_nhwc(x, store)
    yt, yd = empty_nhwc(2, 96, 20, 20, store)
    filler = []
    for wt, p in ((w1, p1), (w2, p2), (w1, p1)):
        plan.set_params(wt, p["biases"], p["scales"], p["mean"], p["var"])
        filler.append(torch.empty(1 << 20, device="cuda"))   # keeps the allocator from handing back the freed address
        plan.forward(xd, yd)                                   # same input and output pointers every time
        torch.cuda.synchronize()
        parity(host_from_nhwc(yt, 96), oracle(x, wt, p, 3), tol, "after set_params")


def test_network_weights_loaded_twice_with_graph_replay(tmp_path):
    cfg, params, net = small_net(tmp_path, seed=32)
    x = synth.seeded_input(cfg, 32)
    s = torch.cuda.Stream()
    xd = torch.from_numpy(x).cuda()
    torch.cuda.synchronize()
    net.enable_graph(True)

    def run():
        for _ in range(3):                             # eager, captured, replayed
            net.forward(xd, stream=s.cuda_stream)
        s.synchronize()
        return net.layer_output(net.n - 1).copy()

    a = run()
    parity(a, orc.forward_network(cfg, params, x)[-1], 1e-2, "first weights")
    params2 = synth.seeded_params(cfg, 33)
    w2 = str(tmp_path / "second.weights")
    synth.write_weights(w2, params2)
    net.load_weights(w2)                               # frees and reallocates every derived tensor
    b = run()
    parity(b, orc.forward_network(cfg, params2, x)[-1], 1e-2, "second weights")
    assert not np.array_equal(a, b)


def test_other_current_device_is_refused(tmp_path):
    n = C.c_int()
    dn.check(dn.lib().dnb_device_count(C.byref(n)))
    if n.value < 2:
        pytest.skip("needs two CUDA devices")
    x, wt, p = make_conv(90, 1, 16, 8, 8, 16, 3)
    plan = dn.ConvPlan(1, 16, 8, 8, 16, 3, 1, 1, 1, True, "leaky").set_params(wt, p["biases"], p["scales"], p["mean"], p["var"])
    xt, xd = dev_nhwc(x)
    yt, yd = empty_nhwc(1, 16, 8, 8)
    cfg, params, net = small_net(tmp_path)
    xin = torch.from_numpy(synth.seeded_input(cfg, 1)).cuda()
    try:
        dn.check(dn.lib().dnb_set_device(1))
        with pytest.raises(dn.DarknetB200Error) as e:
            plan.forward(xd, yd)
        assert e.value.status == dn.EINVAL and "device" in str(e.value)
        with pytest.raises(dn.DarknetB200Error) as e:
            net.forward(xin)
        assert e.value.status == dn.EINVAL
    finally:
        dn.check(dn.lib().dnb_set_device(0))
    plan.forward(xd, yd)
    torch.cuda.synchronize()


@pytest.mark.parametrize("mode", [dn.MODE_TF32, dn.MODE_BF16])
def test_stride_three_runs_on_the_cuda_core_kernel(mode):
    x, wt, p = make_conv(91, 2, 16, 17, 17, 24, 3, stride=3)
    plan = dn.ConvPlan(2, 16, 17, 17, 24, 3, 3, 1, 1, True, "leaky", False, mode)
    plan.set_params(wt, p["biases"], p["scales"], p["mean"], p["var"])
    assert plan.kernel == "direct_fp32"
    from gpu_util import dev_nchw, empty_nchw
    xt, xd = dev_nchw(x)
    yt, yd = empty_nchw(2, 24, plan.out_h, plan.out_w)
    plan.forward(xd, yd)
    torch.cuda.synchronize()
    parity(yt.cpu().numpy(), oracle(x, wt, p, 3, stride=3), 1e-5, "stride 3")
