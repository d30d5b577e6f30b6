"""The allocation-free learnGradient entry point against the ordinary ordered-sum entry point.

`mlp_learn_gradient_ordered_noalloc` exists for hosts that may not call the CUDA allocator while they
train (an engine that sub-allocates one up-front device-memory budget, or a frame loop that cannot
take cudaMalloc's device-wide synchronisation): its scratch lives in a fixed area inside the library.
It must produce exactly what "learnGradient_simt" with MLP_FLAG_SEQUENTIAL_SUM produces, also on a
second call that finds the first call's leftovers in the shared area, and it must refuse batches that
do not fit the area.  Collected last so that a failure here cannot hide another test's result.
"""
import ctypes

import numpy as np
import pytest

from slang_b200 import config as C

from mlp_testlib import make_problem

pytestmark = pytest.mark.gpu


def _run_both(device, cfg, p0, x, t, count):
    from slang_b200.api import FLAG_SEQUENTIAL_SUM, LearnGradParamsEx, Trainer
    from slang_b200.lib import check, load
    xb = device.create_buffer(x.nbytes, x)
    tb = device.create_buffer(t.nbytes, t)
    ref = Trainer(device, cfg, p0, learn_entry="learnGradient_simt")
    ref.learn_gradient(xb.address, tb.address, count, FLAG_SEQUENTIAL_SUM)
    g_ref, l_ref = ref.read_grads(), ref.loss.read(np.uint32).copy()

    new = Trainer(device, cfg, p0, learn_entry="learnGradient_simt")  # only for its buffers
    new.loss.clear()
    device.wait()
    args = LearnGradParamsEx(new.network.address, new.loss.address, xb.address, tb.address, count, 0)
    check(load().mlp_learn_gradient_ordered_noalloc(device.ordinal, None, ctypes.byref(cfg), ctypes.byref(args)))
    import torch
    torch.cuda.synchronize()  # the call ran on the legacy default stream
    g_new, l_new = new.read_grads(), new.loss.read(np.uint32).copy()
    xb.destroy(); tb.destroy()
    return g_ref, l_ref, g_new, l_new


def test_noalloc_entry_point_matches_ordered_sum_twice():
    from slang_b200.api import Device
    device = Device(0)
    try:
        # first call: config 1, a ragged batch; second call: a different network and batch, so the
        # shared area still holds the first call's vectors when the second one starts
        for name, count, seed in (("c1", 1000, 31), ("c2", 300, 32)):
            cfg, p0, batches = make_problem(name, count, seed=seed, steps=1)
            x, t = batches[0]
            g_ref, l_ref, g_new, l_new = _run_both(device, cfg, p0, x, t, count)
            assert np.any(g_ref != 0)
            assert np.array_equal(g_new.view(np.uint32), g_ref.view(np.uint32)), name
            assert l_new[0] == l_ref[0]
            a, b = l_new[1:2].view(np.float32)[0], l_ref[1:2].view(np.float32)[0]
            assert abs(a - b) <= 1e-5 * abs(b)  # the loss sum is an atomic float add in both
    finally:
        device.destroy()


def test_noalloc_entry_point_rejects_oversized_batches():
    from slang_b200.api import Device, LearnGradParamsEx
    from slang_b200.lib import load
    device = Device(0)
    try:
        cfg = C.named_config("c1")
        args = LearnGradParamsEx(1, 1, 1, 1, 10592, 0)  # one sample more than fits 2^20 floats at 99 per sample
        rc = load().mlp_learn_gradient_ordered_noalloc(0, None, ctypes.byref(cfg), ctypes.byref(args))
        assert rc == -2
        assert b"10591" in load().mlp_last_error_string()
    finally:
        device.destroy()
