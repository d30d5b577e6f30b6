"""The allocation-free learnGradient entry point against the ordinary ordered-sum entry point.

`mlp_learn_gradient_ordered_noalloc` exists for hosts that may not call the CUDA allocator while they
train (an engine that sub-allocates one up-front device-memory budget, or a frame loop that cannot
take cudaMalloc's device-wide synchronisation): its scratch lives in a fixed area inside the library.
It must produce exactly what "learnGradient_simt" with MLP_FLAG_SEQUENTIAL_SUM produces, also on a
second call that finds the first call's leftovers in the shared area, it must refuse batches that do
not fit the area, refuse every config and flag the other entry points refuse (before any CUDA call),
leave the amount of free device memory and the caller's current device as it found them, and work on a
caller's stream.  Collected last so that a failure here cannot hide another test's result.
"""
import ctypes

import numpy as np
import pytest

from slang_b200 import config as C

from mlp_testlib import make_problem


def _call(ordinal, stream, cfg, args):
    from slang_b200.lib import load
    return load().mlp_learn_gradient_ordered_noalloc(ordinal, stream, ctypes.byref(cfg), ctypes.byref(args))


# ---- refusals: decided on the host before the first CUDA call, so they run without a GPU ----------
def test_noalloc_refuses_bad_configs_and_flags_before_any_launch():
    from slang_b200.api import FLAG_INPUT_GRADIENT, LearnGradParamsEx
    from slang_b200.lib import load
    ok_args = LearnGradParamsEx(1, 1, 1, 1, 16, 0)

    cfg = C.named_config("c1")
    cfg.dtype = 7  # not an MlpDType: the kernels would read 4-byte elements from a 2-byte buffer
    assert _call(0, None, cfg, ok_args) == -2
    assert b"dtype" in load().mlp_last_error_string()

    cfg = C.named_config("c1")
    cfg.target_dtype = -1
    assert _call(0, None, cfg, ok_args) == -2

    cfg = C.named_config("c1")  # dims[0] = 2
    cfg.encoding = C.ENC_FREQ2D
    assert _call(0, None, cfg, ok_args) == -2
    assert b"frequency encoding" in load().mlp_last_error_string()

    cfg = C.named_config("c1")
    cfg.encoding = 5
    assert _call(0, None, cfg, ok_args) == -2

    cfg = C.named_config("c1")
    cfg.input_width = 3
    assert _call(0, None, cfg, ok_args) == -2

    cfg = C.named_config("c1")
    assert _call(0, None, cfg, LearnGradParamsEx(1, 1, 1, 1, 16, FLAG_INPUT_GRADIENT)) == -3
    assert _call(0, None, cfg, LearnGradParamsEx(1, 1, 1, 1, 16, 8)) == -2
    assert _call(0, None, cfg, LearnGradParamsEx(0, 1, 1, 1, 16, 0)) == -2  # null network address
    assert _call(-1, None, cfg, ok_args) == -2
    assert _call(64, None, cfg, ok_args) == -2


def test_noalloc_rejects_oversized_batches():
    from slang_b200.api import LearnGradParamsEx
    from slang_b200.lib import load
    cfg = C.named_config("c1")
    args = LearnGradParamsEx(1, 1, 1, 1, 10592, 0)  # one sample more than fits 2^20 floats at 99 per sample
    assert _call(0, None, cfg, args) == -2
    assert b"10591" in load().mlp_last_error_string()


# ---- results ------------------------------------------------------------------------------------
def _reference(device, cfg, p0, xb, tb, count):
    from slang_b200.api import FLAG_SEQUENTIAL_SUM, Trainer
    ref = Trainer(device, cfg, p0, learn_entry="learnGradient_simt")
    ref.learn_gradient(xb.address, tb.address, count, FLAG_SEQUENTIAL_SUM)
    return ref.read_grads(), ref.loss.read(np.uint32).copy()


def _noalloc(device, cfg, p0, xb, tb, count, stream=None):
    """Runs the new entry point on `stream` (a torch stream, or None = the legacy default stream)."""
    import torch
    from slang_b200.api import LearnGradParamsEx, Trainer
    from slang_b200.lib import check
    new = Trainer(device, cfg, p0, learn_entry="learnGradient_simt")  # only for its buffers
    new.loss.clear()
    device.wait()
    args = LearnGradParamsEx(new.network.address, new.loss.address, xb.address, tb.address, count, 0)
    check(_call(device.ordinal, None if stream is None else ctypes.c_void_p(stream.cuda_stream), cfg, args))
    torch.cuda.synchronize(device.ordinal)
    return new.read_grads(), new.loss.read(np.uint32).copy()


def _same(g_new, l_new, g_ref, l_ref, what):
    assert np.any(g_ref != 0)
    assert np.array_equal(g_new.view(np.uint32), g_ref.view(np.uint32)), what
    assert l_new[0] == l_ref[0]
    a, b = l_new[1:2].view(np.float32)[0], l_ref[1:2].view(np.float32)[0]
    assert abs(a - b) <= 1e-5 * abs(b)  # the loss sum is an atomic float add in both


@pytest.mark.gpu
def test_noalloc_entry_point_matches_ordered_sum_twice():
    import torch
    from slang_b200.api import Device, LearnGradParamsEx, Trainer
    from slang_b200.lib import check
    device = Device(0)
    try:
        # A count of zero is the documented start-up call: it resolves the area's address, launches
        # nothing and succeeds.
        cfg0 = C.named_config("c1")
        check(_call(0, None, cfg0, LearnGradParamsEx(1, 1, 0, 0, 0, 0)))
        torch.cuda.synchronize(0)
        # first call: config 1, a ragged batch; second call: a different network and batch, so the
        # shared area still holds the first call's vectors when the second one starts; third call:
        # config 1 at exactly the documented limit, so the last slot of the area is written and read.
        for name, count, seed in (("c1", 1000, 31), ("c2", 300, 32), ("c1", 10591, 33)):
            cfg, p0, batches = make_problem(name, count, seed=seed, steps=1)
            x, t = batches[0]
            xb, tb = device.create_buffer(x.nbytes, x), device.create_buffer(t.nbytes, t)
            g_ref, l_ref = _reference(device, cfg, p0, xb, tb, count)
            # the reference path above may allocate (its scratch buffer); measure around the new call only
            new = Trainer(device, cfg, p0, learn_entry="learnGradient_simt")  # only for its buffers
            new.loss.clear()
            device.wait()
            new_buffers_free = torch.cuda.mem_get_info(0)[0]
            args = LearnGradParamsEx(new.network.address, new.loss.address, xb.address, tb.address, count, 0)
            check(_call(0, None, cfg, args))
            torch.cuda.synchronize(0)
            assert torch.cuda.mem_get_info(0)[0] == new_buffers_free, "the call changed the free device memory"
            g_new, l_new = new.read_grads(), new.loss.read(np.uint32).copy()
            _same(g_new, l_new, g_ref, l_ref, name)
            xb.destroy(); tb.destroy()
    finally:
        device.destroy()


@pytest.mark.gpu
def test_noalloc_entry_point_on_a_caller_stream():
    import torch
    from slang_b200.api import Device
    device = Device(0)
    try:
        cfg, p0, batches = make_problem("c1", 777, seed=41, steps=1)
        x, t = batches[0]
        xb, tb = device.create_buffer(x.nbytes, x), device.create_buffer(t.nbytes, t)
        g_ref, l_ref = _reference(device, cfg, p0, xb, tb, 777)
        stream = torch.cuda.Stream(device=0)
        g_new, l_new = _noalloc(device, cfg, p0, xb, tb, 777, stream)
        _same(g_new, l_new, g_ref, l_ref, "caller stream")
    finally:
        device.destroy()


@pytest.mark.gpu
def test_noalloc_entry_point_on_a_second_device_keeps_the_current_device():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs: the area's address is looked up once per device")
    from cuda.bindings import runtime as cudart
    from slang_b200.api import Device, LearnGradParamsEx, Trainer
    from slang_b200.lib import check
    device = Device(1)
    try:
        cfg, p0, batches = make_problem("c1", 500, seed=43, steps=1)
        x, t = batches[0]
        xb, tb = device.create_buffer(x.nbytes, x), device.create_buffer(t.nbytes, t)
        g_ref, l_ref = _reference(device, cfg, p0, xb, tb, 500)
        new = Trainer(device, cfg, p0, learn_entry="learnGradient_simt")  # only for its buffers
        new.loss.clear()
        device.wait()
        # The current device is a property of the calling thread in the driver, so any binding of the runtime
        # sets and sees it.  The handle-based calls above left device 1 current; make it device 0 and check
        # that the call on device 1 puts device 0 back.
        assert int(cudart.cudaSetDevice(0)[0]) == 0
        args = LearnGradParamsEx(new.network.address, new.loss.address, xb.address, tb.address, 500, 0)
        check(_call(1, None, cfg, args))
        err, cur = cudart.cudaGetDevice()
        assert int(err) == 0 and cur == 0
        torch.cuda.synchronize(1)
        _same(new.read_grads(), new.loss.read(np.uint32).copy(), g_ref, l_ref, "device 1")
    finally:
        device.destroy()
