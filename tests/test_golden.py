"""Golden fixtures (tests/golden/*.npz, written by tests/golden/make_golden.py).

CPU: the oracle still reproduces them bit for bit.  GPU: the kernels match them within the bars."""
import os

import numpy as np
import pytest

from slang_b200 import config as C

from mlp_testlib import gpu_trajectory, make_problem, oracle_trajectory, per_layer_rel_errs, rel_err

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
NAMES = ["c1", "c2", "c3", "c4"]


def _load(name):
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    cfg, p0, batches = make_problem(name, int(g["count"]), seed=int(g["seed"]), steps=int(g["steps"]))
    assert np.array_equal(np.asarray(p0).view(np.uint8), g["params0"].view(np.uint8)), "seeded initialisation changed"
    return g, cfg, p0, batches


@pytest.mark.parametrize("name", NAMES)
def test_oracle_reproduces_golden(name):
    g, cfg, p0, batches = _load(name)
    p, losses, g0, states = oracle_trajectory(cfg, p0, batches)
    assert np.array_equal(g0.view(np.uint32), g["grads0"].view(np.uint32))
    assert np.array_equal(np.asarray(p).view(np.uint8), g["params"].view(np.uint8))
    assert np.array_equal(np.array(losses, dtype=np.float64), g["losses"])
    assert np.array_equal(states["iteration"], g["iteration"])


@pytest.mark.gpu
@pytest.mark.parametrize("name", NAMES)
def test_gpu_matches_golden(name):
    from slang_b200.api import Device, FLAG_SEQUENTIAL_SUM
    g, cfg, p0, batches = _load(name)
    dev = Device(0)
    try:
        if name == "c1":
            p, losses, g0, _, _ = gpu_trajectory(dev, cfg, p0, batches, "learnGradient_simt", FLAG_SEQUENTIAL_SUM)
            assert np.array_equal(g0.view(np.uint32), g["grads0"].view(np.uint32))
            assert np.array_equal(p.view(np.uint32), g["params"].view(np.uint32))
        else:
            p, losses, g0, _, tr = gpu_trajectory(dev, cfg, p0, batches)
            assert rel_err(g0, g["grads0"]) < 1e-2
            errs = per_layer_rel_errs(cfg, C.from_storage(p, cfg.dtype), C.from_storage(g["params"], cfg.dtype))
            assert max(errs) < 2e-2, (tr.k_learn.implementation, errs)
        for (mx, mean), (rmx, rmean) in zip(losses, g["losses"]):
            assert abs(mean - rmean) <= 1e-2 * abs(rmean)
            assert abs(mx - rmx) <= 1e-2 * abs(rmx)
    finally:
        dev.destroy()
