"""The NCCL-bound gradient exchange of the C ABI (mlp_comm_*, mlp_allreduce_grads).

One rank on one GPU: the exchange is the identity.  Two ranks (needs two GPUs): child processes, one
per GPU, each running learnGradient on its half of every batch, the exchange, and adjustParameters;
the replicas must stay bit-identical, match a one-GPU run within the summation-order bar, and with the
rank-ordered sum match the ordered sum of the two gradient segments bit for bit.  NVLS is switched
off in the children (plain peer transfers)."""
import os
import subprocess
import sys

import numpy as np
import pytest

from slang_b200 import config as C
from mlp_testlib import make_problem, rel_err

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def device():
    from slang_b200.api import Device
    d = Device(0)
    yield d
    d.destroy()


def test_single_rank_exchange_is_identity(device):
    from slang_b200.api import Comm, Trainer, comm_unique_id
    cfg, p0, batches = make_problem("c1", 512, seed=3, steps=1)
    tr = Trainer(device, cfg, p0)
    x, t = batches[0]
    xb, tb = device.create_buffer(x.nbytes, x), device.create_buffer(t.nbytes, t)
    tr.learn_gradient(xb.address, tb.address, x.shape[0])
    g0, l0 = tr.read_grads().copy(), tr.read_loss()
    comm = Comm(device, 1, 0, comm_unique_id())
    for ordered in (False, True):
        comm.allreduce_grads(tr, rank_ordered=ordered)
        device.wait()
        assert np.array_equal(tr.read_grads().view(np.uint32), g0.view(np.uint32))
        assert tr.read_loss() == l0
    comm.destroy()


CHILD = r"""
import os, sys, time
import numpy as np
sys.path.insert(0, {root!r}); sys.path.insert(0, os.path.join({root!r}, "tests"))
from slang_b200 import config as C
from slang_b200.api import Comm, Device, Trainer, comm_unique_id
from slang_b200.dist import shard_range
from mlp_testlib import make_problem
rank, world, out, ordered = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4] == "1"
idf = os.path.join(out, "id.bin")
if rank == 0:
    uid = comm_unique_id()
    with open(idf + ".tmp", "wb") as f: f.write(uid)
    os.replace(idf + ".tmp", idf)
else:
    for _ in range(600):
        if os.path.exists(idf): break
        time.sleep(0.1)
    uid = open(idf, "rb").read()
dev = Device(rank)
comm = Comm(dev, world, rank, uid)
cfg, p0, batches = make_problem({name!r}, {count}, seed=4, steps={steps})
tr = Trainer(dev, cfg, p0)
local = []
for x, t in batches:
    b, e = shard_range(x.shape[0], rank, world)
    xs, ts = np.ascontiguousarray(x[b:e]), np.ascontiguousarray(t[b:e])
    xb, tb = dev.create_buffer(xs.nbytes, xs), dev.create_buffer(ts.nbytes, ts)
    tr.learn_gradient(xb.address, tb.address, e - b)
    local.append(tr.read_grads().copy())
    comm.allreduce_grads(tr, rank_ordered=ordered)
    summed = tr.read_grads().copy()
    tr.adjust_parameters()
    dev.wait()
np.savez(os.path.join(out, "rank%d.npz" % rank), params=tr.read_params(), last_local=local[-1], last_sum=summed,
         loss=np.array(tr.read_loss()))
comm.destroy()
dev.destroy()
"""


def _run_ranks(tmp_path, name, count, steps, ordered):
    script = tmp_path / "child.py"
    script.write_text(CHILD.format(root=ROOT, name=name, count=count, steps=steps))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, str(script), str(r), "2", str(tmp_path), "1" if ordered else "0"], env=env)
             for r in range(2)]
    try:
        for p in procs:
            assert p.wait(timeout=300) == 0
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    return [np.load(tmp_path / ("rank%d.npz" % r)) for r in range(2)]


def _gpu_count():
    import torch
    return torch.cuda.device_count()


@pytest.mark.parametrize("ordered", [False, True])
def test_two_rank_step(tmp_path, device, ordered):
    if _gpu_count() < 2:
        pytest.skip("needs two GPUs")
    from slang_b200.api import Trainer
    name, count, steps = "c4", 4096, 3
    r = _run_ranks(tmp_path, name, count, steps, ordered)
    assert np.array_equal(r[0]["params"], r[1]["params"]), "replicas diverged"
    assert np.array_equal(r[0]["last_sum"].view(np.uint32), r[1]["last_sum"].view(np.uint32))
    if ordered:
        want = r[0]["last_local"] + r[1]["last_local"]
        assert np.array_equal(r[0]["last_sum"].view(np.uint32), want.view(np.uint32))
    # one GPU over the whole batch
    cfg, p0, batches = make_problem(name, count, seed=4, steps=steps)
    tr = Trainer(device, cfg, p0)
    for x, t in batches:
        xb, tb = device.create_buffer(x.nbytes, x), device.create_buffer(t.nbytes, t)
        tr.learn_gradient(xb.address, tb.address, x.shape[0])
        tr.adjust_parameters()
    device.wait()
    one = C.from_storage(tr.read_params(), cfg.dtype)
    two = C.from_storage(r[0]["params"], cfg.dtype)
    assert rel_err(two, one) <= 2e-2
    mx, sm = tr.read_loss()
    assert abs(r[0]["loss"][0] - mx) <= 1e-2 * abs(mx) and abs(r[0]["loss"][1] - sm) <= 1e-2 * abs(sm)
