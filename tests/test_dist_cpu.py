"""Host-side logic of the data-parallel step on CPU ranks (gloo, world size 2): each rank runs the
oracle on its shard, the flat gradient buffers are summed with the same helper the GPU path uses, and
the result must match a single process over the whole batch."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir, deterministic=False):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch.distributed as dist
    from oracle import oracle
    from slang_b200 import config as C
    from slang_b200.dist import allreduce_gradients, shard_range
    from mlp_testlib import make_problem
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg, p0, batches = make_problem("c1", 1000, seed=4, steps=3)
    _, _, total = C.param_layout(cfg)
    params = p0.copy()
    states = np.zeros(total, dtype=C.ADAM_STATE_DTYPE)
    states["master"] = p0
    for x, t in batches:
        b, e = shard_range(x.shape[0], rank, world)
        grads = np.zeros(total, dtype=np.float32)
        words = np.zeros(2, dtype=np.uint32)
        oracle.learn_gradient(cfg, params, grads, x[b:e].copy(), t[b:e].copy(), e - b, words)
        g_t = torch.from_numpy(grads)
        w_t = torch.from_numpy(words.view(np.float32))
        allreduce_gradients(g_t, w_t, deterministic=deterministic)
        oracle.adjust_parameters(cfg, states, params, grads)
    np.save(os.path.join(out_dir, "params_%d.npy" % rank), params)
    np.save(os.path.join(out_dir, "loss_%d.npy" % rank), words.view(np.float32))
    dist.destroy_process_group()


def test_two_rank_step_matches_single_process(tmp_path):
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from slang_b200 import config as C
    from mlp_testlib import make_problem, oracle_trajectory
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    p = [np.load(tmp_path / ("params_%d.npy" % r)) for r in range(world)]
    assert np.array_equal(p[0].view(np.uint32), p[1].view(np.uint32)), "replicas diverged"
    cfg, p0, batches = make_problem("c1", 1000, seed=4, steps=3)
    p_ref, l_ref, _, _ = oracle_trajectory(cfg, p0, batches)
    # the two half-batch sums are added in a different order than one sequential pass
    assert np.max(np.abs(p[0] - p_ref)) <= 1e-5 * np.max(np.abs(p_ref))
    loss = np.load(tmp_path / "loss_0.npy")
    assert abs(loss[0] - l_ref[-1][0]) <= 1e-6 * abs(l_ref[-1][0])
    assert abs(loss[1] / 1000 - l_ref[-1][1]) <= 1e-5 * abs(l_ref[-1][1])


def test_deterministic_sum_is_rank_ordered(tmp_path):
    """deterministic=True: every rank adds the ranks' segments in ascending rank order, so the result is
    bit-identical to one process that forms the per-shard sums and adds them in that order."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle import oracle
    from slang_b200 import config as C
    from slang_b200.dist import shard_range
    from mlp_testlib import make_problem
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path), True), nprocs=world, join=True)
    p = [np.load(tmp_path / ("params_%d.npy" % r)) for r in range(world)]
    assert np.array_equal(p[0].view(np.uint32), p[1].view(np.uint32)), "replicas diverged"
    cfg, p0, batches = make_problem("c1", 1000, seed=4, steps=3)
    _, _, total = C.param_layout(cfg)
    params = p0.copy()
    states = np.zeros(total, dtype=C.ADAM_STATE_DTYPE)
    states["master"] = p0
    for x, t in batches:
        acc = None
        for r in range(world):
            b, e = shard_range(x.shape[0], r, world)
            g = np.zeros(total, dtype=np.float32)
            oracle.learn_gradient(cfg, params, g, x[b:e].copy(), t[b:e].copy(), e - b, np.zeros(2, dtype=np.uint32))
            acc = g if acc is None else acc + g
        oracle.adjust_parameters(cfg, states, params, acc)
    assert np.array_equal(p[0].view(np.uint32), params.view(np.uint32))


def test_shard_ranges_cover_the_batch():
    from slang_b200.dist import shard_range
    for count in (0, 1, 7, 64, 1000, 1 << 26):
        for world in (1, 2, 3, 4, 8):
            edges = [shard_range(count, r, world) for r in range(world)]
            assert edges[0][0] == 0 and edges[-1][1] == count
            assert all(edges[i][1] == edges[i + 1][0] for i in range(world - 1))
    with pytest.raises(ValueError):
        shard_range(10, 2, 2)
