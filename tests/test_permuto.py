"""Permutohedral-lattice encoder: the oracle against the reference's own known answers (CPU), and the CUDA
kernels against the oracle and the same known answers (GPU)."""
import ctypes
import json
import os

import numpy as np
import pytest

from oracle import permuto as OP
from slang_b200 import config as C
from slang_b200 import permuto as P

GOLD = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "permuto_reference.json")))
EPS = 0.1   # the reference tests' own tolerance (tests/neural/permuto-encoder-test.slang:31)


def reference_case(cfg_source):
    """The configuration of tests/neural/permuto-encoder-test.slang:10-27: 2-D positions at the cell centres
    of a 16 x 16 grid, 4 levels, 2 features per entry, 2^8 entries per level, table[i] = i."""
    cfg = cfg_source(2, 2, 8, 4, 4.0, 1.5, 1.1, 1337, C.F32)
    idx = np.arange(256)
    pos = np.stack([(idx % 16 + 0.5) / 16.0, (idx // 16 + 0.5) / 16.0], axis=1).astype(np.float32)
    table = np.arange(2048, dtype=np.float32)
    return cfg, pos, table


def oracle_prepare(*a):
    return OP.prepare(P.PermutoConfig, *a)


def check_against_reference(out, dpos, dtable):
    vp = GOLD["verify_positions"]
    want = np.array(GOLD["forward"], dtype=np.float32).reshape(16, 8)
    assert np.max(np.abs(out[vp] - want)) <= EPS
    wantp = np.array(GOLD["dl_dpos"], dtype=np.float32).reshape(16, 2)
    assert np.max(np.abs(dpos[vp] - wantp)) <= EPS
    wantt = np.array(GOLD["dl_dparams"], dtype=np.float32)
    assert np.max(np.abs(dtable[GOLD["verify_param_indices"]] - wantt)) <= EPS


def test_hashes_match_reference_known_answers():
    """tests/neural/hash-function-test.slang:100-121: five hashes x four dimensionalities, then the
    dispatcher for Prime and BaseConvert in 3-D.  Both the oracle and the library's host function."""
    pos = GOLD["hash_positions"]
    for fn in (OP.grid_hash, P.grid_hash):
        got = [fn(t, p) for t in (P.HASH_PRIME, P.HASH_COHERENT_PRIME, P.HASH_REVERSED_PRIME, P.HASH_BASE_CONVERT, P.HASH_RNG)
               for p in pos]
        got += [fn(P.HASH_PRIME, pos[2]), fn(P.HASH_BASE_CONVERT, pos[2])]
        assert got == GOLD["hashes"]


def test_level_constants_match_reference():
    """tests/neural/permuto-encoder-precomputed-constants.slang:24-55."""
    k = GOLD["constants"]
    for prep in (oracle_prepare, P.prepare):
        cfg = prep(2, 2, 8, 4, 4.0, 1.5, 1.1, 1337, C.F32)
        assert abs(cfg.max_level - k["lc_maxLevel"]) < 1e-6
        for l in range(4):
            li = cfg.levels[l]
            assert (li.level_index, li.table_offset, li.table_size) == (l, k["lc_offsets"][l], k["lc_tableSizes"][l])
            assert abs(li.scale - k["lc_scales"][l]) <= 2e-6 * k["lc_scales"][l]
            for d in range(2):
                assert abs(li.scales_per_dim[d] - k["lc_scalesPerDim"][2 * l + d]) <= 2e-6 * k["lc_scalesPerDim"][2 * l + d]
                assert abs(li.shifts_per_dim[d] - k["lc_shiftsPerDim"][2 * l + d]) <= 2e-6
    a, b = oracle_prepare(3, 4, 10, 7, 2.0, 0.8, 1.1, 99, C.F16), P.prepare(3, 4, 10, 7, 2.0, 0.8, 1.1, 99, C.F16)
    assert bytes(a) == bytes(b)


def test_oracle_matches_reference_known_answers():
    """tests/neural/permuto-reference-data.slang: 16 positions x 8 forward values, their position gradients
    and 64 feature-table gradients for an all-ones upstream gradient."""
    cfg, pos, table = reference_case(oracle_prepare)
    out = OP.encode(cfg, pos, table)
    dtable = np.zeros_like(table)
    dpos = OP.backward(cfg, pos, table, np.ones_like(out), dtable)
    check_against_reference(out, dpos, dtable)
    # every position spreads weight 1 per level: the table gradient sums to positions x levels x features
    assert abs(float(dtable.sum()) - 256 * 4 * 2) < 1e-2


def test_oracle_properties():
    """Size-independent properties: barycentric weights sum to one (a constant table encodes to that
    constant), levels past max_level are zero, the encoding is linear in the table."""
    rng = np.random.default_rng(0)
    for dims in (1, 2, 3, 4):
        cfg = oracle_prepare(dims, 2, 10, 6, 1.5, 1.0, 0.5, 7, C.F32)   # max_level = 3: levels 3.. are zero? no: index >= 3.001
        pos = rng.uniform(0, 1, (500, dims)).astype(np.float32)
        const = np.full(cfg.table_values, 2.5, dtype=np.float32)
        out = OP.encode(cfg, pos, const)
        live = [l for l in range(6) if float(l) < cfg.max_level + 1e-3]
        assert live == [0, 1, 2, 3]
        assert np.allclose(out[:, :8], 2.5, atol=1e-4) and not out[:, 8:].any()
        t1, t2 = rng.normal(size=cfg.table_values).astype(np.float32), rng.normal(size=cfg.table_values).astype(np.float32)
        assert np.allclose(OP.encode(cfg, pos, t1 + t2), OP.encode(cfg, pos, t1) + OP.encode(cfg, pos, t2), atol=1e-4)
        # the reverse pass is the transpose of the forward pass: <encode(t), g> == <t, backward(g)>
        g = rng.normal(size=(500, 12)).astype(np.float32)
        dt = np.zeros_like(t1)
        OP.backward(cfg, pos, t1, g, dt)
        assert abs(float((OP.encode(cfg, pos, t1).astype(np.float64) * g).sum()) - float((t1.astype(np.float64) * dt).sum())) < 2e-2


def test_oracle_position_gradient_matches_finite_differences():
    rng = np.random.default_rng(3)
    cfg = oracle_prepare(3, 2, 12, 3, 1.0, 0.5, 1.1, 5, C.F32)
    table = rng.normal(size=cfg.table_values).astype(np.float32)
    pos = rng.uniform(0.2, 0.8, (40, 3)).astype(np.float32)
    g = rng.normal(size=(40, 6)).astype(np.float32)
    dpos = OP.backward(cfg, pos, table, g, np.zeros_like(table))
    h = 1e-3
    ok = 0
    for d in range(3):
        e = np.zeros(3, dtype=np.float32); e[d] = h
        num = ((OP.encode(cfg, pos + e, table).astype(np.float64) - OP.encode(cfg, pos - e, table)) * g).sum(axis=1) / (2 * h)
        ok += np.sum(np.abs(num - dpos[:, d]) <= 2e-2 * (1 + np.abs(num)))
    assert ok >= 0.9 * 120   # the encoding is piecewise linear: a step that crosses a simplex face is off


# ---- CUDA kernels ----------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def device():
    from slang_b200.api import Device
    d = Device(0)
    yield d
    d.destroy()


def gpu_run(device, cfg, pos, table, d_out=None, want_dpos=True):
    enc = P.PermutoEncoder(device, cfg)
    n = pos.shape[0]
    nf = cfg.n_features
    pb = device.create_buffer(max(pos.nbytes, 4), pos if n else None)
    tb = device.create_buffer(table.nbytes, table)
    ob = device.create_buffer(max(n * nf * table.itemsize, 4))
    enc.encode(pb.address, tb.address, ob.address, n)
    out = ob.read(table.dtype)[: n * nf].reshape(n, nf).copy()
    if d_out is None:
        return out
    gb = device.create_buffer(max(d_out.nbytes, 4), np.ascontiguousarray(d_out) if n else None)
    dtb = device.create_buffer(table.nbytes)
    dpb = device.create_buffer(max(n * cfg.dims * 4, 4))
    enc.backward(pb.address, tb.address, gb.address, dtb.address, dpb.address if want_dpos else 0, n)
    device.wait()
    return out, dpb.read(np.float32)[: n * cfg.dims].reshape(n, cfg.dims).copy(), dtb.read(table.dtype).copy()


@pytest.mark.gpu
def test_gpu_matches_reference_known_answers(device):
    cfg, pos, table = reference_case(P.prepare)
    out, dpos, dtable = gpu_run(device, cfg, pos, table, np.ones((256, 8), dtype=np.float32))
    check_against_reference(out, dpos, dtable)


@pytest.mark.gpu
@pytest.mark.parametrize("dims", [1, 2, 3, 4])
@pytest.mark.parametrize("features", [1, 2, 4, 8])
def test_gpu_matches_oracle_f32(device, dims, features):
    """Forward and position gradients bit for bit (same expressions, same order, no contraction); table
    gradients within the order-of-addition bar (atomics)."""
    rng = np.random.default_rng(dims * 10 + features)
    cfg = P.prepare(dims, features, 12, 5, 2.0, 1.0, 1.1, 1337 + dims, C.F32)
    n = 3001   # ragged: not a multiple of the block's positions
    pos = rng.uniform(-0.5, 1.5, (n, dims)).astype(np.float32)
    table = rng.normal(size=cfg.table_values).astype(np.float32)
    g = rng.normal(size=(n, cfg.n_features)).astype(np.float32)
    out, dpos, dtable = gpu_run(device, cfg, pos, table, g)
    want = OP.encode(cfg, pos, table)
    wdt = np.zeros_like(table)
    wdpos = OP.backward(cfg, pos, table, g, wdt)
    assert np.array_equal(out.view(np.uint32), want.view(np.uint32))
    assert np.array_equal(dpos.view(np.uint32), wdpos.view(np.uint32))
    assert np.max(np.abs(dtable - wdt)) <= 1e-5 * max(1.0, float(np.max(np.abs(wdt))))


@pytest.mark.gpu
def test_gpu_half_tables(device):
    rng = np.random.default_rng(21)
    cfg = P.prepare(3, 2, 10, 4, 2.0, 1.0, 1.1, 7, C.F16)
    n = 2000
    pos = rng.uniform(0, 1, (n, 3)).astype(np.float32)
    table = rng.normal(size=cfg.table_values).astype(np.float16)
    g = (rng.normal(size=(n, cfg.n_features)) * 0.01).astype(np.float16)
    out, dpos, dtable = gpu_run(device, cfg, pos, table, g)
    want = OP.encode(cfg, pos, table)
    wdt = np.zeros_like(table)
    wdpos = OP.backward(cfg, pos, table, g, wdt)
    assert np.array_equal(out.view(np.uint16), want.view(np.uint16))
    assert np.array_equal(dpos.view(np.uint32), wdpos.view(np.uint32))
    # half accumulation in another order: a few half ulps of the largest entry
    assert np.max(np.abs(dtable.astype(np.float32) - wdt.astype(np.float32))) <= 2e-2 * max(1e-3, float(np.max(np.abs(wdt.astype(np.float32)))))


@pytest.mark.gpu
def test_gpu_edge_cases(device):
    from slang_b200.lib import MlpError
    cfg = P.prepare(2, 2, 8, 4, 4.0, 1.5, 0.5, 1337, C.F32)   # max_level 2: levels 3 is dead (index >= 2.001 -> levels 3 only? 2 < 2.001)
    rng = np.random.default_rng(1)
    table = rng.normal(size=cfg.table_values).astype(np.float32)
    # empty batch
    assert gpu_run(device, cfg, np.zeros((0, 2), np.float32), table).shape == (0, 8)
    # dead levels write zeros and take no gradient; one position; no position gradient requested
    pos = np.array([[0.3, 0.9]], dtype=np.float32)
    g = np.ones((1, 8), dtype=np.float32)
    out, _, dtable = gpu_run(device, cfg, pos, table, g, want_dpos=False)
    want = OP.encode(cfg, pos, table)
    assert np.array_equal(out, want) and not out[0, 6:].any() and out[0, :6].all()
    assert not dtable[3 * 256 * 2:].any() and abs(dtable.sum() - 6.0) < 1e-4
    # all positions on one vertex set: heavy atomic collisions still add up
    same = np.tile(pos, (4096, 1))
    _, _, dt = gpu_run(device, cfg, same, table, np.ones((4096, 8), dtype=np.float32))
    assert abs(float(dt.sum()) - 4096 * 6.0) < 0.5
    bad = P.prepare(2, 2, 8, 4, 4.0, 1.5, 1.1, 1337, C.F32)
    bad.features_per_entry = 3
    with pytest.raises(MlpError):
        P.PermutoEncoder(device, bad).encode(1, 1, 1, 1)
    with pytest.raises(MlpError):
        P.prepare(5, 2, 8, 4, 4.0, 1.5)


@pytest.mark.gpu
def test_gpu_large_batch_properties(device):
    """2^22 positions, 16 levels of 2^19 entries: constant table encodes to the constant, the table gradient
    of an all-ones upstream sums to positions x live levels x features."""
    cfg = P.prepare(3, 2, 19, 16, 16.0, 0.5, 1.1, 1337, C.F32)
    n = 1 << 22
    rng = np.random.default_rng(4)
    pos = rng.uniform(0, 1, (n, 3)).astype(np.float32)
    table = np.full(cfg.table_values, 1.5, dtype=np.float32)
    g = np.ones((n, cfg.n_features), dtype=np.float32)
    out, dpos, dtable = gpu_run(device, cfg, pos, table, g)
    assert np.allclose(out, 1.5, atol=1e-4)
    assert abs(float(dtable.astype(np.float64).sum()) / (n * 32.0) - 1.0) < 1e-4
    sub = slice(0, 4096)
    assert np.array_equal(out[sub], OP.encode(cfg, pos[sub], table))
