"""Parameter layout converter against the reference's own unit-test model
(tools/gfx-unit-test/neural-slang-network-converter.cpp): network 5 -> 13 -> 7 -> 19 with biases on
layers 0 and 2, 321 logical and 1088 physical elements, values (i*37+19)%257 - 128 scaled by 1/8."""
import ctypes

import numpy as np
import pytest

from oracle import layout_oracle as LO
from slang_b200 import config as C
from mlp_testlib import gpu_trajectory, oracle_trajectory, per_layer_rel_errs

DIMS, MASK = [5, 13, 7, 19], 0b101


def test_reference_element_counts():
    assert LO.sizes(DIMS, MASK) == (321, 1088)
    from slang_b200 import lib
    lo, po = ctypes.c_int64(), ctypes.c_int64()
    shape = C.network_shape(DIMS, MASK, 4)
    assert lib.load().mlp_layout_sizes(ctypes.byref(shape), ctypes.byref(lo), ctypes.byref(po)) == 0
    assert (lo.value, po.value) == (321, 1088)
    bad = C.network_shape(DIMS, MASK, 3)
    assert lib.load().mlp_layout_sizes(ctypes.byref(bad), ctypes.byref(lo), ctypes.byref(po)) < 0


def test_oracle_tile_order_is_a_permutation():
    pos = sorted(LO.native_tile_pos(r, c) for r in range(16) for c in range(16))
    assert pos == list(range(256))
    # first B-fragment register of lane 0 holds rows 0,1 of column 0; lane 1 rows 2,3
    assert LO.native_tile_pos(0, 0) == 0 and LO.native_tile_pos(1, 0) == 1 and LO.native_tile_pos(2, 0) == 8
    assert LO.native_tile_pos(8, 0) == 2 and LO.native_tile_pos(0, 8) == 4 and LO.native_tile_pos(0, 1) == 32


@pytest.mark.gpu
@pytest.mark.parametrize("elem", ["f32", "f16"])
def test_converter_round_trip_on_gpu(elem):
    from slang_b200 import lib
    from slang_b200.api import Device
    from slang_b200.lib import check
    dev = Device(0)
    try:
        vals = LO.reference_test_values(321)
        portable = vals if elem == "f32" else vals.astype(np.float16)
        expect = LO.to_optimal(portable, DIMS, MASK)
        shape = C.network_shape(DIMS, MASK, portable.itemsize)
        pb = dev.create_buffer(portable.nbytes, portable)
        ob = dev.create_buffer(1088 * portable.itemsize, np.full(1088, 7, dtype=portable.dtype))
        check(lib.load().mlp_layout_to_optimal(dev.handle, ctypes.byref(shape), pb.address, ob.address))
        got = ob.read(portable.dtype)
        assert np.array_equal(got.view(np.uint8), expect.view(np.uint8))
        back = dev.create_buffer(portable.nbytes)
        check(lib.load().mlp_layout_to_portable(dev.handle, ctypes.byref(shape), ob.address, back.address))
        assert np.array_equal(back.read(portable.dtype).view(np.uint8), portable.view(np.uint8))
        # a larger network with widths that are multiples of 16 and every bias present
        dims, mask = [64, 128, 128, 64], 0b111
        lo, po = LO.sizes(dims, mask)
        p2 = np.random.default_rng(1).normal(size=lo).astype(portable.dtype)
        shape2 = C.network_shape(dims, mask, p2.itemsize)
        pb2 = dev.create_buffer(p2.nbytes, p2); ob2 = dev.create_buffer(po * p2.itemsize)
        check(lib.load().mlp_layout_to_optimal(dev.handle, ctypes.byref(shape2), pb2.address, ob2.address))
        assert np.array_equal(ob2.read(p2.dtype).view(np.uint8), LO.to_optimal(p2, dims, mask).view(np.uint8))
    finally:
        dev.destroy()


def test_fflayer_optimal_layout_envelope():
    """tests/neural/fflayer-wavetangled-vector-tiled-test.slang:87-180: a 4 -> 2 layer in OptimalLayout has
    ParameterCount 10, WeightStorageSize 256, BiasStorageSize 16, StorageSize 272, its bias at element 256;
    the layer without a bias keeps the 272-element envelope (ParameterCount 8)."""
    assert LO.sizes([4, 2], 0b1) == (10, 272)
    assert LO.sizes([4, 2], 0b0) == (8, 272)
    w_off, b_off, total = C.optimal_layout_offsets([4, 2])
    assert (w_off, b_off, total) == ([0], [256], 272)
    portable = np.array([1, 2, 3, 4, 5, 6, 7, 8, 9, 10], dtype=np.float32)   # W = [[1..4],[5..8]], b = [9, 10]
    opt = LO.to_optimal(portable, [4, 2], 0b1)
    assert opt.size == 272 and list(opt[256:258]) == [9.0, 10.0] and not opt[258:].any()
    assert np.count_nonzero(opt[:256]) == 8
    from slang_b200 import lib
    lo, po = ctypes.c_int64(), ctypes.c_int64()
    for mask, want in ((1, (10, 272)), (0, (8, 272))):
        shape = C.network_shape([4, 2], mask, 4)
        assert lib.load().mlp_layout_sizes(ctypes.byref(shape), ctypes.byref(lo), ctypes.byref(po)) == 0
        assert (lo.value, po.value) == want


@pytest.mark.gpu
@pytest.mark.parametrize("dims,dtype,entry", [
    ([4, 2], "f32", "forward_simt"),               # the tiled test's own layer: [39, 80]
    ([4, 4, 2], "f16", "forward"),                 # padded 64-wide tensor-core kernel
    ([64, 64, 64, 64, 64], "f16", "forward"),      # constant-width tensor-core kernel
    ([128, 128, 128, 128, 128], "bf16", "forward"),
    ([32, 128, 128, 3], "f16", "forward"),         # wide tensor-core kernel
    ([5, 13, 7, 19], "f32", "forward_simt"),       # the converter test's shape, nothing a multiple of 16
])
def test_forward_reads_optimal_layout_in_place(dims, dtype, entry):
    """The forward entry points read OptimalLayout parameters where they lie (FFLayer's storage,
    source/standard-modules/neural/layers.slang:53-71): same outputs, bit for bit, as the same network in the
    row-major layout; the 4 -> 2 layer of fflayer-wavetangled-vector-tiled-test.slang:93-110 gives [39, 80]."""
    from slang_b200 import lib
    from slang_b200.api import Device, OptimalLayoutNetwork, Trainer
    from slang_b200.lib import check
    dt = {"f32": C.F32, "f16": C.F16, "bf16": C.BF16}[dtype]
    dev = Device(0)
    try:
        rng = np.random.default_rng(sum(dims))
        act = C.ACT_IDENTITY if dims == [4, 2] else C.ACT_RELU
        cfg = C.make_config(dims, dtype=dt, hidden_act=act, input_dtype=dt if dt != C.F32 else C.F32, target_dtype=C.F32)
        w_off, b_off, total = C.param_layout(cfg)
        p = np.zeros(total, dtype=np.float32)
        for l in range(cfg.n_layers):
            n = dims[l] * dims[l + 1]
            p[w_off[l]:w_off[l] + n] = rng.uniform(-1, 1, n) * (2.0 / dims[l]) ** 0.5
            p[b_off[l]:b_off[l] + dims[l + 1]] = rng.uniform(-0.5, 0.5, dims[l + 1])
        if dims == [4, 2]:
            p[w_off[0]:w_off[0] + 8] = np.arange(1, 9)
            p[b_off[0]:b_off[0] + 2] = [9, 10]
        ps = C.to_storage(p, dt)
        count = 300
        x = rng.uniform(-1, 1, (count, dims[0])).astype(np.float32)
        if dims == [4, 2]:
            x[:] = [1, 2, 3, 4]
        xs = C.to_storage(x, cfg.input_dtype)
        xb = dev.create_buffer(xs.nbytes, xs)
        # row-major reference run
        tr = Trainer(dev, cfg, ps, forward_entry=entry)
        yb = dev.create_buffer(count * dims[-1] * 4)
        tr.forward(xb.address, yb.address, count)
        want = yb.read(np.float32).copy()
        # portable (unpadded) parameters -> OptimalLayout with the library's converter, then used in place
        portable = np.concatenate([np.concatenate([ps[w_off[l]:w_off[l] + dims[l] * dims[l + 1]], ps[b_off[l]:b_off[l] + dims[l + 1]]])
                                   for l in range(cfg.n_layers)])
        mask = (1 << cfg.n_layers) - 1
        lo, po = LO.sizes(dims, mask)
        assert portable.size == lo and po == C.optimal_layout_offsets(dims)[2]
        shape = C.network_shape(dims, mask, portable.itemsize)
        pb = dev.create_buffer(portable.nbytes, portable)
        ob = dev.create_buffer(po * portable.itemsize)
        check(lib.load().mlp_layout_to_optimal(dev.handle, ctypes.byref(shape), pb.address, ob.address))
        cfg_opt = C.make_config(dims, dtype=dt, hidden_act=act, input_dtype=cfg.input_dtype, target_dtype=C.F32)
        cfg_opt.param_layout = C.PARAMS_OPTIMAL
        net = OptimalLayoutNetwork(dev, cfg_opt, ob.address, forward_entry=entry)
        assert net.k_forward.implementation == tr.k_forward.implementation
        y2 = dev.create_buffer(count * dims[-1] * 4)
        net.forward(xb.address, y2.address, count)
        got = y2.read(np.float32)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        if dims == [4, 2]:
            assert np.all(got.reshape(count, 2) == [39.0, 80.0])
        # the training entry points take the layout too (test_training_on_optimal_layout_parameters_in_place)
        assert dev.kernel("learnGradient", cfg_opt).implementation == dev.kernel("learnGradient", cfg).implementation
    finally:
        dev.destroy()


@pytest.mark.gpu
@pytest.mark.parametrize("dims,dtype,act,entry", [
    ([2, 16, 16, 1], "f32", C.ACT_RELU, "learnGradient"),                 # one thread per sample
    ([20, 48, 64, 3], "f16", C.ACT_LEAKY_RELU, "learnGradient"),          # padded 64-wide tensor-core kernel, ragged tiles
    ([4, 32, 32, 32, 32, 4], "f16", C.ACT_LEAKY_RELU, "learnGradient"),   # its 32-wide build
    ([64, 128, 128, 128, 128, 64], "bf16", C.ACT_GELU_TANH, "learnGradient"),  # wide tensor-core kernel
    ([32, 96, 128, 10], "f16", C.ACT_RELU, "learnGradient"),              # wide kernel, widths that are not tile multiples
    ([20, 48, 64, 3], "f16", C.ACT_LEAKY_RELU, "learnGradient_simt"),
])
def test_training_on_optimal_layout_parameters_in_place(dims, dtype, act, entry):
    """learnGradient + adjustParameters on parameters that stay in OptimalLayout (what a Slang shader's FFLayer
    reads, source/standard-modules/neural/layers.slang:53-71): after three steps the parameters, converted back
    with the numpy layout oracle's index map, equal those of the same run on row-major parameters (to the order
    of the atomic adds), and the loss words agree; both runs are held against the CPU oracle's trajectory."""
    from slang_b200.api import Device
    dt = {"f32": C.F32, "f16": C.F16, "bf16": C.BF16}[dtype]
    dev = Device(0)
    try:
        rng = np.random.default_rng(sum(dims) + len(entry))
        in_dt = dt if max(dims) > 64 else C.F32
        cfg = C.make_config(dims, dtype=dt, hidden_act=act, act_alpha=0.02, input_dtype=in_dt, target_dtype=C.F32, lr=1e-3,
                            adam_master=0 if dt == C.F32 else 1)
        cfg_opt = C.make_config(dims, dtype=dt, hidden_act=act, act_alpha=0.02, input_dtype=in_dt, target_dtype=C.F32, lr=1e-3,
                                adam_master=0 if dt == C.F32 else 1)
        cfg_opt.param_layout = C.PARAMS_OPTIMAL
        p0 = C.init_params(cfg, seed=11, scheme="xavier")
        w_off, b_off, total = C.param_layout(cfg)
        ow, ob, ototal = C.param_layout(cfg_opt)
        assert (ow, ob, ototal) == C.optimal_layout_offsets(dims)
        for l in range(cfg.n_layers):
            p0[b_off[l]:b_off[l] + dims[l + 1]] = C.to_storage(rng.uniform(-0.2, 0.2, dims[l + 1]).astype(np.float32), dt)

        def index_map(l):
            """optimal element offset of weight (o, i) of layer l, from the layout oracle's tile order"""
            in16, out16 = LO.align16(dims[l]), LO.align16(dims[l + 1])
            m = np.empty((dims[l + 1], dims[l]), dtype=np.int64)
            for o in range(dims[l + 1]):
                for i in range(dims[l]):
                    tile = (i // 16) * (out16 // 16) + (o // 16)
                    m[o, i] = ow[l] + tile * 256 + LO.native_tile_pos(i % 16, o % 16)
            return m

        maps = [index_map(l) for l in range(cfg.n_layers)]

        def to_opt(flat):
            out = np.zeros(ototal, dtype=flat.dtype)
            for l in range(cfg.n_layers):
                out[maps[l].ravel()] = flat[w_off[l]:w_off[l] + dims[l] * dims[l + 1]]
                out[ob[l]:ob[l] + dims[l + 1]] = flat[b_off[l]:b_off[l] + dims[l + 1]]
            return out

        def to_rows(opt):
            out = np.zeros(total, dtype=opt.dtype)
            for l in range(cfg.n_layers):
                out[w_off[l]:w_off[l] + dims[l] * dims[l + 1]] = opt[maps[l].ravel()]
                out[b_off[l]:b_off[l] + dims[l + 1]] = opt[ob[l]:ob[l] + dims[l + 1]]
            return out

        count = 128 * 3 + 77
        batches = []
        for _ in range(3):
            x = C.to_storage(rng.uniform(-1, 1, (count, dims[0])).astype(np.float32), in_dt)
            t = rng.uniform(-1, 1, (count, dims[-1])).astype(np.float32)
            batches.append((x, t))
        p_rows, l_rows, g_rows, _, tr_rows = gpu_trajectory(dev, cfg, p0, batches, entry)
        p_opt, l_opt, g_opt, _, tr_opt = gpu_trajectory(dev, cfg_opt, to_opt(p0), batches, entry)
        assert tr_opt.k_learn.implementation == tr_rows.k_learn.implementation
        assert tr_opt.k_learn.implementation == ("simt" if dt == C.F32 or entry.endswith("simt") else "tcgen05")
        # the padding of the tiled buffer stays zero: gradients and parameters
        used = np.zeros(ototal, dtype=bool)
        for l in range(cfg.n_layers):
            used[maps[l].ravel()] = True
            used[ob[l]:ob[l] + dims[l + 1]] = True
        assert not g_opt[~used].any() and not C.from_storage(p_opt, dt)[~used].any()
        tol = 1e-5 if dt == C.F32 else 2e-3
        assert max(per_layer_rel_errs(cfg, to_rows(g_opt), g_rows)) <= tol
        assert max(per_layer_rel_errs(cfg, C.from_storage(to_rows(p_opt), dt), C.from_storage(p_rows, dt))) <= 10 * tol
        for (m1, s1), (m2, s2) in zip(l_opt, l_rows):
            assert abs(s1 - s2) <= 10 * tol * abs(s2) and abs(m1 - m2) <= 10 * tol * abs(m2)
        # and against the oracle
        _, l_ref, g_ref, _ = oracle_trajectory(cfg, p0, batches, n_threads=4)
        assert max(per_layer_rel_errs(cfg, to_rows(g_opt), g_ref)) <= (1e-5 if dt == C.F32 else 1e-2)
    finally:
        dev.destroy()
