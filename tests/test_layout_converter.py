"""Parameter layout converter against the reference's own unit-test model
(tools/gfx-unit-test/neural-slang-network-converter.cpp): network 5 -> 13 -> 7 -> 19 with biases on
layers 0 and 2, 321 logical and 1088 physical elements, values (i*37+19)%257 - 128 scaled by 1/8."""
import ctypes

import numpy as np
import pytest

from oracle import layout_oracle as LO
from slang_b200 import config as C

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
