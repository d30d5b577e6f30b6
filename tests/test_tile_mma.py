"""Cooperative-matrix multiply-add (mlp_tile_mma, include/slang_b200_tile_mma.h) against the reference's known
answers (tests/cooperative-matrix/{mat-mul-add,int8,uint8,int8-saturating,uint8-saturating,fp8-cuda,
fp8-cuda-half-acc}.slang) and against the numpy oracle on random problems."""
import ctypes

import numpy as np
import pytest

from oracle import tile_mma_oracle as O

# e4m3 encodings written out in tests/cooperative-matrix/fp8-cuda.slang:32-38
E4M3_ONE, E4M3_TWO, E4M3_THREE, E4M3_FOUR = 0x38, 0x40, 0x44, 0x48


def _identity_problem(input_type):
    """A = 16x16 identity, B = first row [1, 2, 3, 4, 0...]: D = B (int8.slang:5-8, fp8-cuda.slang:8-9)."""
    if input_type in (O.S8, O.U8):
        a = np.eye(16, dtype=np.uint8)
        b = np.zeros((16, 16), dtype=np.uint8)
        b[0, :4] = [1, 2, 3, 4]
    else:
        a = np.zeros((16, 16), dtype=np.uint8)
        a[np.arange(16), np.arange(16)] = E4M3_ONE
        b = np.zeros((16, 16), dtype=np.uint8)
        b[0, :4] = [E4M3_ONE, E4M3_TWO, E4M3_THREE, E4M3_FOUR]
    return a, b


KAT_IDENTITY = [(O.S8, O.ACC_S32, False), (O.S8, O.ACC_S32, True), (O.U8, O.ACC_S32, False), (O.U8, O.ACC_S32, True),
                (O.E4M3, O.ACC_F32, False), (O.E4M3, O.ACC_F16, False)]


def _half_bits(x):
    return np.asarray(x, dtype=np.float16).view(np.uint16)


def _bf16_bits(x):
    u = np.asarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


# ---- CPU: the oracle on the reference's known answers ----------------------------------------------
@pytest.mark.parametrize("input_type,acc_type,sat", KAT_IDENTITY)
def test_oracle_identity_known_answers(input_type, acc_type, sat):
    a, b = _identity_problem(input_type)
    d = O.mat_mul_add(input_type, acc_type, a, b, None, sat)
    assert list(d.ravel()[:4]) == [1, 2, 3, 4] and not d.ravel()[4:].any()


def test_oracle_mat_mul_add_known_answers():
    # ( 3.0 * 5.0 ) * 16 + 1.0 = 241.0 (mat-mul-add.slang:63-68)
    a, b = _half_bits(np.full((16, 16), 3.0)), _half_bits(np.full((16, 16), 5.0))
    d = O.mat_mul_add(O.F16, O.ACC_F32, a, b, np.full((16, 16), 1.0, np.float32))
    assert d.dtype == np.float32 and (d == 241.0).all()
    # ( 3 * 5 ) * 32 + 1 = 481 and the wrap-around of ( 3 * 5 ) * 32 + 0x7FFFFFFF = -2147483169 (:76-111)
    a8, b8 = np.full((16, 32), 3, np.uint8), np.full((32, 16), 5, np.uint8)
    assert (O.mat_mul_add(O.S8, O.ACC_S32, a8, b8, np.full((16, 16), 1, np.int32)) == 481).all()
    wrap = O.mat_mul_add(O.S8, O.ACC_S32, a8, b8, np.full((16, 16), 0x7FFFFFFF, np.int32))
    assert (wrap == -2147483169).all()
    sat = O.mat_mul_add(O.S8, O.ACC_S32, a8, b8, np.full((16, 16), 0x7FFFFFFF, np.int32), saturate=True)
    assert (sat == 0x7FFFFFFF).all()


def test_oracle_fp8_codes():
    assert list(O.decode_e4m3(np.array([E4M3_ONE, E4M3_TWO, E4M3_THREE, E4M3_FOUR, 0x7E, 0x01], np.uint8))) == \
        [1.0, 2.0, 3.0, 4.0, 448.0, 2.0 ** -9]
    assert list(O.decode_e5m2(np.array([0x3C, 0x40, 0x42, 0x7B], np.uint8))) == [1.0, 2.0, 3.0, 57344.0]
    assert list(O.encode_e4m3([1.0, 2.0, 3.0, 4.0, -0.5])) == [E4M3_ONE, E4M3_TWO, E4M3_THREE, E4M3_FOUR, 0xB0]


def test_entry_refuses_without_device():
    from slang_b200.lib import load
    from slang_b200.tile_mma import TileMmaDesc
    desc = TileMmaDesc(O.F16, O.ACC_F32, 16, 16, 16, 0, 0, 0, 16, 16, 16, 256, 256, 256, 0, 1)
    assert load().mlp_tile_mma(None, ctypes.byref(desc), 1, 1, 0, 1) == -2   # MLP_E_INVALID_ARG


# ---- GPU ------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def device():
    from slang_b200.api import Device
    d = Device(0)
    yield d
    d.destroy()


@pytest.mark.gpu
@pytest.mark.parametrize("input_type,acc_type,sat", KAT_IDENTITY)
def test_gpu_identity_known_answers(device, input_type, acc_type, sat):
    from slang_b200.tile_mma import tile_mma
    a, b = _identity_problem(input_type)
    d = tile_mma(device, a, b, None, input_type, acc_type, saturate=sat)
    assert d.shape == (16, 16)
    assert list(d.ravel()[:4]) == [1, 2, 3, 4] and not d.ravel()[4:].any()


@pytest.mark.gpu
def test_gpu_mat_mul_add_known_answers(device):
    from slang_b200.tile_mma import tile_mma
    a, b = _half_bits(np.full((16, 16), 3.0)), _half_bits(np.full((16, 16), 5.0))
    d = tile_mma(device, a, b, np.full((16, 16), 1.0, np.float32), O.F16, O.ACC_F32)
    assert (d == 241.0).all()
    d = tile_mma(device, _bf16_bits(np.full((16, 16), 3.0)), _bf16_bits(np.full((16, 16), 5.0)),
                 np.full((16, 16), 1.0, np.float32), O.BF16, O.ACC_F32)
    assert (d == 241.0).all()
    a8, b8 = np.full((16, 32), 3, np.uint8), np.full((32, 16), 5, np.uint8)
    for n in (16, 8):   # the m16n16k32 and m16n8k32 shapes of mat-mul-add.slang:76-111
        assert (tile_mma(device, a8, b8[:, :n], np.full((16, n), 1, np.int32), O.S8, O.ACC_S32) == 481).all()
        wrap = tile_mma(device, a8, b8[:, :n], np.full((16, n), 0x7FFFFFFF, np.int32), O.S8, O.ACC_S32)
        assert (wrap == -2147483169).all()
        sat = tile_mma(device, a8, b8[:, :n], np.full((16, n), 0x7FFFFFFF, np.int32), O.S8, O.ACC_S32, saturate=True)
        assert (sat == 0x7FFFFFFF).all()
    # the other end of the range: -128 * 127 summed onto INT32_MIN + 5
    an, bp = np.full((16, 32), -128, np.int8).view(np.uint8), np.full((32, 16), 127, np.uint8)
    lo = np.full((16, 16), -2 ** 31 + 5, np.int32)
    assert (tile_mma(device, an, bp, lo, O.S8, O.ACC_S32, saturate=True) == -2 ** 31).all()
    assert (tile_mma(device, an, bp, lo, O.S8, O.ACC_S32) == O.mat_mul_add(O.S8, O.ACC_S32, an, bp, lo)).all()


@pytest.mark.gpu
@pytest.mark.parametrize("input_type", [O.S8, O.U8])
@pytest.mark.parametrize("layouts", [(0, 0, 0), (1, 0, 1), (0, 1, 0), (1, 1, 1)])
def test_gpu_integer_products_exact(device, input_type, layouts):
    """Ragged sizes (rows past one 128-row block, K not a multiple of 32, N not a multiple of 16), a batch, every
    combination of layouts: bit-identical to the oracle."""
    from slang_b200.tile_mma import tile_mma
    rng = np.random.default_rng(11 + input_type + sum(layouts))
    count, m, n, k = 3, 130, 24, 100
    a = rng.integers(0, 256, (count, m, k), dtype=np.uint8)
    b = rng.integers(0, 256, (count, k, n), dtype=np.uint8)
    c = rng.integers(-2 ** 20, 2 ** 20, (count, m, n)).astype(np.int32)
    d = tile_mma(device, a, b, c, input_type, O.ACC_S32, a_layout=layouts[0], b_layout=layouts[1], cd_layout=layouts[2])
    ref = np.stack([O.mat_mul_add(input_type, O.ACC_S32, a[i], b[i], c[i]) for i in range(count)])
    assert d.dtype == np.int32 and (d == ref).all()


@pytest.mark.gpu
@pytest.mark.parametrize("input_type,acc_type", [(O.F16, O.ACC_F32), (O.BF16, O.ACC_F32), (O.F16, O.ACC_F16),
                                                 (O.E4M3, O.ACC_F32), (O.E5M2, O.ACC_F32), (O.E5M2, O.ACC_F16)])
def test_gpu_floating_products(device, input_type, acc_type):
    """Random problems over several K panels and both layouts.  Every product is exact in fp32; what the
    hardware's sum may differ in is the order and the alignment of its partial sums, so the bound is a few
    fp32 rounding steps of the sum of the magnitudes (plus one rounding to half for half accumulators).
    Small-integer inputs must come out exact."""
    from slang_b200.tile_mma import tile_mma
    rng = np.random.default_rng(5 + input_type * 3 + acc_type)
    count, m, n, k = 2, 200, 72, 176
    if input_type == O.F16:
        a, b = _half_bits(rng.uniform(-1, 1, (count, m, k))), _half_bits(rng.uniform(-1, 1, (count, k, n)))
    elif input_type == O.BF16:
        a, b = _bf16_bits(rng.uniform(-1, 1, (count, m, k))), _bf16_bits(rng.uniform(-1, 1, (count, k, n)))
    else:
        # random finite fp8 bit patterns of moderate magnitude: exponent field at most 9 keeps every sum finite in half
        def fp8(shape):
            bits = rng.integers(0, 256, shape, dtype=np.uint8)
            if input_type == O.E4M3:
                e = (bits >> 3) & 0xF
                bits = np.where(e > 9, bits & 0xC7, bits).astype(np.uint8)   # exponent cleared: subnormal range
            else:
                e = (bits >> 2) & 0x1F
                bits = np.where(e > 16, bits & 0x83, bits).astype(np.uint8)
            return bits
        a, b = fp8((count, m, k)), fp8((count, k, n))
    acc_dt = np.float16 if acc_type == O.ACC_F16 else np.float32
    c = rng.uniform(-1, 1, (count, m, n)).astype(acc_dt)
    for layouts in ((0, 0, 0), (1, 1, 1)):
        d = tile_mma(device, a, b, c, input_type, acc_type, a_layout=layouts[0], b_layout=layouts[1], cd_layout=layouts[2])
        for i in range(count):
            ad, bd = O.decode(input_type, a[i]), O.decode(input_type, b[i])
            exact = ad @ bd + c[i].astype(np.float64)
            mag = np.abs(ad) @ np.abs(bd) + np.abs(c[i].astype(np.float64))
            tol = 8 * 2.0 ** -24 * mag + (2.0 ** -11 * np.abs(exact) + 2.0 ** -24 if acc_type == O.ACC_F16 else 0)
            assert d[i].dtype == acc_dt
            assert (np.abs(d[i].astype(np.float64) - exact) <= tol).all(), np.max(np.abs(d[i] - exact) / mag)
    # small integers: exact whatever the order
    ai = rng.integers(-3, 4, (m, k)).astype(np.float64)
    bi = rng.integers(-3, 4, (k, n)).astype(np.float64)
    if input_type == O.F16:
        ab, bb = _half_bits(ai), _half_bits(bi)
    elif input_type == O.BF16:
        ab, bb = _bf16_bits(ai), _bf16_bits(bi)
    elif input_type == O.E4M3:
        ab, bb = O.encode_e4m3(ai), O.encode_e4m3(bi)
    else:
        ab, bb = (_half_bits(ai) >> 8).astype(np.uint8), (_half_bits(bi) >> 8).astype(np.uint8)
    d = tile_mma(device, ab, bb, None, input_type, acc_type)
    assert (d.astype(np.float64) == ai @ bi).all()


@pytest.mark.gpu
def test_gpu_refusals(device):
    from slang_b200.lib import MlpError
    from slang_b200.tile_mma import tile_mma
    a, b = np.zeros((16, 16), np.uint8), np.zeros((16, 16), np.uint8)
    for kwargs in (dict(input_type=O.E4M3, acc_type=O.ACC_S32), dict(input_type=O.S8, acc_type=O.ACC_F32),
                   dict(input_type=O.E4M3, acc_type=O.ACC_F32, saturate=True)):
        with pytest.raises(MlpError) as e:
            tile_mma(device, a, b, None, **kwargs)
        assert e.value.code == -2
    with pytest.raises(MlpError):
        tile_mma(device, np.zeros((16, 16), np.uint16), np.zeros((16, 16), np.uint16), None, O.BF16, O.ACC_F16)
    with pytest.raises(MlpError):
        tile_mma(device, np.zeros((16, 16), np.uint8), np.zeros((16, 264), np.uint8), None, O.U8, O.ACC_S32)
    device.wait()
