"""The oracle's number formats and elementary functions against the reference's own CPU prelude.

oracle/_ref/libref_prelude.so is the reference's prelude/slang-cpp-prelude.h behind a C wrapper
(oracle/ref_prelude_check.cpp), compiled from the reference tree where it lies; the built library travels
with the working copy, the sources do not.  The example kernels cannot be built from the reference (they
need its compiler and a SPIR-V target), so what is pinned here is the arithmetic they are made of on the
reference's CPU target: half conversions, half add and multiply, exp / sin / cos / tanh / sqrt.
"""
import ctypes
import os
import subprocess

import numpy as np
import pytest

from oracle import oracle
from slang_b200 import config as C

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_DIR = os.path.join(os.path.dirname(HERE), "oracle")
REF_SO = os.path.join(ORACLE_DIR, "_ref", "libref_prelude.so")


@pytest.fixture(scope="module")
def ref():
    if os.path.exists("/root/reference/prelude/slang-cpp-prelude.h"):
        subprocess.check_call(["make", "-C", ORACLE_DIR, "-s", "ref"])
    if not os.path.exists(REF_SO):
        pytest.skip("oracle/_ref/libref_prelude.so is not built and the reference tree is not present")
    lib = ctypes.CDLL(REF_SO)
    for name in ("ref_f16tof32", "ref_F32_exp", "ref_F32_sin", "ref_F32_cos", "ref_F32_tanh", "ref_F32_sqrt"):
        getattr(lib, name).restype = ctypes.c_float
    for name in ("ref_F32_exp", "ref_F32_sin", "ref_F32_cos", "ref_F32_tanh", "ref_F32_sqrt", "ref_f32tof16", "ref_half_from_float"):
        getattr(lib, name).argtypes = [ctypes.c_float]
    lib.ref_f16tof32.argtypes = [ctypes.c_uint]
    return lib


def test_half_to_float_is_exact_for_every_pattern(ref):
    bits = np.arange(65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.array([ref.ref_f16tof32(int(b)) for b in bits], dtype=np.float32)
    finite = np.isfinite(want)
    assert np.array_equal(got[finite].view(np.uint32), want[finite].view(np.uint32))
    assert np.all(np.isnan(got[np.isnan(want)])) and np.array_equal(np.isinf(got), np.isinf(want))


def test_float_to_half_matches_the_oracle(ref):
    """The prelude's `half` is the compiler's _Float16 with GCC 12 or later (IEEE round to nearest even, what
    the oracle and the GPU's conversion instructions do).  Its own f32tof16 (the fallback type's conversion,
    also the example host's floatToHalf) truncates to eleven bits and adds the dropped bit back: it differs
    from round-to-nearest-even exactly where the oracle's test of the example's host conversion says it
    does, and nowhere among values that are already halves."""
    rng = np.random.default_rng(11)
    v = np.concatenate([rng.normal(size=200000), rng.uniform(-70000, 70000, 50000), rng.normal(size=50000) * 1e-6,
                        np.array([0.0, -0.0, 1.0, 65504.0, 65520.0, 1e-8, 6e-8, 6.1e-5])]).astype(np.float32)
    out = np.zeros(v.size, dtype=np.uint16)
    oracle.lib().mlp_oracle_convert_from_f32(C.F16, v.ctypes.data_as(ctypes.c_void_p), out.ctypes.data_as(ctypes.c_void_p), ctypes.c_int64(v.size))
    assert ref.ref_half_is_builtin() == 1
    got = np.array([ref.ref_half_from_float(float(x)) for x in v[:60000]], dtype=np.uint16)
    assert np.array_equal(got, out[:60000])
    # the fallback conversion: equal to the example's host conversion that the oracle restates
    fb = np.array([ref.ref_f32tof16(float(x)) for x in v[:60000]], dtype=np.uint16)
    ex = np.array([oracle.example_float_to_half(float(x)) for x in v[:60000]], dtype=np.uint16)
    normal = np.abs(v[:60000]) < 65000
    assert np.array_equal(fb[normal], ex[normal])
    # and it agrees with round-to-nearest-even except on a small share of values (dropped bit set, rounds up)
    assert np.mean(fb[normal] != out[:60000][normal]) < 0.51


def test_half_arithmetic_rounds_every_operation(ref):
    """a + b and a * b on halves: one rounding per operation, as the oracle's -fexcess-precision=16 build does."""
    rng = np.random.default_rng(12)
    a = rng.normal(size=20000).astype(np.float16)
    b = (rng.normal(size=20000) * 3).astype(np.float16)
    add = np.array([ref.ref_half_add(int(x), int(y)) for x, y in zip(a.view(np.uint16), b.view(np.uint16))], dtype=np.uint16)
    mul = np.array([ref.ref_half_mul(int(x), int(y)) for x, y in zip(a.view(np.uint16), b.view(np.uint16))], dtype=np.uint16)
    assert np.array_equal(add, (a + b).view(np.uint16))
    assert np.array_equal(mul, (a * b).view(np.uint16))


def test_elementary_functions_are_the_same_calls(ref):
    """F32_exp / F32_sin / F32_cos / F32_tanh / F32_sqrt against the oracle's activations built on them."""
    rng = np.random.default_rng(13)
    xs = np.concatenate([rng.normal(size=20000) * 3, rng.uniform(-50, 50, 5000)]).astype(np.float32)
    for act, fn, dfn in ((C.ACT_EXP, ref.ref_F32_exp, ref.ref_F32_exp), (C.ACT_SINE, ref.ref_F32_sin, ref.ref_F32_cos),
                         (C.ACT_TANH, ref.ref_F32_tanh, None)):
        for x in xs[:8000]:
            x = float(x)
            assert oracle.activation(act, 0.0, x) == fn(x) or (np.isnan(fn(x)) and np.isnan(oracle.activation(act, 0.0, x)))
            if dfn is not None:
                assert oracle.activation_deriv(act, 0.0, x) == dfn(x) or np.isinf(dfn(x))
    for x in (0.0, 1.0, 2.0, 1e-8, 12345.678):
        assert ref.ref_F32_sqrt(x) == np.float32(np.sqrt(np.float32(x)))
