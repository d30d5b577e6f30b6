"""CPU restatement of the cooperative-matrix multiply-add D = A . B + C (TEST INFRASTRUCTURE ONLY).

Follows linalg::coopMatMulAdd as the reference implements it on CUDA (prelude/slang-cuda-prelude.h:8599-8642):
integer inputs accumulate in int32, wrapping, or clamped to the int32 range with saturatingAccumulation
(:8342-8463); floating inputs (f16, bf16, e4m3, e5m2; :8145-8340, :8465-8590) accumulate in fp32, or in half when
the accumulator fragment is half.  The floating products are exact in fp32; the order and the internal width
of the hardware's sum are not specified, so this restatement sums in float64 and rounds once: integer-valued
cases are exact, the others agree with any fp32 summation order to a few units in the last place of the
largest partial sum.  Pinned on the known answers of tests/cooperative-matrix/*.slang (tests/test_tile_mma.py).
"""
import numpy as np

F16, BF16, S8, U8, E4M3, E5M2 = 1, 2, 3, 4, 5, 6
ACC_F32, ACC_F16, ACC_S32 = 0, 1, 2


def decode_e4m3(bits):
    """OCP FP8 E4M3 (finite-only variant: no infinities, 0x7f / 0xff are NaN), the format of __nv_fp8_e4m3."""
    b = np.asarray(bits, dtype=np.uint8).astype(np.int32)
    sign = np.where(b & 0x80, -1.0, 1.0)
    e = (b >> 3) & 0xF
    m = b & 7
    v = np.where(e == 0, m / 8.0 * 2.0 ** -6, (1.0 + m / 8.0) * 2.0 ** (e - 7.0))
    v = np.where((e == 15) & (m == 7), np.nan, v)
    return (sign * v).astype(np.float64)


def decode_e5m2(bits):
    """OCP FP8 E5M2 (IEEE-like: infinities and NaNs), the format of __nv_fp8_e5m2: the top byte of a half."""
    b = np.asarray(bits, dtype=np.uint8).astype(np.uint16) << 8
    return b.view(np.float16).astype(np.float64)


def encode_e4m3(values):
    """Nearest representable E4M3 bits (ties to even) of finite values within +-448; helper for building inputs."""
    table = decode_e4m3(np.arange(256, dtype=np.uint8))
    order = [i for i in range(256) if not np.isnan(table[i]) and not (i == 0x80)]
    grid = np.array([table[i] for i in order])
    out = np.empty(np.shape(values), dtype=np.uint8)
    flat = np.asarray(values, dtype=np.float64).ravel()
    res = out.ravel()
    for j, v in enumerate(flat):
        d = np.abs(grid - v)
        best = np.flatnonzero(d == d.min())
        pick = best[0] if len(best) == 1 else [i for i in best if (order[i] & 1) == 0][0]
        res[j] = order[pick]
    return out


def decode(input_type, bits):
    bits = np.asarray(bits)
    if input_type == F16:
        return bits.view(np.float16).astype(np.float64)
    if input_type == BF16:
        return (bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    if input_type == S8:
        return bits.view(np.int8).astype(np.int64)
    if input_type == U8:
        return bits.view(np.uint8).astype(np.int64)
    if input_type == E4M3:
        return decode_e4m3(bits.view(np.uint8))
    if input_type == E5M2:
        return decode_e5m2(bits.view(np.uint8))
    raise ValueError("input type")


def mat_mul_add(input_type, acc_type, a_bits, b_bits, c=None, saturate=False, k_step=None):
    """a_bits [M, K], b_bits [K, N] stored bits; c [M, N] of the accumulator type or None.

    k_step: with saturation, the K extent after which the running sum is clamped (the reference clamps after
    every 16-deep mma.sync; any value gives the same result while no intermediate sum leaves the int32 range)."""
    a, b = decode(input_type, a_bits), decode(input_type, b_bits)
    m, k = a.shape
    n = b.shape[1]
    if acc_type == ACC_S32:
        acc = np.zeros((m, n), dtype=np.int64) if c is None else np.asarray(c, dtype=np.int32).astype(np.int64)
        step = k_step or k
        for k0 in range(0, k, step):
            acc = acc + a[:, k0:k0 + step] @ b[k0:k0 + step]
            if saturate:
                acc = np.clip(acc, -2 ** 31, 2 ** 31 - 1)
            else:
                acc = ((acc + 2 ** 31) % 2 ** 32) - 2 ** 31
        return acc.astype(np.int32)
    acc = a @ b
    if c is not None:
        acc = acc + np.asarray(c).astype(np.float64)
    return acc.astype(np.float16 if acc_type == ACC_F16 else np.float32)
