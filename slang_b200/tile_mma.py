"""Host mirror of the cooperative-matrix multiply-add entry (include/slang_b200_tile_mma.h): D = A . B + C on the
tcgen05 tensor cores, the counterpart of linalg::coopMatMulAdd (prelude/slang-cuda-prelude.h:8599-8642)."""
import ctypes

import numpy as np

from .lib import check, load

TILE_F16, TILE_BF16, TILE_S8, TILE_U8, TILE_E4M3, TILE_E5M2 = 1, 2, 3, 4, 5, 6
ACC_F32, ACC_F16, ACC_S32 = 0, 1, 2
ROW_MAJOR, COLUMN_MAJOR = 0, 1

_INPUT_BYTES = {TILE_F16: 2, TILE_BF16: 2, TILE_S8: 1, TILE_U8: 1, TILE_E4M3: 1, TILE_E5M2: 1}
_ACC_DTYPE = {ACC_F32: np.float32, ACC_F16: np.float16, ACC_S32: np.int32}


class TileMmaDesc(ctypes.Structure):
    """MlpTileMmaDesc."""
    _fields_ = [("input_type", ctypes.c_int32), ("acc_type", ctypes.c_int32),
                ("m", ctypes.c_int32), ("n", ctypes.c_int32), ("k", ctypes.c_int32),
                ("a_layout", ctypes.c_int32), ("b_layout", ctypes.c_int32), ("cd_layout", ctypes.c_int32),
                ("lda", ctypes.c_int64), ("ldb", ctypes.c_int64), ("ldcd", ctypes.c_int64),
                ("stride_a", ctypes.c_int64), ("stride_b", ctypes.c_int64), ("stride_cd", ctypes.c_int64),
                ("saturate", ctypes.c_int32), ("count", ctypes.c_int32)]


def tile_mma_raw(device, desc, a_address, b_address, c_address, d_address):
    """mlp_tile_mma on device addresses."""
    check(load().mlp_tile_mma(device.handle, ctypes.byref(desc), a_address, b_address, c_address, d_address))


def tile_mma(device, a_bits, b_bits, c, input_type, acc_type, saturate=False, a_layout=ROW_MAJOR, b_layout=ROW_MAJOR,
             cd_layout=ROW_MAJOR):
    """D = A . B + C for a batch of problems held in numpy arrays.

    a_bits [count, M, K] and b_bits [count, K, N] hold the stored bits of the input type (uint16 for the 16-bit
    types, uint8 / int8 for the 8-bit ones) in LOGICAL index order; the layout arguments choose how they are
    laid out in device memory.  c is [count, M, N] of the accumulator type, or None.  Returns D like c."""
    a_bits, b_bits = np.asarray(a_bits), np.asarray(b_bits)
    if a_bits.ndim == 2:
        a_bits, b_bits = a_bits[None], b_bits[None]
        c = None if c is None else np.asarray(c)[None]
        squeeze = True
    else:
        squeeze = False
    count, m, k = a_bits.shape
    n = b_bits.shape[2]
    assert b_bits.shape[:2] == (count, k) and a_bits.dtype.itemsize == _INPUT_BYTES[input_type] == b_bits.dtype.itemsize
    acc_dt = _ACC_DTYPE[acc_type]

    def lay(x, layout):
        return np.ascontiguousarray(x if layout == ROW_MAJOR else x.transpose(0, 2, 1))

    a_host = lay(a_bits, a_layout)
    a_dev = device.create_buffer(a_host.nbytes, a_host)
    b_host = lay(b_bits, b_layout)
    b_dev = device.create_buffer(b_host.nbytes, b_host)
    d_host = np.zeros((count, m, n) if cd_layout == ROW_MAJOR else (count, n, m), dtype=acc_dt)
    d_dev = device.create_buffer(d_host.nbytes, d_host)
    c_dev = None
    if c is not None:
        c = np.asarray(c, dtype=acc_dt)
        assert c.shape == (count, m, n)
        c_host = lay(c, cd_layout)
        c_dev = device.create_buffer(c_host.nbytes, c_host)
    desc = TileMmaDesc(input_type, acc_type, m, n, k, a_layout, b_layout, cd_layout,
                       k if a_layout == ROW_MAJOR else m, n if b_layout == ROW_MAJOR else k,
                       n if cd_layout == ROW_MAJOR else m, m * k, k * n, m * n, 1 if saturate else 0, count)
    tile_mma_raw(device, desc, a_dev.address, b_dev.address, c_dev.address if c_dev else 0, d_dev.address)
    device.wait()
    out = d_dev.read(acc_dt).reshape(d_host.shape)
    for buf in (a_dev, b_dev, d_dev, c_dev):
        if buf is not None:
            buf.destroy()
    if cd_layout != ROW_MAJOR:
        out = out.transpose(0, 2, 1)
    out = np.ascontiguousarray(out)
    return out[0] if squeeze else out
