"""ctypes front end of the permutohedral-encoder oracle (oracle/permuto_oracle.cpp).  TEST INFRASTRUCTURE ONLY."""
import ctypes

import numpy as np

from .oracle import _p, lib


def _lib():
    L = lib()
    L.permuto_oracle_grid_hash.restype = ctypes.c_uint32
    return L


def grid_hash(hash_type, position_grid):
    p = (ctypes.c_uint32 * len(position_grid))(*position_grid)
    return int(_lib().permuto_oracle_grid_hash(hash_type, len(position_grid), p))


def prepare(cfg_type, dims, features, log2_size, n_levels, base_scale, log2_per_level_scale, max_level_ratio=1.1,
            seed=1337, dtype=0):
    """cfg_type: the ctypes struct class laid out like MlpPermutoConfig."""
    cfg = cfg_type()
    rc = _lib().permuto_oracle_prepare(dims, features, log2_size, n_levels, ctypes.c_float(base_scale),
                                       ctypes.c_float(log2_per_level_scale), ctypes.c_float(max_level_ratio),
                                       ctypes.c_uint32(seed), dtype, ctypes.byref(cfg))
    assert rc == 0
    return cfg


def encode(cfg, positions, table):
    positions = np.ascontiguousarray(positions, dtype=np.float32)
    count = positions.shape[0]
    out = np.zeros((count, cfg.n_levels * cfg.features_per_entry), dtype=table.dtype)
    rc = _lib().permuto_oracle_encode(ctypes.byref(cfg), _p(positions), _p(table), _p(out), ctypes.c_uint32(count))
    assert rc == 0
    return out


def backward(cfg, positions, table, d_out, d_table):
    """Adds into d_table in place; returns the position gradients."""
    positions = np.ascontiguousarray(positions, dtype=np.float32)
    count = positions.shape[0]
    dpos = np.zeros((count, cfg.dims), dtype=np.float32)
    rc = _lib().permuto_oracle_backward(ctypes.byref(cfg), _p(positions), _p(table), _p(np.ascontiguousarray(d_out)),
                                        _p(d_table), _p(dpos), ctypes.c_uint32(count))
    assert rc == 0
    return dpos
