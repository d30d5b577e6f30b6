"""Host side of the permutohedral-lattice encoder (include/slang_b200_permuto.h).

Mirrors PermutoEncoder of the reference's neural module (source/standard-modules/neural/
permuto-encoder.slang): hyper-parameters prepared per level on the host, `encode` for a batch of
positions, and the reverse pass that accumulates the feature-table gradient."""
import ctypes

import numpy as np

from .lib import check, load

MAX_DIMS, MAX_LEVELS = 4, 32
HASH_PRIME, HASH_COHERENT_PRIME, HASH_REVERSED_PRIME, HASH_RNG, HASH_BASE_CONVERT = range(5)


class PermutoLevelInfo(ctypes.Structure):
    _fields_ = [("level_index", ctypes.c_uint32), ("table_offset", ctypes.c_uint32), ("table_size", ctypes.c_uint32),
                ("scale", ctypes.c_float), ("scales_per_dim", ctypes.c_float * MAX_DIMS),
                ("shifts_per_dim", ctypes.c_float * MAX_DIMS)]


class PermutoConfig(ctypes.Structure):
    _fields_ = [("dims", ctypes.c_int32), ("features_per_entry", ctypes.c_int32), ("log2_hashmap_size", ctypes.c_int32),
                ("n_levels", ctypes.c_int32), ("dtype", ctypes.c_int32), ("max_level", ctypes.c_float),
                ("levels", PermutoLevelInfo * MAX_LEVELS)]

    @property
    def n_features(self):
        return self.n_levels * self.features_per_entry

    @property
    def table_values(self):
        return self.n_levels * (1 << self.log2_hashmap_size) * self.features_per_entry


def prepare(dims, features_per_entry, log2_hashmap_size, n_levels, base_scale, log2_per_level_scale,
            max_level_ratio=1.1, seed=1337, dtype=0):
    cfg = PermutoConfig()
    check(load().mlp_permuto_prepare(dims, features_per_entry, log2_hashmap_size, n_levels, base_scale,
                                     log2_per_level_scale, max_level_ratio, seed, dtype, ctypes.byref(cfg)))
    return cfg


def grid_hash(hash_type, position_grid):
    p = (ctypes.c_uint32 * len(position_grid))(*position_grid)
    return int(load().mlp_grid_hash(hash_type, len(position_grid), p))


class PermutoEncoder:
    """Encoder bound to a device: buffers are device addresses (ints)."""

    def __init__(self, device, cfg):
        self.device, self.cfg = device, cfg

    def encode(self, positions, table, out, count):
        check(load().mlp_permuto_encode(self.device.handle, ctypes.byref(self.cfg), positions, table, out, count))

    def backward(self, positions, table, d_out, d_table, d_positions, count):
        check(load().mlp_permuto_backward(self.device.handle, ctypes.byref(self.cfg), positions, table, d_out, d_table,
                                          d_positions or 0, count))
