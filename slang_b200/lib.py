"""Loads the C-ABI shared library and declares its entry points for ctypes.

There is no fallback: if the library has not been built, or no sm_100 device is present when a device
handle is requested, the caller gets an exception.
"""
import ctypes
import os

from .config import MlpConfig

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libslang_b200_mlp.so")

# Every symbol include/slang_b200_mlp.h declares.
EXPORTS = [
    "mlp_device_create", "mlp_device_create_on_stream", "mlp_device_destroy", "mlp_wait",
    "mlp_buffer_create", "mlp_buffer_wrap", "mlp_buffer_destroy", "mlp_buffer_address", "mlp_buffer_clear",
    "mlp_buffer_read", "mlp_buffer_write",
    "mlp_kernel_get", "mlp_kernel_load", "mlp_kernel_get_for_config", "mlp_kernel_destroy", "mlp_kernel_implementation",
    "mlp_dispatch", "mlp_device_launch_count", "mlp_param_layout", "mlp_last_error_string",
    "mlp_learn_gradient_ordered_noalloc", "mlp_selftest_bounded_wait", "mlp_tile_mma",
    "mlp_layout_sizes", "mlp_layout_to_optimal", "mlp_layout_to_portable",
    "mlp_matrix_size", "mlp_matrix_convert",
    "mlp_permuto_prepare", "mlp_grid_hash", "mlp_permuto_encode", "mlp_permuto_backward",
    "mlp_comm_unique_id", "mlp_comm_init", "mlp_comm_destroy", "mlp_allreduce_grads", "mlp_comm_wait",
]

# Stand-alone device module with the literal example entry points (built next to the library).
CUBIN_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "mlp_training_kernels.cubin")

_lib = None


class MlpError(RuntimeError):
    def __init__(self, code, text):
        super().__init__("mlp error %d: %s" % (code, text))
        self.code = code


def load():
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError("%s is missing: run `python -m slang_b200.build` (there is no fallback path)" % LIB_PATH)
    L = ctypes.CDLL(LIB_PATH)
    vp, u64, u32, i32, sz = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int32, ctypes.c_size_t
    pp = ctypes.POINTER(ctypes.c_void_p)
    L.mlp_device_create.argtypes = [i32, pp]
    L.mlp_device_create_on_stream.argtypes = [i32, vp, pp]
    L.mlp_device_destroy.argtypes = [vp]
    L.mlp_wait.argtypes = [vp]
    L.mlp_buffer_create.argtypes = [vp, sz, vp, pp]
    L.mlp_buffer_wrap.argtypes = [vp, u64, sz, pp]
    L.mlp_buffer_destroy.argtypes = [vp]
    L.mlp_buffer_address.argtypes = [vp]
    L.mlp_buffer_address.restype = u64
    L.mlp_buffer_clear.argtypes = [vp, vp, sz, sz]
    L.mlp_buffer_read.argtypes = [vp, vp, sz, sz, vp]
    L.mlp_buffer_write.argtypes = [vp, vp, sz, sz, vp]
    L.mlp_kernel_get.argtypes = [vp, ctypes.c_char_p, pp]
    f32 = ctypes.c_float
    L.mlp_permuto_prepare.argtypes = [i32, i32, i32, i32, f32, f32, f32, u32, i32, vp]
    L.mlp_grid_hash.argtypes = [i32, i32, vp]
    L.mlp_grid_hash.restype = u32
    L.mlp_permuto_encode.argtypes = [vp, vp, u64, u64, u64, u32]
    L.mlp_permuto_backward.argtypes = [vp, vp, u64, u64, u64, u64, u64, u32]
    L.mlp_matrix_size.argtypes = [u32, u32, i32, i32, u64, ctypes.POINTER(u64)]
    L.mlp_matrix_convert.argtypes = [vp, u64, vp, u64, vp, u32]
    L.mlp_comm_unique_id.argtypes = [vp, sz]
    L.mlp_comm_init.argtypes = [vp, i32, i32, vp, sz, pp]
    L.mlp_comm_destroy.argtypes = [vp]
    L.mlp_allreduce_grads.argtypes = [vp, vp, u64, sz, u64, u32]
    L.mlp_comm_wait.argtypes = [vp, vp, u32]
    L.mlp_kernel_load.argtypes = [vp, ctypes.c_char_p, sz, ctypes.c_char_p, pp]
    L.mlp_kernel_get_for_config.argtypes = [vp, ctypes.POINTER(MlpConfig), ctypes.c_char_p, pp]
    L.mlp_kernel_destroy.argtypes = [vp]
    L.mlp_kernel_implementation.argtypes = [vp]
    L.mlp_kernel_implementation.restype = ctypes.c_char_p
    L.mlp_dispatch.argtypes = [vp, vp, vp, sz, u32, u32, u32]
    L.mlp_device_launch_count.argtypes = [vp]
    L.mlp_device_launch_count.restype = u64
    L.mlp_param_layout.argtypes = [ctypes.POINTER(MlpConfig), ctypes.POINTER(ctypes.c_int64),
                                   ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64)]
    L.mlp_last_error_string.restype = ctypes.c_char_p
    L.mlp_layout_sizes.argtypes = [vp, ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64)]
    L.mlp_layout_to_optimal.argtypes = [vp, vp, u64, u64]
    L.mlp_layout_to_portable.argtypes = [vp, vp, u64, u64]
    L.mlp_selftest_bounded_wait.argtypes = [vp, u32]
    L.mlp_tile_mma.argtypes = [vp, vp, u64, u64, u64, u64]
    L.mlp_learn_gradient_ordered_noalloc.argtypes = [i32, vp, ctypes.POINTER(MlpConfig), vp]
    for name in EXPORTS:
        fn = getattr(L, name)
        if fn.restype is ctypes.c_int:
            fn.restype = i32
    _lib = L
    return L


def check(rc):
    if rc != 0:
        raise MlpError(rc, load().mlp_last_error_string().decode("utf-8", "replace"))
