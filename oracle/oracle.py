"""ctypes front end of the CPU oracle (oracle/mlp_oracle.cpp).

TEST INFRASTRUCTURE ONLY.  Tests, the smoke check and the benchmark's CPU baseline may import this
module; the product package must not.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build(force=False):
    so = os.path.join(_HERE, "libmlp_oracle.so")
    srcs = [os.path.join(_HERE, f) for f in ("mlp_oracle.cpp", "permuto_oracle.cpp")]
    if force or not os.path.exists(so) or os.path.getmtime(so) < max(os.path.getmtime(f) for f in srcs):
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B" if force else "-s"])
    return so


def build_ref():
    """oracle/_ref/libref_prelude.so: the reference's CPU prelude behind a C wrapper, compiled from the
    reference tree where it lies (a no-op that keeps a prebuilt library where the tree is absent)."""
    subprocess.check_call(["make", "-C", _HERE, "-s", "ref"])
    return os.path.join(_HERE, "_ref", "libref_prelude.so")


def lib():
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(build())
        _LIB.mlp_oracle_activation.restype = ctypes.c_float
        _LIB.mlp_oracle_activation.argtypes = [ctypes.c_int, ctypes.c_float, ctypes.c_float]
        _LIB.mlp_oracle_activation_deriv.restype = ctypes.c_float
        _LIB.mlp_oracle_activation_deriv.argtypes = [ctypes.c_int, ctypes.c_float, ctypes.c_float]
        _LIB.mlp_oracle_example_float_to_half.restype = ctypes.c_uint16
        _LIB.mlp_oracle_example_float_to_half.argtypes = [ctypes.c_float]
    return _LIB


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def param_layout(cfg):
    w = (ctypes.c_int64 * 8)()
    b = (ctypes.c_int64 * 8)()
    t = ctypes.c_int64()
    rc = lib().mlp_oracle_param_layout(ctypes.byref(cfg), w, b, ctypes.byref(t))
    assert rc == 0
    return list(w)[:cfg.n_layers], list(b)[:cfg.n_layers], t.value


def forward(cfg, params, inputs, count, acc_mode=0):
    out = np.zeros((count, cfg.dims[cfg.n_layers]), dtype=np.float32)
    rc = lib().mlp_oracle_forward(ctypes.byref(cfg), _p(params), _p(inputs), ctypes.c_int64(count), _p(out),
                                  ctypes.c_int(acc_mode))
    assert rc == 0
    return out


def learn_gradient(cfg, params, grads, inputs, targets, count, loss_words=None, acc_mode=0, n_threads=1):
    """grads (float32, padded layout) is accumulated in place; returns the two loss words."""
    assert grads.dtype == np.float32
    if loss_words is None:
        loss_words = np.zeros(2, dtype=np.uint32)
    rc = lib().mlp_oracle_learn_gradient(ctypes.byref(cfg), _p(params), _p(grads), _p(inputs), _p(targets),
                                         ctypes.c_int64(count), _p(loss_words), ctypes.c_int(acc_mode),
                                         ctypes.c_int(n_threads))
    assert rc == 0
    return loss_words


def adjust_parameters(cfg, states, params, grads, count=None):
    if count is None:
        count = grads.size
    rc = lib().mlp_oracle_adjust_parameters(ctypes.byref(cfg), _p(states), _p(params), _p(grads),
                                            ctypes.c_int64(count))
    assert rc == 0


def activation(act, alpha, x):
    return float(lib().mlp_oracle_activation(act, alpha, x))


def activation_deriv(act, alpha, x):
    return float(lib().mlp_oracle_activation_deriv(act, alpha, x))


def example_float_to_half(v):
    return int(lib().mlp_oracle_example_float_to_half(v))


def learn_gradient_inputs(cfg, params, grads, inputs, targets, count, loss_words=None):
    """learn_gradient that also returns d loss / d inputs, [count][dims[0]] fp32."""
    assert grads.dtype == np.float32
    ig = np.zeros((count, cfg.dims[0]), dtype=np.float32)
    rc = lib().mlp_oracle_learn_gradient_inputs(ctypes.byref(cfg), _p(params), _p(grads), _p(inputs), _p(targets),
                                                ctypes.c_int64(count), _p(loss_words), _p(ig))
    assert rc == 0
    return ig


def example_learn_gradient(network_ptrs, loss_word, inputs, count):
    """network_ptrs: uint64 array [2][4] of host addresses (weights, weightsGrad, biases, biasesGrad)."""
    rc = lib().mlp_oracle_example_learn_gradient(_p(network_ptrs), _p(loss_word), _p(inputs), ctypes.c_uint32(count))
    assert rc == 0


def example_adjust_parameters(states, params, grads, count):
    rc = lib().mlp_oracle_example_adjust_parameters(_p(states), _p(params), _p(grads), ctypes.c_uint32(count))
    assert rc == 0


# ---- the example kernels behind the CPU compute entry-point calling convention ------------------
class _Uint3(ctypes.Structure):
    _fields_ = [("x", ctypes.c_uint32), ("y", ctypes.c_uint32), ("z", ctypes.c_uint32)]


class ComputeVaryingInput(ctypes.Structure):
    """prelude/slang-cpp-types.h:1343-1347"""
    _fields_ = [("startGroupID", _Uint3), ("endGroupID", _Uint3)]


class ComputeThreadVaryingInput(ctypes.Structure):
    """prelude/slang-cpp-types.h:1337-1341"""
    _fields_ = [("groupID", _Uint3), ("groupThreadID", _Uint3)]


class EntryParams(ctypes.Structure):
    """Packed uniform parameters of either example kernel: three addresses and a count (28 bytes used)."""
    _fields_ = [("p0", ctypes.c_uint64), ("p1", ctypes.c_uint64), ("p2", ctypes.c_uint64), ("count", ctypes.c_uint32)]


def cpu_entry_range(name, params, start_group, end_group):
    """Calls `name` (learnGradient / adjustParameters) over the groups [start_group, end_group)."""
    v = ComputeVaryingInput(_Uint3(start_group, 0, 0), _Uint3(end_group, 1, 1))
    getattr(lib(), name)(ctypes.byref(v), ctypes.byref(params), None)


def cpu_entry_group(name, params, group):
    v = ComputeVaryingInput(_Uint3(group, 0, 0), _Uint3(group + 1, 1, 1))
    getattr(lib(), name + "_Group")(ctypes.byref(v), ctypes.byref(params), None)


def cpu_entry_thread(name, params, group, thread):
    v = ComputeThreadVaryingInput(_Uint3(group, 0, 0), _Uint3(thread, 0, 0))
    getattr(lib(), name + "_Thread")(ctypes.byref(v), ctypes.byref(params), None)


def example_coopvec_learn_gradient(network_ptrs, loss_word, inputs, count):
    """The cooperative-vector example's learnGradient; weightsGrad points at 16x16 training-optimal tiles."""
    rc = lib().mlp_oracle_example_coopvec_learn_gradient(_p(network_ptrs), _p(loss_word), _p(inputs), ctypes.c_uint32(count))
    assert rc == 0
