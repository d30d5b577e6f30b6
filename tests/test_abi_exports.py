"""CPU-side checks of the boundary: the library loads, exports every declared symbol, and refuses to
work without a GPU instead of falling back."""
import ctypes
import os
import re

import numpy as np
import pytest

from slang_b200 import config as C
from slang_b200 import lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_header_symbols_are_exported():
    inc = os.path.join(ROOT, "include")
    text = "".join(open(os.path.join(inc, f)).read() for f in sorted(os.listdir(inc)) if f.endswith(".h"))
    declared = set(re.findall(r"\b(mlp_[a-z_]+)\s*\(", text))
    assert declared, "no declarations found"
    L = lib.load()
    missing = [n for n in sorted(declared) if not hasattr(L, n)]
    assert not missing, missing
    assert declared == set(lib.EXPORTS)


def test_config_struct_matches_c_layout():
    # 27 four-byte fields, no padding holes.
    assert ctypes.sizeof(C.MlpConfig) == 27 * 4
    assert C.ADAM_STATE_DTYPE.itemsize == 16 and C.EXAMPLE_ADAM_STATE_DTYPE.itemsize == 8


def test_layout_through_abi_matches_host_restatement():
    L = lib.load()
    for name in ["c1", "c2", "c3", "c4", "c5_w64"]:
        cfg = C.named_config(name)
        w = (ctypes.c_int64 * 8)(); b = (ctypes.c_int64 * 8)(); t = ctypes.c_int64()
        assert L.mlp_param_layout(ctypes.byref(cfg), w, b, ctypes.byref(t)) == 0
        pw, pb, pt = C.param_layout(cfg)
        assert list(w)[:cfg.n_layers] == pw and list(b)[:cfg.n_layers] == pb and t.value == pt


def test_no_cpu_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    L = lib.load()
    h = ctypes.c_void_p()
    rc = L.mlp_device_create(0, ctypes.byref(h))
    assert rc < 0 and b"no CPU fallback" in L.mlp_last_error_string()


def test_bf16_helpers_round_to_nearest_even():
    x = np.array([1.0, 1.0 + 2.0 ** -8, 1.0 + 3 * 2.0 ** -8, -0.3, 1e-40, np.inf], dtype=np.float32)
    b = C.f32_to_bf16_bits(x)
    assert list(b[:3]) == [0x3F80, 0x3F80, 0x3F82]
    back = C.bf16_bits_to_f32(b)
    assert back[5] == np.inf and abs(back[3] + 0.3) < 2e-3
