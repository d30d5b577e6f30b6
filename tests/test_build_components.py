"""A build may leave optional components out (python -m slang_b200.build --without ... --out ...): every symbol
the headers declare stays present and the left-out entry points answer MLP_E_NOT_AVAILABLE."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_build_without_components(tmp_path):
    from slang_b200 import build as B
    out = str(tmp_path / "libslang_b200_partial.so")
    assert B.build(without=["comm", "permuto", "tile_mma"], out=out) == out
    lib = ctypes.CDLL(out)
    lib.mlp_last_error_string.restype = ctypes.c_char_p
    inc = os.path.join(ROOT, "include")
    text = "".join(open(os.path.join(inc, f)).read() for f in sorted(os.listdir(inc)) if f.endswith(".h"))
    names = set(re.findall(r"\b(mlp_[a-z0-9_]+)\s*\(", text))
    assert len(names) > 30
    for n in names:
        assert hasattr(lib, n), n
    assert lib.mlp_comm_unique_id(None, 0) == -3 and b"left out" in lib.mlp_last_error_string()
    assert lib.mlp_tile_mma(None, None, 0, 0, 0, 0) == -3
    assert lib.mlp_permuto_encode(None, None, 0, 0, 0, 0) == -3
    # what stays in still answers as usual (an argument check that needs no device)
    assert lib.mlp_wait(None) == -2
    with pytest.raises(ValueError):
        B.build(without=["comm"])                 # the in-tree library is always the full one
    with pytest.raises(ValueError):
        B.build(without=["adam"], out=out)
