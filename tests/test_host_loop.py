"""The example's host program as C++ against the public header (tests/host_loop/mlp_training_host.cpp).

CPU: g++ compiles it with warnings as errors and links it against the built library, so the header is
seen by a C++ compiler exactly as a client sees it, and a plain C compiler parses the headers too.
GPU: the program runs its 1000 iterations; the loss words it prints match the oracle driven through the
same seeded initialisation (bit for bit at the start, within the 16-bit tolerance to the end) and fall.
"""
import ctypes
import os
import re
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "host_loop", "mlp_training_host.cpp")
LIBDIR = os.path.join(ROOT, "slang_b200")


def _build(out):
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"), SRC,
                           "-o", out, "-L", LIBDIR, "-lslang_b200_mlp", "-Wl,-rpath," + LIBDIR])


def test_host_program_compiles_and_links_against_the_public_header(tmp_path):
    from slang_b200 import build
    build.build()
    _build(str(tmp_path / "mlp_training_host"))
    # the headers are C as well as C++
    c_src = tmp_path / "c_client.c"
    c_src.write_text('#include "slang_b200_mlp.h"\n#include "slang_b200_permuto.h"\n'
                     "int main(void) { MlpConfig c; (void)c; return sizeof(MlpLearnGradParamsEx) == 40 ? 0 : 1; }\n")
    subprocess.check_call(["gcc", "-std=c99", "-Wall", "-Werror", "-pedantic", "-fsyntax-only", "-I", os.path.join(ROOT, "include"), str(c_src)])


@pytest.mark.gpu
def test_host_program_trains_like_the_oracle(tmp_path):
    from oracle import oracle
    from slang_b200 import config as C
    exe = str(tmp_path / "mlp_training_host")
    _build(exe)
    out = subprocess.run([exe, "1000"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    words = [int(m.group(1), 16) for m in re.finditer(r"\[0x([0-9a-f]{8})\]", out.stdout)]
    assert len(words) == 100
    assert "launches: 2000" in out.stdout

    # the same run on the oracle (examples/mlp-training/mlp-training.cpp:106-212)
    libc = ctypes.CDLL("libc.so.6")
    libc.srand(1072)
    RAND_MAX = 2147483647
    host = np.zeros(384, dtype=np.uint16)
    for i in range(192):
        v = np.float32(libc.rand()) / np.float32(RAND_MAX)
        host[i] = oracle.example_float_to_half(float(np.float32(v * np.float32(2.0) - np.float32(1.0))))
    inputs = np.array([np.float32(libc.rand()) / np.float32(RAND_MAX) for _ in range(32)], dtype=np.float32)
    base = host.ctypes.data
    offs = [(0, 128), (192, 320)]
    net = np.array([[base + w, base + 384 + w, base + b, base + 384 + b] for w, b in offs], dtype=np.uint64)
    st = np.zeros(192, dtype=C.EXAMPLE_ADAM_STATE_DTYPE)
    ref = []
    for k in range(1000):
        loss = np.zeros(2, dtype=np.uint32)
        oracle.example_learn_gradient(net, loss, inputs, 16)
        oracle.example_adjust_parameters(st, host[:192], host[192:], 192)
        if k % 10 == 0:
            ref.append(int(loss[0]))
    assert words[:2] == ref[:2], "the first printed loss words differ from the oracle's"
    got = np.array(words, dtype=np.uint32).view(np.float32)
    want = np.array(ref, dtype=np.uint32).view(np.float32)
    assert got[-1] < 0.2 * got[0], "the loss did not fall"
    # half-precision Adam drifts over hundreds of steps: compare the printed losses loosely
    assert np.max(np.abs(got - want)) <= 5e-2 * np.max(want)
