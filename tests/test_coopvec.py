"""The cooperative-vector example's host calls and kernel (examples/mlp-training-coopvec):
getCooperativeVectorMatrixSize, convertCooperativeVectorMatrix, learnGradient in the coopvec flavour."""
import ctypes

import numpy as np
import pytest

from oracle import layout_oracle as LO
from oracle import oracle
from slang_b200 import config as C

NP = {C.F32: np.float32, C.F16: np.float16}


def test_matrix_size_matches_layout_model():
    from slang_b200.api import matrix_size
    from slang_b200.lib import MlpError
    for rows, cols in [(16, 4), (4, 16), (1, 1), (17, 33), (128, 128), (5, 13)]:
        for dt, es in [(C.F16, 2), (C.F32, 4), (C.BF16, 2)]:
            for layout in range(4):
                assert matrix_size(rows, cols, dt, layout) == LO.matrix_size(rows, cols, es, layout)
            assert matrix_size(rows, cols, dt, 0, 512) == LO.matrix_size(rows, cols, es, 0, 512)
            assert matrix_size(rows, cols, dt, 1, 512) == LO.matrix_size(rows, cols, es, 1, 512)
    # the example's two weight matrices in the training-optimal layout: one 16x16 tile of halfs each
    assert matrix_size(16, 4, C.F16, 3) == 512 and matrix_size(4, 16, C.F16, 3) == 512
    for bad in [(0, 4, C.F16, 0), (4, 4, 9, 0), (4, 4, C.F16, 7)]:
        with pytest.raises(MlpError):
            matrix_size(*bad)


def test_coopvec_oracle_differs_from_software_flavour_only_where_stated():
    """Same parameters and inputs through both flavours of the oracle: the bias gradient of the output
    layer is identical when no output is negative-sloped (the two differ in slope handling and summation
    start), and the coopvec weight gradient lands in the 16x16 tile positions."""
    rng = np.random.default_rng(2)
    init = np.zeros(384 + 512, dtype=np.uint16)     # segment 1, segment 2, two 256-element tiles
    init[:192] = rng.uniform(-1, 1, 192).astype(np.float16).view(np.uint16)
    inputs = rng.uniform(0, 1, 32).astype(np.float32)
    host = init.copy()
    base = host.ctypes.data
    offs = [(0, 128), (192, 320)]
    net = np.array([[base + w, base + 768 + 512 * l, base + b, base + 384 + b] for l, (w, b) in enumerate(offs)], dtype=np.uint64)
    loss = np.zeros(2, dtype=np.uint32)
    oracle.example_coopvec_learn_gradient(net, loss, inputs, 16)
    t1 = host[384:384 + 256].view(np.float16).reshape(16, 16)   # layer 1: 16 x 4
    t2 = host[384 + 256:].view(np.float16).reshape(16, 16)      # layer 2: 4 x 16
    assert np.any(t1[:, :4] != 0) and not np.any(t1[:, 4:] != 0)
    assert np.any(t2[:4, :] != 0) and not np.any(t2[4:, :] != 0)
    assert loss[0] != 0
    # row-major weight-gradient slots of segment 2 are untouched by the kernel (the host converts later)
    assert not host[192:192 + 64].any() and not host[192 + 96:192 + 160].any()


@pytest.fixture(scope="module")
def device():
    from slang_b200.api import Device
    d = Device(0)
    yield d
    d.destroy()


@pytest.mark.gpu
def test_matrix_convert_matches_layout_model(device):
    from slang_b200.api import MatrixDesc, matrix_size
    from slang_b200.lib import MlpError
    rng = np.random.default_rng(8)
    cases = [(16, 4, C.F16, 3, 0, C.F16, 0, 0), (4, 16, C.F16, 3, 0, C.F16, 0, 8 * 2 * 2),
             (37, 19, C.F32, 0, 0, C.F16, 2, 0), (37, 19, C.F16, 2, 0, C.F32, 1, 0),
             (128, 128, C.F16, 1, 0, C.F16, 3, 0), (5, 13, C.F32, 1, 64, C.F32, 0, 128),
             (33, 17, C.F16, 3, 0, C.F16, 2, 0)]
    for rows, cols, sdt, slay, sstr, ddt, dlay, dstr in cases:
        m = rng.uniform(-2, 2, (rows, cols)).astype(np.float16).astype(np.float32)   # exact in every type used
        src = LO.matrix_to_bytes(m, NP[sdt], slay, sstr)
        want = LO.matrix_to_bytes(m, NP[ddt], dlay, dstr, fill=0xAB)
        ssz, dsz = matrix_size(rows, cols, sdt, slay, sstr), matrix_size(rows, cols, ddt, dlay, dstr)
        assert ssz == src.nbytes and dsz == want.nbytes
        buf = device.create_buffer(256 + ssz + 256 + dsz + 256, np.concatenate([np.zeros(256, np.uint8), src, np.full(256 + dsz + 256, 0xAB, np.uint8)]))
        sd = MatrixDesc(rows, cols, sdt, slay, ssz, 256, sstr)
        dd = MatrixDesc(rows, cols, ddt, dlay, dsz, 256 + ssz + 256, dstr)
        device.matrix_convert(buf.address, [dd], buf.address, [sd])
        got = buf.read(np.uint8)
        assert np.array_equal(got[256 + ssz + 256: 256 + ssz + 256 + dsz], want), (rows, cols, slay, dlay)
        assert np.all(got[256 + ssz: 256 + ssz + 256] == 0xAB) and np.all(got[-256:] == 0xAB)   # nothing outside
        assert np.array_equal(got[256:256 + ssz], src)
    # overlapping ranges and mismatched extents are refused
    buf = device.create_buffer(4096)
    a = MatrixDesc(16, 16, C.F16, 0, 512, 0, 0)
    with pytest.raises(MlpError):
        device.matrix_convert(buf.address, [MatrixDesc(16, 16, C.F16, 3, 512, 256, 0)], buf.address, [a])
    with pytest.raises(MlpError):
        device.matrix_convert(buf.address, [MatrixDesc(16, 8, C.F16, 3, 512, 1024, 0)], buf.address, [a])


@pytest.mark.gpu
def test_coopvec_example_loop_matches_oracle(device):
    """The host loop of examples/mlp-training-coopvec/mlp-training-coopvec.cpp:106-262: three segments
    (parameters, row-major gradients, training-optimal weight gradients), every element of the buffer
    initialised from srand(1072), per step: clear loss, clear segment 3, learnGradient, convert the
    weight gradients to row-major, adjustParameters over segment 2."""
    from slang_b200.api import AdjustParamsParams, LearnGradParams, MatrixDesc, matrix_size
    libc = ctypes.CDLL("libc.so.6")
    libc.srand(1072)
    RAND_MAX = 2147483647
    sizes = [4, 16, 4]
    seg = 384                                   # bytes of segments 1 and 2 (64-byte sub-allocations)
    tsz = [matrix_size(sizes[i + 1], sizes[i], C.F16, 3) for i in range(2)]
    assert tsz == [512, 512]
    total = 2 * seg + sum(tsz)
    init = np.zeros(total // 2, dtype=np.uint16)
    for i in range(total // 2):
        v = np.float32(libc.rand() / np.float32(RAND_MAX))
        init[i] = oracle.example_float_to_half(float(np.float32(v * np.float32(2.0) - np.float32(1.0))))
    inputs = np.array([libc.rand() / np.float32(RAND_MAX) for _ in range(32)], dtype=np.float32)
    offs = [(0, 128), (192, 320)]               # (weights, bias) byte offsets inside a segment
    toff = [2 * seg, 2 * seg + tsz[0]]
    steps = 60

    def descs():
        src = [MatrixDesc(sizes[i + 1], sizes[i], C.F16, 3, tsz[i], toff[i], 0) for i in range(2)]
        dst = [MatrixDesc(sizes[i + 1], sizes[i], C.F16, 0, sizes[i] * sizes[i + 1] * 2, seg + offs[i][0], sizes[i] * 2) for i in range(2)]
        return dst, src

    # oracle on host memory (layout conversion by the numpy model)
    host = init.copy()
    base = host.ctypes.data
    net = np.array([[base + w, base + toff[l], base + b, base + seg + b] for l, (w, b) in enumerate(offs)], dtype=np.uint64)
    n_adam = seg // 2
    st = np.zeros(n_adam, dtype=C.EXAMPLE_ADAM_STATE_DTYPE)
    ref_losses = []
    for k in range(steps):
        loss = np.zeros(2, dtype=np.uint32)
        host[seg:] = 0                          # clear segment 3 (element index seg = byte 2 * seg)
        oracle.example_coopvec_learn_gradient(net, loss, inputs, 16)
        for l in range(2):
            tile = host[toff[l] // 2: toff[l] // 2 + 256].view(np.float16).reshape(16, 16)
            rm = tile[:sizes[l + 1], :sizes[l]].reshape(-1)
            o = (seg + offs[l][0]) // 2
            host[o:o + rm.size] = rm.view(np.uint16)
        oracle.example_adjust_parameters(st, host[:n_adam], host[n_adam:2 * n_adam], n_adam)
        ref_losses.append(int(loss[0]))

    buf = device.create_buffer(init.nbytes, init)
    states = device.create_buffer(n_adam * 8)
    netd = np.array([[buf.address + w, buf.address + toff[l], buf.address + b, buf.address + seg + b] for l, (w, b) in enumerate(offs)], dtype=np.uint64)
    netb = device.create_buffer(netd.nbytes, netd)
    inb = device.create_buffer(inputs.nbytes, inputs)
    lossb = device.create_buffer(8)
    k_learn, k_adjust = device.kernel("learnGradient_coopvec"), device.kernel("adjustParameters")
    dst, src = descs()
    gpu_losses = []
    for k in range(steps):
        lossb.clear()
        buf.clear(2 * seg, sum(tsz))
        k_learn.dispatch(LearnGradParams(netb.address, lossb.address, inb.address, 16), 1)
        device.matrix_convert(buf.address, dst, buf.address, src)
        k_adjust.dispatch(AdjustParamsParams(states.address, buf.address, buf.address + seg, n_adam), 1)
        gpu_losses.append(int(lossb.read(np.uint32)[0]))
    got = buf.read(np.uint16)
    first_loss_mismatch = next((k for k in range(steps) if gpu_losses[k] != ref_losses[k]), steps)
    print("coopvec example: loss words identical for the first %d of %d steps" % (first_loss_mismatch, steps))
    assert first_loss_mismatch >= 20
    a = got[:n_adam].view(np.float16).astype(np.float32); b = host[:n_adam].view(np.float16).astype(np.float32)
    assert np.max(np.abs(a - b)) <= 2e-2 * np.max(np.abs(b))
