"""GPU parity of the forward kernels (tensor-core and one-thread-per-sample) against the CPU oracle."""
import numpy as np
import pytest

from oracle import oracle
from slang_b200 import config as C

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def device():
    from slang_b200.api import Device
    d = Device(0)
    yield d
    d.destroy()


def _forward(device, cfg, params, x, count, entry):
    from slang_b200.api import Trainer
    tr = Trainer(device, cfg, params, forward_entry=entry)
    xin = np.ascontiguousarray(x).view(np.uint8).reshape(-1)
    if xin.size < 16:
        xin = np.concatenate([xin, np.zeros(16 - xin.size, dtype=np.uint8)])
    xb = device.create_buffer(xin.size, xin)
    ob = device.create_buffer(max(count * cfg.out_dim * 4, 16))
    tr.forward(xb.address, ob.address, count)
    device.wait()
    out = ob.read(np.float32)[:count * cfg.out_dim].reshape(count, cfg.out_dim)
    impl = tr.k_forward.implementation
    xb.destroy(); ob.destroy()
    return out, impl


@pytest.mark.parametrize("width", [16, 32, 64, 128])
@pytest.mark.parametrize("count", [1, 127, 128, 1000, 128 * 148 * 2 + 77])
def test_constant_width_forward_sweep(device, width, count):
    """Depth-4 ReLU networks of constant width, fp16 weights from seed 7, inputs uniform in [-1, 1]:
    fp32 outputs against the oracle, elementwise within 2e-3 of the output tensor's largest magnitude
    (both sides round every inter-layer vector to fp16; only the fp32 summation order differs)."""
    name = "c5_w%d" % width
    cfg = C.named_config(name)
    params = C.init_params(cfg, seed=7, scheme="kaiming")
    # non-zero biases so that the bias path is exercised
    w_off, b_off, total = C.param_layout(cfg)
    pf = C.from_storage(params, cfg.dtype).copy()
    rng = np.random.default_rng(width)
    for l in range(cfg.n_layers):
        pf[b_off[l]:b_off[l] + width] = rng.uniform(-0.2, 0.2, width)
    params = C.to_storage(pf, cfg.dtype)
    x, _ = C.synthetic_batch(name, cfg, count, seed=7)
    ref = oracle.forward(cfg, params, x, count)
    out, impl = _forward(device, cfg, params, x, count, "forward")
    assert impl == "tcgen05"
    scale = max(float(np.max(np.abs(ref))), 1e-6)
    err = float(np.max(np.abs(out - ref))) / scale
    print("forward width %d count %d: max err / max|out| = %.3g" % (width, count, err))
    assert err < 2e-3
    out2, impl2 = _forward(device, cfg, params, x, min(count, 4096), "forward_simt")
    assert impl2 == "simt"
    n = min(count, 4096)
    assert float(np.max(np.abs(out2 - ref[:n]))) / scale < 2e-3


@pytest.mark.parametrize("count", [100, 128 * 300 + 5])
def test_wide_network_forward(device, count):
    """64-128-128-128-128-64 bf16 with GELU (the teacher of the training benchmark)."""
    cfg = C.named_config("c4")
    params = C.init_params(cfg, seed=5, scheme="xavier")
    rng = np.random.default_rng(9)
    x = C.to_storage(rng.normal(size=(count, 64)).astype(np.float32), C.BF16)
    ref = oracle.forward(cfg, params, x, count)
    out, impl = _forward(device, cfg, params, x, count, "forward")
    assert impl == "tcgen05"
    scale = float(np.max(np.abs(ref)))
    err = float(np.max(np.abs(out - ref))) / scale
    print("wide forward count %d: max err / max|out| = %.3g" % (count, err))
    assert err < 1e-2


def test_forward_output_in_storage_type(device):
    """MLP_FLAG_OUTPUT_STORAGE_TYPE: the same outputs rounded to bf16, as another network's targets."""
    from slang_b200.api import FLAG_OUTPUT_STORAGE_TYPE, Trainer
    cfg = C.named_config("c4")
    params = C.init_params(cfg, seed=5, scheme="xavier")
    count = 777
    x = C.to_storage(np.random.default_rng(2).normal(size=(count, 64)).astype(np.float32), C.BF16)
    tr = Trainer(device, cfg, params)
    xb = device.create_buffer(x.nbytes, x)
    o32 = device.create_buffer(count * 64 * 4)
    o16 = device.create_buffer(count * 64 * 2)
    tr.forward(xb.address, o32.address, count)
    tr.forward(xb.address, o16.address, count, FLAG_OUTPUT_STORAGE_TYPE)
    device.wait()
    a = o32.read(np.float32)
    b = o16.read(np.uint16)
    assert np.array_equal(C.f32_to_bf16_bits(a), b)


@pytest.mark.parametrize("case", ["c2", "c3", "tanh_bf16", "tiny", "relu3"])
@pytest.mark.parametrize("count", [1, 130, 128 * 148 * 2 + 9])
def test_narrow_network_forward_on_tensor_cores(device, case, count):
    """Networks of any widths up to 64 (any activation, input conversion or the frequency encoding) run
    their forward pass through the padded tensor-core kernel; outputs against the oracle."""
    rng = np.random.default_rng(count % 97 + len(case))
    if case in ("c2", "c3"):
        cfg = C.named_config(case)
        params = C.init_params(cfg, seed=3, scheme="xavier" if case == "c2" else "kaiming")
        x, _ = C.synthetic_batch(case, cfg, count, seed=3)
    else:
        dims, dtype, act = {"tanh_bf16": ([20, 64, 33, 40], C.BF16, C.ACT_TANH), "tiny": ([3, 16, 7], C.F16, C.ACT_SILU),
                            "relu3": ([32, 64, 64, 3], C.F16, C.ACT_RELU)}[case]
        cfg = C.make_config(dims, dtype=dtype, hidden_act=act, output_act=C.ACT_SIGMOID if case == "relu3" else C.ACT_IDENTITY)
        params = C.init_params(cfg, seed=3, scheme="xavier")
        x = rng.uniform(-1, 1, (count, dims[0])).astype(np.float32)
    # non-zero biases
    w_off, b_off, total = C.param_layout(cfg)
    pf = C.from_storage(params, cfg.dtype).copy()
    for l in range(cfg.n_layers):
        pf[b_off[l]:b_off[l] + cfg.dims[l + 1]] = rng.uniform(-0.2, 0.2, cfg.dims[l + 1])
    params = C.to_storage(pf, cfg.dtype)
    ref = oracle.forward(cfg, params, x, count)
    out, impl = _forward(device, cfg, params, x, count, "forward")
    assert impl == "tcgen05"
    scale = max(float(np.max(np.abs(ref))), 1e-6)
    err = float(np.max(np.abs(out - ref))) / scale
    print("narrow forward %s count %d: max err / max|out| = %.3g" % (case, count, err))
    assert err < (1e-2 if cfg.dtype == C.BF16 else 3e-3)
