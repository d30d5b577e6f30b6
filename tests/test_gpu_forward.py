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
    xb = device.create_buffer(max(x.nbytes, 16), x if x.nbytes else None)
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
