"""Input gradients of learnGradient and the encoder-in-front composition (positions -> permutohedral
features -> MLP), against the oracle doing the same three stages on the CPU."""
import numpy as np
import pytest

from oracle import oracle
from oracle import permuto as OP
from slang_b200 import config as C
from slang_b200 import permuto as P
from mlp_testlib import make_problem, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def device():
    from slang_b200.api import Device
    d = Device(0)
    yield d
    d.destroy()


@pytest.mark.parametrize("name,count", [("c1", 1000), ("c2", 777), ("c4", 300)])
def test_input_gradients_match_oracle(device, name, count):
    from slang_b200.api import Trainer
    cfg, p0, batches = make_problem(name, count, seed=9, steps=1)
    x, t = batches[0]
    _, _, total = C.param_layout(cfg)
    g_ref = np.zeros(total, dtype=np.float32)
    words = np.zeros(2, dtype=np.uint32)
    ig_ref = oracle.learn_gradient_inputs(cfg, p0, g_ref, x, t, count, words)
    tr = Trainer(device, cfg, p0)
    xb, tb = device.create_buffer(x.nbytes, x), device.create_buffer(t.nbytes, t)
    igb = device.create_buffer(count * cfg.dims[0] * 4)
    tr.learn_gradient(xb.address, tb.address, count, input_grads_address=igb.address)
    device.wait()
    ig = igb.read(np.float32).reshape(count, cfg.dims[0])
    if cfg.dtype == C.F32:
        assert np.array_equal(ig.view(np.uint32), ig_ref.view(np.uint32))     # per-sample work is bit-exact
    else:
        assert rel_err(ig, ig_ref) <= 1e-2
    assert rel_err(tr.read_grads(), g_ref) <= (1e-5 if cfg.dtype == C.F32 else 1e-2)
    # the flag needs the longer argument struct and a destination
    from slang_b200.api import FLAG_INPUT_GRADIENT
    from slang_b200.lib import MlpError
    with pytest.raises(MlpError):
        tr.learn_gradient(xb.address, tb.address, count, flags=FLAG_INPUT_GRADIENT)


@pytest.mark.parametrize("dims,dtype,act", [([32, 128, 128, 3], C.F16, C.ACT_RELU), ([64, 96, 128, 128, 64], C.BF16, C.ACT_GELU_TANH),
                                            ([8, 128, 16], C.F16, C.ACT_TANH)])
def test_input_gradients_from_the_wide_kernel(device, dims, dtype, act):
    """Networks with a hidden width above 64 and 16-bit inputs: the wide tensor-core kernel writes the input
    gradients itself (one more product per tile, W_0^T . dZ_0^T), ragged last tile included."""
    from slang_b200.api import Trainer
    rng = np.random.default_rng(sum(dims))
    count = 64 * 7 + 19
    cfg = C.make_config(dims, dtype=dtype, hidden_act=act, input_dtype=dtype, target_dtype=C.F32, adam_master=1)
    p0 = C.init_params(cfg, seed=4, scheme="xavier")
    x = C.to_storage(rng.uniform(-1, 1, (count, dims[0])).astype(np.float32), dtype)
    t = rng.uniform(-1, 1, (count, dims[-1])).astype(np.float32)
    _, _, total = C.param_layout(cfg)
    g_ref = np.zeros(total, dtype=np.float32)
    words = np.zeros(2, dtype=np.uint32)
    ig_ref = oracle.learn_gradient_inputs(cfg, p0, g_ref, x, t, count, words)
    tr = Trainer(device, cfg, p0)
    assert tr.k_learn.implementation == "tcgen05"
    xb, tb = device.create_buffer(x.nbytes, x), device.create_buffer(t.nbytes, t)
    igb = device.create_buffer(count * dims[0] * 4)
    for _ in range(2):      # twice: the second launch must not see state of the first
        tr.grads.clear()
        tr.loss.clear()
        tr.learn_gradient(xb.address, tb.address, count, input_grads_address=igb.address)
    device.wait()
    ig = igb.read(np.float32).reshape(count, dims[0])
    assert np.isfinite(ig).all() and rel_err(ig, ig_ref) <= 1e-2
    assert rel_err(tr.read_grads(), g_ref) <= 1e-2
    mx, sm = tr.read_loss()
    assert abs(sm - float(words[1:].view(np.float32)[0])) <= 1e-2 * abs(sm)


@pytest.mark.parametrize("dtype,hidden", [(C.F32, 16), (C.F16, 16), (C.F16, 128)])
def test_encoder_in_front_of_the_network_trains_like_the_oracle(device, dtype, hidden):
    """fp32 network: one thread per sample; fp16 networks: the tensor-core kernel that runs learnGradient writes
    the input gradients (the padded 64-wide one; for 128 hidden units the wide one, whose fp32 feature rows
    are rounded to fp16 by a launch in front of it)."""
    from slang_b200.encoded import EncodedTrainer
    rng = np.random.default_rng(12)
    pcfg = P.prepare(2, 2, 10, 4, 2.0, 1.0, 1.1, 1337, C.F32)
    cfg = C.make_config([8, hidden, hidden, 3], dtype=dtype, hidden_act=C.ACT_RELU, lr=1e-2, adam_master=0 if dtype == C.F32 else 1)
    p0 = C.init_params(cfg, seed=2, scheme="kaiming")
    table0 = rng.uniform(-1e-1, 1e-1, pcfg.table_values).astype(np.float32)
    count, steps = 2000, 5
    tcfg = C.make_config([1, 1], dtype=C.F32, lr=1e-2)
    # oracle
    params, table = p0.copy(), table0.copy()
    _, _, total = C.param_layout(cfg)
    st = np.zeros(total, dtype=C.ADAM_STATE_DTYPE); st["master"] = C.from_storage(p0, cfg.dtype)
    tst = np.zeros(table.size, dtype=C.ADAM_STATE_DTYPE); tst["master"] = table0
    batches, ref_losses = [], []
    for k in range(steps):
        pos = rng.uniform(0, 1, (count, 2)).astype(np.float32)
        tgt = np.stack([np.sin(6 * pos[:, 0]), np.cos(5 * pos[:, 1]), pos[:, 0] * pos[:, 1]], axis=1).astype(np.float32)
        batches.append((pos, tgt))
        feats = OP.encode(pcfg, pos, table)
        grads = np.zeros(total, dtype=np.float32)
        words = np.zeros(2, dtype=np.uint32)
        ig = oracle.learn_gradient_inputs(cfg, params, grads, feats, tgt, count, words)
        dtable = np.zeros_like(table)
        OP.backward(pcfg, pos, table, ig, dtable)
        oracle.adjust_parameters(cfg, st, params, grads)
        oracle.adjust_parameters(tcfg, tst, table, dtable)
        ref_losses.append(float(words[1:].view(np.float32)[0]) / count)
    # library
    et = EncodedTrainer(device, pcfg, cfg, table0, p0, max_count=count)
    assert et.trainer.k_learn.implementation == ("simt" if dtype == C.F32 else "tcgen05")
    tol_loss, tol_par = (1e-4, 1e-3) if dtype == C.F32 else (1e-2, 2e-2)
    gpu_losses = []
    for pos, tgt in batches:
        pb, tb = device.create_buffer(pos.nbytes, pos), device.create_buffer(tgt.nbytes, tgt)
        et.learn_gradient(pb.address, tb.address, count)
        gpu_losses.append(et.trainer.read_loss()[1] / count)
        et.adjust_parameters()
    device.wait()
    print("losses gpu", gpu_losses, "ref", ref_losses)
    assert ref_losses[-1] < ref_losses[0]
    for a, b in zip(gpu_losses, ref_losses):
        assert abs(a - b) <= tol_loss * abs(b)
    assert rel_err(C.from_storage(et.trainer.read_params(), cfg.dtype), C.from_storage(params, cfg.dtype)) <= tol_par
    assert rel_err(et.read_table(), table) <= tol_par
    assert not et.read_table_grads().any()     # Adam cleared the table gradient
