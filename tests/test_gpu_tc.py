"""GPU parity of the tensor-core learnGradient (64-128-128-128-128-64) against the CPU oracle and
against the one-thread-per-sample kernel, through the C ABI."""
import numpy as np
import pytest

from slang_b200 import config as C

from mlp_testlib import gpu_trajectory, layer_rel_errs, make_problem, oracle_trajectory, per_layer_rel_errs, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def device():
    from slang_b200.api import Device
    d = Device(0)
    yield d
    d.destroy()


def _grad_layer_errs(cfg, g, g_ref):
    return max(layer_rel_errs(cfg, g, g_ref))


def test_c4_kernel_is_tensor_core(device):
    k = device.kernel("learnGradient", C.named_config("c4"))
    assert k.implementation == "tcgen05"
    assert device.kernel("learnGradient_simt", C.named_config("c4")).implementation == "simt"


@pytest.mark.parametrize("count", [64, 1, 63, 65, 100, 512, 4096 + 17])
def test_c4_gradients_match_oracle(device, count):
    """One learnGradient: gradients per tensor within 1e-2 of the oracle (relative to the tensor's
    largest magnitude), loss words within 1e-2 relative."""
    cfg, p0, batches = make_problem("c4", count, seed=11, steps=1)
    _, l_ref, g_ref, _ = oracle_trajectory(cfg, p0, batches, n_threads=8)
    _, l_gpu, g_gpu, _, tr = gpu_trajectory(device, cfg, p0, batches)
    assert tr.k_learn.implementation == "tcgen05"
    err = _grad_layer_errs(cfg, g_gpu, g_ref)
    print("c4 count=%d worst per-tensor gradient rel err %.3g; loss gpu %s ref %s" % (count, err, l_gpu[0], l_ref[0]))
    assert err < 1e-2
    assert abs(l_gpu[0][1] - l_ref[0][1]) <= 1e-2 * abs(l_ref[0][1])
    assert abs(l_gpu[0][0] - l_ref[0][0]) <= 1e-2 * abs(l_ref[0][0])


def test_c4_many_tiles_per_cta(device):
    """More tiles than SMs, so every CTA accumulates several tiles in tensor memory, plus a ragged tail."""
    count = 64 * 148 * 3 + 5
    cfg, p0, batches = make_problem("c4", count, seed=12, steps=1)
    _, l_ref, g_ref, _ = oracle_trajectory(cfg, p0, batches, n_threads=8)
    _, l_gpu, g_gpu, _, _ = gpu_trajectory(device, cfg, p0, batches)
    err = _grad_layer_errs(cfg, g_gpu, g_ref)
    print("c4 count=%d worst per-tensor gradient rel err %.3g" % (count, err))
    assert err < 1e-2
    assert abs(l_gpu[0][1] - l_ref[0][1]) <= 1e-2 * abs(l_ref[0][1])


def test_c4_trajectory(device):
    """bf16 bar: per-step loss within 1e-2 relative, final parameters within 2e-2 relative
    (per layer, weights and biases together, relative to the layer's largest magnitude)."""
    cfg, p0, batches = make_problem("c4", 2048, seed=13, steps=8)
    p_ref, l_ref, _, _ = oracle_trajectory(cfg, p0, batches, n_threads=8)
    p_gpu, l_gpu, _, _, _ = gpu_trajectory(device, cfg, p0, batches)
    for (mg, sg), (mr, sr) in zip(l_gpu, l_ref):
        assert abs(sg - sr) <= 1e-2 * abs(sr)
    pg, pr = C.from_storage(p_gpu, cfg.dtype), C.from_storage(p_ref, cfg.dtype)
    errs = per_layer_rel_errs(cfg, pg, pr)
    print("c4 trajectory: worst per-layer parameter rel err %.3g (per tensor, biases alone: %.3g)"
          % (max(errs), max(layer_rel_errs(cfg, pg, pr))))
    assert max(errs) < 2e-2


def test_c4_tensor_core_matches_simt_on_large_batch(device):
    """2^17 samples: too many for the scalar oracle in a test, so the tensor-core kernel is checked
    against the one-thread-per-sample kernel (itself pinned to the oracle), and the gradient of the
    whole batch against the sum of the gradients of its two halves."""
    from slang_b200.api import Trainer
    count = 1 << 17
    cfg = C.named_config("c4")
    p0 = C.init_params(cfg, seed=21, scheme="xavier")
    rng = np.random.default_rng(5)
    x = C.to_storage(rng.normal(size=(count, 64)).astype(np.float32), C.BF16)
    t = C.to_storage(rng.normal(size=(count, 64)).astype(np.float32) * 0.3, C.BF16)
    xb = device.create_buffer(x.nbytes, x); tb = device.create_buffer(t.nbytes, t)
    tr_tc = Trainer(device, cfg, p0)
    tr_simt = Trainer(device, cfg, p0, learn_entry="learnGradient_simt")
    tr_tc.learn_gradient(xb.address, tb.address, count)
    tr_simt.learn_gradient(xb.address, tb.address, count)
    g_tc, g_simt = tr_tc.read_grads(), tr_simt.read_grads()
    err = _grad_layer_errs(cfg, g_tc, g_simt)
    print("c4 2^17: tensor-core vs one-thread-per-sample gradient rel err %.3g" % err)
    assert err < 1e-2
    l_tc, l_simt = tr_tc.read_loss(), tr_simt.read_loss()
    assert abs(l_tc[1] - l_simt[1]) <= 1e-3 * abs(l_simt[1])
    assert abs(l_tc[0] - l_simt[0]) <= 1e-2 * abs(l_simt[0])
    # additivity over a split of the batch
    tr_tc.grads.clear()
    half = count // 2
    tr_tc.learn_gradient(xb.address, tb.address, half)
    tr_tc.k_learn.dispatch(__import__("slang_b200.api", fromlist=["LearnGradParamsEx"]).LearnGradParamsEx(
        tr_tc.network.address, tr_tc.loss.address, xb.address + half * 128, tb.address + half * 128, half, 0), (half + 255) // 256)
    g_split = tr_tc.read_grads()
    assert _grad_layer_errs(cfg, g_split, g_tc) < 1e-4


@pytest.mark.parametrize("name", ["c2", "c3"])
@pytest.mark.parametrize("count", [1, 127, 129, 1024, 128 * 148 * 2 + 5])
def test_narrow_networks_on_tensor_cores(device, name, count):
    """fp16 4-32-32-32-32-4 (LeakyReLU) and enc(2->32)-64-64-64-3 (ReLU, sigmoid output, L2) through the
    padded 64-wide tensor-core kernel: gradients per tensor within 1e-2, loss words within 1e-2."""
    cfg, p0, batches = make_problem(name, count, seed=17, steps=1)
    _, l_ref, g_ref, _ = oracle_trajectory(cfg, p0, batches, n_threads=8)
    _, l_gpu, g_gpu, _, tr = gpu_trajectory(device, cfg, p0, batches)
    assert tr.k_learn.implementation == "tcgen05"
    err = _grad_layer_errs(cfg, g_gpu, g_ref)
    print("%s count=%d worst per-tensor gradient rel err %.3g; loss gpu %s ref %s" % (name, count, err, l_gpu[0], l_ref[0]))
    assert err < 1e-2
    assert abs(l_gpu[0][1] - l_ref[0][1]) <= 1e-2 * abs(l_ref[0][1])
    assert abs(l_gpu[0][0] - l_ref[0][0]) <= 1e-2 * abs(l_ref[0][0])


@pytest.mark.parametrize("dims", [[8, 48, 24], [20, 64, 33, 40], [64, 64, 64, 64, 64, 64], [3, 16, 7]])
def test_narrow_kernel_other_shapes(device, dims):
    """Shapes that exercise each column split of the padded kernel's epilogue (output width <= 16, <= 32,
    larger), odd widths, bf16, tanh hidden units."""
    from oracle import oracle
    rng = np.random.default_rng(sum(dims))
    cfg = C.make_config(dims, dtype=C.BF16, hidden_act=C.ACT_TANH, output_act=C.ACT_IDENTITY, adam_master=1)
    p0 = C.init_params(cfg, seed=5, scheme="xavier")
    count = 128 * 3 + 17
    x = rng.uniform(-1, 1, (count, dims[0])).astype(np.float32)
    t = rng.uniform(-1, 1, (count, dims[-1])).astype(np.float32)
    _, l_ref, g_ref, _ = oracle_trajectory(cfg, p0, [(x, t)])
    _, l_gpu, g_gpu, _, tr = gpu_trajectory(device, cfg, p0, [(x, t)])
    assert tr.k_learn.implementation == "tcgen05"
    err = _grad_layer_errs(cfg, g_gpu, g_ref)
    print(dims, "worst per-tensor gradient rel err %.3g" % err)
    assert err < 1e-2
    assert abs(l_gpu[0][1] - l_ref[0][1]) <= 1e-2 * abs(l_ref[0][1])
    assert abs(l_gpu[0][0] - l_ref[0][0]) <= 1e-2 * abs(l_ref[0][0])


@pytest.mark.parametrize("dims,dtype", [([32, 64, 64, 3], C.F16), ([10, 40, 12], C.BF16), ([64, 64, 64, 64, 32], C.BF16)])
def test_narrow_kernel_two_tiles_in_flight(device, dims, dtype):
    """ReLU networks of up to four layers run two tiles per CTA once there are more tiles than SMs; the
    derivative is recovered from the stored activation (negative zero marks a zero pre-activation).  Inputs
    with many exact zeros exercise the tie: zero inputs and zero biases give zero pre-activations."""
    rng = np.random.default_rng(len(dims) * 7 + dims[0])
    cfg = C.make_config(dims, dtype=dtype, hidden_act=C.ACT_RELU, output_act=C.ACT_IDENTITY, adam_master=1)
    p0 = C.init_params(cfg, seed=8, scheme="kaiming")   # biases start at zero
    count = 128 * 148 * 2 + 77
    x = rng.uniform(-1, 1, (count, dims[0])).astype(np.float32)
    x[::5] = 0.0                                         # every fifth sample: all pre-activations of layer 0 are zero
    t = rng.uniform(-1, 1, (count, dims[-1])).astype(np.float32)
    _, l_ref, g_ref, _ = oracle_trajectory(cfg, p0, [(x, t)], n_threads=8)
    _, l_gpu, g_gpu, _, tr = gpu_trajectory(device, cfg, p0, [(x, t)])
    assert tr.k_learn.implementation == "tcgen05"
    err = _grad_layer_errs(cfg, g_gpu, g_ref)
    print(dims, "worst per-tensor gradient rel err %.3g" % err)
    assert err < 1e-2
    assert abs(l_gpu[0][1] - l_ref[0][1]) <= 1e-2 * abs(l_ref[0][1])
    assert abs(l_gpu[0][0] - l_ref[0][0]) <= 1e-2 * abs(l_ref[0][0])


@pytest.mark.parametrize("name,count,steps", [("c2", 2048, 10), ("c3", 1024, 10)])
def test_narrow_network_trajectories(device, name, count, steps):
    cfg, p0, batches = make_problem(name, count, seed=3, steps=steps)
    p_ref, l_ref, _, _ = oracle_trajectory(cfg, p0, batches)
    p_gpu, l_gpu, _, _, tr = gpu_trajectory(device, cfg, p0, batches)
    assert tr.k_learn.implementation == "tcgen05"
    for (mg, sg), (mr, sr) in zip(l_gpu, l_ref):
        assert abs(sg - sr) <= 1e-2 * abs(sr)
    errs = per_layer_rel_errs(cfg, C.from_storage(p_gpu, cfg.dtype), C.from_storage(p_ref, cfg.dtype))
    print(name, "trajectory: worst per-layer parameter rel err %.3g" % max(errs))
    assert max(errs) < 2e-2


def test_c4_large_batch_properties(device):
    """2^22 samples (one sixteenth of the benchmark batch; the kernel walks 443 tiles per CTA):
    size-independent properties instead of an oracle run.  (1) Additivity: the gradient of the batch
    equals the sum of the gradients of its four quarters, and so does the loss sum.  (2) A zero
    residual gives a zero gradient: when the targets are the network's own outputs (rounded to bf16 by
    the forward kernel), every output difference is at most one rounding step of the output layer."""
    import torch
    from slang_b200.api import FLAG_OUTPUT_STORAGE_TYPE
    from slang_b200.torch_api import TorchTrainer
    count = 1 << 22
    cfg = C.named_config("c4")
    p0 = C.init_params(cfg, seed=33, scheme="xavier")
    gen = torch.Generator(device="cuda"); gen.manual_seed(5)
    x = torch.randn((count, 64), device="cuda", generator=gen).to(torch.bfloat16)
    t = (torch.randn((count, 64), device="cuda", generator=gen) * 0.3).to(torch.bfloat16)
    tt = TorchTrainer(cfg, p0)
    tt.learn_gradient(x, t)
    whole = tt.grads.clone()
    loss_whole = tt.loss()
    tt.grads.zero_()
    q = count // 4
    sums, mx = 0.0, 0.0
    for i in range(4):
        tt.learn_gradient(x[i * q:(i + 1) * q], t[i * q:(i + 1) * q])
        l = tt.loss()
        sums += l[1]; mx = max(mx, l[0])
    parts = tt.grads.clone()
    scale = whole.abs().max().item()
    assert (parts - whole).abs().max().item() <= 1e-4 * scale
    assert abs(sums - loss_whole[1]) <= 1e-4 * abs(loss_whole[1]) and mx == loss_whole[0]
    # zero residual
    own = torch.empty((count, 64), dtype=torch.bfloat16, device="cuda")
    tt.trainer.forward(x.data_ptr(), own.data_ptr(), count, FLAG_OUTPUT_STORAGE_TYPE)
    tt.grads.zero_()
    tt.learn_gradient(x, own)
    assert tt.grads.abs().max().item() <= 2e-3 * scale
    assert tt.loss()[0] < 1e-4


@pytest.mark.parametrize("dims,dtype,act,tdtype", [
    ([32, 128, 128, 3], C.F16, C.ACT_RELU, C.F32),            # odd output width: targets read by the epilogue
    ([64, 96, 96, 64], C.BF16, C.ACT_GELU_TANH, C.BF16),       # hidden widths padded to 128, targets by TMA
    ([16, 128, 8], C.F16, C.ACT_LEAKY_RELU, C.F16),            # two layers
    ([8, 100, 120, 60, 24], C.BF16, C.ACT_TANH, C.BF16),       # widths that are not multiples of 8 or 16, run-time activation
    ([64, 128, 128, 128, 128, 64], C.F16, C.ACT_SIGMOID, C.F16),  # the benchmark shape with a run-time activation
    ([40, 72, 64, 128, 33], C.F16, C.ACT_RELU, C.F16),
])
def test_wide_kernel_other_shapes(device, dims, dtype, act, tdtype):
    """Networks with a width above 64 run the wide tensor-core kernel zero-padded to 64 -> 128 -> ... -> 64:
    two to five layers, inputs a multiple of 8 up to 64, hidden widths up to 128, up to 64 outputs; gradients
    per tensor within 1e-2 of the oracle, loss words within 1e-2.  More tiles than SMs and a ragged tail."""
    rng = np.random.default_rng(sum(dims))
    cfg = C.make_config(dims, dtype=dtype, hidden_act=act, output_act=C.ACT_IDENTITY, act_alpha=0.02,
                        input_dtype=dtype, target_dtype=tdtype, adam_master=1)
    p0 = C.from_storage(C.init_params(cfg, seed=5, scheme="xavier"), dtype).copy()
    w_off, b_off, _ = C.param_layout(cfg)
    for l in range(cfg.n_layers):
        p0[b_off[l]:b_off[l] + dims[l + 1]] = rng.uniform(-0.2, 0.2, dims[l + 1])
    p0 = C.to_storage(p0, dtype)
    count = 64 * 148 + 64 * 3 + 11
    x = C.to_storage(rng.uniform(-1, 1, (count, dims[0])).astype(np.float32), dtype)
    t = C.to_storage(rng.uniform(-1, 1, (count, dims[-1])).astype(np.float32), tdtype)
    _, l_ref, g_ref, _ = oracle_trajectory(cfg, p0, [(x, t)], n_threads=8)
    _, l_gpu, g_gpu, _, tr = gpu_trajectory(device, cfg, p0, [(x, t)])
    assert tr.k_learn.implementation == "tcgen05"
    err = _grad_layer_errs(cfg, g_gpu, g_ref)
    print(dims, "worst per-tensor gradient rel err %.3g; loss gpu %s ref %s" % (err, l_gpu[0], l_ref[0]))
    assert err < 1e-2
    assert abs(l_gpu[0][1] - l_ref[0][1]) <= 1e-2 * abs(l_ref[0][1])
    assert abs(l_gpu[0][0] - l_ref[0][0]) <= 1e-2 * abs(l_ref[0][0])
    # the padding beyond each sub-allocation's real elements stays untouched
    _, _, total = C.param_layout(cfg)
    mask = np.ones(total, dtype=bool)
    for l in range(cfg.n_layers):
        mask[w_off[l]:w_off[l] + dims[l] * dims[l + 1]] = False
        mask[b_off[l]:b_off[l] + dims[l + 1]] = False
    assert not g_gpu[mask].any()
    # the forward entry point of the same shape runs the same kernel without its backward half
    from oracle import oracle
    from slang_b200.api import Trainer
    fresh = Trainer(device, cfg, p0)
    assert fresh.k_forward.implementation == "tcgen05"
    xb = device.create_buffer(x.nbytes, x)
    yb = device.create_buffer(count * dims[-1] * 4, np.full(count * dims[-1], 7.0, dtype=np.float32))
    fresh.forward(xb.address, yb.address, count)
    y = yb.read(np.float32).reshape(count, dims[-1])
    y_ref = oracle.forward(cfg, p0, x, count)
    step = 2.0 ** -7 if dtype == C.BF16 else 2.0 ** -10
    assert np.max(np.abs(y - y_ref)) <= 4 * step * max(1.0, float(np.max(np.abs(y_ref))))


@pytest.mark.parametrize("dims,op,act", [
    ([16, 64, 64, 8], C.F16, C.ACT_RELU),                 # padded 64-wide kernel
    ([4, 32, 32, 32, 4], C.BF16, C.ACT_LEAKY_RELU),       # its 32-wide build
    ([64, 128, 128, 64], C.BF16, C.ACT_GELU_TANH),        # wide kernel (16-bit inputs)
    ([32, 96, 128, 10], C.F16, C.ACT_TANH),               # wide kernel, run-time activation, targets read directly
])
def test_fp32_storage_with_16bit_operands(device, dims, op, act):
    """fp32 parameters, gradients and optimiser with 16-bit tensor-core operands (MlpConfig.operand_dtype): the
    neural module's T = float on its tensor-core path converts both matrix operands to half
    (source/standard-modules/neural/mma-tiled-cuda.slang:104-118, WaveMatrix.slang:62-64).  Gradients per
    tensor within 1e-2 of the oracle in the same mode, loss within 1e-2; the one-thread-per-sample kernel in
    the same mode agrees with the oracle to fp32 rounding; two Adam steps keep the parameters fp32."""
    rng = np.random.default_rng(sum(dims) + op)
    wide = max(dims) > 64
    in_dt = op if wide else C.F32
    cfg = C.make_config(dims, dtype=C.F32, hidden_act=act, act_alpha=0.03, input_dtype=in_dt, target_dtype=C.F32,
                        operand_dtype=op, lr=1e-3)
    p0 = C.init_params(cfg, seed=9, scheme="xavier")
    assert p0.dtype == np.float32
    w_off, b_off, _ = C.param_layout(cfg)
    for l in range(cfg.n_layers):
        p0[b_off[l]:b_off[l] + dims[l + 1]] = rng.uniform(-0.2, 0.2, dims[l + 1])
    count = 128 * 5 + 37
    batches = []
    for _ in range(2):
        x = C.to_storage(rng.uniform(-1, 1, (count, dims[0])).astype(np.float32), in_dt)
        t = rng.uniform(-1, 1, (count, dims[-1])).astype(np.float32)
        batches.append((x, t))
    p_ref, l_ref, g_ref, _ = oracle_trajectory(cfg, p0, batches, n_threads=4)
    p_gpu, l_gpu, g_gpu, _, tr = gpu_trajectory(device, cfg, p0, batches)
    assert tr.k_learn.implementation == "tcgen05" and tr.k_forward.implementation == "tcgen05"
    err = _grad_layer_errs(cfg, g_gpu, g_ref)
    print(dims, "fp32 storage, 16-bit operands: worst per-tensor gradient rel err %.3g" % err)
    assert err < 1e-2
    for (mg, sg), (mr, sr) in zip(l_gpu, l_ref):
        assert abs(sg - sr) <= 1e-2 * abs(sr) and abs(mg - mr) <= 1e-2 * abs(mr)
    assert p_gpu.dtype == np.float32 and max(per_layer_rel_errs(cfg, p_gpu, p_ref)) < 2e-2
    _, l_simt, g_simt, _, _ = gpu_trajectory(device, cfg, p0, batches[:1], "learnGradient_simt")
    assert _grad_layer_errs(cfg, g_simt, g_ref) < 1e-4
    # without the operand switch the same fp32 network stays on the exact one-thread-per-sample path
    cfg32 = C.make_config(dims, dtype=C.F32, hidden_act=act, act_alpha=0.03, input_dtype=C.F32, target_dtype=C.F32)
    assert device.kernel("learnGradient", cfg32).implementation == "simt"
