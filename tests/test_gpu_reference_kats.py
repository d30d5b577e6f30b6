"""The reference's own known answers and activation set through the GPU entry points.

* tests/neural/fflayer-wavetangled-vector-test.slang:95-153 (the tensor-core matvec's test: 4 -> 2 layer,
  W = [[1..4],[5..8]], b = [9,10], x = [1..4]; forward [39, 80], dX = [6,8,10,12], dW = B * [1..4] per
  row, db = B for B = 32, 64, 128) through the tcgen05 entry point "learnGradient" in fp16 and bf16.
* source/standard-modules/neural/activations.slang:27-228 (all nine activations) plus the two this
  library adds (GELU-tanh, the cooperative-vector example's max form): value and derivative through
  "forward" and "learnGradient" on the one-thread-per-sample kernels and on the padded tcgen05 kernel,
  against the oracle, which tests/test_oracle_kat.py pins on activation-functions-test.slang:31-154.
* config 2 at its stated 1000 steps on a reduced batch.
"""
import numpy as np
import pytest

from slang_b200 import config as C

from mlp_testlib import gpu_trajectory, layer_rel_errs, make_problem, oracle_trajectory, per_layer_rel_errs

pytestmark = pytest.mark.gpu

ALL_ACTS = [C.ACT_IDENTITY, C.ACT_RELU, C.ACT_LEAKY_RELU, C.ACT_SIGMOID, C.ACT_TANH, C.ACT_EXP, C.ACT_SINE,
            C.ACT_SILU, C.ACT_QUICK_GELU, C.ACT_GELU_TANH, C.ACT_LEAKY_MAX]
ACT_NAME = {C.ACT_IDENTITY: "identity", C.ACT_RELU: "relu", C.ACT_LEAKY_RELU: "leaky", C.ACT_SIGMOID: "sigmoid",
            C.ACT_TANH: "tanh", C.ACT_EXP: "exp", C.ACT_SINE: "sine", C.ACT_SILU: "silu",
            C.ACT_QUICK_GELU: "quickgelu", C.ACT_GELU_TANH: "gelu_tanh", C.ACT_LEAKY_MAX: "leaky_max"}


@pytest.fixture(scope="module")
def device():
    from slang_b200.api import Device
    d = Device(0)
    yield d
    d.destroy()


@pytest.mark.parametrize("dtype", [C.F16, C.BF16])
@pytest.mark.parametrize("batch", [32, 64, 128])
def test_wavetangled_known_answers_through_tcgen05(device, dtype, batch):
    """Identity layer 4 -> 4 in front of the test's 4 -> 2 layer so that dX of the tested layer shows up
    as the bias gradient of the layer before it (the learnGradient contract returns parameter
    gradients).  L2 loss with targets [38.5, 79.5] makes the output gradient exactly 1 per component."""
    from slang_b200.api import Trainer
    cfg = C.make_config([4, 4, 2], dtype, C.ACT_IDENTITY, loss=C.LOSS_L2_SUM, input_dtype=C.F32, target_dtype=C.F32)
    w_off, b_off, total = C.param_layout(cfg)
    p = np.zeros(total, dtype=np.float32)
    p[w_off[0]:w_off[0] + 16] = np.eye(4).reshape(-1)
    p[w_off[1]:w_off[1] + 8] = np.arange(1, 9)
    p[b_off[1]:b_off[1] + 2] = [9, 10]
    tr = Trainer(device, cfg, C.to_storage(p, dtype))
    assert tr.k_learn.implementation == "tcgen05" and tr.k_forward.implementation == "tcgen05"
    xs = np.tile(np.array([1, 2, 3, 4], dtype=np.float32), (batch, 1))
    ts = np.tile(np.array([38.5, 79.5], dtype=np.float32), (batch, 1))
    xb = device.create_buffer(xs.nbytes, xs); tb = device.create_buffer(ts.nbytes, ts)
    yb = device.create_buffer(batch * 2 * 4)
    tr.forward(xb.address, yb.address, batch)
    y = yb.read(np.float32).reshape(batch, 2)
    assert np.all(y[:, 0] == 39.0) and np.all(y[:, 1] == 80.0)
    tr.learn_gradient(xb.address, tb.address, batch)
    g = tr.read_grads()
    assert list(g[w_off[1]:w_off[1] + 8]) == [batch * v for v in [1, 2, 3, 4, 1, 2, 3, 4]]   # dW = B * x per row
    assert list(g[b_off[1]:b_off[1] + 2]) == [batch, batch]                                   # db = B
    assert list(g[b_off[0]:b_off[0] + 4]) == [batch * v for v in [6, 8, 10, 12]]              # B * dX
    mx, sm = tr.read_loss()
    assert mx == 0.5 and sm == 0.5 * batch


def _act_problem(hidden, output, dtype, count, seed):
    rng = np.random.default_rng(seed)
    dims = [6, 24, 17, 5]
    cfg = C.make_config(dims, dtype=dtype, hidden_act=hidden, output_act=output, act_alpha=0.05, adam_master=1)
    p0 = C.from_storage(C.init_params(cfg, seed=seed, scheme="xavier"), dtype).copy()
    w_off, b_off, _ = C.param_layout(cfg)
    if hidden == C.ACT_EXP or output == C.ACT_EXP:
        p0 *= 0.25  # exp of exp of exp: keep the pre-activations small enough to stay finite
    for l in range(cfg.n_layers):  # non-zero biases so that pre-activations are not centred on the tie points
        p0[b_off[l]:b_off[l] + dims[l + 1]] = rng.uniform(-0.3, 0.3, dims[l + 1])
    p0 = C.to_storage(p0, dtype)
    x = rng.uniform(-1.5, 1.5, (count, dims[0])).astype(np.float32)
    t = rng.uniform(-1, 1, (count, dims[-1])).astype(np.float32)
    return cfg, p0, x, t


@pytest.mark.parametrize("act", ALL_ACTS, ids=[ACT_NAME[a] for a in ALL_ACTS])
def test_every_activation_one_thread_per_sample(device, act):
    """fp32, hidden and output activation both `act`: bit-identical gradients with ordered sums (the
    kernels evaluate expf/sinf/tanhf with the CUDA math library, the oracle with glibc: the last-bit
    differences of those functions are what the 2e-6 below allows; piecewise-linear ones are exact)."""
    from oracle import oracle
    from slang_b200.api import FLAG_SEQUENTIAL_SUM, Trainer
    count = 300
    cfg, p0, x, t = _act_problem(act, act, C.F32, count, 100 + act)
    _, l_ref, g_ref, _ = oracle_trajectory(cfg, p0, [(x, t)])
    _, l_gpu, g_gpu, _, tr = gpu_trajectory(device, cfg, p0, [(x, t)], "learnGradient_simt", FLAG_SEQUENTIAL_SUM)
    assert tr.k_learn.implementation == "simt"
    err = max(layer_rel_errs(cfg, g_gpu, g_ref))
    exact = act in (C.ACT_IDENTITY, C.ACT_RELU, C.ACT_LEAKY_RELU, C.ACT_LEAKY_MAX)
    print(ACT_NAME[act], "simt fp32 gradient rel err %.3g" % err)
    assert np.all(np.isfinite(g_ref)) and np.any(g_ref != 0)
    assert err == 0.0 if exact else err < 2e-6
    assert abs(l_gpu[0][1] - l_ref[0][1]) <= 2e-6 * abs(l_ref[0][1])
    yb = device.create_buffer(count * cfg.out_dim * 4)
    xb = device.create_buffer(x.nbytes, x)
    tr2 = Trainer(device, cfg, p0, forward_entry="forward_simt")
    tr2.forward(xb.address, yb.address, count)
    y = yb.read(np.float32).reshape(count, cfg.out_dim)
    y_ref = oracle.forward(cfg, p0, x, count)
    assert np.max(np.abs(y - y_ref)) <= 2e-6 * max(1.0, float(np.max(np.abs(y_ref))))


@pytest.mark.parametrize("dtype", [C.F16, C.BF16], ids=["f16", "bf16"])
@pytest.mark.parametrize("act", ALL_ACTS, ids=[ACT_NAME[a] for a in ALL_ACTS])
def test_every_activation_on_the_padded_tensor_core_kernel(device, act, dtype):
    """16-bit storage, hidden and output activation both `act`, through "learnGradient" and "forward" of
    the padded tcgen05 kernel: gradients per tensor within 1e-2, loss within 1e-2, outputs within one
    storage rounding step of the oracle."""
    from oracle import oracle
    from slang_b200.api import Trainer
    count = 128 * 3 + 9
    cfg, p0, x, t = _act_problem(act, act, dtype, count, 200 + act)
    _, l_ref, g_ref, _ = oracle_trajectory(cfg, p0, [(x, t)])
    _, l_gpu, g_gpu, _, tr = gpu_trajectory(device, cfg, p0, [(x, t)])
    assert tr.k_learn.implementation == "tcgen05" and tr.k_forward.implementation == "tcgen05"
    err = max(layer_rel_errs(cfg, g_gpu, g_ref))
    print(ACT_NAME[act], "tcgen05 gradient rel err %.3g" % err)
    assert np.all(np.isfinite(g_ref)) and np.any(g_ref != 0)
    assert err < 1e-2
    assert abs(l_gpu[0][1] - l_ref[0][1]) <= 1e-2 * abs(l_ref[0][1])
    assert abs(l_gpu[0][0] - l_ref[0][0]) <= 1e-2 * abs(l_ref[0][0])
    xb = device.create_buffer(x.nbytes, x)
    yb = device.create_buffer(count * cfg.out_dim * 4)
    fresh = Trainer(device, cfg, p0)  # the trajectory above ended with an Adam step: forward with the initial parameters
    fresh.forward(xb.address, yb.address, count)
    y = yb.read(np.float32).reshape(count, cfg.out_dim)
    y_ref = oracle.forward(cfg, p0, x, count)
    step = 2.0 ** -7 if dtype == C.BF16 else 2.0 ** -10
    assert np.max(np.abs(y - y_ref)) <= 4 * step * max(1.0, float(np.max(np.abs(y_ref))))


def test_config2_trajectory_at_its_stated_length(device):
    """Config 2 (fp16 4-32-32-32-32-4, LeakyReLU, Adam 1e-3) for the 1000 steps the configuration names,
    on a batch of 4096.  Training is sensitive to rounding: two runs of the CPU oracle that differ only
    in how the batch is split over threads (a different grouping of the same fp32 sums) agree to 1e-5
    over the first hundred steps and drift apart by 16 % in per-step loss and 4 % in parameters by step
    1000 (fp64 accumulation against fp32: 23 % and more than 100 %).  So the stated bar (per-step loss
    within 1e-2, parameters within 2e-2) is checked where it is a property of the implementation, the
    first 150 steps, and the rest of the run is held to the oracle's own spread: the GPU's drift from the
    8-thread oracle stays within 3x the drift of the 1-thread oracle from the 8-thread oracle, and both
    runs converge to the same loss level."""
    count, steps = 4096, 1000
    cfg, p0, batches = make_problem("c2", count, seed=21, steps=steps)
    p_ref, l_ref, _, _ = oracle_trajectory(cfg, p0, batches, n_threads=8)
    p_alt, l_alt, _, _ = oracle_trajectory(cfg, p0, batches, n_threads=1)
    p_gpu, l_gpu, _, _, tr = gpu_trajectory(device, cfg, p0, batches)
    assert tr.k_learn.implementation == "tcgen05"
    dev_gpu = np.array([abs(sg - sr) / abs(sr) for (_, sg), (_, sr) in zip(l_gpu, l_ref)])
    dev_alt = np.array([abs(sa - sr) / abs(sr) for (_, sa), (_, sr) in zip(l_alt, l_ref)])
    fs = lambda p: C.from_storage(p, cfg.dtype)
    perr_gpu = max(per_layer_rel_errs(cfg, fs(p_gpu), fs(p_ref)))
    perr_alt = max(per_layer_rel_errs(cfg, fs(p_alt), fs(p_ref)))
    # parameters after the first 150 steps, from a second pair of runs
    p_ref150, _, _, _ = oracle_trajectory(cfg, p0, batches[:150], n_threads=8)
    p_gpu150, _, _, _, _ = gpu_trajectory(device, cfg, p0, batches[:150])
    perr150 = max(per_layer_rel_errs(cfg, fs(p_gpu150), fs(p_ref150)))
    tail = lambda l: float(np.mean([s for _, s in l[-50:]]))
    print("c2 x %d steps: per-step loss rel dev, steps 0-149: gpu %.3g (oracle spread %.3g); whole run: gpu %.3g (oracle spread %.3g); "
          "parameters after 150 steps %.3g, after 1000: gpu %.3g (oracle spread %.3g); loss %.4f -> %.4f (gpu %.4f)"
          % (steps, dev_gpu[:150].max(), dev_alt[:150].max(), dev_gpu.max(), dev_alt.max(), perr150, perr_gpu, perr_alt,
             l_ref[0][1], tail(l_ref), tail(l_gpu)))
    assert dev_gpu[:150].max() <= 1e-2
    assert perr150 < 2e-2
    assert dev_gpu.max() <= 3 * max(dev_alt.max(), 1e-2)
    assert perr_gpu <= 3 * max(perr_alt, 2e-2)
    assert abs(tail(l_gpu) - tail(l_ref)) <= 5e-2 * tail(l_ref)


def _run_learn(device, cfg, p, x, t, entry="learnGradient"):
    from slang_b200.api import Trainer
    tr = Trainer(device, cfg, p, learn_entry=entry)
    xs, ts = C.to_storage(x, cfg.input_dtype), C.to_storage(t, cfg.target_dtype)
    xb, tb = device.create_buffer(xs.nbytes, xs), device.create_buffer(ts.nbytes, ts)
    tr.learn_gradient(xb.address, tb.address, x.shape[0])
    return tr, tr.read_grads()


@pytest.mark.parametrize("entry", ["learnGradient", "learnGradient_simt"], ids=["tcgen05", "simt"])
@pytest.mark.parametrize("dtype", [C.F16, C.BF16], ids=["f16", "bf16"])
@pytest.mark.parametrize("size", [16, 32, 64])
def test_tiled_backward_identity_known_answer(device, size, dtype, entry):
    """tests/neural/mma-tiled-backward-test.slang:67-127: W = identity, input ones, dOut of thread t equal to
    t + 1 in every component, 32 threads: dInput = W^T dOut = dOut.  Here the tested layer is the second of
    two identity layers, so its dInput shows up as the first layer's bias gradient: sum over the 32 samples
    of (t + 1) = 528 per component; the tested layer's own dW and db are 528 as well (inputs are ones)."""
    batch = 32
    cfg = C.make_config([size, size, size], dtype, C.ACT_IDENTITY, loss=C.LOSS_L2_SUM, input_dtype=C.F32, target_dtype=C.F32)
    w_off, b_off, total = C.param_layout(cfg)
    p = np.zeros(total, dtype=np.float32)
    for l in range(2):
        p[w_off[l]:w_off[l] + size * size] = np.eye(size).reshape(-1)
    x = np.ones((batch, size), dtype=np.float32)
    # dOut = 2 (out - target) with out = 1  ->  target = 1 - (t + 1) / 2
    t = np.repeat((1.0 - (np.arange(batch) + 1) / 2.0)[:, None], size, axis=1).astype(np.float32)
    tr, g = _run_learn(device, cfg, C.to_storage(p, dtype), x, t, entry)
    assert tr.k_learn.implementation == ("tcgen05" if entry == "learnGradient" else "simt")
    want = batch * (batch + 1) / 2
    assert np.all(g[b_off[0]:b_off[0] + size] == want)                      # sum of dInput of the tested layer
    assert np.all(g[b_off[1]:b_off[1] + size] == want)                      # its bias gradient
    assert np.all(g[w_off[1]:w_off[1] + size * size] == want)               # its weight gradient (inputs are ones)


@pytest.mark.parametrize("dtype", [C.F16, C.BF16], ids=["f16", "bf16"])
@pytest.mark.parametrize("m", [3, 15, 23, 47])
def test_bias_sum_reduce_known_answer(device, m, dtype):
    """tests/neural/bias-sum-reduce.slang:38-67: every one of 128 threads holds dOut[i] = (i + 1) / 128 for an
    output width of 3, 15, 23 or 47; the reduced bias gradient is i + 1 (tolerance 0.001 there, exact here).
    Zero weights make the outputs zero, so the L2 targets -(i + 1) / 256 give exactly that dOut."""
    batch = 128
    cfg = C.make_config([8, 8, m], dtype, C.ACT_IDENTITY, loss=C.LOSS_L2_SUM, input_dtype=C.F32, target_dtype=C.F32)
    w_off, b_off, total = C.param_layout(cfg)
    p = np.zeros(total, dtype=np.float32)
    p[w_off[0]:w_off[0] + 64] = np.eye(8).reshape(-1)
    x = np.ones((batch, 8), dtype=np.float32)
    t = np.tile(-(np.arange(m) + 1) / 256.0, (batch, 1)).astype(np.float32)
    tr, g = _run_learn(device, cfg, C.to_storage(p, dtype), x, t)
    assert tr.k_learn.implementation == "tcgen05"
    assert list(g[b_off[1]:b_off[1] + m]) == [float(i + 1) for i in range(m)]


@pytest.mark.parametrize("dtype", [C.F16, C.BF16], ids=["f16", "bf16"])
@pytest.mark.parametrize("k,m", [(8, 8), (16, 32), (32, 16), (64, 64), (24, 40)])
def test_outer_product_accumulate_known_answer(device, k, m, dtype):
    """tests/neural/outerproduct-accumulate-test.slang:47-92: 128 threads, input[j] = (j + 1)(t + 1) / 128,
    dOut[i] = (M - i) / 128; the accumulated outer product is dW[i][j] = (M - i)(j + 1) * 129 / 256 within
    WorkgroupSize * 0.016 = 2.05 (the test's tolerance for half inputs), and within 1e-2 relative of the
    oracle, which rounds the inputs to the storage type as the kernel does."""
    batch = 128
    cfg = C.make_config([k, k, m], dtype, C.ACT_IDENTITY, loss=C.LOSS_L2_SUM, input_dtype=C.F32, target_dtype=C.F32)
    w_off, b_off, total = C.param_layout(cfg)
    p = np.zeros(total, dtype=np.float32)
    p[w_off[0]:w_off[0] + k * k] = np.eye(k).reshape(-1)
    x = ((np.arange(k) + 1)[None, :] * (np.arange(batch) + 1)[:, None] / 128.0).astype(np.float32)
    t = np.tile(-(m - np.arange(m)) / 256.0, (batch, 1)).astype(np.float32)
    ps = C.to_storage(p, dtype)
    tr, g = _run_learn(device, cfg, ps, x, t)
    assert tr.k_learn.implementation == "tcgen05"
    got = g[w_off[1]:w_off[1] + m * k].reshape(m, k)
    want = (m - np.arange(m))[:, None] * (np.arange(k) + 1)[None, :] * (129.0 / 256.0)
    assert np.max(np.abs(got - want)) <= 128 * 0.016
    _, _, g_ref, _ = oracle_trajectory(cfg, ps, [(x, t)])
    ref = g_ref[w_off[1]:w_off[1] + m * k].reshape(m, k)
    assert np.max(np.abs(got - ref)) <= 1e-2 * np.max(np.abs(ref))
