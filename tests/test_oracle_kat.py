"""The oracle against the known answers held by the reference's own tests.

Each case names the reference test file and lines that state the expected numbers.
"""
import numpy as np
import pytest

from oracle import oracle
from slang_b200 import config as C


def _params(cfg, layers):
    """layers: list of (W [out][in], b [out]) -> padded storage-type segment."""
    w_off, b_off, total = C.param_layout(cfg)
    p = np.zeros(total, dtype=np.float32)
    for l, (w, b) in enumerate(layers):
        w = np.asarray(w, dtype=np.float32).reshape(-1)
        b = np.asarray(b, dtype=np.float32).reshape(-1)
        p[w_off[l]:w_off[l] + w.size] = w
        p[b_off[l]:b_off[l] + b.size] = b
    return C.to_storage(p, cfg.dtype)


def _grad_with_unit_dout(cfg, params, x, y, count=1, preset=None):
    """Gradients for dL/dout = `dout` using the L2 loss: target = out - dout/2."""
    w_off, b_off, total = C.param_layout(cfg)
    grads = np.zeros(total, dtype=np.float32) if preset is None else preset
    xs = np.tile(np.asarray(x, dtype=np.float32), (count, 1))
    tg = np.tile(np.asarray(y, dtype=np.float32), (count, 1))
    oracle.learn_gradient(cfg, params, grads, C.to_storage(xs, cfg.input_dtype), tg, count)
    return grads, w_off, b_off


def test_layout_matches_python_restatement():
    for name in ["c1", "c2", "c3", "c4", "c5_w16", "c5_w128"]:
        cfg = C.named_config(name)
        assert oracle.param_layout(cfg) == C.param_layout(cfg)
    # Appendix shapes: logical parameter counts of the benchmark configurations.
    assert C.logical_param_count(C.named_config("c1")) == 609
    assert C.logical_param_count(C.named_config("c2")) == 3460
    assert C.logical_param_count(C.named_config("c3")) == 10627
    assert C.logical_param_count(C.named_config("c4")) == 66112


def test_ffn_forward_known_answer():
    # tests/neural/basic-ilayer-ffn-forward-test.slang:56-68 : y = -40.5
    cfg = C.make_config([2, 2, 1], C.F32, C.ACT_IDENTITY, loss=C.LOSS_L2_SUM)
    p = _params(cfg, [([[2, -1], [0.5, 3]], [1, -2]), ([[-2, 4]], [0.5])])
    y = oracle.forward(cfg, p, np.array([[1.5, -2.0]], dtype=np.float32), 1)
    assert y.shape == (1, 1) and y[0, 0] == -40.5


def test_ffn_backward_known_answer():
    # tests/neural/basic-ilayer-ffn-backward-test.slang:76-93 : nine gradients for dL/dy = 1
    cfg = C.make_config([2, 2, 1], C.F32, C.ACT_IDENTITY, loss=C.LOSS_L2_SUM)
    p = _params(cfg, [([[2, -1], [0.5, 3]], [1, -2]), ([[-2, 4]], [0.5])])
    g, w_off, b_off = _grad_with_unit_dout(cfg, p, [1.5, -2.0], [-40.5 - 0.5])
    assert list(g[w_off[0]:w_off[0] + 4]) == [-3.0, 4.0, 6.0, -8.0]
    assert list(g[b_off[0]:b_off[0] + 2]) == [-2.0, 4.0]
    assert list(g[w_off[1]:w_off[1] + 2]) == [6.0, -7.25]
    assert list(g[b_off[1]:b_off[1] + 1]) == [1.0]


@pytest.mark.parametrize("dtype", [C.F32, C.F16])
@pytest.mark.parametrize("batch", [32, 64, 128])
def test_fflayer_batch_known_answer(dtype, batch):
    # tests/neural/fflayer-wavetangled-vector-test.slang:95-153 : forward [39, 80]; dInput [6,8,10,12];
    # dW = BatchSize * [[1,2,3,4],[1,2,3,4]]; dBias = [BatchSize, BatchSize].
    # An identity first layer exposes dInput of the tested layer as that layer's bias gradient.
    cfg = C.make_config([4, 4, 2], dtype, C.ACT_IDENTITY, loss=C.LOSS_L2_SUM)
    p = _params(cfg, [(np.eye(4), np.zeros(4)), ([[1, 2, 3, 4], [5, 6, 7, 8]], [9, 10])])
    x = [1.0, 2.0, 3.0, 4.0]
    y = oracle.forward(cfg, p, C.to_storage(np.array([x], dtype=np.float32), cfg.input_dtype), 1)
    assert list(y[0]) == [39.0, 80.0]
    g, w_off, b_off = _grad_with_unit_dout(cfg, p, x, [39.0 - 0.5, 80.0 - 0.5], count=batch)
    assert list(g[w_off[1]:w_off[1] + 8]) == [batch * v for v in [1, 2, 3, 4, 1, 2, 3, 4]]
    assert list(g[b_off[1]:b_off[1] + 2]) == [batch, batch]
    assert list(g[b_off[0]:b_off[0] + 4]) == [batch * v for v in [6, 8, 10, 12]]


def test_activation_known_answers():
    # tests/neural/activation-functions-test.slang:31-154
    A = oracle.activation
    assert [A(C.ACT_IDENTITY, 0, v) for v in (-1.0, 0.0, 2.5)] == [-1.0, 0.0, 2.5]
    assert [A(C.ACT_RELU, 0, v) for v in (-2.0, 0.0, 3.0)] == [0.0, 0.0, 3.0]
    np.testing.assert_allclose([A(C.ACT_LEAKY_RELU, 0.1, v) for v in (-2.0, 0.0, 3.0)], [-0.2, 0.0, 3.0], atol=1e-6)
    np.testing.assert_allclose([A(C.ACT_SIGMOID, 0, v) for v in (0.0, 1.0, -1.0)], [0.5, 0.7310586, 0.2689414], atol=1e-3)
    np.testing.assert_allclose([A(C.ACT_TANH, 0, v) for v in (0.0, 1.0, -1.0)], [0.0, 0.7615942, -0.7615942], atol=1e-3)
    np.testing.assert_allclose([A(C.ACT_EXP, 0, v) for v in (0.0, 1.0, -1.0)], [1.0, 2.7182818, 0.3678794], atol=1e-3)
    np.testing.assert_allclose([A(C.ACT_SINE, 0, v) for v in (0.0, np.pi / 2, np.pi)], [0.0, 1.0, 0.0], atol=1e-3)
    np.testing.assert_allclose([A(C.ACT_SILU, 0, v) for v in (0.0, 1.0, -1.0)], [0.0, 0.7310586, -0.2689414], atol=1e-3)
    np.testing.assert_allclose([A(C.ACT_QUICK_GELU, 0, v) for v in (0.0, 1.0, -1.0)], [0.0, 0.8458, -0.1542], atol=1e-3)


def test_activation_derivatives_against_finite_differences():
    D, A = oracle.activation_deriv, oracle.activation
    for act in range(11):
        for x in (-1.7, -0.3, 0.4, 2.1):
            h = 1e-3
            fd = (A(act, 0.01, x + h) - A(act, 0.01, x - h)) / (2 * h)
            assert abs(D(act, 0.01, x) - fd) < 2e-3, (act, x)


def test_max_tie_rule():
    # source/slang/diff.meta.slang:2268-2273 : a tie in max() sends half of the gradient to each side,
    # so ReLU = max(x, 0) has derivative 1/2 at exactly zero; the select form of LeakyReLU has 1.
    assert oracle.activation_deriv(C.ACT_RELU, 0.0, 0.0) == 0.5
    assert oracle.activation_deriv(C.ACT_LEAKY_RELU, 0.01, 0.0) == 1.0
    assert abs(oracle.activation_deriv(C.ACT_LEAKY_MAX, 0.001, 0.0) - 0.5005) < 1e-6


@pytest.mark.parametrize("acc_mode", [0, 1, 2])
def test_coopvec_matrix_mul_bias(acc_mode):
    # tests/cooperative-vector/matrix-mul-bias.slang:8-12 (runs on the reference's CPU target)
    cfg = C.make_config([4, 4], C.F16, C.ACT_IDENTITY, input_dtype=C.F16)
    p = _params(cfg, [(np.arange(1, 17).reshape(4, 4), [5, 6, 7, 8])])
    x = C.to_storage(np.array([[1, 2, 3, 4]], dtype=np.float32), C.F16)
    y = oracle.forward(cfg, p, x, 1, acc_mode=acc_mode)
    assert list(y[0]) == [35.0, 76.0, 117.0, 158.0]


def test_coopvec_outer_product_and_reduce_sum_accumulate():
    # tests/cooperative-vector/outer-product.slang:9-41 : A=[1..4], B=[1..8], output[0] preset to 111
    # tests/cooperative-vector/reduce-sum-accumulate.slang:9-13 : [111+1, 2, 3, 4]
    cfg = C.make_config([8, 4], C.F16, C.ACT_IDENTITY, loss=C.LOSS_L2_SUM, input_dtype=C.F16)
    p = _params(cfg, [(np.zeros((4, 8)), np.zeros(4))])
    w_off, b_off, total = C.param_layout(cfg)
    preset = np.zeros(total, dtype=np.float32)
    preset[w_off[0]] = 111.0
    preset[b_off[0]] = 111.0
    # out = 0, so target = -dout/2 gives dL/dout = [1, 2, 3, 4]
    g, _, _ = _grad_with_unit_dout(cfg, p, np.arange(1, 9), [-0.5, -1.0, -1.5, -2.0], preset=preset)
    expect = np.outer(np.arange(1, 5), np.arange(1, 9)).astype(np.float32).reshape(-1)
    expect[0] += 111.0
    assert list(g[w_off[0]:w_off[0] + 32]) == list(expect)
    assert list(g[b_off[0]:b_off[0] + 4]) == [112.0, 2.0, 3.0, 4.0]


def test_example_float_to_half_rounds_half_up():
    # examples/mlp-training/mlp-training.cpp:314-339
    f2h = oracle.example_float_to_half
    assert f2h(0.0) == 0 and f2h(1.0) == 0x3C00 and f2h(-2.0) == 0xC000
    assert f2h(65536.0) == 0x7C00 and f2h(1e-9) == 0
    # 1 + 2^-11 sits exactly between two halves: ties go up here, to even in IEEE.
    assert f2h(1.0 + 2.0 ** -11) == 0x3C01
    assert int(np.float16(1.0 + 2.0 ** -11).view(np.uint16)) == 0x3C00
    rng = np.random.default_rng(0)
    for v in rng.uniform(-1, 1, 200).astype(np.float32):
        got = np.array([f2h(float(v))], dtype=np.uint16).view(np.float16)[0]
        assert abs(float(got) - float(v)) <= 2.0 ** -11 * max(abs(float(v)), 2.0 ** -14)


def test_example_kernels_quirks():
    # examples/mlp-training/mlp_sw.slang:22-24 vs 35-39: negatives are scaled by 0.001 going forward
    # but their gradients by 0.01 going back; kernels.slang:22-27: the loss word is a running max.
    params = np.zeros(192, dtype=np.float16)
    grads = np.zeros(192, dtype=np.float16)
    # layer 1 (16x4) at 0, bias at 64; layer 2 (4x16) at 96, bias at 160 (64-byte sub-allocations of halfs)
    w1 = params[0:64].reshape(16, 4); b1 = params[64:80]
    w2 = params[96:160].reshape(4, 16); b2 = params[160:164]
    w1[0, 0] = -1.0
    w2[0, 0] = 1.0
    base_p, base_g = params.ctypes.data, grads.ctypes.data
    net = np.array([[base_p + 0, base_g + 0, base_p + 128, base_g + 128],
                    [base_p + 192, base_g + 192, base_p + 320, base_g + 320]], dtype=np.uint64)
    loss = np.zeros(2, dtype=np.uint32)
    x = np.array([[0.5, 0.25]], dtype=np.float32)
    oracle.example_learn_gradient(net, loss, x, 1)
    h = np.float16(-0.5) * np.float16(0.001)
    out0 = np.float16(h * np.float16(0.001))      # layer 2 applies the same leaky step to its own negative output
    gt0 = np.float16((0.5 + 0.25) / (1 + 0.25 * 0.25))
    diff0 = np.float16(out0 - gt0)
    g_out0 = np.float16(diff0 + diff0)           # out0 < 0, so the backward slope applies
    g_out0 = np.float16(g_out0 * np.float16(0.01))
    assert grads[160] == g_out0
    assert grads[96] == np.float16(g_out0 * h)
    assert loss[0] > 0
    before = int(loss[0])
    oracle.example_learn_gradient(net, loss, np.zeros((1, 2), dtype=np.float32), 1)
    assert int(loss[0]) == before  # a smaller loss does not lower the word


def test_example_half_arithmetic_rounds_every_operation():
    """The example oracle must round each half operation on its own (IEEE half arithmetic), not keep
    float intermediates: checked against a numpy float16 restatement of one sample."""
    rng = np.random.default_rng(1)
    params = rng.uniform(-1, 1, 192).astype(np.float16)
    grads = np.zeros(192, dtype=np.float16)
    P = params.copy()
    bp, bg = P.ctypes.data, grads.ctypes.data
    net = np.array([[bp, bg, bp + 128, bg + 128], [bp + 192, bg + 192, bp + 320, bg + 320]], dtype=np.uint64)
    loss = np.zeros(2, dtype=np.uint32)
    oracle.example_learn_gradient(net, loss, np.array([[0.3, 0.8]], dtype=np.float32), 1)
    h = np.float16

    def layer(W, b, xv, n_in, n_out):
        y = []
        for i in range(n_out):
            r = h(b[i])
            for j in range(n_in):
                r = h(r + h(W[i * n_in + j] * xv[j]))
            y.append(r)
        return [h(v * h(0.001)) if v < 0 else v for v in y]

    x, y = h(0.3), h(0.8)
    enc = [x, y, h(x * x), h(y * y)]
    h1 = layer(params[0:64], params[64:80], enc, 4, 16)
    out = layer(params[96:160], params[160:164], h1, 16, 4)
    gt = [h(h(x + y) / h(h(1) + h(y * y))), h(h(h(2) * x) + y),
          h(h(h(h(0.5) * x) * x) + h(h(1.2) * y)), h(x + h(h(h(0.5) * y) * y))]
    d = [h(out[k] - gt[k]) for k in range(4)]
    g2 = [h(d[k] + d[k]) for k in range(4)]
    g2 = [h(g2[k] * h(0.01)) if out[k] < 0 else g2[k] for k in range(4)]
    dW2 = np.array([h(g2[i] * h1[j]) for i in range(4) for j in range(16)], dtype=np.float16)
    assert np.array_equal(dW2.view(np.uint16), grads[96:160].view(np.uint16))
    assert np.array_equal(np.array(g2, dtype=np.float16).view(np.uint16), grads[160:164].view(np.uint16))
    total = h(0)
    for k in range(4):
        total = h(total + h(d[k] * d[k]))
    assert np.float32(total) == loss[:1].view(np.float32)[0]


def test_example_cpu_entry_point_flavours_agree():
    """The example kernels behind the CPU compute calling convention (docs/cpu-target.md:363-424): the
    group-range function, the per-group function and the per-thread function, driven in ascending
    order, leave the same bytes as the plain sequential loop."""
    rng = np.random.default_rng(11)
    count = 300   # two groups of 256, the second ragged
    init = np.zeros(384, dtype=np.uint16)
    init[:192] = rng.uniform(-1, 1, 192).astype(np.float16).view(np.uint16)
    inputs = rng.uniform(0, 1, 2 * count).astype(np.float32)
    offs = [(0, 128), (192, 320)]

    def run(mode):
        host = init.copy()
        base = host.ctypes.data
        net = np.array([[base + w, base + 384 + w, base + b, base + 384 + b] for w, b in offs], dtype=np.uint64)
        st = np.zeros(192, dtype=C.EXAMPLE_ADAM_STATE_DTYPE)
        loss = np.zeros(2, dtype=np.uint32)
        lp = oracle.EntryParams(net.ctypes.data, loss.ctypes.data, inputs.ctypes.data, count)
        ap = oracle.EntryParams(st.ctypes.data, base, base + 384, 192)
        for _ in range(2):
            if mode == "plain":
                oracle.example_learn_gradient(net, loss, inputs, count)
                oracle.example_adjust_parameters(st, host[:192], host[192:], 192)
            elif mode == "range":
                oracle.cpu_entry_range("learnGradient", lp, 0, 2)
                oracle.cpu_entry_range("adjustParameters", ap, 0, 1)
            elif mode == "split":
                oracle.cpu_entry_range("learnGradient", lp, 0, 1)
                oracle.cpu_entry_range("learnGradient", lp, 1, 2)
                oracle.cpu_entry_range("adjustParameters", ap, 0, 1)
            elif mode == "group":
                for g in range(2):
                    oracle.cpu_entry_group("learnGradient", lp, g)
                oracle.cpu_entry_group("adjustParameters", ap, 0)
            else:
                for g in range(2):
                    for t in range(256):
                        oracle.cpu_entry_thread("learnGradient", lp, g, t)
                for t in range(256):
                    oracle.cpu_entry_thread("adjustParameters", ap, 0, t)
        return host.copy(), st.copy(), loss.copy()

    ref = run("plain")
    assert ref[2][0] != 0 and np.any(ref[0][:192] != init[:192])
    for mode in ("range", "split", "group", "thread"):
        got = run(mode)
        assert np.array_equal(got[0], ref[0]), mode
        assert got[1].tobytes() == ref[1].tobytes(), mode
        assert np.array_equal(got[2], ref[2]), mode


# ---- summation order (MlpConfig.sum_order) -------------------------------------------------------
def _order_cfg(order):
    cfg = C.make_config([4, 1], C.F32, C.ACT_IDENTITY, loss=C.LOSS_L2_SUM, sum_order=order)
    return cfg


def test_neural_order_sums_from_zero_and_adds_the_bias_last():
    """source/standard-modules/neural/inline-vector.slang:101-110, 131-132: `output[row] += data[col] *
    rowAddr[col]` from a zero vector, then `output[i] + biasAddress[i]`.  With bias 2^27 (spacing 16) and
    four terms of 3 the order is visible: 12 + 2^27 rounds up to 2^27 + 16, while a sum that starts at the
    bias loses every term (examples/mlp-training/mlvec_sw.slang:31-34 starts from the bias)."""
    x = np.array([[3, 3, 3, 3]], dtype=np.float32)
    big = float(2 ** 27)
    for order, expect in ((C.SUM_NEURAL, big + 16.0), (C.SUM_BIAS_FIRST_FUSED, big)):
        cfg = _order_cfg(order)
        p = _params(cfg, [([[1, 1, 1, 1]], [big])])
        assert oracle.forward(cfg, p, x, 1)[0, 0] == expect


def test_neural_order_rounds_each_product_before_adding():
    """inline-vector.slang:108 multiplies and adds as two operations (and :156-157, :171-173 name the
    product `prod` before the add); source/slang/hlsl.meta.slang:33266-33274 does the same for the outer
    product.  -1 + (1 + 2^-12)^2: the rounded product is 1 + 2^-11, so the two-operation sum is 2^-11;
    a fused multiply-add keeps the 2^-24."""
    e = np.float32(2.0 ** -12)
    x = np.array([[1, 1 + e, 0, 0]], dtype=np.float32)
    w = [[-1, 1 + e, 0, 0]]
    for order, expect in ((C.SUM_NEURAL, 2.0 ** -11), (C.SUM_BIAS_FIRST_FUSED, 2.0 ** -11 + 2.0 ** -24)):
        cfg = _order_cfg(order)
        p = _params(cfg, [(w, [0])])
        assert oracle.forward(cfg, p, x, 1)[0, 0] == np.float32(expect)
    # dW = x * dy as a rounded product added to the running gradient: start the gradient at -1.
    for order, expect in ((C.SUM_NEURAL, 2.0 ** -11), (C.SUM_BIAS_FIRST_FUSED, 2.0 ** -11 + 2.0 ** -24)):
        cfg = C.make_config([1, 1], C.F32, C.ACT_IDENTITY, loss=C.LOSS_L2_SUM, sum_order=order)
        p = _params(cfg, [([[0]], [0])])
        w_off, _, total = C.param_layout(cfg)
        g = np.zeros(total, dtype=np.float32)
        g[w_off[0]] = -1.0
        # output 0, target -(1+e)/2  ->  dy = 2 * (0 + (1+e)/2) = 1 + e ; x = 1 + e
        oracle.learn_gradient(cfg, p, g, np.array([[1 + e]], dtype=np.float32), np.array([[-(1 + e) / 2]], dtype=np.float32), 1)
        assert g[w_off[0]] == np.float32(expect)


def test_config1_under_both_orders_stays_within_the_bar():
    """Config 1, 100 steps x 4096: the two orders are different roundings of the same sums; their
    parameters differ in the last bits and agree within the 1e-5 bar of the fp32 configuration."""
    import sys, os
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from mlp_testlib import layer_rel_errs, make_problem, oracle_trajectory
    cfg, p0, batches = make_problem("c1", 4096, seed=0, steps=100)
    assert cfg.sum_order == C.SUM_NEURAL
    p_neural, l_neural, _, _ = oracle_trajectory(cfg, p0, batches)
    cfg.sum_order = C.SUM_BIAS_FIRST_FUSED
    p_fused, l_fused, _, _ = oracle_trajectory(cfg, p0, batches)
    errs = layer_rel_errs(cfg, p_fused, p_neural)
    print("config 1 after 100 steps: bias-first/fused vs neural order, worst per-tensor rel diff %.3g; final mean loss %.6g vs %.6g"
          % (max(errs), l_fused[-1][1], l_neural[-1][1]))
    assert not np.array_equal(p_fused.view(np.uint32), p_neural.view(np.uint32))
    assert max(errs) < 1e-5
