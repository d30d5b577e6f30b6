"""Problem descriptions for the small-MLP training step and the host-side parameter layout.

`MlpConfig` mirrors `struct MlpConfig` of include/slang_b200_mlp_config.h field by field.  The
reference fixes the same facts at compile time (examples/mlp-training/network.slang:8-9,
examples/mlp-training/adam.slang:15-19, kLayerSizes in examples/mlp-training/mlp-training.cpp:24).

`param_layout` restates allocateNetworkParameterStorage (examples/mlp-training/mlp-training.cpp:217-250):
segment 1 is W0|b0|W1|b1|..., every sub-allocation rounded up to 64 bytes of the storage type; the
gradient segment and the Adam states use the same element offsets.
"""
import ctypes
import math

import numpy as np

MLP_MAX_LAYERS = 8

F32, F16, BF16 = 0, 1, 2
(ACT_IDENTITY, ACT_RELU, ACT_LEAKY_RELU, ACT_SIGMOID, ACT_TANH, ACT_EXP, ACT_SINE, ACT_SILU,
 ACT_QUICK_GELU, ACT_GELU_TANH, ACT_LEAKY_MAX) = range(11)
LOSS_MSE_MEAN, LOSS_L2_SUM = 0, 1
ENC_NONE, ENC_FREQ2D = 0, 1
# MlpSumOrder: neural module / cooperative-vector fallback order (zero start, rounded products, bias
# last) and the example's order (bias first, fused multiply-adds).
SUM_NEURAL, SUM_BIAS_FIRST_FUSED = 0, 1
# MlpParamLayout: the example's row-major weights, or the neural module's OptimalLayout (16x16 tiles in
# tensor-core B-fragment order, a padded bias slot behind every layer's weights).
PARAMS_ROW_MAJOR, PARAMS_OPTIMAL = 0, 1

DTYPE_SIZE = {F32: 4, F16: 2, BF16: 2}
DTYPE_NAME = {F32: "f32", F16: "f16", BF16: "bf16"}


class MlpConfig(ctypes.Structure):
    _fields_ = [
        ("n_layers", ctypes.c_int32),
        ("dims", ctypes.c_int32 * (MLP_MAX_LAYERS + 1)),
        ("dtype", ctypes.c_int32),
        ("input_dtype", ctypes.c_int32),
        ("target_dtype", ctypes.c_int32),
        ("hidden_act", ctypes.c_int32),
        ("output_act", ctypes.c_int32),
        ("act_alpha", ctypes.c_float),
        ("loss", ctypes.c_int32),
        ("encoding", ctypes.c_int32),
        ("input_width", ctypes.c_int32),
        ("lr", ctypes.c_float),
        ("beta1", ctypes.c_float),
        ("beta2", ctypes.c_float),
        ("eps", ctypes.c_float),
        ("adam_master", ctypes.c_int32),
        ("sum_order", ctypes.c_int32),
        ("param_layout", ctypes.c_int32),
        ("operand_dtype", ctypes.c_int32),
    ]

    @property
    def layer_dims(self):
        return [int(self.dims[i]) for i in range(self.n_layers + 1)]

    @property
    def out_dim(self):
        return int(self.dims[self.n_layers])


class MlpNetworkShape(ctypes.Structure):
    """Mirrors struct MlpNetworkShape: layer widths and one bias bit per layer."""
    _fields_ = [("n_layers", ctypes.c_int32), ("dims", ctypes.c_int32 * (MLP_MAX_LAYERS + 1)),
                ("bias_mask", ctypes.c_uint64), ("elem_bytes", ctypes.c_int32), ("reserved", ctypes.c_int32)]


def network_shape(dims, bias_mask, elem_bytes):
    s = MlpNetworkShape()
    s.n_layers = len(dims) - 1
    for i, d in enumerate(dims):
        s.dims[i] = d
    s.bias_mask, s.elem_bytes = bias_mask, elem_bytes
    return s


class MlpAdamState(ctypes.Structure):
    _fields_ = [("mean", ctypes.c_float), ("variance", ctypes.c_float),
                ("iteration", ctypes.c_int32), ("master", ctypes.c_float)]


ADAM_STATE_DTYPE = np.dtype([("mean", "<f4"), ("variance", "<f4"), ("iteration", "<i4"), ("master", "<f4")])
EXAMPLE_ADAM_STATE_DTYPE = np.dtype([("mean", "<u2"), ("variance", "<u2"), ("iteration", "<i4")])


def make_config(dims, dtype=F32, hidden_act=ACT_RELU, output_act=ACT_IDENTITY, act_alpha=0.01,
                loss=LOSS_MSE_MEAN, encoding=ENC_NONE, input_dtype=F32, target_dtype=F32,
                lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, adam_master=0, sum_order=SUM_NEURAL, operand_dtype=0):
    dims = list(dims)
    if not (1 <= len(dims) - 1 <= MLP_MAX_LAYERS):
        raise ValueError("layer count out of range")
    c = MlpConfig()
    c.n_layers = len(dims) - 1
    for i, d in enumerate(dims):
        c.dims[i] = d
    c.dtype, c.input_dtype, c.target_dtype = dtype, input_dtype, target_dtype
    c.hidden_act, c.output_act, c.act_alpha = hidden_act, output_act, act_alpha
    c.loss, c.encoding = loss, encoding
    c.input_width = 2 if encoding == ENC_FREQ2D else dims[0]
    c.lr, c.beta1, c.beta2, c.eps = lr, beta1, beta2, eps
    c.adam_master = adam_master
    c.sum_order = sum_order
    c.operand_dtype = operand_dtype  # F16 / BF16 with dtype F32: fp32 storage, 16-bit tensor-core operands
    return c


def named_config(name):
    """The benchmark configurations, in the order the baseline file lists them.

    c1: fp32 2-16-16-16-1, ReLU, linear output, MSE, Adam 1e-3.
    c2: fp16 4-32-32-32-32-4, LeakyReLU(0.01), MSE, Adam 1e-3, fp32 accumulate and moments.
    c3: fp16 frequency encoding (2 -> 32) then 32-64-64-64-3, ReLU, sigmoid output, L2, Adam 1e-2.
    c4: bf16 64-128-128-128-128-64, GELU (tanh form), MSE, Adam 3e-4.
    c5_w<w>: forward-only depth-4 ReLU MLP of constant width w, fp16 weights, fp32 outputs.
    """
    if name == "c1":
        return make_config([2, 16, 16, 16, 1], F32, ACT_RELU, lr=1e-3)
    if name == "c2":
        return make_config([4, 32, 32, 32, 32, 4], F16, ACT_LEAKY_RELU, act_alpha=0.01, lr=1e-3,
                           input_dtype=F32, target_dtype=F32, adam_master=1)
    if name == "c3":
        return make_config([32, 64, 64, 64, 3], F16, ACT_RELU, output_act=ACT_SIGMOID, loss=LOSS_L2_SUM,
                           encoding=ENC_FREQ2D, lr=1e-2, input_dtype=F32, target_dtype=F16, adam_master=1)
    if name == "c4":
        return make_config([64, 128, 128, 128, 128, 64], BF16, ACT_GELU_TANH, lr=3e-4,
                           input_dtype=BF16, target_dtype=BF16, adam_master=1)
    if name.startswith("c5_w"):
        w = int(name[4:])
        return make_config([w] * 5, F16, ACT_RELU, input_dtype=F16, target_dtype=F32)
    raise KeyError(name)


def param_layout(cfg):
    """Element offsets (weights, biases) per layer and the padded element count (of the row-major segment, or of
    the OptimalLayout buffer when cfg.param_layout says so)."""
    if cfg.param_layout == PARAMS_OPTIMAL:
        return optimal_layout_offsets(cfg.layer_dims)
    align = 64 // DTYPE_SIZE[cfg.dtype]
    off = 0
    w_off, b_off = [], []
    dims = cfg.layer_dims
    for l in range(cfg.n_layers):
        nw = dims[l] * dims[l + 1]
        w_off.append(off)
        off += (nw + align - 1) // align * align
        b_off.append(off)
        off += (dims[l + 1] + align - 1) // align * align
    return w_off, b_off, off


def optimal_layout_offsets(dims):
    """Element offsets (weights, biases) per layer and the element count of a network in OptimalLayout:
    per layer align16(in) * align16(out) weights, then align16(out) bias slots (reserved for every layer)."""
    a16 = lambda v: (v + 15) // 16 * 16
    off, w_off, b_off = 0, [], []
    for l in range(len(dims) - 1):
        w_off.append(off)
        off += a16(dims[l]) * a16(dims[l + 1])
        b_off.append(off)
        off += a16(dims[l + 1])
    return w_off, b_off, off


def logical_param_count(cfg):
    dims = cfg.layer_dims
    return sum(dims[l] * dims[l + 1] + dims[l + 1] for l in range(cfg.n_layers))


def flops_per_sample(cfg, training=True):
    """2W forward, 2W for dW and 2(W - in0*out0) for dX (the first layer's input gradient is dead)."""
    dims = cfg.layer_dims
    w = sum(dims[l] * dims[l + 1] for l in range(cfg.n_layers))
    if not training:
        return 2 * w
    return 2 * w + 2 * w + 2 * (w - dims[0] * dims[1])


# ----------------------------------------------------------------------------------------------
# 16-bit storage types as numpy uint16 bit patterns (numpy has no bfloat16).
# ----------------------------------------------------------------------------------------------
def f32_to_bf16_bits(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = (u + (0x7FFF + ((u >> 16) & 1))) >> 16
    r = np.where(nan, (u >> 16) | 0x40, r)
    return r.astype(np.uint16)


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def to_storage(x, dtype):
    """float array -> array in the storage type (float32, float16, or uint16 bf16 bit patterns)."""
    x = np.asarray(x, dtype=np.float32)
    if dtype == F32:
        return np.ascontiguousarray(x)
    if dtype == F16:
        return np.ascontiguousarray(x.astype(np.float16))
    return f32_to_bf16_bits(x)


def from_storage(a, dtype):
    if dtype == F32:
        return np.asarray(a, dtype=np.float32)
    if dtype == F16:
        return np.asarray(a).view(np.float16).astype(np.float32)
    return bf16_bits_to_f32(np.asarray(a).view(np.uint16))


def storage_np_dtype(dtype):
    return {F32: np.float32, F16: np.float16, BF16: np.uint16}[dtype]


# ----------------------------------------------------------------------------------------------
# Seeded initialisation and synthetic batches.
# ----------------------------------------------------------------------------------------------
def init_params(cfg, seed=0, scheme="kaiming"):
    """Padded parameter segment in the storage type: uniform weights, zero biases, zero padding.

    kaiming: bound sqrt(6 / fan_in); xavier: bound sqrt(6 / (fan_in + fan_out)).
    """
    rng = np.random.Generator(np.random.Philox(seed))
    w_off, b_off, total = param_layout(cfg)
    p = np.zeros(total, dtype=np.float32)
    dims = cfg.layer_dims
    for l in range(cfg.n_layers):
        fan_in, fan_out = dims[l], dims[l + 1]
        bound = math.sqrt(6.0 / fan_in) if scheme == "kaiming" else math.sqrt(6.0 / (fan_in + fan_out))
        w = rng.uniform(-bound, bound, size=fan_in * fan_out).astype(np.float32)
        p[w_off[l]:w_off[l] + w.size] = w
    return to_storage(p, cfg.dtype)


def unit_vectors(seed, n, dim):
    rng = np.random.Generator(np.random.Philox(seed))
    v = rng.normal(size=(n, dim))
    return (v / np.linalg.norm(v, axis=1, keepdims=True)).astype(np.float32)


def gaussian_blobs(seed, n_blobs=16, channels=3):
    rng = np.random.Generator(np.random.Philox(seed))
    centres = rng.uniform(0.0, 1.0, size=(channels, n_blobs, 2))
    sigma = rng.uniform(0.01, 0.1, size=(channels, n_blobs))
    return centres, sigma


def synthetic_batch(name, cfg, count, seed, step=0, teacher_forward=None):
    """Inputs and targets of one step, in the buffers' storage types.

    c1: x ~ U[-1,1]^2, target sin(pi x0) cos(pi x1).
    c2: x ~ U[0,1]^4, target_k = sin(2 pi x.w_k) for four fixed seeded unit vectors.
    c3: pixel centres of a sqrt(count)^2 grid (or seeded uniform coordinates when count is not a
        square), target = per-channel sum of 16 seeded Gaussian blobs.
    c4: x ~ N(0,1)^64 rounded to bf16, target = teacher_forward(x) (a frozen network of the same shape).
    c5: x ~ U[-1,1]^w, no target.
    """
    rng = np.random.Generator(np.random.Philox(key=seed, counter=[step, 0, 0, 0]))
    if name == "c1":
        x = rng.uniform(-1.0, 1.0, size=(count, 2)).astype(np.float32)
        t = (np.sin(np.pi * x[:, 0].astype(np.float64)) * np.cos(np.pi * x[:, 1].astype(np.float64)))
        return x, t.astype(np.float32).reshape(count, 1)
    if name == "c2":
        x = rng.uniform(0.0, 1.0, size=(count, 4)).astype(np.float32)
        w = unit_vectors(1234, 4, 4)
        t = np.sin(2.0 * np.pi * (x.astype(np.float64) @ w.T.astype(np.float64)))
        return x, t.astype(np.float32)
    if name == "c3":
        side = int(round(math.sqrt(count)))
        if side * side == count:
            ys, xs = np.divmod(np.arange(count), side)
            x = np.stack([(xs + 0.5) / side, (ys + 0.5) / side], axis=1).astype(np.float32)
        else:
            x = rng.uniform(0.0, 1.0, size=(count, 2)).astype(np.float32)
        centres, sigma = gaussian_blobs(4321)
        t = np.zeros((count, 3), dtype=np.float64)
        xd = x.astype(np.float64)
        for ch in range(3):
            for b in range(centres.shape[1]):
                d2 = ((xd - centres[ch, b]) ** 2).sum(axis=1)
                t[:, ch] += np.exp(-d2 / (2.0 * sigma[ch, b] ** 2))
        return x, to_storage(np.clip(t, 0.0, 1.0).astype(np.float32), cfg.target_dtype)
    if name == "c4":
        x = to_storage(rng.normal(size=(count, 64)).astype(np.float32), BF16)
        t = teacher_forward(x)
        return x, to_storage(t, cfg.target_dtype)
    if name.startswith("c5"):
        w = cfg.dims[0]
        x = rng.uniform(-1.0, 1.0, size=(count, w)).astype(np.float32)
        return to_storage(x, cfg.input_dtype), None
    raise KeyError(name)
