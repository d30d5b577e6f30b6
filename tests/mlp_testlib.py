"""Shared pieces of the parity tests: seeded problems, the oracle trajectory and the GPU trajectory."""
import numpy as np

from oracle import oracle
from slang_b200 import config as C


def make_problem(name, count, seed=0, steps=1):
    """Config, initial parameters and `steps` seeded batches of `count` samples."""
    cfg = C.named_config(name)
    scheme = "kaiming" if name in ("c1", "c3") or name.startswith("c5") else "xavier"
    params0 = C.init_params(cfg, seed=seed, scheme=scheme)
    teacher = None
    if name == "c4":
        tparams = C.init_params(cfg, seed=seed + 1000, scheme="xavier")
        teacher = lambda x: oracle.forward(cfg, tparams, x, x.shape[0])
    batches = [C.synthetic_batch(name, cfg, count, seed, step=s, teacher_forward=teacher) for s in range(steps)]
    return cfg, params0, batches


def oracle_trajectory(cfg, params0, batches, acc_mode=0, n_threads=1):
    """Runs learnGradient + adjustParameters per batch on the CPU oracle.

    Returns (final params, per-step (max loss, mean loss), gradients of the first step, final states)."""
    _, _, total = C.param_layout(cfg)
    params = params0.copy()
    grads = np.zeros(total, dtype=np.float32)
    states = np.zeros(total, dtype=C.ADAM_STATE_DTYPE)
    states["master"] = C.from_storage(params0, cfg.dtype)
    losses, first_grads = [], None
    for x, t in batches:
        count = x.shape[0]
        words = np.zeros(2, dtype=np.uint32)
        oracle.learn_gradient(cfg, params, grads, x, t, count, words, acc_mode=acc_mode, n_threads=n_threads)
        if first_grads is None:
            first_grads = grads.copy()
        losses.append((float(words[:1].view(np.float32)[0]), float(words[1:].view(np.float32)[0]) / max(count, 1)))
        oracle.adjust_parameters(cfg, states, params, grads)
    return params, losses, first_grads, states


def gpu_trajectory(device, cfg, params0, batches, learn_entry="learnGradient", flags=0):
    from slang_b200.api import Trainer
    tr = Trainer(device, cfg, params0, learn_entry=learn_entry)
    losses, first_grads = [], None
    for x, t in batches:
        count = x.shape[0]
        xb = device.create_buffer(max(x.nbytes, 1), x if x.nbytes else None)
        tb = device.create_buffer(max(t.nbytes, 1), t if t.nbytes else None)
        tr.learn_gradient(xb.address, tb.address, count, flags)
        if first_grads is None:
            first_grads = tr.read_grads()
        mx, sm = tr.read_loss()
        losses.append((mx, sm / max(count, 1)))
        tr.adjust_parameters()
        device.wait()
        xb.destroy(); tb.destroy()
    return tr.read_params(), losses, first_grads, tr.read_states(), tr


def rel_err(a, b):
    """Largest absolute difference relative to the largest magnitude of the reference b."""
    a = np.asarray(a, dtype=np.float64); b = np.asarray(b, dtype=np.float64)
    scale = max(float(np.max(np.abs(b))), 1e-30)
    return float(np.max(np.abs(a - b))) / scale


def layer_rel_errs(cfg, a, b):
    """rel_err per weight matrix and per bias vector (parameters given as float arrays, padded layout)."""
    w_off, b_off, _ = C.param_layout(cfg)
    dims = cfg.layer_dims
    out = []
    for l in range(cfg.n_layers):
        nw = dims[l] * dims[l + 1]
        out.append(rel_err(a[w_off[l]:w_off[l] + nw], b[w_off[l]:w_off[l] + nw]))
        bb = b[b_off[l]:b_off[l] + dims[l + 1]]
        if np.max(np.abs(bb)) > 0:
            out.append(rel_err(a[b_off[l]:b_off[l] + dims[l + 1]], bb))
    return out


def per_layer_rel_errs(cfg, a, b):
    """rel_err per layer with the weight matrix and the bias vector taken together.

    Zero-initialised biases move by about +-lr per Adam step in the first steps whatever the size of
    their gradient, so the sign of a near-zero gradient decides a bias's early path; measured against
    the layer's own parameter scale that effect is small, measured against the bias vector alone it is not."""
    w_off, b_off, _ = C.param_layout(cfg)
    dims = cfg.layer_dims
    out = []
    for l in range(cfg.n_layers):
        nw = dims[l] * dims[l + 1]
        ia = np.concatenate([a[w_off[l]:w_off[l] + nw], a[b_off[l]:b_off[l] + dims[l + 1]]])
        ib = np.concatenate([b[w_off[l]:w_off[l] + nw], b[b_off[l]:b_off[l] + dims[l + 1]]])
        out.append(rel_err(ia, ib))
    return out
