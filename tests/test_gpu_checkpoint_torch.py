"""Checkpoint/resume and the torch-tensor front end."""
import numpy as np
import pytest

from slang_b200 import config as C

from mlp_testlib import make_problem

pytestmark = pytest.mark.gpu


def test_resume_reproduces_the_next_steps(tmp_path):
    """Six steps in one go against three steps, checkpoint, fresh trainer, three more: identical
    parameters and optimiser state (config 1 with ordered sums, so every step is deterministic)."""
    from slang_b200 import checkpoint
    from slang_b200.api import Device, FLAG_SEQUENTIAL_SUM, Trainer
    cfg, p0, batches = make_problem("c1", 777, seed=8, steps=6)
    dev = Device(0)
    try:
        def run(tr, some):
            for x, t in some:
                xb, tb = dev.create_buffer(x.nbytes, x), dev.create_buffer(t.nbytes, t)
                tr.learn_gradient(xb.address, tb.address, x.shape[0], FLAG_SEQUENTIAL_SUM)
                tr.adjust_parameters()
                dev.wait()
                xb.destroy(); tb.destroy()
        a = Trainer(dev, cfg, p0, learn_entry="learnGradient_simt")
        run(a, batches)
        b = Trainer(dev, cfg, p0, learn_entry="learnGradient_simt")
        run(b, batches[:3])
        path = str(tmp_path / "ckpt.bin")
        checkpoint.save(path, b, seed=8, step=3)
        cfg2, params, states, seed, step = checkpoint.load(path)
        assert (seed, step) == (8, 3) and bytes(cfg2) == bytes(cfg)
        c = Trainer(dev, cfg2, p0, learn_entry="learnGradient_simt")
        checkpoint.restore(c, params, states)
        run(c, batches[step:])
        assert np.array_equal(c.read_params().view(np.uint32), a.read_params().view(np.uint32))
        sa, sc = a.read_states(), c.read_states()
        for f in ("mean", "variance", "master"):
            assert np.array_equal(sa[f].view(np.uint32), sc[f].view(np.uint32))
        assert np.array_equal(sa["iteration"], sc["iteration"])
    finally:
        dev.destroy()


def test_torch_front_end_matches_buffer_front_end():
    import torch
    from slang_b200.api import Device, Trainer
    from slang_b200.torch_api import TorchTrainer
    cfg, p0, batches = make_problem("c2", 1000, seed=9, steps=1)
    x, t = batches[0]
    tt = TorchTrainer(cfg, p0)
    xt, ttg = torch.from_numpy(x).cuda(), torch.from_numpy(t).cuda()
    tt.learn_gradient(xt, ttg)
    g_torch = tt.grads.cpu().numpy()
    dev = Device(0)
    try:
        tr = Trainer(dev, cfg, p0)
        xb, tb = dev.create_buffer(x.nbytes, x), dev.create_buffer(t.nbytes, t)
        tr.learn_gradient(xb.address, tb.address, 1000)
        g_buf = tr.read_grads()
    finally:
        dev.destroy()
    scale = np.max(np.abs(g_buf))
    assert np.max(np.abs(g_torch - g_buf)) <= 1e-5 * scale  # same kernel; only the atomic order differs
    with pytest.raises(ValueError):
        tt.learn_gradient(xt[:, :2], ttg)
    # strided views: every other row of a taller tensor, a column slice of a wider one, a transposed target
    wide_x = torch.zeros((2000, 6), device="cuda")
    wide_x[::2, 1:5] = xt
    t_t = ttg.t().contiguous().t()          # same values, column-major strides
    assert not wide_x[::2, 1:5].is_contiguous() and not t_t.is_contiguous()
    tt.grads.zero_()
    tt.learn_gradient(wide_x[::2, 1:5], t_t)
    g_view = tt.grads.cpu().numpy()
    assert np.max(np.abs(g_view - g_buf)) <= 1e-5 * scale
    out_wide = torch.zeros((1000, 8), device="cuda")
    y = tt.forward(xt)
    tt.forward(wide_x[::2, 1:5], out=out_wide[:, 2:6])
    assert torch.equal(out_wide[:, 2:6], y) and not out_wide[:, :2].any() and not out_wide[:, 6:].any()
    tt.adjust_parameters()
    torch.cuda.synchronize()
    assert torch.isfinite(tt.params.float()).all()
