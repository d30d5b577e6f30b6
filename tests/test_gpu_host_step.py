"""HostStepper (the step whose batch starts in pinned host memory) against Trainer.learn_gradient on
resident data: same gradients and loss, with targets from the host and with targets from a teacher
network computed on the device; the copies are ordered against the kernels' own stream."""
import numpy as np
import pytest

from slang_b200 import config as C

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("with_teacher", [False, True], ids=["host_targets", "teacher"])
def test_host_step_matches_resident_step(with_teacher):
    import torch
    from slang_b200.api import FLAG_OUTPUT_STORAGE_TYPE, Device, Trainer
    from slang_b200.host_step import HostStepper
    torch.cuda.set_device(0)
    stream = torch.cuda.Stream(device=0)      # not the current stream: ordering must not depend on that
    device = Device(0, stream.cuda_stream)
    try:
        cfg = C.named_config("c4")
        count = 5 * 4096 + 333                  # several pieces and a ragged last one
        p0 = C.init_params(cfg, seed=4, scheme="xavier")
        gen = torch.Generator(device="cuda"); gen.manual_seed(9)
        x = torch.randn((count, 64), device="cuda", generator=gen).to(torch.bfloat16)
        teacher = Trainer(device, cfg, C.init_params(cfg, seed=5, scheme="xavier")) if with_teacher else None
        t = torch.empty((count, 64), dtype=torch.bfloat16, device="cuda")
        if with_teacher:
            torch.cuda.synchronize()
            teacher.forward(x.data_ptr(), t.data_ptr(), count, FLAG_OUTPUT_STORAGE_TYPE)
            device.wait()
        else:
            t.copy_((torch.randn((count, 64), device="cuda", generator=gen) * 0.3).to(torch.bfloat16))
        torch.cuda.synchronize()
        ref = Trainer(device, cfg, p0)
        ref.learn_gradient(x.data_ptr(), t.data_ptr(), count)
        g_ref, l_ref = ref.read_grads(), ref.read_loss()

        tr = Trainer(device, cfg, p0)
        xh = torch.empty((count, 64), dtype=torch.bfloat16, pin_memory=True); xh.copy_(x)
        th = None
        if not with_teacher:
            th = torch.empty((count, 64), dtype=torch.bfloat16, pin_memory=True); th.copy_(t)
        torch.cuda.synchronize()
        stepper = HostStepper(tr, chunk_samples=4096, teacher=teacher)
        grads_before_adam = {}
        orig_adjust = tr.adjust_parameters
        tr.adjust_parameters = lambda: grads_before_adam.setdefault("g", tr.read_grads())  # keep the gradients
        mx, mean = stepper.step(xh, th)
        g = grads_before_adam["g"]
        scale = float(np.max(np.abs(g_ref)))
        assert np.max(np.abs(g - g_ref)) <= 1e-4 * scale      # pieces add in a different order than one launch
        assert abs(mean * count - l_ref[1]) <= 1e-4 * abs(l_ref[1]) and mx == l_ref[0]
        assert stepper.h2d_bytes == count * 128 * (1 if with_teacher else 2) and stepper.d2h_bytes == 8
        tr.adjust_parameters = orig_adjust
    finally:
        device.destroy()


def test_host_step_refuses_a_device_with_a_private_stream():
    from slang_b200.api import Device, Trainer
    from slang_b200.host_step import HostStepper
    device = Device(0)
    try:
        cfg = C.named_config("c2")
        tr = Trainer(device, cfg, C.init_params(cfg, seed=1, scheme="xavier"))
        with pytest.raises(ValueError):
            HostStepper(tr)
    finally:
        device.destroy()
