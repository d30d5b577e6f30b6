"""Driving the step from torch tensors.

The reference's other caller of this path passes torch tensors to Slang kernels through
TorchTensorViewAddress / TensorView (source/standard-modules/neural/bindless-storage.slang:247-336,
prelude/slang-cuda-prelude.h:5958): the kernels read device pointers and strides of tensors the
framework owns.  `TorchTrainer` does the same for this library: parameters and gradients live in
torch tensors (so torch.distributed collectives see them), inputs and targets are passed as tensors,
and every kernel is issued on torch's current CUDA stream.
"""
import torch

from . import config as C
from .api import Device, Trainer

TORCH_DTYPE = {C.F32: torch.float32, C.F16: torch.float16, C.BF16: torch.bfloat16}


class TorchTrainer:
    def __init__(self, cfg, params_init, device_index=None):
        if not torch.cuda.is_available():
            raise RuntimeError("a CUDA device is required (the library has no CPU fallback)")
        idx = torch.cuda.current_device() if device_index is None else device_index
        self.cfg = cfg
        self.stream = torch.cuda.current_stream(idx)
        self.device = Device(idx, self.stream.cuda_stream)
        _, _, total = C.param_layout(cfg)
        dev = torch.device("cuda", idx)
        self.params = torch.zeros(total, dtype=TORCH_DTYPE[cfg.dtype], device=dev)
        self.grads = torch.zeros(total, dtype=torch.float32, device=dev)
        self.trainer = Trainer(self.device, cfg, params_init, param_memory=(self.params.data_ptr(), self.grads.data_ptr()))

    def _check(self, t, width, dtype, what):
        if not (t.is_cuda and t.is_contiguous() and t.dim() == 2 and t.shape[1] == width and t.dtype == TORCH_DTYPE[dtype]):
            raise ValueError("%s must be a contiguous CUDA tensor [count, %d] of %s" % (what, width, TORCH_DTYPE[dtype]))

    def learn_gradient(self, inputs, targets, flags=0):
        self._check(inputs, self.cfg.input_width, self.cfg.input_dtype, "inputs")
        self._check(targets, self.cfg.out_dim, self.cfg.target_dtype, "targets")
        if inputs.shape[0] != targets.shape[0]:
            raise ValueError("inputs and targets disagree on the sample count")
        self.trainer.learn_gradient(inputs.data_ptr(), targets.data_ptr(), inputs.shape[0], flags)

    def adjust_parameters(self):
        self.trainer.adjust_parameters()

    def forward(self, inputs):
        self._check(inputs, self.cfg.input_width, self.cfg.input_dtype, "inputs")
        out = torch.empty((inputs.shape[0], self.cfg.out_dim), dtype=torch.float32, device=inputs.device)
        self.trainer.forward(inputs.data_ptr(), out.data_ptr(), inputs.shape[0])
        return out

    def loss(self):
        return self.trainer.read_loss()
