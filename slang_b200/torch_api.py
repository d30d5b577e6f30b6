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

    def _rows(self, t, width, dtype, what):
        """The tensor as dense rows.  The kernels read dense [count, width] rows; a strided view (a column
        slice, a transposed or stepped view: what the reference's TensorView reads through its strides,
        bindless-storage.slang:247-336) is packed by one strided copy on the same stream first."""
        if not (t.is_cuda and t.dim() == 2 and t.shape[1] == width and t.dtype == TORCH_DTYPE[dtype]):
            raise ValueError("%s must be a CUDA tensor [count, %d] of %s" % (what, width, TORCH_DTYPE[dtype]))
        if t.device.index != self.device.ordinal:
            raise ValueError("%s lives on another device" % what)
        return t if t.is_contiguous() else t.contiguous()

    def learn_gradient(self, inputs, targets, flags=0):
        inputs = self._rows(inputs, self.cfg.input_width, self.cfg.input_dtype, "inputs")
        targets = self._rows(targets, self.cfg.out_dim, self.cfg.target_dtype, "targets")
        if inputs.shape[0] != targets.shape[0]:
            raise ValueError("inputs and targets disagree on the sample count")
        self.trainer.learn_gradient(inputs.data_ptr(), targets.data_ptr(), inputs.shape[0], flags)

    def adjust_parameters(self):
        self.trainer.adjust_parameters()

    def forward(self, inputs, out=None):
        """Network outputs as fp32 [count, out_dim]; `out` may be any fp32 view of that shape (a strided one is
        filled through a dense temporary)."""
        inputs = self._rows(inputs, self.cfg.input_width, self.cfg.input_dtype, "inputs")
        dense = torch.empty((inputs.shape[0], self.cfg.out_dim), dtype=torch.float32, device=inputs.device)
        if out is not None:
            if not (out.is_cuda and out.dtype == torch.float32 and tuple(out.shape) == tuple(dense.shape)):
                raise ValueError("out must be a CUDA fp32 tensor [count, %d]" % self.cfg.out_dim)
            if out.is_contiguous():
                dense = out
        self.trainer.forward(inputs.data_ptr(), dense.data_ptr(), inputs.shape[0])
        if out is not None and dense is not out:
            out.copy_(dense)
            return out
        return dense

    def loss(self):
        return self.trainer.read_loss()
