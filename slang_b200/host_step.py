"""A whole training step whose inputs and targets start in host memory.

This is the call a host program makes when its batch is not already on the GPU: the batch is cut
into pieces, each piece is copied from pinned host memory on a copy stream while the previous piece
runs learnGradient on the compute stream, gradients accumulate across the pieces, an optional
all-reduce sums them over the data-parallel ranks, adjustParameters runs once, and the two loss words
are read back.  torch supplies the streams, events and pinned/device memory; all arithmetic is in
the library's kernels.
"""
import torch

from . import config as C

_TORCH_DTYPE = {C.F32: torch.float32, C.F16: torch.float16, C.BF16: torch.bfloat16}


class HostStepper:
    """trainer: the network being trained.  teacher: optional Trainer of a frozen network whose
    outputs are the targets; when given, only the inputs cross the host-device link and the targets
    are computed on the device, piece by piece, with the teacher's forward kernel."""

    def __init__(self, trainer, chunk_samples=1 << 21, allreduce=None, teacher=None):
        self.tr = trainer
        self.teacher = teacher
        cfg = trainer.cfg
        self.chunk = chunk_samples
        self.allreduce = allreduce
        dev = torch.device("cuda", trainer.device.ordinal)
        # The copies are ordered against the kernels with events, so the kernels' stream must be one
        # this class can record on and wait on: the stream the Device was created on.
        if trainer.device.stream is None:
            raise ValueError("HostStepper needs a Device created on a caller's stream (Device(ordinal, stream=...)): "
                             "the library's own private stream cannot be ordered against the copies")
        if teacher is not None and teacher.device is not trainer.device:
            raise ValueError("the teacher must run on the trainer's Device (same stream)")
        self.compute = (torch.cuda.default_stream(dev) if trainer.device.stream == 0
                        else torch.cuda.ExternalStream(trainer.device.stream, device=dev))
        self.x_dev = [torch.empty((chunk_samples, cfg.input_width), dtype=_TORCH_DTYPE[cfg.input_dtype], device=dev) for _ in range(2)]
        self.t_dev = [torch.empty((chunk_samples, cfg.out_dim), dtype=_TORCH_DTYPE[cfg.target_dtype], device=dev) for _ in range(2)]
        self.copy_stream = torch.cuda.Stream(device=dev)
        self.copy_done = [torch.cuda.Event() for _ in range(2)]
        self.compute_done = [torch.cuda.Event() for _ in range(2)]
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def step(self, x_host, t_host=None):
        """x_host, t_host: pinned CPU tensors [count, width] (t_host is None with a teacher).
        Returns (max loss, mean loss) of this rank's samples."""
        from .api import FLAG_OUTPUT_STORAGE_TYPE
        count = x_host.shape[0]
        compute = self.compute
        self.h2d_bytes = x_host.numel() * x_host.element_size()
        if self.teacher is None:
            self.h2d_bytes += t_host.numel() * t_host.element_size()
        n_chunks = (count + self.chunk - 1) // self.chunk
        for i in range(n_chunks):
            b = i & 1
            i0, i1 = i * self.chunk, min(count, (i + 1) * self.chunk)
            n = i1 - i0
            if i >= 2:
                self.copy_stream.wait_event(self.compute_done[b])
            with torch.cuda.stream(self.copy_stream):
                self.x_dev[b][:n].copy_(x_host[i0:i1], non_blocking=True)
                if self.teacher is None:
                    self.t_dev[b][:n].copy_(t_host[i0:i1], non_blocking=True)
                self.copy_done[b].record(self.copy_stream)
            compute.wait_event(self.copy_done[b])
            if self.teacher is not None:
                self.teacher.forward(self.x_dev[b].data_ptr(), self.t_dev[b].data_ptr(), n, FLAG_OUTPUT_STORAGE_TYPE)
            self.tr.learn_gradient(self.x_dev[b].data_ptr(), self.t_dev[b].data_ptr(), n, clear_loss=(i == 0))
            self.compute_done[b].record(compute)
        if self.allreduce is not None:
            self.allreduce()
        self.tr.adjust_parameters()
        mx, sm = self.tr.read_loss()  # device -> host, waits for the step
        self.d2h_bytes = 8
        return mx, sm / max(count, 1)
