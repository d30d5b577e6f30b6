"""Host-side mirror of the reference example's host program over the C ABI.

`Device`, `Buffer` and `Kernel` wrap the opaque handles; `Trainer` plays the part of
ExampleProgram::execute (examples/mlp-training/mlp-training.cpp:92-214): it lays the parameters out
in the example's two-segment buffer, builds the network constant buffer of per-layer device
addresses, owns the Adam-state and loss buffers, and issues learnGradient / adjustParameters with the
grid the example would use, ceil(count / 256).
"""
import ctypes

import numpy as np

from . import config as C
from .lib import check, load


class LearnGradParams(ctypes.Structure):
    _fields_ = [("networkBuffer", ctypes.c_uint64), ("lossBuffer", ctypes.c_uint64),
                ("inputs", ctypes.c_uint64), ("count", ctypes.c_uint32)]


class AdjustParamsParams(ctypes.Structure):
    _fields_ = [("adamStates", ctypes.c_uint64), ("params", ctypes.c_uint64),
                ("gradients", ctypes.c_uint64), ("count", ctypes.c_uint32)]


class LearnGradParamsEx(ctypes.Structure):
    _fields_ = [("networkBuffer", ctypes.c_uint64), ("lossBuffer", ctypes.c_uint64),
                ("inputs", ctypes.c_uint64), ("targets", ctypes.c_uint64),
                ("count", ctypes.c_uint32), ("flags", ctypes.c_uint32)]


class LearnGradParamsEx2(ctypes.Structure):
    _fields_ = [("base", LearnGradParamsEx), ("inputGradients", ctypes.c_uint64)]


class ForwardParams(ctypes.Structure):
    _fields_ = [("networkBuffer", ctypes.c_uint64), ("inputs", ctypes.c_uint64),
                ("outputs", ctypes.c_uint64), ("count", ctypes.c_uint32), ("flags", ctypes.c_uint32)]


FLAG_SEQUENTIAL_SUM = 1
FLAG_OUTPUT_STORAGE_TYPE = 2
FLAG_INPUT_GRADIENT = 4


class Buffer:
    def __init__(self, device, handle, size):
        self.device, self.handle, self.size = device, handle, size
        self.address = load().mlp_buffer_address(handle)

    def clear(self, offset=0, size=None):
        check(load().mlp_buffer_clear(self.device.handle, self.handle, offset, self.size - offset if size is None else size))

    def read(self, dtype=np.uint8, offset=0, size=None):
        size = self.size - offset if size is None else size
        out = np.empty(size, dtype=np.uint8)
        check(load().mlp_buffer_read(self.device.handle, self.handle, offset, size, out.ctypes.data_as(ctypes.c_void_p)))
        return out.view(dtype)

    def write(self, array, offset=0):
        a = np.ascontiguousarray(array)
        check(load().mlp_buffer_write(self.device.handle, self.handle, offset, a.nbytes, a.ctypes.data_as(ctypes.c_void_p)))
        self.device.wait()  # the source array may be a temporary

    def destroy(self):
        if self.handle:
            load().mlp_buffer_destroy(self.handle)
            self.handle = None


class Kernel:
    def __init__(self, device, handle):
        self.device, self.handle = device, handle
        self.implementation = load().mlp_kernel_implementation(handle).decode()

    def dispatch(self, args, groups):
        check(load().mlp_dispatch(self.device.handle, self.handle, ctypes.byref(args), ctypes.sizeof(args), groups, 1, 1))


class Device:
    def __init__(self, ordinal=0, stream=None):
        h = ctypes.c_void_p()
        if stream is None:
            check(load().mlp_device_create(ordinal, ctypes.byref(h)))
        else:
            # `stream` is a cudaStream_t as an integer (0 = the legacy default stream)
            check(load().mlp_device_create_on_stream(ordinal, ctypes.c_void_p(stream), ctypes.byref(h)))
        self.handle = h
        self.ordinal = ordinal
        # the cudaStream_t the kernels run on when the caller supplied it; None when the library
        # created its own stream, which a caller cannot order other work against
        self.stream = stream

    def create_buffer(self, size, init=None):
        h = ctypes.c_void_p()
        if init is not None:
            init = np.ascontiguousarray(init)
            assert init.nbytes == size
            ptr = init.ctypes.data_as(ctypes.c_void_p)
        else:
            ptr = None
        check(load().mlp_buffer_create(self.handle, size, ptr, ctypes.byref(h)))
        b = Buffer(self, h, size)
        if init is None:
            b.clear()
        return b

    def wrap_buffer(self, address, size):
        h = ctypes.c_void_p()
        check(load().mlp_buffer_wrap(self.handle, address, size, ctypes.byref(h)))
        return Buffer(self, h, size)

    def kernel(self, entry_point, cfg=None):
        h = ctypes.c_void_p()
        if cfg is None:
            check(load().mlp_kernel_get(self.handle, entry_point.encode(), ctypes.byref(h)))
        else:
            check(load().mlp_kernel_get_for_config(self.handle, ctypes.byref(cfg), entry_point.encode(), ctypes.byref(h)))
        return Kernel(self, h)

    def matrix_convert(self, dst_address, dst_descs, src_address, src_descs):
        """convertCooperativeVectorMatrix: lists of MatrixDesc of equal length."""
        n = len(dst_descs)
        assert n == len(src_descs)
        d = (MatrixDesc * n)(*dst_descs)
        s_ = (MatrixDesc * n)(*src_descs)
        check(load().mlp_matrix_convert(self.handle, dst_address, d, src_address, s_, n))

    def load_kernel(self, image, entry_point):
        """A kernel from a caller-supplied device module (cubin or PTX bytes); dispatch passes the argument
        bytes as the packed parameter buffer, block (256,1,1)."""
        h = ctypes.c_void_p()
        check(load().mlp_kernel_load(self.handle, image, len(image), entry_point.encode(), ctypes.byref(h)))
        return Kernel(self, h)

    def wait(self):
        check(load().mlp_wait(self.handle))

    @property
    def launch_count(self):
        return int(load().mlp_device_launch_count(self.handle))

    def destroy(self):
        if self.handle:
            load().mlp_device_destroy(self.handle)
            self.handle = None


def groups_for(count):
    return (count + 255) // 256


MATRIX_ROW_MAJOR, MATRIX_COLUMN_MAJOR, MATRIX_INFERENCING_OPTIMAL, MATRIX_TRAINING_OPTIMAL = 0, 1, 2, 3


class MatrixDesc(ctypes.Structure):
    """MlpMatrixDesc: one matrix inside a buffer (component_type is an MlpDType)."""
    _fields_ = [("rows", ctypes.c_uint32), ("cols", ctypes.c_uint32), ("component_type", ctypes.c_int32),
                ("layout", ctypes.c_int32), ("size", ctypes.c_uint64), ("offset", ctypes.c_uint64),
                ("row_col_stride", ctypes.c_uint64)]


def matrix_size(rows, cols, component_type, layout, stride=0):
    out = ctypes.c_uint64()
    check(load().mlp_matrix_size(rows, cols, component_type, layout, stride, ctypes.byref(out)))
    return int(out.value)


COMM_ID_BYTES = 128
COMM_RANK_ORDERED_SUM = 1


def comm_unique_id():
    """128 bytes that rank 0 creates and hands to the other ranks (file, socket, store ...)."""
    buf = ctypes.create_string_buffer(COMM_ID_BYTES)
    check(load().mlp_comm_unique_id(buf, COMM_ID_BYTES))
    return buf.raw


class Comm:
    """The gradient exchange of a data-parallel run, one object per rank (mlp_comm_*)."""

    def __init__(self, device, nranks, rank, unique_id):
        assert len(unique_id) == COMM_ID_BYTES
        h = ctypes.c_void_p()
        check(load().mlp_comm_init(device.handle, nranks, rank, unique_id, COMM_ID_BYTES, ctypes.byref(h)))
        self.device, self.handle, self.nranks, self.rank = device, h, nranks, rank

    def allreduce_grads(self, trainer, with_loss=True, rank_ordered=False):
        check(load().mlp_allreduce_grads(self.device.handle, self.handle, trainer.grads.address, trainer.total,
                                         trainer.loss.address if with_loss else 0,
                                         COMM_RANK_ORDERED_SUM if rank_ordered else 0))

    def wait(self, timeout_ms=30000):
        """Host wait for the stream with the collective library's asynchronous errors polled; raises
        MlpError (MLP_E_COMM) after an error or the time limit, with the communicator aborted."""
        check(load().mlp_comm_wait(self.device.handle, self.handle, timeout_ms))

    def destroy(self):
        if self.handle:
            load().mlp_comm_destroy(self.handle)
            self.handle = None


class Trainer:
    """The example's host program for an arbitrary MlpConfig.

    Buffers (all device-local, created through the C ABI):
      params  segment 1: W0|b0|W1|b1|... in the storage type, 64-byte sub-allocations
      grads   segment 2: same element offsets, fp32
      states  MlpAdamState per element of segment 1
      network MlpLayerPointers per layer
      loss    two 32-bit words, cleared before every learnGradient
    """

    def __init__(self, device, cfg, params_init, learn_entry="learnGradient", forward_entry="forward",
                 param_memory=None):
        self.device, self.cfg = device, cfg
        self.w_off, self.b_off, self.total = C.param_layout(cfg)
        esz = C.DTYPE_SIZE[cfg.dtype]
        params_init = np.ascontiguousarray(params_init)
        assert params_init.nbytes == self.total * esz, "params_init must be the padded segment in the storage type"
        if param_memory is None:
            self.params = device.create_buffer(self.total * esz, params_init)
            self.grads = device.create_buffer(self.total * 4)
        else:
            # (params_address, grads_address): memory owned by the caller, e.g. tensors that a
            # collective library also sees.
            self.params = device.wrap_buffer(param_memory[0], self.total * esz)
            self.grads = device.wrap_buffer(param_memory[1], self.total * 4)
            self.params.write(params_init)
            self.grads.clear()
        states = np.zeros(self.total, dtype=C.ADAM_STATE_DTYPE)
        states["master"] = C.from_storage(params_init, cfg.dtype)
        self.states = device.create_buffer(states.nbytes, states)
        net = np.zeros((cfg.n_layers, 4), dtype=np.uint64)
        for l in range(cfg.n_layers):
            net[l] = [self.params.address + self.w_off[l] * esz, self.grads.address + self.w_off[l] * 4,
                      self.params.address + self.b_off[l] * esz, self.grads.address + self.b_off[l] * 4]
        self.network = device.create_buffer(net.nbytes, net)
        self.loss = device.create_buffer(8)
        self.k_learn = device.kernel(learn_entry, cfg)
        self.k_adjust = device.kernel("adjustParameters", cfg)
        self.k_forward = device.kernel(forward_entry, cfg)

    def learn_gradient(self, inputs_address, targets_address, count, flags=0, clear_loss=True, input_grads_address=0):
        """One learnGradient dispatch.  Gradients and the loss words accumulate across dispatches, so a
        batch may be fed in several pieces with clear_loss=False after the first.  With
        input_grads_address the gradient with respect to the inputs ([count][dims[0]] fp32) is written too."""
        if clear_loss:
            self.loss.clear()
        args = LearnGradParamsEx(self.network.address, self.loss.address, inputs_address, targets_address, count, flags)
        if input_grads_address:
            args.flags |= FLAG_INPUT_GRADIENT
            args = LearnGradParamsEx2(args, input_grads_address)
        self.k_learn.dispatch(args, groups_for(count))

    def adjust_parameters(self):
        args = AdjustParamsParams(self.states.address, self.params.address, self.grads.address, self.total)
        self.k_adjust.dispatch(args, groups_for(self.total))

    def forward(self, inputs_address, outputs_address, count, flags=0):
        args = ForwardParams(self.network.address, inputs_address, outputs_address, count, flags)
        self.k_forward.dispatch(args, groups_for(count))

    def read_loss(self):
        """(largest per-sample loss, sum of per-sample losses) of the last learnGradient."""
        w = self.loss.read(np.uint32)
        return float(w[:1].view(np.float32)[0]), float(w[1:2].view(np.float32)[0])

    def read_params(self):
        return self.params.read(C.storage_np_dtype(self.cfg.dtype))

    def read_grads(self):
        return self.grads.read(np.float32)

    def read_states(self):
        return self.states.read(np.uint8).view(C.ADAM_STATE_DTYPE)


class OptimalLayoutNetwork:
    """Forward pass over parameters that lie in the neural module's OptimalLayout (16x16 tiles in tensor-core
    B-fragment order, a padded bias slot behind every layer's weights: FFLayer's storage,
    source/standard-modules/neural/layers.slang:53-71), used in place: the per-layer device addresses point
    into the caller's buffer, nothing is converted.  `params_address` is that buffer on the device
    (C.optimal_layout_offsets gives its element offsets)."""

    def __init__(self, device, cfg, params_address, forward_entry="forward"):
        assert cfg.param_layout == C.PARAMS_OPTIMAL
        self.device, self.cfg = device, cfg
        esz = C.DTYPE_SIZE[cfg.dtype]
        w_off, b_off, self.total = C.optimal_layout_offsets(cfg.layer_dims)
        net = np.zeros((cfg.n_layers, 4), dtype=np.uint64)
        for l in range(cfg.n_layers):
            net[l] = [params_address + w_off[l] * esz, 0, params_address + b_off[l] * esz, 0]
        self.network = device.create_buffer(net.nbytes, net)
        self.k_forward = device.kernel(forward_entry, cfg)

    def forward(self, inputs_address, outputs_address, count, flags=0):
        args = ForwardParams(self.network.address, inputs_address, outputs_address, count, flags)
        self.k_forward.dispatch(args, groups_for(count))
