"""Checkpoint and resume of a training run.

The reference has no training checkpoint (its nearest relatives are serialized modules and API
record/replay, docs/repro.md, docs/replays.md).  Here a checkpoint is one flat file holding everything
a step depends on: the padded parameter segment, the Adam state of every element (moments, per-element
iteration count, fp32 master copy), the configuration bytes, and the data position (seed, step), so
that a resumed run produces the same next step as an uninterrupted one.
"""
import ctypes
import io
import json

import numpy as np

from . import config as C

MAGIC = b"MLPB200CKPT1\n"


def save(path, trainer, seed, step):
    trainer.device.wait()
    params = trainer.read_params()
    states = trainer.read_states()
    cfg_bytes = bytes(ctypes.string_at(ctypes.addressof(trainer.cfg), ctypes.sizeof(trainer.cfg)))
    header = json.dumps({"seed": int(seed), "step": int(step), "total": int(trainer.total),
                         "params_bytes": int(params.nbytes), "states_bytes": int(states.nbytes),
                         "config_bytes": len(cfg_bytes)}).encode()
    with open(path, "wb") as f:
        f.write(MAGIC)
        f.write(len(header).to_bytes(4, "little"))
        f.write(header)
        f.write(cfg_bytes)
        f.write(np.ascontiguousarray(params).tobytes())
        f.write(np.ascontiguousarray(states).tobytes())


def load(path):
    """Returns (config, params array in the storage type, Adam states, seed, step)."""
    with open(path, "rb") as f:
        data = f.read()
    if not data.startswith(MAGIC):
        raise ValueError("not a checkpoint of this library")
    buf = io.BytesIO(data[len(MAGIC):])
    n = int.from_bytes(buf.read(4), "little")
    h = json.loads(buf.read(n))
    cfg = C.MlpConfig.from_buffer_copy(buf.read(h["config_bytes"]))
    params = np.frombuffer(buf.read(h["params_bytes"]), dtype=C.storage_np_dtype(cfg.dtype)).copy()
    states = np.frombuffer(buf.read(h["states_bytes"]), dtype=C.ADAM_STATE_DTYPE).copy()
    if params.size != h["total"] or states.size != h["total"]:
        raise ValueError("checkpoint is truncated")
    return cfg, params, states, h["seed"], h["step"]


def restore(trainer, params, states):
    """Loads parameters and optimiser state into an existing trainer of the same configuration."""
    trainer.params.write(params)
    trainer.states.write(states)
    trainer.grads.clear()
    trainer.device.wait()
