"""Per-step records of a training run: phase times from CUDA events and a JSON-lines log.

The reference's example reports one number, the loss word it reads back every tenth iteration
(examples/mlp-training/mlp-training.cpp:205-211), and its neural module has compile-time switches for
timing the three backward pieces separately (accelerate-vector-coopmat.slang:5-15).  Here a step's phases
(learnGradient, the gradient exchange between GPUs, adjustParameters) are bracketed by CUDA events on the
stream the kernels run on, read after the run without stalling it, and written one JSON object per step.
"""
import json
import time

import torch


class PhaseTimer:
    """Events around named phases of consecutive steps on one CUDA stream.

        timer = PhaseTimer(stream)
        for step in ...:
            timer.begin_step()
            learn(); timer.mark("learn_gradient")
            exchange(); timer.mark("exchange")
            adjust(); timer.mark("adjust_parameters")
        rows = timer.collect()   # synchronises once; one dict of milliseconds per step
    """

    def __init__(self, stream=None):
        self.stream = stream
        self._steps = []

    def _event(self):
        e = torch.cuda.Event(enable_timing=True)
        e.record(self.stream) if self.stream is not None else e.record()
        return e

    def begin_step(self):
        self._steps.append([("begin", self._event())])

    def mark(self, name):
        self._steps[-1].append((name, self._event()))

    def collect(self):
        if self._steps:
            self._steps[-1][-1][1].synchronize()
        rows = []
        for marks in self._steps:
            row = {}
            for (_, e0), (name, e1) in zip(marks[:-1], marks[1:]):
                row[name + "_ms"] = e0.elapsed_time(e1)
            row["step_ms"] = marks[0][1].elapsed_time(marks[-1][1])
            rows.append(row)
        self._steps = []
        return rows


class JsonlLogger:
    """One JSON object per line: step index, phase times, throughput, loss words when the caller has them."""

    def __init__(self, path):
        self.f = open(path, "w")
        self.t0 = time.time()

    def log(self, step, samples, phases, loss_max=None, loss_mean=None, **extra):
        rec = {"step": int(step), "samples": int(samples), "wall_s": time.time() - self.t0}
        rec.update(phases)
        if phases.get("step_ms"):
            rec["samples_per_s"] = samples / (phases["step_ms"] * 1e-3)
        if loss_max is not None:
            rec["loss_max"] = float(loss_max)
        if loss_mean is not None:
            rec["loss_mean"] = float(loss_mean)
        rec.update(extra)
        self.f.write(json.dumps(rec) + "\n")
        self.f.flush()

    def close(self):
        self.f.close()
