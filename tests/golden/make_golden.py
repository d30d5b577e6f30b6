"""Writes the golden fixtures of the parity tests from the CPU oracle.

    python tests/golden/make_golden.py

For each named configuration: seeded parameters and batches (slang_b200.config.synthetic_batch), a
few learnGradient + adjustParameters steps on the oracle (fp32 accumulate, one thread, ascending
sample order), and the results: gradients of the first step, per-step loss words, final parameters.
The reference itself cannot be built or run here (its compiler needs submodules that are not
vendored), so these vectors come from the oracle, whose per-operation behaviour is pinned by
tests/test_oracle_kat.py against the reference's own known answers.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from mlp_testlib import make_problem, oracle_trajectory  # noqa: E402

CASES = {"c1": (512, 5), "c2": (256, 4), "c3": (256, 4), "c4": (192, 3)}


def main():
    for name, (count, steps) in CASES.items():
        cfg, p0, batches = make_problem(name, count, seed=7, steps=steps)
        p, losses, g0, states = oracle_trajectory(cfg, p0, batches)
        np.savez_compressed(os.path.join(HERE, "%s.npz" % name), params0=p0, params=p, grads0=g0,
                            losses=np.array(losses, dtype=np.float64), iteration=states["iteration"],
                            count=count, steps=steps, seed=7)
        print(name, "written:", count, "samples x", steps, "steps")


if __name__ == "__main__":
    main()
