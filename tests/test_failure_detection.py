"""Failure detection without a GPU fault.

CPU (gloo, world size 2): a rank that leaves between steps, and a rank that dies silently, are seen by
the survivor on the host before it enters the next collective: it gets an exception within the time
limit instead of a deadlock (slang_b200.dist.Membership).
GPU: a bounded device wait that runs out (an mbarrier nobody arrives on, a few thousand polls) ends
the kernel normally and surfaces as MLP_E_DEVICE_STATUS from mlp_wait exactly once; a collective whose
library reports an asynchronous error, or that does not finish in time, surfaces as MLP_E_COMM from
mlp_comm_wait (checked against a stand-in collective library built by the test).
"""
import os
import socket
import subprocess
import sys
import time

import numpy as np
import pytest
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _member(rank, world, port, out_dir, mode):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from slang_b200.dist import Membership, RankLeft, RankTimeout, allreduce_gradients
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    m = Membership(rank, world)
    g = torch.ones(16)
    outcome = "finished"
    t0 = time.monotonic()
    try:
        for step in range(4):
            if rank == 1 and step == 2:
                # between steps: the last exchange has completed, nothing of this rank is in flight
                if mode == "leave":
                    m.leave()
                os._exit(0)  # "silent": no announcement at all
            m.arrive(step, timeout_s=3.0)
            allreduce_gradients(g)
    except RankLeft as e:
        outcome = "left:%d:step%d" % (e.rank, step)
    except RankTimeout as e:
        outcome = "timeout:%d:step%d" % (e.rank, step)
    with open(os.path.join(out_dir, "outcome_%d.txt" % rank), "w") as f:
        f.write("%s %.2f %g" % (outcome, time.monotonic() - t0, float(g[0])))
    os._exit(0)  # the group is broken on purpose: no collective teardown


@pytest.mark.parametrize("mode", ["leave", "silent"])
def test_survivor_learns_of_a_missing_rank_before_the_next_collective(tmp_path, mode):
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_member, args=(r, 2, port, str(tmp_path), mode)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert p.exitcode == 0, "a rank hung or crashed"
    outcome, seconds, g0 = open(tmp_path / "outcome_0.txt").read().split()
    # two exchanges completed (1 -> 2 -> 4), the third was never entered
    assert float(g0) == 4.0
    if mode == "leave":
        assert outcome == "left:1:step2"
        assert float(seconds) < 3.0
    else:
        assert outcome == "timeout:1:step2"
        assert float(seconds) < 10.0


# ---- GPU --------------------------------------------------------------------------------------
@pytest.mark.gpu
def test_bounded_wait_that_runs_out_is_reported_once():
    from slang_b200.api import Device
    from slang_b200.lib import MlpError, check, load
    dev = Device(0)
    try:
        dev.wait()  # clean to begin with
        check(load().mlp_selftest_bounded_wait(dev.handle, 2000))
        with pytest.raises(MlpError) as info:
            dev.wait()
        assert info.value.code == -5
        assert "0x40000000" in str(info.value)  # the intended wait ran out; the "late" bit is not set
        dev.wait()  # reported once, then cleared
        # the context is intact: a real kernel still runs and is correct afterwards
        from slang_b200 import config as C
        from slang_b200.api import Trainer
        from mlp_testlib import make_problem
        cfg, p0, batches = make_problem("c2", 256, seed=3, steps=1)
        tr = Trainer(dev, cfg, p0)
        x, t = batches[0]
        xb, tb = dev.create_buffer(x.nbytes, x), dev.create_buffer(t.nbytes, t)
        tr.learn_gradient(xb.address, tb.address, 256)
        dev.wait()
        assert np.any(tr.read_grads() != 0)
    finally:
        dev.destroy()


FAKE_NCCL = r"""
// Stand-in for the collective library: every call succeeds and moves no data; the asynchronous error
// query starts failing after FAKE_NCCL_FAIL_AFTER calls (never, when that is negative), and the
// collectives park the stream behind a host callback for FAKE_NCCL_STALL_MS milliseconds.
#include <cuda_runtime.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>
typedef struct { char internal[128]; } ncclUniqueId;
typedef void* ncclComm_t;
static int queries = 0, aborted = 0;
static void stall(void* ms) { usleep(1000 * (long)(size_t)ms); }
int ncclGetUniqueId(ncclUniqueId* id) { memset(id, 7, sizeof *id); return 0; }
int ncclCommInitRank(ncclComm_t* c, int n, ncclUniqueId id, int r) { *c = (void*)0x1; return 0; }
int ncclCommDestroy(ncclComm_t c) { return 0; }
int ncclCommAbort(ncclComm_t c) { aborted = 1; const char* f = getenv("FAKE_NCCL_ABORT_FILE"); if (f) { FILE* h = fopen(f, "w"); if (h) fclose(h); } return 0; }
int ncclAllReduce(const void* s, void* d, size_t n, int t, int op, ncclComm_t c, cudaStream_t st)
{
    const char* ms = getenv("FAKE_NCCL_STALL_MS");
    if (ms && atol(ms) > 0) cudaLaunchHostFunc(st, stall, (void*)(size_t)atol(ms));
    return 0;
}
int ncclAllGather(const void* s, void* d, size_t n, int t, ncclComm_t c, cudaStream_t st) { return 0; }
int ncclGroupStart(void) { return 0; }
int ncclGroupEnd(void) { return 0; }
const char* ncclGetErrorString(int r) { return r == 0 ? "no error" : "remote process exited or there was a network error"; }
int ncclCommGetAsyncError(ncclComm_t c, int* out)
{
    const char* a = getenv("FAKE_NCCL_FAIL_AFTER");
    long after = a ? atol(a) : -1;
    ++queries;
    *out = (after >= 0 && queries > after) ? 6 /* ncclRemoteError */ : 0;
    return 0;
}
"""


def _comm_child(fake_lib, fail_after, stall_ms, timeout_ms, abort_file):
    """Runs in a fresh process so that the library binds the stand-in instead of the real NCCL."""
    code = r"""
import ctypes, os, sys
sys.path.insert(0, %r)
from slang_b200.api import Device, Comm, comm_unique_id
from slang_b200.lib import load
dev = Device(0)
comm = Comm(dev, 1, 0, comm_unique_id())
buf = dev.create_buffer(4096)
rc = load().mlp_allreduce_grads(dev.handle, comm.handle, buf.address, 1024, 0, 0)
assert rc == 0, rc
rc = load().mlp_comm_wait(dev.handle, comm.handle, %d)
print("RC", rc, load().mlp_last_error_string().decode())
""" % (ROOT, timeout_ms)
    env = dict(os.environ, SLANG_B200_NCCL_LIBRARY=fake_lib, FAKE_NCCL_FAIL_AFTER=str(fail_after),
               FAKE_NCCL_STALL_MS=str(stall_ms), FAKE_NCCL_ABORT_FILE=abort_file)
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("RC ")][-1]
    return int(line.split()[1]), line


@pytest.mark.gpu
def test_collective_errors_and_time_limits_surface_on_the_host(tmp_path):
    src = tmp_path / "fake_nccl.c"
    src.write_text("#include <stdio.h>\n" + FAKE_NCCL)
    lib = str(tmp_path / "libfake_nccl.so")
    subprocess.check_call(["gcc", "-shared", "-fPIC", "-O1", "-I/usr/local/cuda/include", str(src), "-o", lib,
                           "-L/usr/local/cuda/lib64", "-Wl,-rpath,/usr/local/cuda/lib64", "-lcudart"])
    # healthy: the wait returns 0 and nothing is aborted
    rc, line = _comm_child(lib, -1, 0, 2000, str(tmp_path / "a0"))
    assert rc == 0, line
    assert not os.path.exists(tmp_path / "a0")
    # the library reports an asynchronous error while the stream is still busy: MLP_E_COMM, communicator aborted
    rc, line = _comm_child(lib, 2, 1500, 10000, str(tmp_path / "a1"))
    assert rc == -6 and "remote process" in line, line
    assert os.path.exists(tmp_path / "a1")
    # no error, but the collective does not finish within the limit: MLP_E_COMM, communicator aborted
    rc, line = _comm_child(lib, -1, 1500, 200, str(tmp_path / "a2"))
    assert rc == -6 and "time limit" in line, line
    assert os.path.exists(tmp_path / "a2")
