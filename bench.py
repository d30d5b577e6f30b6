"""Benchmark of the small-MLP training step (learnGradient + gradient all-reduce + adjustParameters).

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--config c4] [--batch B]

Workload (default): the wide bf16 network 64-128-128-128-128-64 with GELU (tanh form), global batch
2^26 split evenly over the N GPUs of one node (strong scaling), MSE against a frozen seeded teacher
network of the same shape, an fp32 all-reduce of the flat gradient buffer (NCCL over NVLink) and a
replicated Adam step.  Inputs are seeded synthetic N(0,1) in bf16; the teacher's outputs are computed
once during set-up.  Two resident batches alternate between steps; each is far larger than L2.

One JSON line is printed by rank 0:
  value      samples/s with the inputs resident in HBM (K steps, CUDA events, max over ranks)
  e2e        samples/s through the host-buffer step (pinned host inputs copied in the timed region)
  roofline   achieved TFLOP/s of the learnGradient kernel against the measured bf16 peak
  cpu_baseline  the CPU oracle timed on this box's host cores on a bounded sample (N = 1 only)
`--impl reference` times the CPU oracle (the reference's CPU-target semantics restated in C++; the
reference itself cannot be built or run here) on all host threads and prints the same line shape.
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "MLP train samples/sec (fwd+bwd+Adam)"
UNIT = "samples/s"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"bf16_burst": d["bf16_tflops"], "bf16_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                "hbm_gbs": d["hbm_gbs"], "source": "measured"}
    return {"bf16_burst": 1590.0, "bf16_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML every 200 ms while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._halt = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
        }
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._halt.wait(0.2)

    def stop(self):
        self._halt.set()
        self.join(timeout=2)
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def oracle_rate(cfg, name, threads, target_seconds):
    """samples/s of the CPU oracle's learnGradient + adjustParameters on a bounded sample."""
    from oracle import oracle
    from slang_b200 import config as C
    p0 = C.init_params(cfg, seed=1, scheme="xavier")
    teacher = C.init_params(cfg, seed=2, scheme="xavier")
    _, _, total = C.param_layout(cfg)

    def run(n):
        rng = np.random.default_rng(3)
        x = C.to_storage(rng.normal(size=(n, cfg.dims[0])).astype(np.float32), cfg.input_dtype)
        t = C.to_storage(oracle.forward(cfg, teacher, x, min(n, 256)).repeat((n + 255) // 256, axis=0)[:n], cfg.target_dtype)
        params = p0.copy()
        grads = np.zeros(total, dtype=np.float32)
        states = np.zeros(total, dtype=C.ADAM_STATE_DTYPE)
        states["master"] = C.from_storage(p0, cfg.dtype)
        t0 = time.perf_counter()
        oracle.learn_gradient(cfg, params, grads, x, t, n, n_threads=threads)
        oracle.adjust_parameters(cfg, states, params, grads)
        return time.perf_counter() - t0

    n = 256 * threads
    run(n)  # first touch of the library, the thread pool and the pages
    dt = run(n)
    n_big = int(max(n, min(1 << 20, n * 0.5 * target_seconds / max(dt, 1e-6))))
    n_big = (n_big + 255) // 256 * 256
    dt = 0.5 * (run(n_big) + run(n_big))  # two passes: a single pass moved by a third between runs on one box
    return n_big / dt, n_big, dt


def reference_arm(args, rank):
    """The reference's CPU implementation of the path, as far as it exists here: the CPU oracle port."""
    if rank != 0:
        return
    from slang_b200 import config as C
    cfg = C.named_config(args.config)
    threads = os.cpu_count() or 1
    rates, sample = [], None
    per_step = max(2.0, min(20.0, 120.0 / max(args.steps + args.warmup, 1)))
    for i in range(args.warmup + args.steps):
        r, n, dt = oracle_rate(cfg, args.config, threads, per_step)
        sample = n
        if i >= args.warmup:
            rates.append((r, dt))
    total_dt = sum(dt for _, dt in rates)
    value = sample * len(rates) / total_dt
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * total_dt / len(rates), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload_name(args), "global_batch": args.batch, "step_sample": sample,
                   "note": "each step is a bounded sample of the workload on host cores"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": "%d samples per step, learnGradient + adjustParameters, %d threads" % (sample, threads)},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_name(args):
    return {"c4": "bf16 MLP 64-128-128-128-128-64 GELU(tanh), MSE vs frozen teacher, Adam lr 3e-4"}.get(args.config, args.config)


def teacher_targets(torch, cfg, x, seed):
    """Outputs of a frozen seeded network of the same shape, in bf16 (set-up only; plain torch)."""
    from slang_b200 import config as C
    tp = C.from_storage(C.init_params(cfg, seed=seed, scheme="xavier"), cfg.dtype)
    w_off, b_off, _ = C.param_layout(cfg)
    dims = cfg.layer_dims
    dev = x.device
    Ws = [torch.from_numpy(tp[w_off[l]:w_off[l] + dims[l] * dims[l + 1]].reshape(dims[l + 1], dims[l]).copy()).to(dev).to(torch.bfloat16) for l in range(cfg.n_layers)]
    out = torch.empty((x.shape[0], dims[-1]), dtype=torch.bfloat16, device=dev)
    step = 1 << 21
    for i0 in range(0, x.shape[0], step):
        a = x[i0:i0 + step]
        for l in range(cfg.n_layers):
            z = (a @ Ws[l].t()).float()
            a = (torch.nn.functional.gelu(z, approximate="tanh") if l < cfg.n_layers - 1 else z).to(torch.bfloat16)
        out[i0:i0 + step] = a
    return out


def measure_forward_points(torch, device, dev_t, widths, batches, warmup, steps):
    """Forward-only points: depth-4 ReLU networks of constant width (fp16 weights, Kaiming-uniform, seed 7;
    inputs uniform in [-1, 1]; fp32 outputs).  Each point: samples/s, achieved HBM GB/s over the
    algorithmic 6w bytes per sample against the measured copy bandwidth, and TFLOP/s.  L2 is flushed
    between timed iterations."""
    from slang_b200 import config as C
    from slang_b200.api import Trainer
    peaks = measured_peaks()
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev_t)
    points = []
    for w in widths:
        cfg = C.named_config("c5_w%d" % w)
        tr = Trainer(device, cfg, C.init_params(cfg, seed=7, scheme="kaiming"))
        assert tr.k_forward.implementation == "tcgen05"
        for n in batches:
            gen = torch.Generator(device=dev_t); gen.manual_seed(7)
            x = torch.empty((n, w), dtype=torch.float16, device=dev_t)
            piece = 1 << 22
            for i0 in range(0, n, piece):
                x[i0:i0 + piece] = (torch.rand((min(piece, n - i0), w), device=dev_t, generator=gen) * 2 - 1).to(torch.float16)
            out = torch.empty((n, w), dtype=torch.float32, device=dev_t)
            times = []
            for it in range(warmup + steps):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                tr.forward(x.data_ptr(), out.data_ptr(), n)
                e1.record()
                torch.cuda.synchronize()
                if it >= warmup:
                    times.append(e0.elapsed_time(e1))
            ms = float(np.median(times))
            sps = n / (ms * 1e-3)
            gbs = sps * 6 * w / 1e9
            points.append({"width": w, "batch": n, "ms": ms, "samples_per_s": sps, "hbm_gbs": gbs,
                           "hbm_frac": gbs / peaks["hbm_gbs"], "tflops": sps * 8 * w * w / 1e12,
                           "tensor_frac_of_burst": sps * 8 * w * w / 1e12 / peaks["bf16_burst"]})
            del x, out
    device.wait()
    del flush
    return points


def sweep_forward(args):
    """Forward-only inference sweep: widths 16/32/64/128, batch 2^20 .. 2^26 in powers of 4."""
    import torch
    from slang_b200.api import Device
    torch.cuda.set_device(0)
    dev_t = torch.device("cuda", 0)
    stream = torch.cuda.Stream(device=dev_t)
    torch.cuda.set_stream(stream)
    device = Device(0, stream.cuda_stream)
    peaks = measured_peaks()
    single = args.config.startswith("c5_w")  # one point: --config c5_w64 --batch N
    widths = (int(args.config[4:]),) if single else (16, 32, 64, 128)
    batches = (args.batch,) if single else (1 << 20, 1 << 22, 1 << 24, 1 << 26)
    points = measure_forward_points(torch, device, dev_t, widths, batches, args.warmup, args.steps)
    best = max(points, key=lambda p: p["hbm_frac"])
    line = {"metric": "MLP forward samples/sec (depth-4 constant width)", "value": best["samples_per_s"], "unit": UNIT,
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": best["ms"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "forward sweep, widths 16-128, batch 2^20-2^26; value is the point with the best HBM fraction",
                       "l2": "512 MB written between timed iterations"},
            "roofline": {"bound": "hbm", "achieved": best["hbm_gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": best["hbm_frac"], "traffic": None, "kernel": "forward_tc_kernel", "peak_source": peaks["source"]},
            "gpu_launches": device.launch_count, "sweep": points}
    print(json.dumps(line), flush=True)
    device.destroy()


def bench_narrow(args):
    """Configurations 2 and 3 at their stated sizes on one GPU (resident inputs, CUDA events)."""
    import torch
    from slang_b200.api import Device
    torch.cuda.set_device(0)
    dev_t = torch.device("cuda", 0)
    stream = torch.cuda.Stream(device=dev_t)
    torch.cuda.set_stream(stream)
    device = Device(0, stream.cuda_stream)
    name = args.config
    count = args.batch if args.batch != (1 << 26) else {"c1": 4096, "c2": 1 << 20}.get(name, 1 << 24)
    line = measure_narrow(torch, device, dev_t, name, count, args.warmup, args.steps)
    print(json.dumps(line), flush=True)
    device.destroy()


def measure_narrow(torch, device, dev_t, name, count, warmup, steps):
    """One of configurations 2 and 3: learnGradient + adjustParameters per step with resident inputs,
    and the forward entry point of the same network; returns the JSON line as a dict."""
    from slang_b200 import config as C
    from slang_b200.api import Trainer
    cfg = C.named_config(name)
    gen = torch.Generator(device=dev_t); gen.manual_seed(11)
    if name == "c1":
        # the CPU-runnable parity configuration: a launch-bound step (4096 samples), reported as ms per step
        x = (torch.rand((count, 2), device=dev_t, generator=gen) * 2 - 1).contiguous()
        t = (torch.sin(np.pi * x[:, 0]) * torch.cos(np.pi * x[:, 1])).reshape(count, 1).contiguous()
        workload = "fp32 MLP 2-16-16-16-1 ReLU, MSE, Adam lr 1e-3 (one thread per sample)"
    elif name == "c2":
        x = torch.rand((count, 4), device=dev_t, generator=gen)
        w = torch.from_numpy(C.unit_vectors(1234, 4, 4)).to(dev_t)
        t = torch.sin(2 * np.pi * (x @ w.t())).contiguous()
        workload = "fp16 MLP 4-32-32-32-32-4 LeakyReLU(0.01), MSE, Adam lr 1e-3"
    else:
        side = int(round(count ** 0.5))
        assert side * side == count
        idx = torch.arange(count, device=dev_t)
        x = torch.stack([((idx % side) + 0.5) / side, ((idx // side) + 0.5) / side], dim=1).float().contiguous()
        centres, sigma = C.gaussian_blobs(4321)
        t = torch.zeros((count, 3), device=dev_t)
        for ch in range(3):
            for b in range(centres.shape[1]):
                cx, cy, sg = float(centres[ch, b, 0]), float(centres[ch, b, 1]), float(sigma[ch, b])
                t[:, ch] += torch.exp(-((x[:, 0] - cx) ** 2 + (x[:, 1] - cy) ** 2) / (2 * sg * sg))
        t = t.clamp(0, 1).to(torch.float16).contiguous()
        workload = "fp16 MLP enc(2->32)-64-64-64-3 ReLU, sigmoid out, L2, Adam lr 1e-2, 4096x4096 grid"
    tr = Trainer(device, cfg, C.init_params(cfg, seed=1, scheme="xavier" if name == "c2" else "kaiming"))
    impl = tr.k_learn.implementation
    kernel_name = "learn_gradient_narrow_kernel" if impl == "tcgen05" else "learn_gradient_simt_kernel"
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev_t)

    def step():
        tr.learn_gradient(x.data_ptr(), t.data_ptr(), count)
        tr.adjust_parameters()

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    times, ktimes = [], []
    launches0 = device.launch_count
    for _ in range(steps):
        flush.zero_()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        tr.learn_gradient(x.data_ptr(), t.data_ptr(), count)
        e1.record()
        tr.adjust_parameters()
        e2.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e2)); ktimes.append(e0.elapsed_time(e1))
    launches = device.launch_count - launches0
    device.wait()
    ms, kms = float(np.mean(times)), float(np.mean(ktimes))
    mx, sm = tr.read_loss()
    # the forward entry point of the same network (outputs fp32), timed the same way
    out = torch.empty((count, cfg.out_dim), dtype=torch.float32, device=dev_t)
    ftimes = []
    for i in range(warmup + steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        tr.forward(x.data_ptr(), out.data_ptr(), count)
        e1.record()
        torch.cuda.synchronize()
        if i >= warmup:
            ftimes.append(e0.elapsed_time(e1))
    fms = float(np.mean(ftimes))
    peaks = measured_peaks()
    flops = C.flops_per_sample(cfg, training=True)
    achieved = flops * count / (kms * 1e-3) / 1e12
    line = {"metric": METRIC, "value": count / (ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": steps, "warmup": warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32" if name == "c1" else "f16", "data": "synthetic",
            "config": {"workload": workload, "global_batch": count, "l2": "512 MB written between timed steps"},
            "gpu_launches": launches, "implementation": impl,
            "forward": {"ms": fms, "samples_per_s": count / (fms * 1e-3), "implementation": tr.k_forward.implementation},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_burst"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["bf16_burst"], "traffic": None, "kernel": kernel_name,
                         "kernel_ms": kms, "flop_per_sample": flops, "peak_source": peaks["source"] + " (burst; kernel timed alone)"},
            "loss": {"max": mx, "mean": sm / count}}
    if name == "c1":
        # launch- and latency-bound: the honest yardstick is HBM bytes (12 B per sample plus the parameters), which it is nowhere near
        _, _, total = C.param_layout(cfg)
        bytes_step = count * 12 + total * 8
        gbs = bytes_step / (kms * 1e-3) / 1e9
        line["roofline"] = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                            "traffic": None, "kernel": kernel_name, "kernel_ms": kms, "flop_per_sample": flops,
                            "peak_source": peaks["source"], "note": "launch- and latency-bound at 4096 samples per step"}
    del x, t, out, flush
    return line


def measure_other_widths(torch, device, dev_t):
    """Networks that are neither a benchmark configuration nor at most 64 wide: learnGradient + adjustParameters
    on 2^20 samples through the shape's fastest kernel and, for scale, through the one-thread-per-sample kernel
    (2^17 samples)."""
    from slang_b200 import config as C
    from slang_b200.api import Trainer
    out = []
    for dims, dtype, act in (([32, 128, 128, 3], C.F16, C.ACT_RELU), ([64, 96, 96, 64], C.BF16, C.ACT_GELU_TANH)):
        cfg = C.make_config(dims, dtype=dtype, hidden_act=act, input_dtype=dtype, target_dtype=dtype, adam_master=1)
        p0 = C.init_params(cfg, seed=1, scheme="xavier")
        tdt = torch.float16 if dtype == C.F16 else torch.bfloat16
        n = 1 << 20
        gen = torch.Generator(device=dev_t); gen.manual_seed(3)
        x = torch.randn((n, dims[0]), device=dev_t, generator=gen).to(tdt)
        t = (torch.randn((n, dims[-1]), device=dev_t, generator=gen) * 0.3).to(tdt)
        rates = {}
        for entry, cnt in (("learnGradient", n), ("learnGradient_simt", 1 << 17)):
            tr = Trainer(device, cfg, p0, learn_entry=entry)
            for _ in range(2):
                tr.learn_gradient(x.data_ptr(), t.data_ptr(), cnt); tr.adjust_parameters()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(3):
                tr.learn_gradient(x.data_ptr(), t.data_ptr(), cnt); tr.adjust_parameters()
            e1.record()
            torch.cuda.synchronize()
            rates[entry] = (3 * cnt / (e0.elapsed_time(e1) * 1e-3), tr.k_learn.implementation)
        out.append({"dims": dims, "dtype": C.DTYPE_NAME[dtype], "samples_per_s": rates["learnGradient"][0],
                    "implementation": rates["learnGradient"][1], "one_thread_per_sample_samples_per_s": rates["learnGradient_simt"][0],
                    "tflops": rates["learnGradient"][0] * C.flops_per_sample(cfg) / 1e12})
        del x, t
    return out


def bench_permuto(args):
    """Permutohedral encoder: 3-D positions, 16 levels of 2^19 entries, 2 features per entry (fp32 or fp16
    tables).  Reports encode and reverse-pass rates; the roofline is HBM against the bytes that must cross
    it when the table stays in L2 (positions in, feature rows out / upstream rows in)."""
    import ctypes
    import torch
    from oracle import permuto as OP
    from slang_b200 import config as C
    from slang_b200 import permuto as P
    from slang_b200.api import Device
    torch.cuda.set_device(0)
    dev_t = torch.device("cuda", 0)
    stream = torch.cuda.Stream(device=dev_t)
    torch.cuda.set_stream(stream)
    device = Device(0, stream.cuda_stream)
    half = args.config.endswith("f16")
    dims, feats, log2, levels = 3, 2, 19, 16
    cfg = P.prepare(dims, feats, log2, levels, 16.0, 0.5, 1.1, 1337, C.F16 if half else C.F32)
    tdt = torch.float16 if half else torch.float32
    es = 2 if half else 4
    count = args.batch if args.batch != (1 << 26) else 1 << 22
    gen = torch.Generator(device=dev_t); gen.manual_seed(5)
    pos = torch.rand((count, dims), device=dev_t, generator=gen)
    table = (torch.rand(cfg.table_values, device=dev_t, generator=gen) * 2e-4 - 1e-4).to(tdt)
    out = torch.empty((count, cfg.n_features), dtype=tdt, device=dev_t)
    g = torch.full((count, cfg.n_features), 1.0 / 64, dtype=tdt, device=dev_t)
    dtable = torch.zeros(cfg.table_values, dtype=tdt, device=dev_t)
    dpos = torch.empty((count, dims), device=dev_t)
    enc = P.PermutoEncoder(device, cfg)
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev_t)

    def fwd():
        enc.encode(pos.data_ptr(), table.data_ptr(), out.data_ptr(), count)

    def bwd():
        enc.backward(pos.data_ptr(), table.data_ptr(), g.data_ptr(), dtable.data_ptr(), dpos.data_ptr(), count)

    for _ in range(args.warmup):
        fwd(); bwd()
    torch.cuda.synchronize()
    # parity spot check against the oracle on the first 4096 positions (checker only, outside the timing)
    want = OP.encode(cfg, pos[:4096].cpu().numpy(), table.cpu().numpy())
    assert np.array_equal(out[:4096].cpu().numpy(), want), "encode differs from the oracle"
    tf, tb = [], []
    launches0 = device.launch_count
    for _ in range(args.steps):
        flush.zero_()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record(); fwd(); e1.record(); bwd(); e2.record()
        torch.cuda.synchronize()
        tf.append(e0.elapsed_time(e1)); tb.append(e1.elapsed_time(e2))
    launches = device.launch_count - launches0
    mf, mb = float(np.mean(tf)), float(np.mean(tb))
    peaks = measured_peaks()
    bytes_f = count * (dims * 4 + cfg.n_features * es)
    bytes_b = count * (dims * 4 + cfg.n_features * es + dims * 4)
    gathered = count * levels * (dims + 1) * feats * es
    line = {"metric": "permuto encoder positions/sec (encode + reverse)", "value": count / ((mf + mb) * 1e-3), "unit": "positions/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": mf + mb, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16" if half else "f32", "data": "synthetic",
            "config": {"workload": "permutohedral encoder, 3-D, 16 levels x 2^19 entries x 2 features, %s tables" % ("fp16" if half else "fp32"),
                       "positions": count, "l2": "512 MB written between timed steps"},
            "gpu_launches": launches,
            "encode": {"ms": mf, "positions_per_s": count / (mf * 1e-3), "gathered_gbs": gathered / (mf * 1e-3) / 1e9},
            "reverse": {"ms": mb, "positions_per_s": count / (mb * 1e-3), "scattered_gbs": gathered / (mb * 1e-3) / 1e9},
            "roofline": {"bound": "hbm", "achieved": bytes_f / (mf * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": bytes_f / (mf * 1e-3) / 1e9 / peaks["hbm_gbs"], "traffic": None, "kernel": "permuto_encode_kernel",
                         "reverse_achieved": bytes_b / (mb * 1e-3) / 1e9, "reverse_frac": bytes_b / (mb * 1e-3) / 1e9 / peaks["hbm_gbs"],
                         "peak_source": peaks["source"]}}
    n_cpu = 1 << 16
    p_h, t_h = pos[:n_cpu].cpu().numpy(), table.cpu().numpy()
    g_h = g[:n_cpu].cpu().numpy()
    t0 = time.perf_counter()
    OP.encode(cfg, p_h, t_h)
    OP.backward(cfg, p_h, t_h, g_h, np.zeros_like(t_h))
    dt = time.perf_counter() - t0
    line["cpu_baseline"] = {"value": n_cpu / dt, "unit": "positions/s", "cores": 1, "kind": "port",
                            "sample": "%d positions, encode + reverse once, %.2f s" % (n_cpu, dt)}
    print(json.dumps(line), flush=True)
    device.destroy()


def bench_encoded(args):
    """Trainable encoder in front of a small network: 3-D positions -> permutohedral features (16 levels x 2)
    -> fp16 MLP 32-64-64-3 (ReLU, sigmoid output, L2).  One step = encode, learnGradient with input
    gradients (tensor cores), the encoder's reverse pass, Adam over the network and over the table."""
    import torch
    from slang_b200 import config as C
    from slang_b200 import permuto as P
    from slang_b200.api import Device
    from slang_b200.encoded import EncodedTrainer
    torch.cuda.set_device(0)
    dev_t = torch.device("cuda", 0)
    stream = torch.cuda.Stream(device=dev_t)
    torch.cuda.set_stream(stream)
    device = Device(0, stream.cuda_stream)
    count = args.batch if args.batch != (1 << 26) else 1 << 22
    pcfg = P.prepare(3, 2, 19, 16, 16.0, 0.5, 1.1, 1337, C.F32)
    cfg = C.make_config([32, 64, 64, 3], dtype=C.F16, hidden_act=C.ACT_RELU, output_act=C.ACT_SIGMOID, loss=C.LOSS_L2_SUM,
                        target_dtype=C.F16, lr=1e-2, adam_master=1)
    rng = np.random.default_rng(3)
    table0 = rng.uniform(-1e-4, 1e-4, pcfg.table_values).astype(np.float32)
    et = EncodedTrainer(device, pcfg, cfg, table0, C.init_params(cfg, seed=1, scheme="kaiming"), max_count=count)
    gen = torch.Generator(device=dev_t); gen.manual_seed(9)
    pos = torch.rand((count, 3), device=dev_t, generator=gen)
    tgt = (0.5 + 0.5 * torch.sin(pos * torch.tensor([7.0, 11.0, 13.0], device=dev_t))).to(torch.float16).contiguous()
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev_t)

    def step():
        et.learn_gradient(pos.data_ptr(), tgt.data_ptr(), count)
        et.adjust_parameters()

    losses = []
    for _ in range(args.warmup):
        step()
        losses.append(et.trainer.read_loss()[1] / count)
    times = []
    launches0 = device.launch_count
    for _ in range(args.steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); step(); e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    launches = device.launch_count - launches0
    losses.append(et.trainer.read_loss()[1] / count)
    ms = float(np.mean(times))
    line = {"metric": "encoder + MLP train positions/sec (encode, fwd+bwd with input gradients, encoder reverse, Adam x2)",
            "value": count / (ms * 1e-3), "unit": "positions/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "permutohedral encoder (3-D, 16 x 2^19 x 2, fp32 table) + fp16 MLP 32-64-64-3", "positions": count,
                       "l2": "512 MB written between timed steps"},
            "gpu_launches": launches, "implementation": et.trainer.k_learn.implementation,
            "loss": {"first_warmup_step": losses[0], "last_step": losses[-1]}}
    print(json.dumps(line), flush=True)
    device.destroy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--config", default="c4")
    ap.add_argument("--batch", type=int, default=1 << 26, help="global batch (samples per step over all GPUs)")
    ap.add_argument("--e2e-steps", type=int, default=10)
    ap.add_argument("--no-sub", action="store_true", help="N=1: skip the block of the other configurations")
    ap.add_argument("--log-jsonl", default=None, help="write one JSON object per timed step (phase times, samples/s) to this file (rank 0)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--deterministic-sum", action="store_true",
                    help="N>1: gather every rank's gradient segment and add in rank order instead of an all-reduce")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        reference_arm(args, rank)
        return
    if args.config in ("c1", "c2", "c3"):
        if rank == 0:
            bench_narrow(args)
        return
    if args.config == "encoded":
        if rank == 0:
            bench_encoded(args)
        return
    if args.config.startswith("permuto"):
        if rank == 0:
            bench_permuto(args)
        return
    if args.config == "c5_sweep" or args.config.startswith("c5_w"):
        if rank == 0:
            sweep_forward(args)
        return

    import torch
    import torch.distributed as dist
    from slang_b200 import config as C
    from slang_b200.api import Device, Trainer
    from slang_b200.host_step import HostStepper

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the library has no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev_t = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev_t)

    cfg = C.named_config(args.config)
    assert args.config == "c4", "the timed workload is the wide bf16 network (c4)"
    count = args.batch // world
    stream = torch.cuda.Stream(device=dev_t)
    torch.cuda.set_stream(stream)  # kernels, collectives and timing events all go to this stream
    device = Device(local_rank, stream.cuda_stream)
    _, _, total = C.param_layout(cfg)

    # Parameters and gradients live in torch tensors so that the collective sees the same memory.
    p0 = C.init_params(cfg, seed=1, scheme="xavier")
    params_t = torch.zeros(total, dtype=torch.bfloat16, device=dev_t)
    grads_t = torch.zeros(total, dtype=torch.float32, device=dev_t)
    trainer = Trainer(device, cfg, p0, param_memory=(params_t.data_ptr(), grads_t.data_ptr()))
    assert trainer.k_learn.implementation == "tcgen05", "the tensor-core kernel did not resolve: %s" % trainer.k_learn.implementation

    n_batches = 2
    gen = torch.Generator(device=dev_t)
    xs, ts = [], []
    for b in range(n_batches):
        gen.manual_seed(1000 + 17 * b + rank)
        x = torch.randn((count, 64), dtype=torch.float32, device=dev_t, generator=gen).to(torch.bfloat16) if count <= (1 << 24) else None
        if x is None:
            x = torch.empty((count, 64), dtype=torch.bfloat16, device=dev_t)
            piece = 1 << 23
            for i0 in range(0, count, piece):
                x[i0:i0 + piece] = torch.randn((min(piece, count - i0), 64), dtype=torch.float32, device=dev_t, generator=gen).to(torch.bfloat16)
        xs.append(x)
        ts.append(teacher_targets(torch, cfg, x, seed=2))
    torch.cuda.synchronize()

    # The gradient exchange goes through the library's own collective entry points (mlp_comm_init /
    # mlp_allreduce_grads, NCCL bound inside the library): the call a C++ host loop makes between its
    # two dispatches.  torch.distributed only carries the communicator id and the timing reductions.
    comm = None
    if world > 1:
        from slang_b200.api import Comm, comm_unique_id
        box = [comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        comm = Comm(device, world, rank, box[0])

    def allreduce():
        if comm is not None:
            # fp32 sum of the flat gradient segment (NCCL over NVLink), stream ordered
            comm.allreduce_grads(trainer, with_loss=False, rank_ordered=args.deterministic_sum)

    def step(i):
        b = i % n_batches
        trainer.learn_gradient(xs[b].data_ptr(), ts[b].data_ptr(), count)
        allreduce()
        trainer.adjust_parameters()

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = device.launch_count
    from slang_b200.metrics import JsonlLogger, PhaseTimer
    phase_timer = PhaseTimer(stream)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(args.steps):
        b = i % n_batches
        phase_timer.begin_step()
        trainer.learn_gradient(xs[b].data_ptr(), ts[b].data_ptr(), count)
        phase_timer.mark("learn_gradient")
        allreduce()
        phase_timer.mark("exchange")
        trainer.adjust_parameters()
        phase_timer.mark("adjust_parameters")
    ev1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    launches = device.launch_count - launches0
    device.wait()  # raises if a kernel set the status word

    elapsed_ms = ev0.elapsed_time(ev1)
    phase_rows = phase_timer.collect()
    # the learn_gradient phase includes the 8-byte clear of the loss words that precedes the kernel
    kernel_ms = float(np.mean([r["learn_gradient_ms"] for r in phase_rows]))
    phases = {k: float(np.mean([r[k] for r in phase_rows])) for k in phase_rows[0]}
    if world > 1:
        # every rank's own GPU: its clock record and its learnGradient time (the step waits for the slowest rank)
        mine = {"rank": rank, "sm_mhz": clocks["sm_mhz"], "reasons": clocks["reasons"], "learn_gradient_ms": kernel_ms}
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
        clocks["per_rank"] = gathered
        clocks["reasons"] = sorted(set(r for g in gathered for r in g["reasons"]))
    if args.log_jsonl and rank == 0:
        log = JsonlLogger(args.log_jsonl)
        for i, r in enumerate(phase_rows):
            log.log(i, args.batch, r, n_gpus=world)
        log.close()
    if world > 1:
        tt = torch.tensor([elapsed_ms, kernel_ms], dtype=torch.float64, device=dev_t)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        elapsed_ms, kernel_ms = float(tt[0]), float(tt[1])
        lt = torch.tensor([launches], dtype=torch.int64, device=dev_t)
        dist.all_reduce(lt)
        launches = int(lt[0])
    value = args.batch * args.steps / (elapsed_ms * 1e-3)
    mx, sm = trainer.read_loss()

    # ---- end to end: pinned host inputs, copies inside the timed region ----
    e2e = None
    if not args.no_e2e:
        # The targets are the frozen teacher's outputs: only the inputs cross the host-device link, the
        # teacher's forward kernel produces each piece's targets on the device inside the timed region.
        teacher = Trainer(device, cfg, C.init_params(cfg, seed=2, scheme="xavier"))
        assert teacher.k_forward.implementation == "tcgen05"
        stepper = HostStepper(trainer, chunk_samples=min(count, 1 << 21), allreduce=allreduce if world > 1 else None, teacher=teacher)
        xh = torch.empty((count, 64), dtype=torch.bfloat16, pin_memory=True)
        xh.copy_(xs[0])
        torch.cuda.synchronize()
        # Ceiling of the host-to-device link as this rank sees it while every rank copies at once: the
        # same pinned buffer into device memory with plain cudaMemcpyAsync, nothing else running.
        if world > 1:
            dist.barrier()
        l0, l1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        xs[1].copy_(xh, non_blocking=True)  # warm-up pass
        l0.record()
        for _ in range(2):
            xs[1].copy_(xh, non_blocking=True)
        l1.record()
        torch.cuda.synchronize()
        link_ms = l0.elapsed_time(l1) / 2
        # (batch 1's inputs are overwritten; the timed region that used them is over)
        stepper.step(xh)  # warm-up
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.e2e_steps):
            stepper.step(xh)
        e1.record()
        torch.cuda.synchronize()
        e2e_ms = e0.elapsed_time(e1)
        wall_ms = (time.perf_counter() - t0) * 1e3
        if world > 1:
            tt = torch.tensor([e2e_ms, link_ms], dtype=torch.float64, device=dev_t)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            e2e_ms, link_ms = float(tt[0]), float(tt[1])
        link_ceiling = stepper.h2d_bytes / (link_ms * 1e-3) / 1e9          # GB/s per rank, slowest rank
        link_used = stepper.h2d_bytes * args.e2e_steps / (e2e_ms * 1e-3) / 1e9
        e2e = {"value": args.batch * args.e2e_steps / (e2e_ms * 1e-3), "unit": UNIT,
               "h2d_bytes_per_step": int(stepper.h2d_bytes) * world, "d2h_bytes_per_step": int(stepper.d2h_bytes) * world,
               "steps": args.e2e_steps, "wall_ms_per_step": wall_ms / args.e2e_steps,
               "link_gbs": link_used, "link_ceiling_gbs": link_ceiling, "link_frac": link_used / link_ceiling,
               "link_note": "GB/s per rank (slowest rank): link_gbs inside the timed end-to-end steps, link_ceiling_gbs a plain "
                            "pinned cudaMemcpyAsync of the same buffer with all ranks copying at once",
               "api": "slang_b200.host_step.HostStepper.step (pinned host inputs, chunked copies overlapped with the "
                      "teacher's forward kernel and learnGradient; targets computed on the device)"}
        del xh

    if rank == 0:
        peaks = measured_peaks()
        flops = C.flops_per_sample(cfg, training=True)
        achieved = flops * count / (kernel_ms * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload_name(args), "global_batch": args.batch, "per_gpu_batch": count,
                       "parallelism": "dp%d" % world, "gradient_sum": ("rank-ordered gather" if args.deterministic_sum else "all-reduce") + " through mlp_allreduce_grads (NCCL bound inside the library)", "l2": "inputs (%.1f GB per step per GPU) larger than L2; two batches alternate" % (count * 256 / 1e9)},
            "clocks": clocks, "gpu_launches": launches, "e2e": e2e, "phases_ms": phases,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_sustained"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["bf16_sustained"], "frac_of_burst": achieved / peaks["bf16_burst"],
                         # DRAM read + write bytes of one launch: a constant from one profiler capture of a
                         # 2^20-sample launch (272.9 MB; the algorithmic bytes are 268.4 MB), scaled by this
                         # launch's samples.  Not measured in this run.
                         "traffic": int(round(272.9e6 / 1048576 * count)), "traffic_static": True,
                         "traffic_source": "static: ncu capture of a 2^20-sample launch, scaled per sample",
                         "algorithmic_bytes": count * 256,
                         "peak_source": peaks["source"] + " (sustained bf16 GEMM; kernel timed inside the step loop)",
                         "kernel": "learn_gradient_wide_kernel", "kernel_ms": kernel_ms, "flop_per_sample": flops,
                         "hbm_gbs": count * 256 / (kernel_ms * 1e-3) / 1e9},
            "loss": {"max": mx, "mean_local": sm / count},
        }
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            r, n, dt = oracle_rate(cfg, args.config, threads, 12.0)
            line["cpu_baseline"] = {"value": r, "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": "%d samples, learnGradient + adjustParameters once, %.1f s" % (n, dt)}
            # The structure of the reference's example kernels on the same GPU: one thread per sample,
            # scalar fused multiply-adds, block-level sums and atomics (learnGradient_simt), on a bounded sample.
            n_simt = min(count, 1 << 18)
            tr_simt = Trainer(device, cfg, p0, learn_entry="learnGradient_simt")
            for _ in range(2):
                tr_simt.learn_gradient(xs[0].data_ptr(), ts[0].data_ptr(), n_simt)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            tr_simt.learn_gradient(xs[0].data_ptr(), ts[0].data_ptr(), n_simt)
            tr_simt.adjust_parameters()
            e1.record()
            torch.cuda.synchronize()
            line["gpu_baseline"] = {"value": n_simt / (e0.elapsed_time(e1) * 1e-3), "unit": UNIT,
                                    "kind": "one thread per sample on the same GPU (the example kernels' structure, this library's learnGradient_simt)",
                                    "sample": "%d samples, learnGradient + adjustParameters once" % n_simt}
        if world == 1 and not args.no_sub:
            # The other configurations under the same clock, in this process: configurations 1, 2 and 3
            # at their stated sizes (training step and forward), configuration 5 at two batch sizes per width.
            del xs, ts
            torch.cuda.empty_cache()
            sub = {}
            for name, n in (("c1", 4096), ("c2", 1 << 20), ("c3", 1 << 24)):
                r = measure_narrow(torch, device, dev_t, name, n, 3, 5)
                sub[name] = {"samples_per_s": r["value"], "ms_per_step": r["ms_per_step"], "kernel_ms": r["roofline"]["kernel_ms"],
                             "tflops": r["roofline"]["flop_per_sample"] * n / (r["roofline"]["kernel_ms"] * 1e-3) / 1e12,
                             "roofline_frac_of_burst": r["roofline"]["flop_per_sample"] * n / (r["roofline"]["kernel_ms"] * 1e-3) / 1e12 / peaks["bf16_burst"],
                             "forward_samples_per_s": r["forward"]["samples_per_s"], "global_batch": n,
                             "implementation": r["implementation"], "workload": r["config"]["workload"]}
            pts = measure_forward_points(torch, device, dev_t, (16, 32, 64, 128), (1 << 20, 1 << 24), 3, 5)
            sub["c5"] = {"points": [{k: p[k] for k in ("width", "batch", "samples_per_s", "hbm_frac", "tflops", "tensor_frac_of_burst")} for p in pts],
                         "workload": "forward only, depth-4 ReLU, fp16 weights, fp32 outputs; hbm_frac = 6w bytes per sample over the measured copy bandwidth"}
            sub["other_widths"] = measure_other_widths(torch, device, dev_t)
            line["sub"] = sub
        print(json.dumps(line), flush=True)
    if comm is not None:
        comm.wait(60000)  # drains the stream with the collective library's asynchronous errors polled
        comm.destroy()
    device.destroy()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
