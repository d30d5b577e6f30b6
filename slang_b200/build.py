"""Builds the sm_100a shared library in-tree with nvcc (no JIT at run time).

    python -m slang_b200.build [--force] [--verbose]

Each translation unit is compiled to an object with its own flags and the objects are linked into
slang_b200/libslang_b200_mlp.so; the literal example entry points are also built into a stand-alone
device module, slang_b200/mlp_training_kernels.cubin.  The CUDA runtime is linked statically so the library has no
dependency beyond the driver.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libslang_b200_mlp.so")
OBJDIR = os.path.join(HERE, "build")
# Stand-alone device module holding the literal example entry points (for cuModuleLoadData hosts).
CUBIN = os.path.join(HERE, "mlp_training_kernels.cubin")
CUBIN_SRC = "example_module.cu"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
          "--expt-relaxed-constexpr"]

# (source, extra flags).  The one-thread-per-sample kernels must not contract a*b+c into an fma on
# their own: their fp32 results are compared bit for bit with a sequential CPU.
UNITS = [
    ("abi.cu", []),
    ("simt_kernels.cu", ["-fmad=false"]),
    ("layout_convert.cu", []),
    ("tc_kernels.cu", []),
    ("tc_forward.cu", []),
    ("tc_train_narrow.cu", []),
    ("comm.cu", []),
    ("matrix_convert.cu", []),
    ("permuto.cu", ["-fmad=false"]),
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    inc = os.path.join(os.path.dirname(HERE), "include")
    hs += [os.path.join(inc, f) for f in os.listdir(inc)]
    return hs


def build(force=False, verbose=False):
    nvcc = _nvcc()
    os.makedirs(OBJDIR, exist_ok=True)
    newest_header = max(os.path.getmtime(h) for h in _headers())
    objs = []
    rebuilt = False
    for src, extra in UNITS:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJDIR, src.replace(".cu", ".o"))
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), newest_header):
            more = os.environ.get("MLPB200_NVCC_FLAGS", "").split()  # experiments only, e.g. -DMLPB200_CH=64
            cmd = [nvcc] + ARCH + COMMON + extra + more + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
            if verbose:
                print(" ".join(cmd), flush=True)
            subprocess.check_call(cmd)
            rebuilt = True
    cs = os.path.join(CSRC, CUBIN_SRC)
    if force or not os.path.exists(CUBIN) or os.path.getmtime(CUBIN) < max(os.path.getmtime(cs), newest_header):
        cmd = [nvcc, "-arch=sm_100a", "-cubin", "-O3", "-std=c++17", "-lineinfo", "-fmad=false", cs, "-o", CUBIN]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
    if rebuilt or not os.path.exists(OUT):
        cmd = [nvcc] + ARCH + ["-shared", "-cudart", "static", "-o", OUT] + objs + ["-ldl"]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
