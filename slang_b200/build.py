"""Builds the sm_100a shared library in-tree with nvcc (no JIT at run time).

    python -m slang_b200.build [--force] [--verbose]

Each translation unit is compiled to an object with its own flags (stale units side by side, one nvcc
process each) and the objects are linked into slang_b200/libslang_b200_mlp.so; the literal example
entry points are also built into a stand-alone device module, slang_b200/mlp_training_kernels.cubin.
A unit is stale when its source, or any header its last compile read (nvcc -MD), is newer than its
object.  The CUDA runtime is linked statically so the library has no dependency beyond the driver.
"""
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

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

# (object name, source, extra flags).  The one-thread-per-sample kernels must not contract a*b+c into
# an fma on their own: their fp32 results are compared bit for bit with a sequential CPU.  The padded
# tensor-core kernel is instantiated some fifty times; its source is compiled in eight parts, the wide
# kernel's in three (training builds, forward-only builds, training builds with the optional outputs).
UNITS = [
    ("abi", "abi.cu", []),
    ("simt_kernels", "simt_kernels.cu", ["-fmad=false"]),
    ("layout_convert", "layout_convert.cu", []),
    ("tc_kernels_0", "tc_kernels.cu", ["-DMLPB200_WIDE_PART=0"]),
    ("tc_kernels_1", "tc_kernels.cu", ["-DMLPB200_WIDE_PART=1"]),
    ("tc_kernels_2", "tc_kernels.cu", ["-DMLPB200_WIDE_PART=2"]),
    ("tc_forward", "tc_forward.cu", []),
    ("comm", "comm.cu", []),
    ("matrix_convert", "matrix_convert.cu", []),
    ("permuto", "permuto.cu", ["-fmad=false"]),
    ("selftest", "selftest.cu", []),
    ("tile_mma", "tile_mma.cu", []),
] + [("tc_train_narrow_%d" % i, "tc_train_narrow.cu", ["-DMLPB200_NARROW_PART=%d" % i]) for i in range(8)]


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _deps(depfile):
    """Prerequisites listed in a make-style dependency file written by nvcc -MD."""
    try:
        text = open(depfile).read()
    except OSError:
        return None
    text = text.replace("\\\n", " ")
    if ":" not in text:
        return None
    return [t for t in text.split(":", 1)[1].split() if t]


def _stale(obj, src, depfile):
    if not os.path.exists(obj):
        return True
    t = os.path.getmtime(obj)
    if os.path.getmtime(src) > t:
        return True
    deps = _deps(depfile)
    if deps is None:
        return True
    for d in deps:
        if d.startswith(("/usr/", "/opt/")):
            continue  # toolkit and system headers
        if not os.path.exists(d) or os.path.getmtime(d) > t:
            return True
    return False


# Components a build may leave out (--without): their units are replaced by stubs that keep every declared
# symbol and answer MLP_E_NOT_AVAILABLE.
OPTIONAL = {"comm": ["comm"], "permuto": ["permuto"], "tile_mma": ["tile_mma"]}


def build(force=False, verbose=False, jobs=None, without=(), out=None):
    """Builds the library.  `without`: names from OPTIONAL to leave out (then `out` must name another output
    file: the in-tree library is always the full one)."""
    nvcc = _nvcc()
    os.makedirs(OBJDIR, exist_ok=True)
    without = [w for w in without if w]
    for w in without:
        if w not in OPTIONAL:
            raise ValueError("unknown component %r (optional components: %s)" % (w, ", ".join(sorted(OPTIONAL))))
    if without and not out:
        raise ValueError("a build without components needs its own output file (--out)")
    skipped = {u for w in without for u in OPTIONAL[w]}
    units = [u for u in UNITS if u[0] not in skipped]
    if without:
        units.append(("stubs_" + "_".join(sorted(without)), "component_stubs.cu",
                      ["-DMLPB200_WITHOUT_" + w.upper() for w in sorted(without)]))
    target = out or OUT
    objs, todo = [], []
    for name, src, extra in units:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJDIR, name + ".o")
        d = os.path.join(OBJDIR, name + ".d")
        objs.append(o)
        if force or _stale(o, s, d):
            cmd = [nvcc] + ARCH + COMMON + extra + (["-Xptxas", "-v"] if verbose else []) + ["-MD", "-MF", d, "-c", s, "-o", o]
            todo.append(cmd)

    def run(cmd):
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        return cmd, r.returncode, r.stdout

    if todo:
        with ThreadPoolExecutor(max_workers=jobs or min(len(todo), os.cpu_count() or 4)) as pool:
            results = list(pool.map(run, todo))
        failed = [(c, out) for c, rc, out in results if rc != 0]
        if verbose or failed:
            for c, rc, out in results:
                if out.strip() and (verbose or rc != 0):
                    print(out, flush=True)
        if failed:
            raise subprocess.CalledProcessError(1, failed[0][0], output=failed[0][1])
    cs = os.path.join(CSRC, CUBIN_SRC)
    cd = os.path.join(OBJDIR, "example_module.d")
    if force or _stale(CUBIN, cs, cd):
        cmd = [nvcc, "-arch=sm_100a", "-cubin", "-O3", "-std=c++17", "-lineinfo", "-fmad=false", "-MD", "-MF", cd, cs, "-o", CUBIN]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
    if todo or not os.path.exists(target):
        cmd = [nvcc] + ARCH + ["-shared", "-cudart", "static", "-o", target] + objs + ["-ldl"]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
    return target


def _option(name):
    return sys.argv[sys.argv.index(name) + 1] if name in sys.argv else None


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv,
                without=(_option("--without") or "").split(","), out=_option("--out")))
