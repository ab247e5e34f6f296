"""Build the native library in-tree: `python -m cagnet_b200.build`.

Compiles every `csrc/*.cu` for sm_100a with nvcc (cross-compiles without a GPU) and links
`cagnet_b200/libcagnet_b200.so`.  The ptxas resource report (registers, spills, shared memory per
kernel) is written next to the objects as `build/ptxas.log`.
"""
import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD_DIR = os.path.join(HERE, "build")
LIB_PATH = os.path.join(HERE, "libcagnet_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def cutlass_include_dirs():
    """The CUTLASS / CuTe header tree that ships inside the flashinfer wheel (include/ and tools/util/include/), or
    [] when it is not installed.  Located without importing the package."""
    import importlib.util
    try:
        spec = importlib.util.find_spec("flashinfer")
    except (ImportError, ValueError):
        spec = None
    for root in (list(spec.submodule_search_locations) if spec and spec.submodule_search_locations else []):
        inc = os.path.join(root, "data", "cutlass", "include")
        if os.path.exists(os.path.join(inc, "cutlass", "gemm", "collective", "builders", "sm100_umma_builder.inl")):
            return [inc, os.path.join(root, "data", "cutlass", "tools", "util", "include")]
    return []


def _nvcc():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the CUDA kernels cannot be built")
    return nvcc


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    """Compile and link; returns the library path.  Re-uses objects that are newer than their sources."""
    nvcc = _nvcc()
    os.makedirs(BUILD_DIR, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "cagnet_b200.h"))
    cutlass = cutlass_include_dirs()
    if not cutlass:
        print("cagnet_b200.build: WARNING: no CUTLASS / CuTe header tree found (looked inside the flashinfer wheel): "
              "the tcgen05 dense-core kernels are NOT built and the fp32-FMA core kernel is used instead",
              file=sys.stderr, flush=True)
    srcs = sources()
    objs = [os.path.join(BUILD_DIR, os.path.basename(s)[:-3] + ".o") for s in srcs]

    def compile_one(pair):
        src, obj = pair
        if not force and not _stale(obj, [src] + headers):
            return ""
        extra = []
        if os.path.basename(src) in ("core_gemm_tc.cu", "core_gemm_int.cu") and cutlass:
            extra = ["--expt-relaxed-constexpr", "-DCAGNET_HAVE_CUTLASS", "-diag-suppress", "20012"]
            for d in cutlass:
                extra += ["-I", d]
        cmd = [nvcc] + NVCC_FLAGS + extra + ["-c", src, "-o", obj]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, p.stdout, p.stderr))
        return "### %s\n%s\n" % (os.path.basename(src), p.stderr)

    with concurrent.futures.ThreadPoolExecutor(max_workers=len(srcs)) as ex:
        logs = list(ex.map(compile_one, zip(srcs, objs)))
    if any(logs):
        with open(os.path.join(BUILD_DIR, "ptxas.log"), "a") as fh:
            fh.write("".join(logs))
    if force or _stale(LIB_PATH, objs):
        cmd = [nvcc, "-shared", "-o", LIB_PATH] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            raise RuntimeError("link failed:\n%s\n%s" % (p.stdout, p.stderr))
    if verbose:
        print("built", LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
