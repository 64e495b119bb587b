"""In-tree build of libhabitat_b200.so (nvcc, sm_100a only).

Run as `python -m habitat_b200.build` or through `__graft_entry__.build()`.
The shared object lands next to the package (habitat_b200/_lib/) so that it
travels with a source snapshot; nothing is installed into site-packages.
"""
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
SRC_DIR = os.path.join(PKG_DIR, "csrc")
LIB_DIR = os.path.join(PKG_DIR, "_lib")
OBJ_DIR = os.path.join(PKG_DIR, "_lib", "obj")
INCLUDE_DIR = os.path.join(os.path.dirname(PKG_DIR), "include")
LIB_PATH = os.path.join(LIB_DIR, "libhabitat_b200.so")

SOURCES = ["hb_error.cu", "wave_scale.cu", "reduce.cu", "peer_exchange.cu", "mlp_chain.cu", "device_probe.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc():
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = os.path.join(cuda_home, "bin", "nvcc")
    return cand if os.path.exists(cand) else (shutil.which("nvcc") or "nvcc")


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


# Sources that carry index checks under -DHB_BOUNDS_CHECK (the checked library reuses the
# ordinary objects of the others).
CHECKED_SOURCES = ["wave_scale.cu"]
CHECKED_LIB_PATH = os.path.join(LIB_DIR, "libhabitat_b200_checked.so")


def build(force=False, verbose=False, ptxas_info=False, checked=False):
    """Compile every CUDA source and link the shared library. Returns its path.
    checked=True builds the variant whose wave-scaling kernels compare every table and element
    index with its bound (libhabitat_b200_checked.so; load it with HABITAT_B200_LIB=...)."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    headers = [os.path.join(SRC_DIR, f) for f in os.listdir(SRC_DIR)
               if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(INCLUDE_DIR, "habitat_b200.h"))
    objs = []
    relink = force
    lib_path = CHECKED_LIB_PATH if checked else LIB_PATH
    for src in SOURCES:
        src_path = os.path.join(SRC_DIR, src)
        with_checks = checked and src in CHECKED_SOURCES
        obj = os.path.join(OBJ_DIR, src.replace(".cu", ".checked.o" if with_checks else ".o"))
        objs.append(obj)
        if force or _stale(obj, [src_path] + headers):
            cmd = [_nvcc()] + NVCC_FLAGS + ["-I", INCLUDE_DIR, "-I", SRC_DIR, "-c", src_path, "-o", obj]
            if with_checks:
                cmd += ["-DHB_BOUNDS_CHECK"]
            if ptxas_info:
                cmd += ["-Xptxas", "-v"]
            if verbose:
                print(" ".join(cmd), file=sys.stderr)
            subprocess.run(cmd, check=True)
            relink = True
    if relink or not os.path.exists(lib_path) or _stale(lib_path, objs):
        cmd = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", lib_path] + objs + ["-cudart", "static"]
        if verbose:
            print(" ".join(cmd), file=sys.stderr)
        subprocess.run(cmd, check=True)
    return lib_path


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv))
    if "--checked" in sys.argv:
        print(build(verbose=True, checked=True))
