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

SOURCES = ["hb_error.cu", "wave_scale.cu", "reduce.cu", "mlp_chain.cu", "device_probe.cu"]

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


def build(force=False, verbose=False, ptxas_info=False):
    """Compile every CUDA source and link the shared library. Returns its path."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    headers = [os.path.join(SRC_DIR, f) for f in os.listdir(SRC_DIR)
               if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(INCLUDE_DIR, "habitat_b200.h"))
    objs = []
    relink = force
    for src in SOURCES:
        src_path = os.path.join(SRC_DIR, src)
        obj = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        objs.append(obj)
        if force or _stale(obj, [src_path] + headers):
            cmd = [_nvcc()] + NVCC_FLAGS + ["-I", INCLUDE_DIR, "-I", SRC_DIR, "-c", src_path, "-o", obj]
            if ptxas_info:
                cmd += ["-Xptxas", "-v"]
            if verbose:
                print(" ".join(cmd), file=sys.stderr)
            subprocess.run(cmd, check=True)
            relink = True
    if relink or not os.path.exists(LIB_PATH):
        cmd = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB_PATH] + objs + ["-cudart", "static"]
        if verbose:
            print(" ".join(cmd), file=sys.stderr)
        subprocess.run(cmd, check=True)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv))
