"""Build recipe for the CPU oracle and the compiled reference -- TEST INFRASTRUCTURE ONLY.

`build_oracle()` compiles the plain-C restatement (habitat_oracle.c) into
oracle/_build/libhabitat_oracle.so.

`build_ref()` compiles, when the reference tree is present, the reference's own
sources from where they lie (nothing is copied) into oracle/_ref/:
  * libhabitat_ref.so   - cpp/src/cuda/kernel.cpp behind a small C-ABI shim;
  * habitat_cuda*.so    - the reference's pybind11 bindings
                          (cpp/src/frontend/model_bindings.cpp) plus a
                          KernelInstance factory, for fixture generation;
  * libtoolkit_occ.so   - the CUDA toolkit's cuda_occupancy.h under Habitat's
                          call convention (covers compute capability >= 8).
The reference's CMake build is not used: it needs CUPTI, gflags and pybind11
submodules that are absent; these three translation units need none of them.
"""
import os
import shutil
import subprocess
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
BUILD_DIR = os.path.join(HERE, "_build")
REF_DIR = os.path.join(HERE, "_ref")
# the reference tree: HABITAT_REFERENCE_ROOT, else a `reference` directory beside this repository
REFERENCE_ROOT = os.environ.get("HABITAT_REFERENCE_ROOT") or os.path.join(
    os.path.dirname(os.path.dirname(HERE)), "reference")
CUDA_INCLUDE = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")


def _run(cmd):
    subprocess.run(cmd, check=True)


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources if os.path.exists(s))


def build_oracle(force=False):
    os.makedirs(BUILD_DIR, exist_ok=True)
    out = os.path.join(BUILD_DIR, "libhabitat_oracle.so")
    srcs = [os.path.join(HERE, "habitat_oracle.c"), os.path.join(HERE, "habitat_oracle.h")]
    if force or _stale(out, srcs):
        _run(["gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off",
              srcs[0], "-o", out, "-lm"])
    return out


def reference_available():
    return os.path.isdir(os.path.join(REFERENCE_ROOT, "cpp", "src", "cuda"))


def build_ref(force=False):
    """Returns the dict of built artefacts (possibly prebuilt ones when the
    reference tree is absent, e.g. on a GPU box)."""
    os.makedirs(REF_DIR, exist_ok=True)
    ext = sysconfig.get_config_var("EXT_SUFFIX")
    outs = {
        "ref": os.path.join(REF_DIR, "libhabitat_ref.so"),
        "pybind": os.path.join(REF_DIR, "habitat_cuda" + ext),
        "toolkit": os.path.join(REF_DIR, "libtoolkit_occ.so"),
    }
    tk_src = os.path.join(HERE, "toolkit_occupancy_shim.cpp")
    if os.path.exists(os.path.join(CUDA_INCLUDE, "cuda_occupancy.h")) and (
            force or _stale(outs["toolkit"], [tk_src])):
        _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-I", CUDA_INCLUDE, tk_src,
              "-o", outs["toolkit"]])
    if not reference_available():
        return {k: v for k, v in outs.items() if os.path.exists(v)}
    src_root = os.path.join(REFERENCE_ROOT, "cpp", "src")
    kernel_cpp = os.path.join(src_root, "cuda", "kernel.cpp")
    shim = os.path.join(HERE, "ref_occupancy_shim.cpp")
    if force or _stale(outs["ref"], [shim, kernel_cpp]):
        _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-I", src_root, shim, kernel_cpp,
              "-o", outs["ref"]])
    pyshim = os.path.join(HERE, "ref_pybind_shim.cpp")
    bindings = os.path.join(src_root, "frontend", "model_bindings.cpp")
    if force or _stale(outs["pybind"], [pyshim, bindings, kernel_cpp]):
        import pybind11
        _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-I", src_root,
              "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"],
              pyshim, bindings, kernel_cpp, "-o", outs["pybind"]])
    return outs


if __name__ == "__main__":
    print(build_oracle(force=True))
    for k, v in build_ref(force=True).items():
        print(k, v)
