"""Build oracle/_ref/quik_ref_ops*.so: the QUIK reference's own CUDA kernels.

Test infrastructure, not product code.  The reference's sources are compiled where they lie (the checkout given by the
environment variable QUIK_REFERENCE_DIR, else a directory `reference` beside this repository): src/asymmetric/{asymmetric,fused_dequantize}.cu,
src/symmetric/{symmetric,fused_dequantize}.cu and src/matmul/matmul.cu with the small binding oracle/ref_binding.cpp,
by nvcc directly (not by the reference's cmake build).  They need CUTLASS headers (the reference's own submodule is not
vendored in the checkout); a CUTLASS header tree installed in the Python environment is used instead.  The cuSPARSELt
path is not enabled.  The reference's module file experiments/qlinear.py is placed unmodified next to the library
(reference_qlinear.py) so that a GPU test can run it against this repository's `quik` package.  Nothing of the reference
enters this repository's history: the output directory is git-ignored.

Usage: python oracle/build_ref.py     (prints the path of the library, or why it was not built, and exits 0)
"""
import glob
import os
import subprocess
import sys
import sysconfig
import time

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
NAME = "quik_ref_ops"


def _cutlass_include():
    """[include dir, tools/util/include dir] of a CUTLASS tree that has both, or None."""
    for mod, rel in (("flashinfer", "data/cutlass"), ("tilelang", "3rdparty/cutlass")):
        try:
            m = __import__(mod)
        except Exception:
            continue
        root = os.path.join(os.path.dirname(m.__file__), rel)
        inc, util = os.path.join(root, "include"), os.path.join(root, "tools", "util", "include")
        if os.path.isfile(os.path.join(inc, "cutlass", "gemm", "device", "gemm.h")) and \
                os.path.isfile(os.path.join(util, "cutlass", "util", "host_reorder.h")):
            return [inc, util]
    return None


def lib_path():
    return os.path.join(OUT_DIR, NAME + sysconfig.get_config_var("EXT_SUFFIX"))


def reference_dir():
    """The reference checkout: QUIK_REFERENCE_DIR, else `reference` beside this repository (may not exist)."""
    return os.environ.get("QUIK_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def module_path():
    return os.path.join(OUT_DIR, "reference_qlinear.py")


def _place_module(ref):
    """The reference's layer module, byte for byte, beside the library (kept out of history with it)."""
    src = os.path.join(ref, "experiments", "qlinear.py")
    if os.path.isfile(src):
        import shutil
        os.makedirs(OUT_DIR, exist_ok=True)
        shutil.copyfile(src, module_path())


def build(verbose=False):
    ref = reference_dir()
    _place_module(ref)
    srcs = [os.path.join(ref, "src", *p) for p in (("asymmetric", "asymmetric.cu"), ("asymmetric", "fused_dequantize.cu"),
                                                   ("symmetric", "symmetric.cu"), ("symmetric", "fused_dequantize.cu"),
                                                   ("matmul", "matmul.cu"))]
    if not all(os.path.isfile(s) for s in srcs):
        return None, f"reference sources not found under {ref}"
    cutlass = _cutlass_include()
    if cutlass is None:
        return None, "no CUTLASS header tree (include + tools/util/include) in this environment"
    import torch
    from torch.utils import cpp_extension as ce

    out = lib_path()
    binding = os.path.join(HERE, "ref_binding.cpp")
    newest = max(os.path.getmtime(s) for s in srcs + [binding, __file__])
    if os.path.isfile(out) and os.path.getmtime(out) >= newest:
        return out, "up to date"
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    inc = [os.path.join(ref, "include"), *cutlass, sysconfig.get_paths()["include"]] + ce.include_paths("cuda")
    # the half-operator switches are the ones the reference's own CMakeLists.txt (lines 77-80) passes to nvcc
    common = ["-O2", "-std=c++17", "-DCUDA_HAS_FP16=1", "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
              "-D__CUDA_NO_HALF2_OPERATORS__", "-D__CUDA_NO_BFLOAT16_CONVERSIONS__",
              "-DTORCH_EXTENSION_NAME=" + NAME, "-DTORCH_API_INCLUDE_EXTENSION_H",
              "-D_GLIBCXX_USE_CXX11_ABI=" + str(int(torch._C._GLIBCXX_USE_CXX11_ABI))] + ["-I" + i for i in inc]
    # the translation units take minutes each (torch and CUTLASS headers under nvcc): compile them side by side
    objs, procs = [], []
    for i, src in enumerate(srcs + [binding]):
        obj = os.path.join(OUT_DIR, f"ref_{i}.o")
        cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "--expt-relaxed-constexpr", "--expt-extended-lambda",
               "-Xcompiler", "-fPIC", "-x", "cu", *common, "-c", src, "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)))
        objs.append(obj)
    failed = None
    limit = float(os.environ.get("QUIK_REF_BUILD_TIMEOUT", "1500"))      # seconds for all translation units together
    deadline = time.monotonic() + limit
    for src, pr in procs:
        try:
            _, err = pr.communicate(timeout=max(1.0, deadline - time.monotonic()))
        except subprocess.TimeoutExpired:
            for _, other in procs:
                if other.poll() is None:
                    other.kill()
            return None, f"compilation did not finish within {limit:.0f} s"
        if pr.returncode != 0 and failed is None:
            lines = [l for l in err.splitlines() if "error" in l]
            failed = f"nvcc failed for {os.path.basename(src)}: " + " | ".join(lines[:4])
        elif verbose and err:
            print(err[-300:], file=sys.stderr)
    if failed:
        return None, failed
    libdirs = ce.library_paths("cuda")
    cmd = [nvcc, "-shared", "-o", out, *objs, *["-L" + d for d in libdirs], "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda",
           "-ltorch", "-ltorch_python", "-lcudart", *["-Xlinker=-rpath=" + d for d in libdirs]]
    r = subprocess.run(cmd, capture_output=True, text=True)
    for o in objs:
        os.remove(o)
    if r.returncode != 0:
        return None, f"link failed: {r.stderr[-2000:]}"
    return out, "built"


def load():
    """Import the built library (None when it is absent, e.g. on a box without the reference checkout at build time)."""
    path = lib_path()
    if not os.path.isfile(path):
        return None
    import importlib.util

    import torch  # noqa: F401  (the library links against torch)
    spec = importlib.util.spec_from_file_location(NAME, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    path, why = build(verbose=True)
    print(path if path else "not built", "-", why)
