"""Build oracle/_ref/quik_ref_ops*.so: the QUIK reference's own quantize / dequantize CUDA kernels.

Test infrastructure, not product code.  The reference's sources are compiled where they lie (the checkout given by
QUIK_REFERENCE_DIR, default /root/reference): src/asymmetric/asymmetric.cu and src/symmetric/symmetric.cu with the
small binding oracle/ref_binding.cpp.  They include one header-only CUTLASS file (cutlass/subbyte_reference.h, for the
packed-int4 reference type), taken from a CUTLASS header tree installed in the Python environment; the reference's GEMM
and fused-dequantize sources need CUTLASS GEMM templates from a submodule that the checkout does not vendor and are
left out.  Nothing of the reference is copied into this repository; the output directory is git-ignored.

Usage: python oracle/build_ref.py     (prints the path of the library, or why it was not built, and exits 0)
"""
import glob
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
NAME = "quik_ref_ops"


def _cutlass_include():
    for mod, rel in (("flashinfer", "data/cutlass/include"), ("tilelang", "3rdparty/cutlass/include")):
        try:
            m = __import__(mod)
        except Exception:
            continue
        path = os.path.join(os.path.dirname(m.__file__), rel)
        if os.path.isfile(os.path.join(path, "cutlass", "subbyte_reference.h")):
            return path
    return None


def lib_path():
    return os.path.join(OUT_DIR, NAME + sysconfig.get_config_var("EXT_SUFFIX"))


def build(verbose=False):
    ref = os.environ.get("QUIK_REFERENCE_DIR", "/root/reference")
    srcs = [os.path.join(ref, "src", "asymmetric", "asymmetric.cu"), os.path.join(ref, "src", "symmetric", "symmetric.cu")]
    if not all(os.path.isfile(s) for s in srcs):
        return None, f"reference sources not found under {ref}"
    cutlass = _cutlass_include()
    if cutlass is None:
        return None, "no CUTLASS header tree with cutlass/subbyte_reference.h in this environment"
    import torch
    from torch.utils import cpp_extension as ce

    out = lib_path()
    binding = os.path.join(HERE, "ref_binding.cpp")
    newest = max(os.path.getmtime(s) for s in srcs + [binding, __file__])
    if os.path.isfile(out) and os.path.getmtime(out) >= newest:
        return out, "up to date"
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    inc = [os.path.join(ref, "include"), cutlass, sysconfig.get_paths()["include"]] + ce.include_paths("cuda")
    # the half-operator switches are the ones the reference's own CMakeLists.txt (lines 77-80) passes to nvcc
    common = ["-O2", "-std=c++17", "-DCUDA_HAS_FP16=1", "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
              "-D__CUDA_NO_HALF2_OPERATORS__", "-D__CUDA_NO_BFLOAT16_CONVERSIONS__",
              "-DTORCH_EXTENSION_NAME=" + NAME, "-DTORCH_API_INCLUDE_EXTENSION_H",
              "-D_GLIBCXX_USE_CXX11_ABI=" + str(int(torch._C._GLIBCXX_USE_CXX11_ABI))] + ["-I" + i for i in inc]
    # the three translation units take minutes each (torch headers under nvcc): compile them side by side
    objs, procs = [], []
    for i, src in enumerate(srcs + [binding]):
        obj = os.path.join(OUT_DIR, f"ref_{i}.o")
        cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "--expt-relaxed-constexpr", "--expt-extended-lambda",
               "-Xcompiler", "-fPIC", "-x", "cu", *common, "-c", src, "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)))
        objs.append(obj)
    failed = None
    for src, pr in procs:
        _, err = pr.communicate()
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
