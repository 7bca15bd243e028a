"""In-tree build of ``libflashck_b200.so`` (sm_100a only) with nvcc.

``python -m flashck_b200.build`` compiles every ``csrc/*.cu`` into ``flashck_b200/_build/*.o`` and links
the shared library next to this file.  Objects are rebuilt only when a source or header is newer.
"""
from __future__ import annotations

import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "_build")
LIB = os.path.join(HERE, "libflashck_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr", "-diag-suppress", "177",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def _newest(paths) -> float:
    return max(os.path.getmtime(p) for p in paths)


def build(force: bool = False, verbose: bool = False) -> str:
    nvcc = _nvcc()
    os.makedirs(OBJ, exist_ok=True)
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")) + \
        glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    hdr_time = _newest(headers) if headers else 0.0

    def compile_one(src: str):
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        if (not force and os.path.exists(obj)
                and os.path.getmtime(obj) >= max(os.path.getmtime(src), hdr_time)):
            return obj, ""
        cmd = [nvcc, *NVCC_FLAGS, "-Xptxas", "-v", "-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        return obj, r.stderr

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(sources))) as ex:
        results = list(ex.map(compile_one, sources))
    objs = [o for o, _ in results]
    if verbose:
        for _, log in results:
            if log:
                sys.stderr.write(log)
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < _newest(objs):
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB, *objs]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


def build_pybind(force: bool = False) -> str:
    """Compiles ``csrc/pybind/flash_ck.cpp`` -- the pybind11 / PyTorch binding over the C++ operator API -- into
    ``flashck_b200/flash_ck<ext suffix>`` with g++, linked against ``libflashck_b200.so`` (found at run time next to the
    module) and the torch libraries of this interpreter."""
    import sysconfig

    import torch
    from torch.utils import cpp_extension as ce
    src = os.path.join(CSRC, "pybind", "flash_ck.cpp")
    out = os.path.join(HERE, "flash_ck" + sysconfig.get_config_var("EXT_SUFFIX"))
    lib = build()
    deps = [src, lib, os.path.join(HERE, "..", "include", "flashck", "fmha", "fmha_fwd.h"),
            os.path.join(HERE, "..", "include", "flashck_b200.h")]
    if not force and os.path.exists(out) and os.path.getmtime(out) >= _newest(deps):
        return out
    gxx = os.environ.get("CXX") or shutil.which("g++")
    if not gxx:
        raise RuntimeError("g++ not found; set CXX")
    cuda_home = os.environ.get("CUDA_HOME") or os.path.dirname(os.path.dirname(_nvcc()))
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = [gxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-Wno-attributes",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", "-DTORCH_EXTENSION_NAME=flash_ck",
           "-DTORCH_API_INCLUDE_EXTENSION_H"]
    for inc in ce.include_paths() + [sysconfig.get_paths()["include"], os.path.join(cuda_home, "include"),
                                     os.path.join(HERE, "..", "include")]:
        cmd += ["-isystem" if "torch" in inc or "cuda" in inc else "-I", inc]
    cmd += [src, "-o", out, "-L", torch_lib, "-ltorch", "-ltorch_cpu", "-lc10", "-lc10_cuda", "-ltorch_python",
            "-L", HERE, "-l:libflashck_b200.so", f"-Wl,-rpath,{torch_lib}", "-Wl,-rpath,$ORIGIN"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"g++ failed for {src}:\n{r.stdout}\n{r.stderr[-6000:]}")
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--no-pybind" not in sys.argv:
        print(build_pybind(force="--force" in sys.argv))
