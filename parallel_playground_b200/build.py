"""Build libmoe_cuda_b200.so (sm_100a only) in-tree with nvcc.

Usage: ``python -m parallel_playground_b200.build [--force] [--verbose]``.
The library has no dependency on torch or on libcuda at link time (the one
driver entry point it needs is resolved at run time), so it loads on machines
without a GPU, where only the symbol table can be checked.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
REPO_ROOT = PKG_DIR.parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "lib"
LIB_PATH = LIB_DIR / "libmoe_cuda_b200.so"

SOURCES = ["api.cu", "router.cu", "route_plan.cu", "quant.cu", "combine.cu", "ep_p2p.cu", "ep_ctx.cu",
           "grouped_gemm.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def find_nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found (set NVCC or add it to PATH)")
    return cand


def _newest_source_mtime() -> float:
    files = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    files.append(REPO_ROOT / "include" / "moe_cuda_b200.h")
    return max(f.stat().st_mtime for f in files)


def needs_build() -> bool:
    return not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < _newest_source_mtime()


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile every .cu file and link the shared library. Returns its path."""
    if not force and not needs_build():
        return LIB_PATH
    nvcc = find_nvcc()
    LIB_DIR.mkdir(exist_ok=True)
    obj_dir = LIB_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)
    include = ["-I", str(REPO_ROOT / "include"), "-I", str(CSRC)]
    procs = []
    for src in SOURCES:
        obj = obj_dir / (Path(src).stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *include, "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE,
                                                  stderr=subprocess.STDOUT, text=True)))
    objs = []
    for src, obj, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
        if verbose and out:
            print(f"--- {src}\n{out}")
        objs.append(str(obj))
    link = [nvcc, "-shared", "-o", str(LIB_PATH), *objs, "-gencode",
            "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC", "-cudart", "static"]
    res = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}")
    return LIB_PATH


EXT_NAME = "moe_cuda_b200_ext"


def extension_path() -> Path:
    import sysconfig
    return LIB_DIR / (EXT_NAME + sysconfig.get_config_var("EXT_SUFFIX"))


def build_extension(force: bool = False) -> Path:
    """Compile csrc/python_api.cpp (pybind11, at::Tensor signatures of the
    reference's C++ API) into lib/moe_cuda_b200_ext.*.so, linked against
    libmoe_cuda_b200.so. Plain g++: no JIT cache outside the tree."""
    import sysconfig

    import torch
    from torch.utils import cpp_extension

    out = extension_path()
    src = CSRC / "python_api.cpp"
    hdr = REPO_ROOT / "include" / "moe_cuda_b200_torch.hpp"
    build_library()
    if (not force and out.exists()
            and out.stat().st_mtime >= max(src.stat().st_mtime, hdr.stat().st_mtime,
                                           LIB_PATH.stat().st_mtime)):
        return out
    gxx = shutil.which("g++")
    if gxx is None:
        raise RuntimeError("g++ not found")
    inc = []
    for p in cpp_extension.include_paths():
        inc += ["-isystem", p]
    inc += ["-isystem", sysconfig.get_paths()["include"], "-isystem", "/usr/local/cuda/include",
            "-I", str(REPO_ROOT / "include")]
    torch_lib = Path(torch.__file__).parent / "lib"
    cmd = [gxx, "-O2", "-std=c++17", "-shared", "-fPIC", f"-DTORCH_EXTENSION_NAME={EXT_NAME}",
           "-D_GLIBCXX_USE_CXX11_ABI=1", *inc, str(src), "-o", str(out),
           f"-L{LIB_DIR}", "-lmoe_cuda_b200", "-Wl,-rpath,$ORIGIN",
           f"-L{torch_lib}", f"-Wl,-rpath,{torch_lib}", "-ltorch", "-ltorch_cpu", "-ltorch_python",
           "-lc10", "-lc10_cuda", "-ltorch_cuda"]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"extension build failed:\n{res.stdout[-6000:]}")
    return out


def load_extension():
    """Import the compiled pybind module (building it if needed)."""
    import importlib.util

    import torch  # noqa: F401  (libtorch must be loaded first)
    path = build_extension()
    spec = importlib.util.spec_from_file_location(EXT_NAME, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas register/spill report")
    args = ap.parse_args()
    path = build_library(force=args.force, verbose=args.verbose)
    print(path)
    return 0


if __name__ == "__main__":
    sys.exit(main())
