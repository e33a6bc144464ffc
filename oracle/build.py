"""Build the CPU oracle (test infrastructure) with gcc.

``python -m oracle.build`` compiles oracle/moe_oracle.c into
oracle/libmoe_oracle.so. Floating-point contraction and fast-math are off so
that every operation is a single correctly rounded IEEE operation, which is
what the bit-exact comparisons with the CUDA kernels rely on.

When the reference checkout is present next to this repository the script
also compiles oracle/ref_fixtures.cpp against the reference's own C++ test
fixtures (test/test_cpp/test_utils.h: quantize_fp8_1d_block,
quantize_fp8_2d_block, calc_diff, grouped-layout generators) into
oracle/_ref/ref_fixtures, from the sources where they lie; nothing is copied.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

ORACLE_DIR = Path(__file__).resolve().parent
REPO_ROOT = ORACLE_DIR.parent
LIB_PATH = ORACLE_DIR / "libmoe_oracle.so"
SRC = ORACLE_DIR / "moe_oracle.c"
DET_MATH_DIR = REPO_ROOT / "parallel_playground_b200" / "csrc"
REF_DIR = ORACLE_DIR / "_ref"
REF_BIN = REF_DIR / "ref_fixtures"
# the reference checkout: named by MOE_REFERENCE_ROOT, else a directory `reference`
# beside this repository (absent on machines that only run the tests)
REFERENCE_ROOT = Path(os.environ["MOE_REFERENCE_ROOT"]) if os.environ.get("MOE_REFERENCE_ROOT") \
    else REPO_ROOT.parent / "reference"


def build_oracle(force: bool = False) -> Path:
    deps = [SRC, DET_MATH_DIR / "det_math.h"]
    if (not force and LIB_PATH.exists()
            and LIB_PATH.stat().st_mtime >= max(d.stat().st_mtime for d in deps)):
        return LIB_PATH
    gcc = shutil.which("gcc")
    if gcc is None:
        raise RuntimeError("gcc not found")
    cmd = [gcc, "-O2", "-std=c11", "-ffp-contract=off", "-fno-fast-math", "-fvisibility=hidden",
           "-shared", "-fPIC", "-I", str(DET_MATH_DIR), str(SRC), "-o", str(LIB_PATH), "-lm"]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"gcc failed:\n{res.stdout}")
    return LIB_PATH


def build_reference_fixtures(force: bool = False) -> Path | None:
    """Compile the reference's libtorch test fixtures; None if unavailable."""
    src = ORACLE_DIR / "ref_fixtures.cpp"
    hdr = REFERENCE_ROOT / "test" / "test_cpp" / "test_utils.h"
    if not src.exists() or not hdr.exists():
        return REF_BIN if REF_BIN.exists() else None
    if not force and REF_BIN.exists() and REF_BIN.stat().st_mtime >= src.stat().st_mtime:
        return REF_BIN
    import torch  # only to locate libtorch
    from torch.utils import cpp_extension

    gxx = shutil.which("g++")
    if gxx is None:
        return None
    REF_DIR.mkdir(exist_ok=True)
    torch_lib = Path(torch.__file__).parent / "lib"
    inc = []
    for p in cpp_extension.include_paths():
        inc += ["-isystem", p]
    inc += ["-I", str(REFERENCE_ROOT / "test" / "test_cpp"),
            "-I", str(REFERENCE_ROOT / "moe_cuda" / "include"),
            "-I", str(REFERENCE_ROOT / "csrc"),
            "-isystem", "/usr/local/cuda/include"]
    cmd = [gxx, "-O1", "-std=c++17", "-D_GLIBCXX_USE_CXX11_ABI=1", *inc, str(src), "-o",
           str(REF_BIN), f"-L{torch_lib}", f"-Wl,-rpath,{torch_lib}", "-ltorch", "-ltorch_cpu",
           "-lc10"]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"reference fixtures failed to compile:\n{res.stdout[-4000:]}")
    return REF_BIN


def main() -> int:
    print(build_oracle(force="--force" in sys.argv))
    if "--ref" in sys.argv:
        print(build_reference_fixtures(force=True))
    return 0


if __name__ == "__main__":
    sys.exit(main())
