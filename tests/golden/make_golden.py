"""Generate tests/golden/reference_vectors.npz from the reference itself.

Run where the reference checkout is present (its location: MOE_REFERENCE_ROOT,
see REFERENCE below for the default):

    python tests/golden/make_golden.py

Two sources, both the reference's own code:
 1. oracle/_ref/ref_fixtures — the reference's C++ test fixtures
    (test/test_cpp/test_utils.h) compiled by `python -m oracle.build --ref`.
 2. The reference's Python helpers python/common.py (quantize_1d_128,
    quantize_2d_128, calc_cosine_diff) and python/benchmark_mlp.py
    (manual_swiglu_ref, reference_fused_silu_mul_quant), imported from the
    checkout. They import the compiled `moe_cuda` extension and
    TransformerEngine at module load; neither exists here, so inert stand-in
    modules are registered first. Only CPU-runnable functions are called.

The GPU box has no reference checkout: tests read the committed .npz only.
"""
from __future__ import annotations

import enum
import os
import struct
import subprocess
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
REFERENCE = Path(os.environ["MOE_REFERENCE_ROOT"]) if os.environ.get("MOE_REFERENCE_ROOT") \
    else REPO.parent / "reference"
OUT = HERE / "reference_vectors.npz"

_NP = {1: np.uint8, 2: np.uint16, 4: np.float32, 8: np.float64}


def read_fixture_records(path: Path) -> dict[int, np.ndarray]:
    data = path.read_bytes()
    off = 0
    out = {}
    int_tags = {11: np.int32, 12: np.int64, 13: np.int32}
    while off < len(data):
        tag, ndim = struct.unpack_from("<ii", data, off)
        off += 8
        dims = struct.unpack_from(f"<{ndim}q", data, off)
        off += 8 * ndim
        (es,) = struct.unpack_from("<i", data, off)
        off += 4
        n = int(np.prod(dims)) if ndim else 1
        dt = int_tags.get(tag, _NP[es])
        out[tag] = np.frombuffer(data, dtype=dt, count=n, offset=off).reshape(dims).copy()
        off += n * es
    return out


class _Stub(types.ModuleType):
    """A module whose every attribute is another inert stand-in."""

    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)
        return _Stub(f"{self.__name__}.{name}")

    def __call__(self, *a, **k):
        return None


def import_reference_python():
    class GemmType(enum.IntEnum):
        Normal = 0
        MGroupedContiguous = 1
        MGroupedMasked = 2
        Batched = 3

    moe_cuda = _Stub("moe_cuda")
    moe_cuda.GemmType = GemmType
    sys.modules["moe_cuda"] = moe_cuda
    for name in ["transformer_engine", "transformer_engine.pytorch",
                 "transformer_engine.common", "transformer_engine.common.recipe",
                 "transformer_engine.pytorch.tensor",
                 "transformer_engine.pytorch.tensor.float8_blockwise_tensor",
                 "transformer_engine_torch"]:
        sys.modules[name] = _Stub(name)
    sys.path.insert(0, str(REFERENCE / "python"))
    import common  # noqa: E402
    import benchmark_mlp  # noqa: E402
    return common, benchmark_mlp, GemmType


def main() -> int:
    fix_bin = REPO / "oracle" / "_ref" / "ref_fixtures"
    if not fix_bin.exists():
        subprocess.check_call([sys.executable, "-m", "oracle.build", "--ref"], cwd=REPO)
    tmp = HERE / "_fixtures.bin"
    subprocess.check_call([str(fix_bin), str(tmp)])
    rec = read_fixture_records(tmp)
    tmp.unlink()
    g = {
        "cpp_x": rec[1], "cpp_q1d": rec[2], "cpp_sf1d_kmajor": rec[3], "cpp_sf1d_mnmajor": rec[4],
        "cpp_w": rec[5], "cpp_q2d": rec[6], "cpp_sf2d": rec[7],
        "cpp_diff_a": rec[8], "cpp_diff_b": rec[9], "cpp_diff": rec[10],
        "cpp_layout_contig": rec[11], "cpp_layout_contig_actual": rec[12],
        "cpp_layout_masked": rec[13],
    }

    common, bmlp, GemmType = import_reference_python()
    torch.manual_seed(0)
    # python quantisers (fp32 tensors holding bf16-representable values, no zero blocks)
    x = torch.randn(8, 256).bfloat16().float()
    q, s = common.quantize_1d_128(x)
    g["py_x"] = x.numpy()
    g["py_q1d"] = q.view(torch.uint8).numpy()
    g["py_sf1d_mn"] = s.numpy()  # [H/128, rows]
    w = (torch.randn(2, 128, 256) * 0.02).bfloat16().float()
    q, s = common.quantize_2d_128(w)
    g["py_w"] = w.numpy()
    g["py_q2d"] = q.view(torch.uint8).numpy()
    g["py_sf2d"] = s.numpy()
    a = torch.randn(64, 32)
    b = a + 0.05 * torch.randn(64, 32)
    g["py_cos_a"], g["py_cos_b"] = a.numpy(), b.numpy()
    g["py_cos_diff"] = np.array([float(common.calc_cosine_diff(a, b))])

    # manual_swiglu_ref: contiguous (3 groups, ragged, -1 padding) and masked
    G, H, I = 3, 256, 128
    actual = [100, 128, 37]
    layout = []
    for gi, m in enumerate(actual):
        layout += [gi] * m + [-1] * ((m + 127) // 128 * 128 - m)
    layout = torch.tensor(layout, dtype=torch.int32)
    A = (torch.randn(layout.numel(), H) * H ** -0.5).bfloat16()
    gate = (torch.randn(G, I, H) * 0.5).bfloat16()
    up = (torch.randn(G, I, H) * 0.5).bfloat16()
    ref = bmlp.manual_swiglu_ref(A=A, gate_weight=gate, up_weight=up, grouped_layout=layout,
                                 gemm_type=GemmType.MGroupedContiguous, num_groups=G)
    bits = lambda t: t.contiguous().view(torch.int16).numpy().view(np.uint16)  # noqa: E731
    g["sw_A"], g["sw_gate"], g["sw_up"] = bits(A), bits(gate), bits(up)
    g["sw_layout"] = layout.numpy()
    g["sw_ref_contig"] = bits(ref)
    max_m = 128
    counts = torch.tensor([128, 50, 0], dtype=torch.int32)
    Am = (torch.randn(G * max_m, H) * H ** -0.5).bfloat16()
    refm = bmlp.manual_swiglu_ref(A=Am, gate_weight=gate, up_weight=up, grouped_layout=counts,
                                  gemm_type=GemmType.MGroupedMasked, num_groups=G, max_m=max_m)
    g["sw_A_masked"] = bits(Am)
    g["sw_counts_masked"] = counts.numpy()
    g["sw_ref_masked"] = bits(refm)

    # reference_fused_silu_mul_quant (bf16 silu(gate)*up)
    go = torch.randn(8, 512).bfloat16()
    g["silu_in"] = bits(go)
    g["silu_ref"] = bits(bmlp.reference_fused_silu_mul_quant(go))

    np.savez_compressed(OUT, **g)
    print(f"wrote {OUT} ({OUT.stat().st_size} bytes, {len(g)} arrays)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
