"""The C-ABI library loads on a machine without a GPU and exports every symbol
include/moe_cuda_b200.h declares; argument validation works without a device."""
import ctypes
import re
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (REPO / "include" / "moe_cuda_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(moeb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = declared_symbols()
    for must in ["moeb_router_logits", "moeb_router_select", "moeb_route_plan", "moeb_permute_quant",
                 "moeb_fp8_grouped_gemm_swiglu", "moeb_fp8_grouped_gemm_nt",
                 "moeb_unpermute_combine", "moeb_moe_forward", "moeb_status_string"]:
        assert must in names


def test_library_exports_every_declared_symbol(lib):
    from parallel_playground_b200 import cabi
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
        assert name in cabi.PROTOTYPES, f"{name} has no ctypes prototype"
    assert set(cabi.PROTOTYPES) <= set(declared_symbols())


def test_host_only_entry_points(lib):
    assert lib.moeb_abi_version() >= 1
    assert lib.moeb_status_string(0) == b"ok"
    assert b"wait" in lib.moeb_status_string(4)
    assert lib.moeb_route_plan_rows(256, 2, 8, 128) == (256 * 2 + 8 * 127 + 127) // 128 * 128
    assert lib.moeb_route_plan_rows(0, 2, 8, 128) == 1024
    assert lib.moeb_route_plan_rows(-1, 2, 8, 128) == -1
    assert lib.moeb_route_plan_workspace_bytes(256, 2, 8) % 256 == 0
    from parallel_playground_b200.cabi import LayerConfig
    cfg = LayerConfig(256, 1024, 512, 8, 2, 0, 1, 1, 1, 1.0)
    assert lib.moeb_moe_forward_workspace_bytes(cfg) > 0
    bad = LayerConfig(256, 1000, 512, 8, 2, 0, 1, 1, 1, 1.0)  # H not a multiple of 128
    assert lib.moeb_moe_forward_workspace_bytes(bad) == 0


def test_invalid_arguments_are_rejected_without_a_device(lib):
    # null pointers / bad shapes return "invalid argument" before any CUDA call
    assert lib.moeb_cast_bf16_to_e4m3(None, None, None, 4, 128, 0, None) == 1
    assert lib.moeb_router_select(None, 1, 8, 2, 0, 1, 1, 1, 1.0, None, None, None) == 1
    assert lib.moeb_fp8_grouped_gemm_nt(None, None, None, None, None, 0, 128, 128, 128, 1, 1, None,
                                        0, None, None) == 1
    assert b"null" in lib.moeb_last_error()
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.addressof(buf)
    p = (p + 255) // 256 * 256
    # K not a multiple of 128
    assert lib.moeb_fp8_grouped_gemm_nt(p, p, p, p, p, 0, 128, 128, 100, 1, 1, p, 0, None, None) == 1
    # Normal / Batched GEMM types are outside the MoE path
    assert lib.moeb_fp8_grouped_gemm_nt(p, p, p, p, p, 0, 128, 128, 128, 1, 0, p, 0, None, None) == 1
    assert lib.moeb_permute_quant(p, p, 4, 40, 128, 512, p, p, None) == 1  # k > 32


def test_missing_library_fails_loudly(tmp_path):
    from parallel_playground_b200 import cabi
    with pytest.raises(ImportError):
        cabi.load(tmp_path / "libmoe_cuda_b200.so")


def test_python_ops_reject_cpu_tensors(lib):
    import torch
    from parallel_playground_b200 import moe_cuda
    x = torch.zeros(4, 128, dtype=torch.bfloat16)
    q = torch.zeros(4, 128, dtype=torch.float8_e4m3fn)
    s = torch.zeros(4, 1)
    with pytest.raises(ValueError):
        moe_cuda.cast(x, q, s)
    with pytest.raises(ValueError):
        moe_cuda.bf16_gemm(x, x, x)          # CPU tensors: there is no CPU path
    with pytest.raises(NotImplementedError):
        moe_cuda.bf16_gemm(x, x, x, gemm_type=moe_cuda.GemmType.Batched)


def test_compiled_extension_exposes_reference_names(lib):
    """The pybind module (C++ host side, at::Tensor signatures of the reference's
    csrc/python_api.cpp) builds, imports without a GPU and carries the op names."""
    from parallel_playground_b200.build import load_extension
    ext = load_extension()
    for name in ["init", "cast", "fused_silu_mul_quant", "fp8_grouped_gemm_nt",
                 "fp8_grouped_gemm_swiglu", "fp8_grouped_gemm_swiglu_contiguous",
                 "fp8_grouped_gemm_swiglu_masked", "fp8_grouped_gemm_swiglu_sub",
                 "fp8_grouped_gemm_swiglu_pp", "fp8_grouped_gemm_swiglu_masked_pp", "bf16_gemm",
                 "fp8_gemm_nt", "All2All", "naive_moe_forward_dispatch", "all2all_symmetric_bytes"]:
        assert hasattr(ext, name), name
    assert ext.all2all_symmetric_bytes(256, 8, 2, 128, 1024, 1) > 0
    assert int(ext.GemmType.MGroupedContiguous) == 1 and int(ext.GemmType.MGroupedMasked) == 2
    ext.init("", "")


def test_router_workspace_query_is_host_only_and_monotone(lib):
    """moeb_router_logits_workspace_bytes: 0 where the tensor-core path does not apply (few
    tokens, up to 64 experts, E % 8 != 0, bad sizes); otherwise a size that also serves
    every smaller token count, so one workspace sized for the most tokens is enough."""
    q = lib.moeb_router_logits_workspace_bytes
    assert q(8192, 4096, 32) == 0 and q(8192, 4096, 64) == 0      # narrow routers
    assert q(512, 4096, 256) == 0                                  # few tokens
    assert q(8192, 4096, 100) == 0                                 # E % 8 != 0
    assert q(8192, 4100, 256) == 0 and q(0, 4096, 256) == 0 and q(8192, 4096, 0) == 0
    big = q(8192, 4096, 256)
    assert big >= 256 * 4096 * 2 + 8192 * 256 * 4
    sizes = [q(t, 4096, 256) for t in (1024, 2048, 4096, 8192, 20000, 65536)]
    assert all(b >= a > 0 for a, b in zip(sizes, sizes[1:]))
    assert sizes[3] == big


def test_ep_mode_query_without_a_context(lib):
    assert lib.moeb_ep_mlp_mode(None) == -1
