"""ctypes binding of libmoe_cuda_b200.so (the C ABI declared in include/moe_cuda_b200.h).

The library is the product: there is no Python or CPU fallback. If it is
missing, loading raises with the build command to run.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_size_t, c_uint32, c_void_p
from pathlib import Path

from .build import LIB_PATH

GEMM_NORMAL = 0
GEMM_M_GROUPED_CONTIGUOUS = 1
GEMM_M_GROUPED_MASKED = 2
GEMM_BATCHED = 3

ROUTER_SOFTMAX = 0
ROUTER_SIGMOID_GROUPED = 1

OUT_BF16 = 0
OUT_F32 = 1

STATUS_DEVICE_TIMEOUT = 4


class LayerConfig(ctypes.Structure):
    """moeb_layer_config"""
    _fields_ = [("T", c_int), ("H", c_int), ("I", c_int), ("E", c_int), ("k", c_int),
                ("router_mode", c_int), ("n_group", c_int), ("topk_group", c_int),
                ("renorm", c_int), ("route_scale", c_float)]


class MoebError(RuntimeError):
    def __init__(self, fn: str, status: int, text: str, detail: str):
        super().__init__(f"{fn} failed: status {status} ({text}) {detail}".rstrip())
        self.status = status


class EpConfig(ctypes.Structure):
    """moeb_ep_config"""
    _fields_ = [("max_tokens", c_int), ("hidden", c_int), ("num_experts", c_int),
                ("top_k", c_int), ("expert_padding", c_int), ("world", c_int), ("rank", c_int),
                ("capacity_rows", c_int), ("transport", c_int)]


class EpView(ctypes.Structure):
    """moeb_ep_view"""
    _fields_ = [("expert_x", c_void_p), ("expert_x_scale", c_void_p), ("grouped_layout", c_void_p),
                ("m_valid", c_void_p), ("tokens_per_expert", c_void_p),
                ("padded_offsets", c_void_p), ("source_rank", c_void_p), ("source_pos", c_void_p),
                ("dst_rank", c_void_p), ("dst_row", c_void_p), ("overflow", c_void_p),
                ("home", c_void_p), ("max_recv_rows", c_int), ("local_experts", c_int),
                ("rows", c_int)]


# name -> (restype, argtypes); every symbol include/moe_cuda_b200.h declares
PROTOTYPES = {
    "moeb_abi_version": (c_int, []),
    "moeb_status_string": (ctypes.c_char_p, [c_int]),
    "moeb_last_error": (ctypes.c_char_p, []),
    "moeb_router_logits": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                   c_void_p]),
    "moeb_router_logits_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "moeb_router_logits_ws": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                      c_void_p, c_size_t, c_void_p, c_void_p]),
    "moeb_router_select": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                   c_float, c_void_p, c_void_p, c_void_p]),
    "moeb_route_plan_rows": (c_int, [c_int, c_int, c_int, c_int]),
    "moeb_route_plan_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "moeb_route_plan": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t,
                                c_void_p]),
    "moeb_route_plan_static_max_ints": (c_int, []),
    "moeb_route_plan_static": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                       c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_void_p]),
    "moeb_cast_bf16_to_e4m3": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                       c_void_p]),
    "moeb_fused_silu_mul_quant": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                          c_void_p]),
    "moeb_permute_quant": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                   c_void_p, c_void_p]),
    "moeb_dispatch_pack": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int,
                                   c_void_p]),
    "moeb_dispatch_pack_q": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                     c_int, c_void_p]),
    "moeb_dispatch_unpack": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                     c_void_p, c_void_p]),
    "moeb_recv_plan": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                               c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "moeb_gather_rows_bf16": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "moeb_fp8_grouped_gemm_swiglu": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                             c_int, c_int, c_void_p, c_int, c_void_p, c_void_p]),
    "moeb_fp8_grouped_gemm_nt": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                         c_int, c_int, c_int, c_int, c_int, c_void_p, c_int,
                                         c_void_p, c_void_p]),
    "moeb_fp8_grouped_gemm_swiglu_dyn": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                 c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                                 c_int, c_int, c_int, c_int, c_void_p, c_int,
                                                 c_void_p, c_void_p]),
    "moeb_fp8_grouped_gemm_nt_dyn": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_int, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                             c_void_p, c_int, c_void_p, c_void_p]),
    "moeb_ep_dest_base": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                  c_void_p]),
    "moeb_ep_dispatch_once": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                      c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "moeb_ep_unstash": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                c_int, c_void_p, c_void_p, c_void_p]),
    "moeb_bf16_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                               c_void_p, c_int, c_void_p, c_void_p]),
    "moeb_ep_barrier": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_uint32,
                                c_void_p, c_void_p]),
    "moeb_ep_dispatch_p2p": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                     c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_void_p, c_void_p, c_void_p]),
    "moeb_fp8_grouped_gemm_nt_scatter": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                 c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                                                 c_int, c_void_p, c_void_p, c_void_p]),
    "moeb_ep_scale_transpose": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "moeb_ep_combine_pull": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                     c_void_p, c_int, c_void_p]),
    "moeb_unpermute_combine": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                       c_int, c_void_p]),
    "moeb_moe_forward_workspace_bytes": (c_size_t, [ctypes.POINTER(LayerConfig)]),
    "moeb_moe_forward": (c_int, [ctypes.POINTER(LayerConfig), c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p,
                                 c_void_p]),
    "moeb_moe_forward_host": (c_int, [ctypes.POINTER(LayerConfig), c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p,
                                      c_void_p]),
    "moeb_ep_max_recv_rows": (c_int, [ctypes.POINTER(EpConfig)]),
    "moeb_ep_symmetric_bytes": (c_size_t, [ctypes.POINTER(EpConfig)]),
    "moeb_ep_local_bytes": (c_size_t, [ctypes.POINTER(EpConfig)]),
    "moeb_ep_create": (c_int, [ctypes.POINTER(EpConfig), c_void_p, c_void_p, c_size_t, c_void_p,
                               ctypes.POINTER(c_void_p)]),
    "moeb_ep_destroy": (c_int, [c_void_p]),
    "moeb_ep_get_view": (c_int, [c_void_p, ctypes.POINTER(EpView)]),
    "moeb_ep_dispatch": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                 c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "moeb_ep_fused_dispatch_swiglu": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                              c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                              c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                              c_void_p, c_void_p]),
    "moeb_ep_fused_gemm_combine": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                           c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "moeb_ep_combine": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                c_void_p, c_void_p]),
    "moeb_ep_moe_forward_workspace_bytes": (c_size_t, [c_void_p, c_int]),
    "moeb_ep_moe_forward": (c_int, [c_void_p, ctypes.POINTER(LayerConfig), c_void_p, c_void_p,
                                    c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t,
                                    c_int, c_void_p, c_void_p]),
    "moeb_ep_mlp_mode": (c_int, [c_void_p]),
    "moeb_ep_set_timing": (c_int, [c_void_p, c_int]),
    "moeb_ep_read_timing": (c_int, [c_void_p, ctypes.POINTER(c_float), ctypes.POINTER(c_int)]),
}

_lib = None


def load(path: str | Path | None = None) -> ctypes.CDLL:
    """Load the shared library and attach prototypes (idempotent)."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = Path(path) if path is not None else LIB_PATH
    if not p.exists():
        raise ImportError(
            f"{p} is missing: build it with `python -m parallel_playground_b200.build` "
            "(needs nvcc; there is no CPU fallback)")
    lib = ctypes.CDLL(str(p))
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    if path is None:
        _lib = lib
    return lib


def check(fn_name: str, status: int) -> None:
    if status != 0:
        lib = load()
        raise MoebError(fn_name, status, lib.moeb_status_string(status).decode(),
                        lib.moeb_last_error().decode())


def call(fn_name: str, *args) -> None:
    """Call a status-returning entry point and raise MoebError on failure."""
    check(fn_name, getattr(load(), fn_name)(*args))
