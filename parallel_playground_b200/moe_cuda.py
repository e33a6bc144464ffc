"""`moe_cuda`-compatible operator module on top of libmoe_cuda_b200.so.

Mirrors the names, positional order and keyword names of the reference's torch
extension (csrc/python_api.cpp:170-533, csrc/tk_bindings.cu:13-94): every op
takes pre-allocated CUDA tensors, writes its outputs in place, returns None and
runs on the current CUDA stream (python_api.cpp:26-28). Errors are Python
exceptions (the reference prints and exits, moe_cuda/include/moe_cuda/error.hpp:11-33).

torch is used for tensor memory, the current stream and torch.distributed
only; all arithmetic happens in the CUDA library. There is no CPU path: CPU
tensors are rejected.

Additions without a reference counterpart (they change no existing signature):
router_topk, route_plan, permute_quant, unpermute_combine, MoELayer.
"""
from __future__ import annotations

import enum
from typing import Optional

import torch

from . import cabi
from .cabi import LayerConfig, MoebError  # noqa: F401  (re-exported)


class GemmType(enum.IntEnum):
    """moe_cuda/include/moe_cuda/types.h:2-10"""
    Normal = 0
    MGroupedContiguous = 1
    MGroupedMasked = 2
    Batched = 3


Normal = GemmType.Normal
MGroupedContiguous = GemmType.MGroupedContiguous
MGroupedMasked = GemmType.MGroupedMasked
Batched = GemmType.Batched

ROUTER_SOFTMAX = cabi.ROUTER_SOFTMAX
ROUTER_SIGMOID_GROUPED = cabi.ROUTER_SIGMOID_GROUPED

_status_words: dict[int, torch.Tensor] = {}


def __getattr__(name):
    # `All2All` lives in ep.py (which imports this module): resolved on first use
    if name in ("All2All", "EPContext"):
        from . import ep
        return getattr(ep, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def init(library_root: str = "", cuda_home: str = "") -> None:
    """python_api.cpp:184-190. The reference sets JIT paths here; this build is
    compiled ahead of time, so the call only makes sure the library loads."""
    cabi.load()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("moe_cuda ops take CUDA tensors (there is no CPU path)")
        if t is not None and not t.is_contiguous():
            raise ValueError("moe_cuda ops take contiguous tensors")


def status_word(device: torch.device | int | None = None) -> torch.Tensor:
    """int32[12] device word that kernels fill when a bounded wait expires:
    [0:4] gate/up GEMM (and what runs before it in a layer call: the router's GEMM, the
    dispatch), [4:8] down GEMM (each zeroed by the call that uses it), [8:12] the
    expert-parallel rank barrier (never zeroed: the first expiry sticks)."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    if dev not in _status_words:
        _status_words[dev] = torch.zeros(12, dtype=torch.int32, device=f"cuda:{dev}")
    return _status_words[dev]


def check_device_status(device=None) -> None:
    """Synchronise and raise if a kernel reported an expired wait."""
    w = status_word(device).cpu().tolist()
    for base in (0, 4):
        if w[base] != 0:
            raise MoebError("device", w[base], cabi.load().moeb_status_string(w[base]).decode(),
                            f"role={w[base + 1]} tile={w[base + 2]} kblock={w[base + 3]}")
    if w[8] != 0:
        raise MoebError("device", w[8], cabi.load().moeb_status_string(w[8]).decode(),
                        f"rank barrier: peer {w[10]} did not arrive (epoch {w[11]})")


# ----------------------------------------------------------------- helpers --
def _mn_major_scale(scale: torch.Tensor, rows: int, n_kb: int, what: str) -> torch.Tensor:
    """Activation scales as [K/128, rows] fp32 contiguous. A [rows, K/128] tensor
    is transposed the way api::fp8_gemm_nt does (csrc/apis/moe.hpp:30)."""
    if scale.dtype != torch.float32:
        raise ValueError(f"{what} must be float32")
    if scale.dim() >= 2 and scale.shape[-2] == n_kb and scale.numel() == rows * n_kb:
        return scale
    if scale.dim() >= 2 and scale.shape[-1] == n_kb and scale.numel() == rows * n_kb:
        return scale.reshape(rows, n_kb).t().contiguous()
    raise ValueError(f"{what} has shape {tuple(scale.shape)}, expected [{n_kb}, {rows}]")


def _gemm_dims(A: torch.Tensor, W: torch.Tensor, gemm_type: GemmType):
    if W.dim() != 3:
        raise ValueError("weights must be [G, N, K]")
    G, N, K = W.shape
    if gemm_type == GemmType.MGroupedMasked:
        if A.dim() != 3 or A.shape[0] != G or A.shape[2] != K:
            raise ValueError("masked layout takes A of shape [G, max_m, K]")
        return A.shape[0] * A.shape[1], N, K, G, A.shape[1]
    if A.dim() != 2 or A.shape[1] != K:
        raise ValueError("contiguous layout takes A of shape [M, K]")
    return A.shape[0], N, K, G, 0


def _check_layout(grouped_layout: torch.Tensor, gemm_type: GemmType, m_total: int, G: int) -> None:
    if grouped_layout.dtype != torch.int32:
        raise ValueError("invalid grouped layout type")  # python_api.cpp:257
    want = G if gemm_type == GemmType.MGroupedMasked else m_total
    if grouped_layout.numel() < want:
        raise ValueError(f"grouped_layout has {grouped_layout.numel()} entries, needs {want}")


# ------------------------------------------------------------------- a5/a6 --
def fp8_grouped_gemm_swiglu(A, scale_a, gate_weight, gate_scale, up_weight, up_scale, D, scale_d,
                            gemm_type, grouped_layout) -> None:
    """python_api.cpp:249-276 -> kernels::fp8_grouped_gemm_swiglu."""
    _need_cuda(A, scale_a, gate_weight, gate_scale, up_weight, up_scale, D, scale_d,
               grouped_layout)
    gemm_type = GemmType(int(gemm_type))
    if gemm_type not in (GemmType.MGroupedContiguous, GemmType.MGroupedMasked):
        raise ValueError("fp8_grouped_gemm_swiglu supports MGroupedContiguous and MGroupedMasked")
    m_total, N, K, G, max_m = _gemm_dims(A, gate_weight, gemm_type)
    if up_weight.shape != gate_weight.shape:
        raise ValueError("gate and up weights must have the same shape")
    if D.shape[-1] // 128 != scale_d.shape[-2]:
        raise ValueError("incorrect output scale d layout")  # python_api.cpp:259
    _check_layout(grouped_layout, gemm_type, m_total, G)
    sa = _mn_major_scale(scale_a, m_total, K // 128, "scale_a")
    cabi.call("moeb_fp8_grouped_gemm_swiglu", _ptr(A), _ptr(sa), _ptr(gate_weight),
              _ptr(gate_scale), _ptr(up_weight), _ptr(up_scale), _ptr(D), _ptr(scale_d), m_total,
              N, K, G, int(gemm_type), _ptr(grouped_layout), max_m, _ptr(status_word(A.device)),
              _stream())


def fp8_grouped_gemm_swiglu_contiguous(A, scale_a, gate_weight, gate_scale, up_weight, up_scale,
                                       D, scale_d, grouped_layout) -> None:
    fp8_grouped_gemm_swiglu(A, scale_a, gate_weight, gate_scale, up_weight, up_scale, D, scale_d,
                            GemmType.MGroupedContiguous, grouped_layout)


def fp8_grouped_gemm_swiglu_masked(A, scale_a, gate_weight, gate_scale, up_weight, up_scale, D,
                                   scale_d, grouped_layout) -> None:
    fp8_grouped_gemm_swiglu(A, scale_a, gate_weight, gate_scale, up_weight, up_scale, D, scale_d,
                            GemmType.MGroupedMasked, grouped_layout)


# The reference ships three schedules of the same computation (kernel3,
# kernel3_sub without MMA/scale interleaving, kernel4 with consumer ping-pong;
# python_api.cpp:311-453). They are numerically the same op; here all names map
# to the one sm_100a kernel.
fp8_grouped_gemm_swiglu_sub = fp8_grouped_gemm_swiglu
fp8_grouped_gemm_swiglu_sub_contiguous = fp8_grouped_gemm_swiglu_contiguous
fp8_grouped_gemm_swiglu_sub_masked = fp8_grouped_gemm_swiglu_masked
fp8_grouped_gemm_swiglu_pp = fp8_grouped_gemm_swiglu
fp8_grouped_gemm_swiglu_contiguous_pp = fp8_grouped_gemm_swiglu_contiguous
fp8_grouped_gemm_swiglu_masked_pp = fp8_grouped_gemm_swiglu_masked


def fp8_grouped_gemm_nt(act, act_scale, weight, weight_scale, output, gemm_type,
                        grouped_layout) -> None:
    """python_api.cpp:233-247 -> kernels::fp8_grouped_gemm_nt (down projection)."""
    _need_cuda(act, act_scale, weight, weight_scale, output, grouped_layout)
    gemm_type = GemmType(int(gemm_type))
    if gemm_type not in (GemmType.MGroupedContiguous, GemmType.MGroupedMasked):
        raise ValueError("fp8_grouped_gemm only supports MGroupedContiguous and MGroupedMasked")
    m_total, N, K, G, max_m = _gemm_dims(act, weight, gemm_type)
    _check_layout(grouped_layout, gemm_type, m_total, G)
    if output.dtype == torch.bfloat16:
        out_dtype = cabi.OUT_BF16
    elif output.dtype == torch.float32:
        out_dtype = cabi.OUT_F32
    else:
        raise ValueError("output must be bfloat16 or float32")
    if output.numel() != m_total * N:
        raise ValueError("output has the wrong number of elements")
    sa = _mn_major_scale(act_scale, m_total, K // 128, "act_scale")
    cabi.call("moeb_fp8_grouped_gemm_nt", _ptr(act), _ptr(sa), _ptr(weight), _ptr(weight_scale),
              _ptr(output), out_dtype, m_total, N, K, G, int(gemm_type), _ptr(grouped_layout),
              max_m, _ptr(status_word(act.device)), _stream())


def bf16_gemm(a, b, d, c=None, gemm_type=GemmType.Normal, compiled_dims="", grouped_layout=None) -> None:
    """python_api.cpp:192-211. d[M,N] = a[M,K] * b[N,K]^T (dense) or the grouped
    forms with b [G,N,K]; bf16 operands, fp32 accumulation, bf16 or fp32 d. `c`
    is accepted and ignored, as in the reference (csrc/apis/moe.hpp:72-98 passes
    it on to a launcher that never reads it). Not on the FP8 MoE path."""
    gemm_type = GemmType(int(gemm_type))
    if gemm_type == GemmType.Batched:
        raise NotImplementedError("bf16_gemm: GemmType.Batched is not built")
    _need_cuda(a, b, d, grouped_layout)
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise ValueError("bf16_gemm takes bfloat16 operands")
    if d.dtype == torch.bfloat16:
        out_dtype = cabi.OUT_BF16
    elif d.dtype == torch.float32:
        out_dtype = cabi.OUT_F32
    else:
        raise ValueError("d must be bfloat16 or float32")
    if gemm_type == GemmType.Normal:
        if a.dim() != 2 or b.dim() not in (2, 3) or (b.dim() == 3 and b.shape[0] != 1):
            raise ValueError("bf16_gemm takes a [M,K] and b [N,K]")
        m_total, K = a.shape
        N, G, max_m = b.shape[-2], 1, 0
        if b.shape[-1] != K:
            raise ValueError("a and b disagree on K")
    else:
        if grouped_layout is None:
            raise ValueError("a grouped gemm_type needs grouped_layout")
        m_total, N, K, G, max_m = _gemm_dims(a, b, gemm_type)
        _check_layout(grouped_layout, gemm_type, m_total, G)
    if d.numel() != m_total * N:
        raise ValueError("d has the wrong number of elements")
    cabi.call("moeb_bf16_gemm", _ptr(a), _ptr(b), _ptr(d), out_dtype, m_total, N, K, G,
              int(gemm_type), _ptr(grouped_layout), max_m, _ptr(status_word(a.device)), _stream())


_zero_layouts: dict[int, torch.Tensor] = {}


def _zero_layout(device: torch.device, rows: int) -> torch.Tensor:
    """int32 zeros [>= rows]: the grouped layout of a single group."""
    dev = torch.device(device).index
    cur = _zero_layouts.get(dev)
    if cur is None or cur.numel() < rows:
        cur = torch.zeros(max(rows, 1), dtype=torch.int32, device=f"cuda:{dev}")
        _zero_layouts[dev] = cur
    return cur


def fp8_gemm_nt(act, act_scale, weight, weight_scale, output, gemm_type=GemmType.Normal,
                compiled_dims="", grouped_layout=None) -> None:
    """python_api.cpp:213-231. Dense FP8 GEMM out[M,N] = act[M,K] * weight[N,K]^T
    with 1x128 activation scales and 128x128 weight scales: run as a grouped GEMM
    with one group (the grouped kernel has no other cost for it). A grouped
    gemm_type forwards to fp8_grouped_gemm_nt; Batched is not built."""
    gemm_type = GemmType(int(gemm_type))
    if gemm_type in (GemmType.MGroupedContiguous, GemmType.MGroupedMasked):
        if grouped_layout is None:
            raise ValueError("a grouped gemm_type needs grouped_layout")
        return fp8_grouped_gemm_nt(act, act_scale, weight, weight_scale, output, gemm_type,
                                   grouped_layout)
    if gemm_type != GemmType.Normal:
        raise NotImplementedError("fp8_gemm_nt: GemmType.Batched is not built")
    _need_cuda(act, act_scale, weight, weight_scale, output)
    if act.dim() != 2 or weight.dim() not in (2, 3) or (weight.dim() == 3 and weight.shape[0] != 1):
        raise ValueError("fp8_gemm_nt takes act [M,K] and weight [N,K]")
    M, K = act.shape
    N = weight.shape[-2]
    if weight.shape[-1] != K or output.numel() != M * N:
        raise ValueError("shape mismatch between act, weight and output")
    if output.dtype == torch.bfloat16:
        out_dtype = cabi.OUT_BF16
    elif output.dtype == torch.float32:
        out_dtype = cabi.OUT_F32
    else:
        raise ValueError("output must be bfloat16 or float32")
    sa = _mn_major_scale(act_scale, M, K // 128, "act_scale")
    cabi.call("moeb_fp8_grouped_gemm_nt", _ptr(act), _ptr(sa), _ptr(weight), _ptr(weight_scale),
              _ptr(output), out_dtype, M, N, K, 1, int(GemmType.MGroupedContiguous),
              _ptr(_zero_layout(act.device, M)), 0, _ptr(status_word(act.device)), _stream())


# ---------------------------------------------------------------------- a3 --
def cast(inp, out, scale=None) -> None:
    """python_api.cpp:455-462. bf16 -> e4m3 with 1x128 scales written row-major
    [rows, H/128] (csrc/kernels/cast.cuh:104-108); a [H/128, rows] scale tensor
    selects the MN-major layout the GEMMs consume."""
    _need_cuda(inp, out, scale)
    if inp.dtype == torch.bfloat16 and out.dtype == torch.float8_e4m3fn:
        if scale is None:
            raise ValueError("cast to float8_e4m3fn needs a scale tensor")
        H = inp.shape[-1]
        rows = inp.numel() // H
        n_kb = H // 128
        mn_major = scale.dim() >= 2 and scale.shape[-2] == n_kb and scale.shape[-1] == rows \
            and not (scale.shape[-1] == n_kb and scale.shape[-2] == rows)
        if scale.numel() != rows * n_kb or scale.dtype != torch.float32:
            raise ValueError("scale must be float32 with rows * H/128 elements")
        cabi.call("moeb_cast_bf16_to_e4m3", _ptr(inp), _ptr(out), _ptr(scale), rows, H,
                  int(mn_major), _stream())
        return
    raise NotImplementedError(
        f"cast {inp.dtype} -> {out.dtype}: only bfloat16 -> float8_e4m3fn is on the MoE path")


def fused_silu_mul_quant(gemm_out, swiglu_out, scale) -> None:
    """python_api.cpp:464-472: [rows, 2I] bf16 (gate | up) -> silu(gate)*up -> e4m3 + scales."""
    _need_cuda(gemm_out, swiglu_out, scale)
    if gemm_out.dtype != torch.bfloat16 or swiglu_out.dtype != torch.float8_e4m3fn:
        raise ValueError("fused_silu_mul_quant takes bfloat16 in, float8_e4m3fn out")
    I = gemm_out.shape[-1] // 2
    rows = gemm_out.numel() // (2 * I)
    n_kb = I // 128
    mn_major = scale.dim() >= 2 and scale.shape[-2] == n_kb and scale.shape[-1] == rows \
        and not (scale.shape[-1] == n_kb and scale.shape[-2] == rows)
    cabi.call("moeb_fused_silu_mul_quant", _ptr(gemm_out), _ptr(swiglu_out), _ptr(scale), rows, I,
              int(mn_major), _stream())


# ---------------------------------------------------------- a1, a2, a4, a7 --
def router_logits_workspace_bytes(T: int, H: int, E: int) -> int:
    """Scratch bytes with which router_logits runs on the tcgen05 tensor cores (many
    tokens, more than 64 experts); 0 where that path does not apply."""
    return int(cabi.load().moeb_router_logits_workspace_bytes(int(T), int(H), int(E)))


_router_scratch: dict = {}


def router_logits(x, w_gate, logits, bias=None, workspace=None) -> None:
    """logits = x @ w_gate (+ bias). `workspace`: uint8 device tensor of
    router_logits_workspace_bytes(T, H, E) bytes; None: a scratch tensor kept per device
    (so that every caller of this module gets the same kernels, and the same bits, as the
    whole-layer calls of the library, which always bring a workspace); False: none, the
    plain kernels."""
    _need_cuda(x, w_gate, logits, bias)
    if workspace is None:
        need = router_logits_workspace_bytes(x.shape[0], x.shape[1], w_gate.shape[1])
        if need > 0:
            key = x.device.index
            if key not in _router_scratch or _router_scratch[key].numel() < need:
                _router_scratch[key] = torch.empty(need, dtype=torch.uint8, device=x.device)
            workspace = _router_scratch[key]
    elif workspace is False:
        workspace = None
    T, H = x.shape
    E = w_gate.shape[1]
    if w_gate.shape[0] != H or x.dtype != torch.bfloat16 or w_gate.dtype != torch.bfloat16 \
            or logits.dtype != torch.float32 or logits.numel() != T * E:
        raise ValueError("router_logits: x [T,H] bf16, w_gate [H,E] bf16, logits [T,E] fp32")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != E):
        raise ValueError("router bias must be float32 [E]")
    if workspace is not None:
        _need_cuda(workspace)
        cabi.call("moeb_router_logits_ws", _ptr(x), _ptr(w_gate), _ptr(bias), _ptr(logits), T, H, E,
                  _ptr(workspace), workspace.numel() * workspace.element_size(),
                  status_word(x.device).data_ptr(), _stream())
        return
    cabi.call("moeb_router_logits", _ptr(x), _ptr(w_gate), _ptr(bias), _ptr(logits), T, H, E,
              _stream())


def router_select(logits, indices, weights, mode=ROUTER_SOFTMAX, n_group=1, topk_group=1,
                  renorm=True, route_scale=1.0) -> None:
    _need_cuda(logits, indices, weights)
    T, E = logits.shape
    k = indices.shape[1]
    if indices.dtype != torch.int32 or weights.dtype != torch.float32 or \
            logits.dtype != torch.float32 or weights.shape != indices.shape:
        raise ValueError("router_select: logits fp32 [T,E], indices int32 [T,k], weights fp32 [T,k]")
    cabi.call("moeb_router_select", _ptr(logits), T, E, k, int(mode), int(n_group),
              int(topk_group), int(bool(renorm)), float(route_scale), _ptr(indices), _ptr(weights),
              _stream())


def router_topk(x, w_gate, indices, weights, logits=None, mode=ROUTER_SOFTMAX, n_group=1,
                topk_group=1, renorm=True, route_scale=1.0, bias=None) -> None:
    """Router: logits = x @ w_gate (+ bias), then softmax / grouped-sigmoid top-k."""
    if logits is None:
        logits = torch.empty((x.shape[0], w_gate.shape[1]), dtype=torch.float32, device=x.device)
    router_logits(x, w_gate, logits, bias)
    router_select(logits, indices, weights, mode, n_group, topk_group, renorm, route_scale)


def route_plan_rows(T: int, k: int, E: int, pad: int = 128) -> int:
    return cabi.load().moeb_route_plan_rows(T, k, E, pad)


class RoutePlan:
    """Device-side routing plan buffers for (T, k, E): counts, padded offsets,
    (token,slot)->row map and its inverse, and the MGroupedContiguous layout."""

    def __init__(self, T: int, k: int, E: int, pad: int = 128, device=None):
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        self.T, self.k, self.E, self.pad = T, k, E, pad
        self.m_cap = route_plan_rows(T, k, E, pad)
        i32 = dict(dtype=torch.int32, device=device)
        self.expert_counts = torch.empty(E, **i32)
        self.padded_offsets = torch.empty(E + 1, **i32)
        self.dst_row = torch.empty((T, k), **i32)
        self.src_token = torch.empty(self.m_cap, **i32)
        self.src_slot = torch.empty(self.m_cap, **i32)
        self.grouped_layout = torch.empty(self.m_cap, **i32)
        ws = cabi.load().moeb_route_plan_workspace_bytes(T, k, E)
        self.workspace = torch.empty(ws, dtype=torch.uint8, device=device)

    def run(self, indices: torch.Tensor) -> "RoutePlan":
        _need_cuda(indices)
        if indices.dtype != torch.int32 or indices.numel() != self.T * self.k:
            raise ValueError("indices must be int32 [T,k]")
        cabi.call("moeb_route_plan", _ptr(indices), self.T, self.k, self.E, self.pad, self.m_cap,
                  _ptr(self.expert_counts), _ptr(self.padded_offsets), _ptr(self.dst_row),
                  _ptr(self.src_token), _ptr(self.src_slot), _ptr(self.grouped_layout),
                  _ptr(self.workspace), self.workspace.numel(), _stream())
        return self


def route_plan(indices: torch.Tensor, num_experts: int, pad: int = 128) -> RoutePlan:
    T, k = indices.shape
    return RoutePlan(T, k, num_experts, pad, indices.device).run(indices)


def permute_quant(x, dst_row, expert_x, expert_x_scale) -> None:
    """Quantise x [T,H] bf16 once per token and write its k copies to
    expert_x [m_cap,H] e4m3 / expert_x_scale [H/128,m_cap] fp32."""
    _need_cuda(x, dst_row, expert_x, expert_x_scale)
    T, H = x.shape
    k = dst_row.shape[1]
    m_cap = expert_x.shape[0]
    if expert_x_scale.shape != (H // 128, m_cap) or dst_row.dtype != torch.int32:
        raise ValueError("permute_quant: expert_x_scale must be [H/128, m_cap], dst_row int32")
    cabi.call("moeb_permute_quant", _ptr(x), _ptr(dst_row), T, k, H, m_cap, _ptr(expert_x),
              _ptr(expert_x_scale), _stream())


def unpermute_combine(expert_y, row_of_slot, weights, out_tokens, accumulate=False) -> None:
    """out[t] = (accumulate ? out[t] : 0) + sum_j weights[t,j] * expert_y[row_of_slot[t,j]]."""
    _need_cuda(expert_y, row_of_slot, weights, out_tokens)
    T, k = row_of_slot.shape
    H = expert_y.shape[-1]
    if expert_y.dtype != torch.bfloat16 or out_tokens.dtype != torch.bfloat16:
        raise ValueError("combine only supports bfloat16")  # a2a_context_tk.hpp:181-182
    cabi.call("moeb_unpermute_combine", _ptr(expert_y), _ptr(row_of_slot), _ptr(weights), T, k, H,
              _ptr(out_tokens), int(bool(accumulate)), _stream())


# ----------------------------------------------------------- whole layer ----
class MoELayer:
    """One-GPU MoE layer (router -> plan -> permute+quant -> gate/up SwiGLU GEMM
    -> down GEMM -> weighted un-permute) behind a single C-ABI call.

    Weights are pre-quantised e4m3 tensors with 128x128 fp32 scales:
    gate/up [E,I,H] + [E,I/128,H/128], down [E,H,I] + [E,H/128,I/128];
    w_router is bf16 [H,E]. The workspace is allocated once."""

    def __init__(self, T, H, I, E, k, w_router, gate, gate_scale, up, up_scale, down, down_scale,
                 router_mode=ROUTER_SOFTMAX, n_group=1, topk_group=1, renorm=True,
                 route_scale=1.0, router_bias=None):
        _need_cuda(w_router, gate, gate_scale, up, up_scale, down, down_scale, router_bias)
        self.router_bias = router_bias
        self.cfg = LayerConfig(T, H, I, E, k, int(router_mode), int(n_group), int(topk_group),
                               int(bool(renorm)), float(route_scale))
        self.device = gate.device
        self.tensors = (w_router, gate, gate_scale, up, up_scale, down, down_scale)
        lib = cabi.load()
        nbytes = lib.moeb_moe_forward_workspace_bytes(self.cfg)
        if nbytes == 0:
            raise ValueError("bad layer configuration (H and I multiples of 128, k <= E)")
        self.workspace = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.indices = torch.empty((T, k), dtype=torch.int32, device=self.device)
        self.weights = torch.empty((T, k), dtype=torch.float32, device=self.device)
        self._dev_x = None
        self._dev_out = None
        self._pipe = None

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> None:
        """Device tensors in, device tensor out (in place), current stream."""
        _need_cuda(x, out)
        w_router, gate, gs, up, us, down, ds = self.tensors
        cabi.call("moeb_moe_forward", self.cfg, _ptr(x), _ptr(w_router), _ptr(self.router_bias),
                  _ptr(gate), _ptr(gs),
                  _ptr(up), _ptr(us), _ptr(down), _ptr(ds), _ptr(out), _ptr(self.indices),
                  _ptr(self.weights), _ptr(self.workspace), self.workspace.numel(),
                  _ptr(status_word(self.device)), _stream())

    def forward_host(self, x_host: torch.Tensor, out_host: torch.Tensor) -> None:
        """(Pinned) host tensors in and out; the copies run on the current stream."""
        if x_host.is_cuda or out_host.is_cuda:
            raise ValueError("forward_host takes host tensors")
        c = self.cfg
        if self._dev_x is None:
            self._dev_x = torch.empty((c.T, c.H), dtype=torch.bfloat16, device=self.device)
            self._dev_out = torch.empty((c.T, c.H), dtype=torch.bfloat16, device=self.device)
        w_router, gate, gs, up, us, down, ds = self.tensors
        cabi.call("moeb_moe_forward_host", self.cfg, x_host.data_ptr(), out_host.data_ptr(),
                  _ptr(self._dev_x), _ptr(self._dev_out), _ptr(w_router), _ptr(self.router_bias),
                  _ptr(gate), _ptr(gs),
                  _ptr(up), _ptr(us), _ptr(down), _ptr(ds), _ptr(self.workspace),
                  self.workspace.numel(), _ptr(status_word(self.device)), _stream())


    def capture(self, x: torch.Tensor, out: torch.Tensor) -> "torch.cuda.CUDAGraph":
        """Records forward(x, out) into a CUDA graph and returns it: `replay()`
        re-runs the nine launches of the layer from one submission, which is what
        a launch-bound size (decode batches, the tiny configuration) needs. The
        library neither allocates nor synchronises, so the whole call is
        capturable. x and out are read and written in place at every replay."""
        _need_cuda(x, out)
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            self.forward(x, out)          # first-call set-up happens outside the capture
        torch.cuda.current_stream(self.device).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.forward(x, out)
        return graph

    def forward_host_batches(self, xs, outs) -> None:
        """A stream of (pinned) host batches: the PCIe copies of neighbouring
        batches overlap the layer (see hostpipe.HostPipeline). Results are
        readable after a synchronize on the current stream."""
        from .hostpipe import HostPipeline
        if self._pipe is None:
            c = self.cfg
            self._pipe = HostPipeline(self.forward, (c.T, c.H), (c.T, c.H), torch.bfloat16,
                                      self.device)
        self._pipe.process(xs, outs)


# ------------------------------------------------- multi-GPU entry points ----
class TKParallelTensor:
    """Stand-in for ThunderKittens' parallel tensor as the reference's Python side
    uses it (python/benchmark_fused_moe.py:519-535, bound in csrc/tk_bindings.cu:13-15):
    `TKParallelTensor(shape, dtype, local_rank, local_world_size, multicast)` owns
    one tensor per rank in peer-mapped memory, `.data()` is this rank's tensor.
    Here it is a torch symmetric-memory allocation (a plain device tensor when the
    process group has one rank). `multicast=True` is refused: no kernel of this
    library reads through NVLink multicast objects."""

    def __init__(self, shape, dtype, local_rank=0, local_world_size=1, multicast=False):
        import torch.distributed as dist
        if multicast:
            raise ValueError("TKParallelTensor(multicast=True) is not supported: this library "
                             "uses plain peer loads and stores only")
        self.shape = tuple(int(v) for v in shape)
        self.dtype = dtype
        self.local_rank = int(local_rank)
        self.local_world_size = int(local_world_size)
        dev = torch.device("cuda", self.local_rank)
        n = 1
        for v in self.shape:
            n *= v
        if self.local_world_size > 1:
            if not (dist.is_available() and dist.is_initialized()):
                raise RuntimeError("TKParallelTensor over several ranks needs torch.distributed")
            import torch.distributed._symmetric_memory as symm_mem
            nbytes = max(n, 1) * torch.empty((), dtype=dtype).element_size()
            self._raw = symm_mem.empty((nbytes + 15) // 16 * 16, dtype=torch.uint8, device=dev)
            self._handle = symm_mem.rendezvous(self._raw, dist.group.WORLD)
            self.raw_ptrs = [int(p) for p in self._handle.buffer_ptrs]
            self._t = self._raw[:n * torch.empty((), dtype=dtype).element_size()].view(dtype)
        else:
            self._t = torch.empty(max(n, 1), dtype=dtype, device=dev)[:n]
            self.raw_ptrs = [self._t.data_ptr()]
        self._t = self._t.view(self.shape)

    def data(self) -> torch.Tensor:
        return self._t


_fused_contexts: dict = {}


def _fused_context(T, E, k, H, device):
    """The process-wide expert-parallel context behind the reference-style fused
    ops, whose own signatures carry no handle."""
    from .ep import EPContext
    key = (int(T), int(E), int(k), int(H), torch.device(device).index)
    ctx = _fused_contexts.get(key)
    if ctx is None:
        ctx = _fused_contexts[key] = EPContext(T, E, k, H, device=key[4])
    return ctx


def _as_tensor(t):
    return t.data() if isinstance(t, TKParallelTensor) else t


def fused_dispatch_grouped_gemm_swiglu(*args, **kwargs):
    """csrc/tk_bindings.cu:17-60: dispatch the tokens to their experts' ranks and
    run the gate/up SwiGLU grouped GEMM over what arrives, as one op.

    Reference form (31 arguments, same order and keywords): in_tokens,
    in_tokens_scales (parallel tensors: e4m3 [T,H], fp32 [H/128,T]),
    expert_x_tokens, expert_x_tokens_scale (out: e4m3 [max_recv,H], fp32
    [H/128,max_recv]), gate, up, C (out: e4m3 [max_recv,I]), scale_gate, scale_up,
    out_scales (out: fp32 [I/128,max_recv]), indices, global_num_routed,
    expert_to_token_map, expert_to_slot_map, padded_expert_counts, src_token_idx,
    src_dev_idx, src_slot_idx, barrier, num_tokens, num_recv_tokens, dp_rank, rank,
    dp_size, cur_dp_group, num_dp_groups, world_size, num_experts,
    experts_per_token, num_comm_sms, num_comp_sms. The routing outputs
    (padded_expert_counts [E/W], src_token_idx / src_dev_idx / src_slot_idx
    [max_recv], num_recv_tokens [1]) are filled as the reference's kernel fills them;
    global_num_routed, the two maps and barrier are scratch of the reference's
    kernel and are left untouched: the state they stand for lives in this
    library's expert-parallel context. max_recv must be the context's
    max_recv_tokens (num_tokens*world*k padded per expert).

    Short form: (a2a, in_tokens, indices, gate, up, C, scale_gate, scale_up,
    out_scales) with a2a an ep.EPContext / ep.All2All (or ep.All2AllP2P) and bf16
    in_tokens; returns the device word holding the rows in use."""
    names31 = ("in_tokens", "in_tokens_scales", "expert_x_tokens", "expert_x_tokens_scale", "gate",
               "up", "C", "scale_gate", "scale_up", "out_scales", "indices", "global_num_routed",
               "expert_to_token_map", "expert_to_slot_map", "padded_expert_counts",
               "src_token_idx", "src_dev_idx", "src_slot_idx", "barrier", "num_tokens",
               "num_recv_tokens", "dp_rank", "rank", "dp_size", "cur_dp_group", "num_dp_groups",
               "world_size", "num_experts", "experts_per_token", "num_comm_sms", "num_comp_sms")
    if len(args) + len(kwargs) == len(names31) and "a2a" not in kwargs:
        a = dict(zip(names31, args))
        a.update(kwargs)
        if set(a) != set(names31):
            raise TypeError("fused_dispatch_grouped_gemm_swiglu: unexpected arguments")
        if a["dp_size"] != 1:
            raise ValueError("dp_size must be 1")   # the reference's dp > 1 path is untested, README.md:49
        xq = _as_tensor(a["in_tokens"])
        xs = _as_tensor(a["in_tokens_scales"])
        T = int(a["num_tokens"])
        H = xq.shape[1]
        _need_cuda(xq, xs, a["expert_x_tokens"], a["expert_x_tokens_scale"], a["gate"], a["up"],
                   a["C"], a["scale_gate"], a["scale_up"], a["out_scales"], a["indices"])
        ctx = _fused_context(xq.shape[0], a["num_experts"], a["experts_per_token"], H, xq.device)
        if ctx.world_size != int(a["world_size"]) or ctx.rank != int(a["rank"]):
            raise ValueError("world_size / rank do not match the process group")
        ctx.fused_dispatch_swiglu(None, a["indices"][:T], a["gate"], a["scale_gate"], a["up"],
                                  a["scale_up"], a["C"], a["out_scales"], fused=True,
                                  x_q=xq[:T], x_scale_mn=xs if T == xs.shape[1] else
                                  xs[:, :T].contiguous(),
                                  out_expert_x=a["expert_x_tokens"],
                                  out_expert_x_scale=a["expert_x_tokens_scale"])
        # routing outputs in the reference's terms
        k = int(a["experts_per_token"])
        off = ctx.padded_offsets
        a["padded_expert_counts"].view(torch.int32)[:ctx.e_local].copy_(off[1:] - off[:-1])
        n = min(a["src_token_idx"].numel(), ctx.m_cap)
        pos = ctx.source_pos[:n]
        live = (ctx.source_rank[:n] >= 0) & (pos >= 0)
        a["src_token_idx"].view(torch.int32)[:n].copy_(torch.where(live, pos // k, -1))
        a["src_slot_idx"].view(torch.int32)[:n].copy_(torch.where(live, pos % k, -1))
        a["src_dev_idx"].view(torch.int32)[:n].copy_(ctx.source_rank[:n])
        a["num_recv_tokens"].view(torch.int32)[:1].copy_(ctx.tokens_per_expert.sum().view(1))
        return ctx.m_valid
    a2a, in_tokens, indices, gate, up, C, scale_gate, scale_up, out_scales = args
    _need_cuda(in_tokens, indices, gate, up, C, scale_gate, scale_up, out_scales)
    ctx = getattr(a2a, "ctx", a2a)
    if hasattr(ctx, "fused_dispatch_swiglu"):
        ctx.fused_dispatch_swiglu(in_tokens, indices, gate, scale_gate, up, scale_up, C, out_scales,
                                  fused=kwargs.get("fused", True))
        return ctx.m_valid
    # ep.All2AllP2P: push dispatch, rank barrier, then the GEMM
    a2a.dispatch_bf16(in_tokens, indices)
    G, I, H = gate.shape
    cabi.call("moeb_fp8_grouped_gemm_swiglu_dyn", _ptr(a2a.expert_x), _ptr(a2a.scale_mn), _ptr(gate),
              _ptr(scale_gate), _ptr(up), _ptr(scale_up), _ptr(C), _ptr(out_scales), a2a.m_cap,
              _ptr(a2a.m_valid), I, H, G, cabi.GEMM_M_GROUPED_CONTIGUOUS, _ptr(a2a.grouped_layout),
              0, _ptr(status_word(in_tokens.device)), _stream())
    return a2a.m_valid


def fused_grouped_gemm_combine(*args, **kwargs):
    """csrc/tk_bindings.cu:62-94 (the reference ships only the launcher, its
    kernel file is empty): the down projection whose store warps send every
    expert-output row straight to the rank its token came from, over NVLink, then
    the weighted reduction of each token's k rows.

    Reference form (21 arguments, same order and keywords): out_tokens (parallel
    tensor or tensor, bf16 [T,H]), expert_y_tokens (e4m3 [max_recv,I]),
    expert_y_tokens_scale (fp32 [I/128,max_recv]), down, scale_down, C (unused
    scratch), weights (fp32 [T,k]), padded_expert_counts, src_token_idx,
    src_dev_idx, src_slot_idx, num_experts, experts_per_token, num_recv_tokens,
    dp_rank, rank, dp_size, cur_dp_group, num_dp_groups, num_comm_sms,
    num_comp_sms. It uses the routing of the preceding
    fused_dispatch_grouped_gemm_swiglu call.

    Short form: (a2a, out_tokens, expert_y_tokens, expert_y_tokens_scale, down,
    scale_down, weights, accumulate=False)."""
    names21 = ("out_tokens", "expert_y_tokens", "expert_y_tokens_scale", "down", "scale_down", "C",
               "weights", "padded_expert_counts", "src_token_idx", "src_dev_idx", "src_slot_idx",
               "num_experts", "experts_per_token", "num_recv_tokens", "dp_rank", "rank", "dp_size",
               "cur_dp_group", "num_dp_groups", "num_comm_sms", "num_comp_sms")
    if len(args) + len(kwargs) == len(names21) and "a2a" not in kwargs:
        a = dict(zip(names21, args))
        a.update(kwargs)
        if set(a) != set(names21):
            raise TypeError("fused_grouped_gemm_combine: unexpected arguments")
        out = _as_tensor(a["out_tokens"])
        _need_cuda(out, a["expert_y_tokens"], a["expert_y_tokens_scale"], a["down"],
                   a["scale_down"], a["weights"])
        T, H = out.shape
        ctx = _fused_context(T, a["num_experts"], a["experts_per_token"], H, out.device)
        n = ctx._n_tokens
        ctx.fused_gemm_combine(a["expert_y_tokens"], a["expert_y_tokens_scale"], a["down"],
                               a["scale_down"], a["weights"][:n], out[:n])
        return None
    a2a, out_tokens, expert_y_tokens, expert_y_tokens_scale, down, scale_down, weights = args[:7]
    accumulate = args[7] if len(args) > 7 else kwargs.get("accumulate", False)
    _need_cuda(out_tokens, expert_y_tokens, expert_y_tokens_scale, down, scale_down, weights)
    ctx = getattr(a2a, "ctx", a2a)
    if hasattr(ctx, "fused_gemm_combine"):
        ctx.fused_gemm_combine(expert_y_tokens, expert_y_tokens_scale, down, scale_down, weights,
                               out_tokens, accumulate)
        return None
    G, H, I = down.shape
    st = status_word(out_tokens.device)
    cabi.call("moeb_fp8_grouped_gemm_nt_scatter", _ptr(expert_y_tokens), _ptr(expert_y_tokens_scale),
              _ptr(down), _ptr(scale_down), _ptr(a2a.peer_home), _ptr(a2a.source_rank),
              _ptr(a2a.sym_pos), a2a.m_cap, _ptr(a2a.m_valid), H, I, G, _ptr(a2a.grouped_layout),
              st[4:].data_ptr(), _stream())
    a2a.combine_home(out_tokens, weights, accumulate)
    return None


def naive_moe_forward_dispatch(all2all, num_experts, experts_per_token, hidden_dim, gemm_type,
                               input, input_scales, gate, gate_scales, up, up_scales, down,
                               down_scales, indices, weights, out_tokens, expert_x,
                               expert_x_scales, inter_y, inter_y_scales, expert_y) -> None:
    """csrc/python_api.cpp:516-532 -> naive_moe_forward (src/moe_ops.cu:153-191):
    dispatch -> gate/up SwiGLU grouped GEMM -> down grouped GEMM -> combine, on the
    caller's buffers. input e4m3 [T,H] with input_scales fp32 [H/128,T]; expert_x
    e4m3 [max_recv_tokens,H] + expert_x_scales [H/128,max_recv_tokens]; inter_y e4m3
    [max_recv_tokens,I] + inter_y_scales [I/128,max_recv_tokens]; expert_y bf16
    [max_recv_tokens,H]; out_tokens bf16 [T,H]. The grouped layout handed to the
    GEMMs is the expert id per row (what they read, kernel3.cuh:136-139), not the
    per-expert counts the reference passes there (src/moe_ops.cu:181-183)."""
    gemm_type = GemmType(int(gemm_type))
    if gemm_type != GemmType.MGroupedContiguous:
        raise NotImplementedError("naive_moe_forward_dispatch: the dispatch delivers the contiguous "
                                  "layout; MGroupedMasked is not built for it")
    ctx = all2all.ctx
    if (ctx.E, ctx.k, ctx.H) != (int(num_experts), int(experts_per_token), int(hidden_dim)):
        raise ValueError("num_experts / experts_per_token / hidden_dim do not match the All2All")
    all2all.dispatch(None, expert_x, expert_x_scales, input, input_scales, indices, weights)
    fp8_grouped_gemm_swiglu(expert_x, expert_x_scales, gate, gate_scales, up, up_scales, inter_y,
                            inter_y_scales, gemm_type, all2all.grouped_layout)
    fp8_grouped_gemm_nt(inter_y, inter_y_scales, down, down_scales, expert_y, gemm_type,
                        all2all.grouped_layout)
    all2all.combine(out_tokens, indices, weights, expert_y)
