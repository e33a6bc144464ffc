"""Seeded synthetic inputs for the five benchmark configurations.

The configurations name well-known models only for their layer SHAPES; no
weights or data of those models are involved. Everything is drawn from
torch's seeded generators, on the CPU so that a CPU checker and a GPU run see
identical bits, and moved to the device by the caller.

Weight pre-quantisation (128x128 blocks, fp32 scales) is offline preparation,
not part of the timed path; it is done with torch tensor ops.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

ROUTER_SOFTMAX = 0
ROUTER_SIGMOID_GROUPED = 1


@dataclass
class LayerShape:
    name: str
    T: int            # tokens per rank
    H: int            # hidden size
    I: int            # intermediate size per expert
    E: int            # experts (global)
    k: int            # experts per token
    router_mode: int = ROUTER_SOFTMAX
    n_group: int = 1
    topk_group: int = 1
    renorm: bool = True
    route_scale: float = 1.0
    zipf_bias: float = 0.0   # > 0: per-expert logit bias log(Zipf(s) pmf)
    seed: int = 0
    extra: dict = field(default_factory=dict)


# BASELINE.json `configs`, in order.
CONFIGS = {
    "tiny": LayerShape("tiny", T=256, H=1024, I=512, E=8, k=2, seed=0),
    "gemm32": LayerShape("gemm32", T=8192, H=4096, I=1536, E=32, k=8, seed=1),
    "mixtral": LayerShape("mixtral", T=16384, H=4096, I=14336, E=8, k=2, zipf_bias=1.1, seed=2),
    "qwen3": LayerShape("qwen3", T=8192, H=2048, I=768, E=128, k=8, seed=3),
    "dsv3_prefill": LayerShape("dsv3_prefill", T=4096, H=7168, I=2048, E=256, k=8,
                               router_mode=ROUTER_SIGMOID_GROUPED, n_group=8, topk_group=4,
                               route_scale=2.5, seed=4),
    "dsv3_decode": LayerShape("dsv3_decode", T=128, H=7168, I=2048, E=256, k=8,
                              router_mode=ROUTER_SIGMOID_GROUPED, n_group=8, topk_group=4,
                              route_scale=2.5, seed=4),
    # one-GPU stand-in for the work of ONE rank of the DeepSeek-V3-shaped layer at EP=8:
    # its 32 experts and as many routed rows (4096 tokens x top-8) as a rank receives
    "dsv3_rank": LayerShape("dsv3_rank", T=4096, H=7168, I=2048, E=32, k=8,
                            router_mode=ROUTER_SIGMOID_GROUPED, n_group=8, topk_group=4,
                            route_scale=2.5, seed=4),
}


def quantize_weights_128x128(w: torch.Tensor):
    """w [G,N,K] (any float dtype) -> (e4m3 [G,N,K], fp32 scales [G,N/128,K/128]).
    scale = amax/448 per 128x128 block (1 for an all-zero block), q = e4m3(clamp(w/scale))
    — python/common.py:212-233 with the zero guard of test/test_cpp/test_utils.h:243-244."""
    G, N, K = w.shape
    assert N % 128 == 0 and K % 128 == 0
    blocks = w.float().view(G, N // 128, 128, K // 128, 128)
    amax = blocks.abs().amax(dim=(2, 4))
    scale = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    q = (blocks / scale[:, :, None, :, None]).clamp(-448.0, 448.0)
    return q.reshape(G, N, K).to(torch.float8_e4m3fn), scale.contiguous()


def zipf_log_bias(E: int, s: float) -> torch.Tensor:
    """log of the Zipf(s) pmf over expert rank 1..E (expert 0 most popular)."""
    r = torch.arange(1, E + 1, dtype=torch.float64)
    pmf = r.pow(-s)
    pmf = pmf / pmf.sum()
    return pmf.log().float()


@dataclass
class LayerInputs:
    shape: LayerShape
    x: torch.Tensor            # [T,H] bf16
    w_router: torch.Tensor     # [H,E] bf16
    router_bias: torch.Tensor | None
    gate: torch.Tensor         # [E_local,I,H] e4m3
    gate_scale: torch.Tensor
    up: torch.Tensor
    up_scale: torch.Tensor
    down: torch.Tensor         # [E_local,H,I] e4m3
    down_scale: torch.Tensor

    def to(self, device) -> "LayerInputs":
        mv = lambda t: None if t is None else t.to(device)  # noqa: E731
        return LayerInputs(self.shape, mv(self.x), mv(self.w_router), mv(self.router_bias),
                           mv(self.gate), mv(self.gate_scale), mv(self.up), mv(self.up_scale),
                           mv(self.down), mv(self.down_scale))


def make_layer_inputs(shape: LayerShape, rank: int = 0, world: int = 1, T: int | None = None,
                      weights_device: str = "cpu") -> LayerInputs:
    """Inputs of one rank. Tokens are seeded per rank (seed*world + rank); the
    router weights are identical on every rank; expert weights are seeded per
    GLOBAL expert id so that any EP split sees the same experts. `weights_device`
    lets large expert weights be generated directly on the GPU."""
    T = shape.T if T is None else T
    E_local = shape.E // world
    g = torch.Generator().manual_seed(shape.seed * world + rank)
    x = torch.randn(T, shape.H, generator=g).bfloat16()
    gr = torch.Generator().manual_seed(1000 + shape.seed)
    w_router = (torch.randn(shape.H, shape.E, generator=gr) * 0.02).bfloat16()
    bias = zipf_log_bias(shape.E, shape.zipf_bias) if shape.zipf_bias > 0 else None

    def expert_weights(tag: int, n: int, k: int):
        qs, ss = [], []
        for e in range(rank * E_local, (rank + 1) * E_local):
            q, s = _one_expert_matrix(shape, tag, e, n, k, weights_device)
            qs.append(q)
            ss.append(s)
        return torch.cat(qs), torch.cat(ss)

    gate, gate_s = expert_weights(1, shape.I, shape.H)
    up, up_s = expert_weights(2, shape.I, shape.H)
    down, down_s = expert_weights(3, shape.H, shape.I)
    return LayerInputs(shape, x, w_router, bias, gate, gate_s, up, up_s, down, down_s)


def _one_expert_matrix(shape: LayerShape, tag: int, e: int, n: int, k: int, weights_device: str):
    """One weight matrix [1,n,k] of GLOBAL expert e, N(0, 0.02), quantised. The
    seed depends on the expert id only, so every EP split sees the same expert;
    the random stream depends on the device kind (CPU and CUDA generators differ)."""
    ge = torch.Generator(device=weights_device).manual_seed((shape.seed * 7919 + tag) * 100003 + e)
    w = torch.randn(1, n, k, generator=ge, device=weights_device) * 0.02
    return quantize_weights_128x128(w.bfloat16())


def make_expert_weights(shape: LayerShape, e: int, weights_device: str = "cpu") -> dict:
    """The three quantised matrices of global expert e, bit-identical to what
    make_layer_inputs(..., weights_device=same kind of device) gives its owner."""
    gate, gate_s = _one_expert_matrix(shape, 1, e, shape.I, shape.H, weights_device)
    up, up_s = _one_expert_matrix(shape, 2, e, shape.I, shape.H, weights_device)
    down, down_s = _one_expert_matrix(shape, 3, e, shape.H, shape.I, weights_device)
    return {"gate": gate, "gate_scale": gate_s, "up": up, "up_scale": up_s, "down": down,
            "down_scale": down_s}


def dirichlet_multinomial_indices(T: int, E: int, k: int, seed: int, alpha: float = 1.0):
    """Routing of the grouped-GEMM-only configuration: p ~ Dirichlet(alpha * 1_E),
    every token draws k distinct experts by multinomial(p). Returns int32 [T,k]
    and uniform weights 1/k."""
    g = torch.Generator().manual_seed(seed)
    gam = torch.distributions.Gamma(torch.full((E,), alpha), torch.ones(E))
    torch.manual_seed(seed)
    p = gam.sample()
    p = p / p.sum()
    idx = torch.multinomial(p.expand(T, E), k, replacement=False, generator=g).int()
    w = torch.full((T, k), 1.0 / k, dtype=torch.float32)
    return idx, w


def layer_flops(shape: LayerShape, routed_rows: int) -> float:
    """Algorithmic FLOPs of the grouped GEMMs: 6 * M * H * I (gate, up, down)."""
    return 6.0 * routed_rows * shape.H * shape.I


def dispatch_row_bytes(H: int) -> int:
    """Bytes of one dispatched row: H e4m3 + H/128 fp32 scales, 16-byte aligned."""
    return (H + 4 * (H // 128) + 15) // 16 * 16
