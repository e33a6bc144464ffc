"""Pins oracle.router_select against a second, independent statement of the two
routers, written with torch's own softmax / sigmoid / topk from the workload
descriptions (softmax -> top-k -> renormalise; sigmoid -> 8 groups -> group
score = sum of the group's two best -> top-4 groups -> top-8 experts among
them -> renormalise -> x 2.5), not from the oracle's or the kernel's code.

The oracle and the CUDA kernel share one exp polynomial and one summation
order, so comparing those two with each other cannot catch a wrong reading of
the routing rule. This file can: logits are tie-free random fp32 values, the
selected experts must be identical and the weights must agree to 1e-6
relative (the torch statement sums in another order and uses libm's exp).
Ties are defined by the oracle alone (lower expert id first) and are checked
separately for that rule.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.timeout(300)


def _tie_free_logits(T, E, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(T, E, generator=g, dtype=torch.float32) * scale).contiguous()


def torch_softmax_topk(logits: torch.Tensor, k: int, renorm: bool):
    p = torch.softmax(logits.double(), dim=-1)
    w, idx = torch.topk(p, k, dim=-1)          # descending by probability
    if renorm:
        w = w / w.sum(-1, keepdim=True)
    return idx.int().numpy(), w.float().numpy()


def torch_grouped_sigmoid_topk(logits: torch.Tensor, k: int, n_group: int, topk_group: int,
                               renorm: bool, route_scale: float):
    T, E = logits.shape
    s = torch.sigmoid(logits.double())
    grouped = s.view(T, n_group, E // n_group)
    group_score = grouped.topk(2, dim=-1).values.sum(-1)              # two best of each group
    keep = group_score.topk(topk_group, dim=-1).indices                # best groups
    mask = torch.zeros(T, n_group, dtype=torch.bool)
    mask.scatter_(1, keep, True)
    masked = s.masked_fill(~mask.unsqueeze(-1).expand(T, n_group, E // n_group).reshape(T, E),
                           float("-inf"))
    idx = masked.topk(k, dim=-1).indices
    w = s.gather(1, idx)
    if renorm:
        w = w / w.sum(-1, keepdim=True)
    w = w * route_scale
    return idx.int().numpy(), w.float().numpy()


@pytest.mark.parametrize("T,E,k,renorm", [(256, 8, 2, True), (512, 128, 8, True),
                                          (300, 64, 6, False), (64, 1024, 12, True)])
def test_softmax_router_matches_torch(oracle_mod, T, E, k, renorm):
    logits = _tie_free_logits(T, E, seed=E + k, scale=2.0)
    idx, w = oracle_mod.router_select(logits.numpy(), k, oracle_mod.ROUTER_SOFTMAX, 1, 1, renorm,
                                      1.0)
    ref_idx, ref_w = torch_softmax_topk(logits, k, renorm)
    assert np.array_equal(idx, ref_idx)
    np.testing.assert_allclose(w, ref_w, rtol=1e-6, atol=0)
    if renorm:
        np.testing.assert_allclose(w.sum(-1), 1.0, rtol=1e-6)


@pytest.mark.parametrize("T,E,k,n_group,topk_group,scale", [
    (512, 256, 8, 8, 4, 2.5),      # the DeepSeek-V3-shaped configuration
    (200, 64, 6, 4, 2, 1.0),
    (128, 256, 8, 1, 1, 2.5),      # no group limit: plain sigmoid top-k
])
def test_grouped_sigmoid_router_matches_torch(oracle_mod, T, E, k, n_group, topk_group, scale):
    logits = _tie_free_logits(T, E, seed=3 * E + k)
    idx, w = oracle_mod.router_select(logits.numpy(), k, oracle_mod.ROUTER_SIGMOID_GROUPED,
                                      n_group, topk_group, True, scale)
    ref_idx, ref_w = torch_grouped_sigmoid_topk(logits, k, n_group, topk_group, True, scale)
    assert np.array_equal(idx, ref_idx)
    np.testing.assert_allclose(w, ref_w, rtol=1e-6, atol=0)
    np.testing.assert_allclose(w.sum(-1), scale, rtol=1e-6)
    # every selected expert lies in one of at most topk_group groups
    groups = idx // (E // n_group)
    assert max(len(set(row)) for row in groups.tolist()) <= max(topk_group, 1) or n_group == 1


def test_ties_go_to_the_lower_expert_id(oracle_mod):
    """Oracle-defined part: equal scores are ordered by expert id."""
    logits = np.zeros((3, 16), dtype=np.float32)
    logits[1, 5] = 1.0
    logits[2, [9, 3]] = 2.0
    idx, w = oracle_mod.router_select(logits, 4, oracle_mod.ROUTER_SOFTMAX, 1, 1, True, 1.0)
    assert idx[0].tolist() == [0, 1, 2, 3]
    assert idx[1].tolist() == [5, 0, 1, 2]
    assert idx[2].tolist() == [3, 9, 0, 1]
    np.testing.assert_allclose(w.sum(-1), 1.0, rtol=1e-6)


def test_workload_router_settings_are_the_configured_ones():
    """The benchmark shapes carry the routing rule of their configuration."""
    from parallel_playground_b200 import workloads as wl
    from parallel_playground_b200 import cabi
    d = wl.CONFIGS["dsv3_prefill"]
    assert (d.E, d.k, d.n_group, d.topk_group, d.route_scale) == (256, 8, 8, 4, 2.5)
    assert d.router_mode == cabi.ROUTER_SIGMOID_GROUPED and d.renorm
    for name in ("tiny", "mixtral", "qwen3"):
        c = wl.CONFIGS[name]
        assert c.router_mode == cabi.ROUTER_SOFTMAX and c.renorm
