"""moeb_route_plan_static: the routing plan for hosts that cannot allocate.

Some users of the library (a server whose memory pool owns the whole GPU, a
host that forbids allocation calls while serving) cannot pass a workspace, so
this entry point keeps its scratch in a fixed device array inside the library.
The test calls it through the C ABI twice in a row, with different inputs, and
requires exactly the outputs of the regular entry point moeb_route_plan
(integer work: equality, no tolerance). The second call also shows that stale
scratch contents of the first call do no harm. The file name makes pytest
collect it last.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _plan_buffers(T, k, E, m_cap):
    i32 = dict(dtype=torch.int32, device=DEV)
    # poison the outputs so that every word must be written by the call
    return [torch.full((n,), -7, **i32) for n in (E, E + 1, max(T * k, 1), m_cap, m_cap, m_cap)]


def _run(lib, name, idx_dev, T, k, E, m_cap, workspace=None):
    from parallel_playground_b200 import cabi
    bufs = _plan_buffers(T, k, E, m_cap)
    stream = torch.cuda.current_stream().cuda_stream
    args = [idx_dev.data_ptr(), T, k, E, 128, m_cap] + [b.data_ptr() for b in bufs]
    if workspace is not None:
        args += [workspace.data_ptr(), workspace.numel()]
    cabi.call(name, *args, stream)
    torch.cuda.synchronize()
    return [b.cpu().numpy() for b in bufs]


def _indices(T, E, k, seed):
    g = torch.Generator().manual_seed(seed)
    if T == 0:
        return torch.zeros((1, k), dtype=torch.int32)[:0]
    return torch.rand(T, E, generator=g).argsort(1)[:, :k].int().contiguous()


def test_static_route_plan_matches_workspace_version_twice(lib):
    torch.cuda.set_device(0)
    # first a large problem (fills much of the scratch), then a small one with
    # other shapes: left-over scratch contents must not leak into the result
    # ... then exactly at the limit of the built-in scratch (ceil(T*k/256)*E ==
    # 131072 entries) and a call without tokens
    assert (8192 * 8 // 256) * 512 == lib.moeb_route_plan_static_max_ints()
    for T, E, k, seed in [(8192, 32, 8, 5), (300, 64, 6, 6), (8192, 512, 8, 7), (0, 256, 8, 8)]:
        idx = _indices(T, E, k, seed).to(DEV)
        m_cap = lib.moeb_route_plan_rows(T, k, E, 128)
        ws = torch.empty(lib.moeb_route_plan_workspace_bytes(T, k, E), dtype=torch.uint8, device=DEV)
        want = _run(lib, "moeb_route_plan", idx, T, k, E, m_cap, ws)
        got = _run(lib, "moeb_route_plan_static", idx, T, k, E, m_cap)
        names = ["expert_counts", "padded_offsets", "dst_row", "src_token", "src_slot",
                 "grouped_layout"]
        for n, a, b in zip(names, want, got):
            assert np.array_equal(a, b), f"{n} differs for T={T} E={E} k={k}"
        assert want[0].sum() == T * k


def test_static_route_plan_rejects_oversized_problems(lib):
    limit = lib.moeb_route_plan_static_max_ints()
    assert limit == 128 * 1024
    T, k, E = 65536, 8, 1024            # ceil(T*k/256) * E = 2048 * 1024 > limit
    assert (T * k // 256) * E > limit
    buf = torch.zeros(16, dtype=torch.int32, device=DEV)
    p = buf.data_ptr()
    m_cap = lib.moeb_route_plan_rows(T, k, E, 128)
    rc = lib.moeb_route_plan_static(p, T, k, E, 128, m_cap, p, p, p, p, p, p, None)
    assert rc == 7
    assert b"exceeds the built-in scratch" in lib.moeb_last_error()
    assert isinstance(ctypes.c_int(rc).value, int)
