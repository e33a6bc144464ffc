"""Expert-parallel layer on real GPUs (one process per GPU, NCCL process group).

The 2- and 4-rank cases run only where that many CUDA devices are visible.
Every rank runs the EP layer over the staged transport (router -> fused
quantise+pack -> NCCL all-to-all dispatch -> grouped GEMMs -> all-to-all
combine) and checks its own tokens against the CPU oracle: a token's result
depends only on its quantised row and on the weights of the experts it is
routed to, not on how experts are spread over ranks, so the one-rank oracle
with all experts is the reference for every rank. The peer-memory transport
(push and pull combine, the fused-op entry points, ranks without tokens, a
receive capacity that is too small) must then give the same bits.
"""
import os
import socket
import sys
import traceback
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

REPO = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    try:
        sys.path.insert(0, str(REPO))
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                          WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
        import dataclasses
        import torch.distributed as dist
        import oracle
        from parallel_playground_b200 import moe_cuda as mc
        from parallel_playground_b200 import workloads as wl
        from parallel_playground_b200.ep import All2AllStaged as All2All, All2AllP2P, \
            ep_moe_forward, ep_moe_forward_p2p

        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        shape = dataclasses.replace(wl.CONFIGS["qwen3"], T=160, H=512, I=256, E=16, k=4)
        inp = wl.make_layer_inputs(shape, rank=rank, world=world)
        full = wl.make_layer_inputs(shape, rank=0, world=1)      # all experts, for the oracle
        d = inp.to(dev)
        a2a = All2All(shape.T, shape.E, shape.k, 128, shape.H, in_dtype=torch.float8_e4m3fn,
                      out_dtype=torch.bfloat16, device=rank)
        assert a2a.world_size == world and a2a.rank == rank
        out = torch.empty((shape.T, shape.H), dtype=torch.bfloat16, device=dev)
        for _ in range(2):   # twice: buffers and plans are reused across calls
            idx, wts = ep_moe_forward(a2a, d.x, d.w_router, None, d.gate, d.gate_scale, d.up,
                                      d.up_scale, d.down, d.down_scale, out, shape)
        torch.cuda.synchronize()
        mc.check_device_status()
        qv = lambda t: t.view(torch.uint8).numpy()  # noqa: E731
        ref = oracle.moe_layer_ref(inp.x, inp.w_router, qv(full.gate), full.gate_scale.numpy(),
                                   qv(full.up), full.up_scale.numpy(), qv(full.down),
                                   full.down_scale.numpy(), shape.k,
                                   indices=idx.cpu().numpy(), weights=wts.cpu().numpy())
        err = (out.float().cpu() - torch.from_numpy(ref.out_f32)).abs()
        max_rel = float(err.max() / np.abs(ref.out_f32).max())
        mean_abs = float(err.mean())
        assert max_rel <= 2e-2 and mean_abs <= 1e-3, (max_rel, mean_abs)
        # per-expert received counts are exact (test_all2all.cpp:621-641)
        counts_all = [torch.zeros(shape.E, dtype=torch.int32, device=dev) for _ in range(world)]
        mine = torch.bincount(idx.flatten().long(), minlength=shape.E).int()
        dist.all_gather(counts_all, mine)
        e_local = shape.E // world
        want = torch.stack(counts_all).sum(0)[rank * e_local:(rank + 1) * e_local]
        assert torch.equal(a2a._tokens_per_expert, want)
        # the peer-memory transport gives the same bits as the staged one: the rows
        # land in the same canonical order and the reduction order is the same
        p2p = All2AllP2P(shape.T, shape.E, shape.k, shape.H, device=rank)
        out2 = torch.empty_like(out)
        work = {}
        for _ in range(3):   # repeated calls reuse the peer buffers
            idx2, wts2 = ep_moe_forward_p2p(p2p, d.x, d.w_router, None, d.gate, d.gate_scale, d.up,
                                            d.up_scale, d.down, d.down_scale, out2, shape, work)
        torch.cuda.synchronize()
        mc.check_device_status()
        assert int(p2p.overflow.item()) == 0
        assert torch.equal(idx2, idx) and torch.equal(wts2, wts)
        assert torch.equal(p2p.tokens_per_expert, want)
        assert torch.equal(out2.view(torch.int16), out.view(torch.int16)), \
            float((out2.float() - out.float()).abs().max())
        # pull-style combine (peer loads) instead of the push-style GEMM epilogue
        out3 = torch.full_like(out, 7.0)
        ep_moe_forward_p2p(p2p, d.x, d.w_router, None, d.gate, d.gate_scale, d.up, d.up_scale,
                           d.down, d.down_scale, out3, shape, work, push_combine=False)
        torch.cuda.synchronize()
        assert torch.equal(out3.view(torch.int16), out.view(torch.int16))
        # the other dispatch form (once per destination rank + owner-side fan-out, or one
        # store per expert copy): same bytes in the experts' buffers, same result
        other = All2AllP2P(shape.T, shape.E, shape.k, shape.H, device=rank,
                           once_per_rank=not p2p.once_per_rank)
        out6 = torch.full_like(out, 6.0)
        for _ in range(2):
            ep_moe_forward_p2p(other, d.x, d.w_router, None, d.gate, d.gate_scale, d.up, d.up_scale,
                               d.down, d.down_scale, out6, shape, {})
        torch.cuda.synchronize()
        mc.check_device_status()
        assert torch.equal(other.tokens_per_expert, want)
        assert torch.equal(out6.view(torch.int16), out.view(torch.int16))
        live = p2p.grouped_layout >= 0
        assert torch.equal(other.grouped_layout, p2p.grouped_layout)
        assert torch.equal(other.expert_x.view(torch.uint8)[live], p2p.expert_x.view(torch.uint8)[live])
        # the two fused-op entry points of the operator module, over the same context
        out4 = torch.full_like(out, 3.0)
        rows_dev = mc.fused_dispatch_grouped_gemm_swiglu(p2p, d.x, idx2, d.gate, d.up, work["inter"],
                                                         d.gate_scale, d.up_scale, work["inter_s"])
        mc.fused_grouped_gemm_combine(p2p, out4, work["inter"], work["inter_s"], d.down,
                                      d.down_scale, wts2)
        torch.cuda.synchronize()
        mc.check_device_status()
        assert int(rows_dev.item()) % 128 == 0 and int(rows_dev.item()) >= int(want.sum())
        assert torch.equal(out4.view(torch.int16), out.view(torch.int16))
        # ragged ranks: odd ranks bring no tokens at all (empty send plan, experts that
        # receive nothing from them); the even ranks' results do not change
        n_tok = 0 if rank % 2 == 1 else shape.T
        out5 = torch.full((n_tok, shape.H), 5.0, dtype=torch.bfloat16, device=dev)
        ep_moe_forward_p2p(p2p, d.x[:n_tok], d.w_router, None, d.gate, d.gate_scale, d.up,
                           d.up_scale, d.down, d.down_scale, out5, shape, {})
        torch.cuda.synchronize()
        mc.check_device_status()
        assert int(p2p.overflow.item()) == 0
        if n_tok:
            assert torch.equal(out5.view(torch.int16), out.view(torch.int16))
        # a capacity that is too small is reported, not written out of bounds
        small = All2AllP2P(shape.T, shape.E, shape.k, shape.H, capacity_rows=256, device=rank)
        ep_moe_forward_p2p(small, d.x, d.w_router, None, d.gate, d.gate_scale, d.up, d.up_scale,
                           d.down, d.down_scale, out2, shape, {})
        torch.cuda.synchronize()
        total = torch.tensor([int(small.overflow.item())], device=dev)
        dist.all_reduce(total)
        assert int(total.item()) > 0
        # dropped copies stay out of the sum in both combine forms: push == pull bits
        # (the home buffer is poisoned first, so a stale row would show)
        small.home.fill_(1000.0)
        out7, out8 = torch.full_like(out, 1.0), torch.full_like(out, 2.0)
        ep_moe_forward_p2p(small, d.x, d.w_router, None, d.gate, d.gate_scale, d.up, d.up_scale,
                           d.down, d.down_scale, out7, shape, {})
        ep_moe_forward_p2p(small, d.x, d.w_router, None, d.gate, d.gate_scale, d.up, d.up_scale,
                           d.down, d.down_scale, out8, shape, {}, push_combine=False)
        torch.cuda.synchronize()
        assert torch.equal(out7.view(torch.int16), out8.view(torch.int16))
        assert float(out7.float().abs().max()) < 100.0
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception:  # noqa: BLE001
        q.put((rank, "FAILED\n" + traceback.format_exc()))


@pytest.mark.parametrize("world", [1, 2, 4])
def test_ep_layer_matches_oracle(world):
    """world = 1 runs the same code (peer buffers, rank barrier, scatter epilogue)
    with this rank as its own and only peer, so a one-GPU box covers it too."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=600) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    assert all(v == "ok" for v in results.values()), results
