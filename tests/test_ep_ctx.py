"""The expert-parallel context of the C ABI (moeb_ep_*) on real GPUs.

One process per GPU; the 2- and 4-rank cases run only where that many devices
are visible, the 1-rank case runs the same kernels with the rank as its own and
only peer. Every rank drives the context through the C ABI alone and checks:
  * the whole-layer call, fused (rows fetched by comm CTAs inside the gate/up
    GEMM) and unfused (rows fetched by a kernel of their own): bit-identical to
    each other and to the staged transport (NCCL all-to-all-v), and within the
    layer tolerances of the CPU oracle;
  * exact per-expert counts (test/test_cpp/test_all2all.cpp:621-641) and the
    same expert-sorted bytes as the staged transport;
  * the split-phase halves of dispatch and combine (do_send / do_recv,
    csrc/all2all/all2all_tk.hpp:292-334, 376-394) with the caller's own GEMMs;
  * pre-quantised tokens as the reference's dispatch takes them;
  * ranks that bring no tokens; a receive capacity that is too small;
  * a bounded wait that runs out is reported, not hung (a tag nobody writes).
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
        from parallel_playground_b200.ep import All2AllStaged, EPContext, ep_moe_forward

        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        shape = dataclasses.replace(wl.CONFIGS["qwen3"], T=160, H=512, I=256, E=16, k=4)
        inp = wl.make_layer_inputs(shape, rank=rank, world=world)
        full = wl.make_layer_inputs(shape, rank=0, world=1)      # all experts, for the oracle
        d = inp.to(dev)
        T, H, I, k = shape.T, shape.H, shape.I, shape.k
        bits = lambda t: t.view(torch.int16)  # noqa: E731

        # reference bits: the staged transport (pack -> NCCL all-to-all-v -> unpack)
        staged = All2AllStaged(T, shape.E, k, 128, H, in_dtype=torch.float8_e4m3fn,
                               out_dtype=torch.bfloat16, device=rank)
        out_ref = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
        idx, wts = ep_moe_forward(staged, d.x, d.w_router, None, d.gate, d.gate_scale, d.up,
                                  d.up_scale, d.down, d.down_scale, out_ref, shape)
        torch.cuda.synchronize()

        ctx = EPContext(T, shape.E, k, H, device=rank)
        assert ctx.world_size == world and ctx.rank == rank
        layer = lambda out, fused, x=d.x: ctx.moe_forward(  # noqa: E731
            x, d.w_router, None, d.gate, d.gate_scale, d.up, d.up_scale, d.down, d.down_scale, out,
            shape, fused=fused)
        # the other way to run the two expert GEMMs of the whole-layer call: in row chunks
        # (the down projection of a chunk beside the gate/up GEMM of the next). Same bits.
        assert ctx.mlp_mode == "seq"
        for mode, extra in (("chunks", {}), ("chunks", {"MOEB_EP_MLP_CHUNKS": "3"}),
                            ("chunks", {"MOEB_EP_MLP_CHUNKS": "8", "MOEB_EP_DOWN_SMS": "30"})):
            os.environ.update(MOEB_EP_MLP=mode, **extra)
            other_mlp = EPContext(T, shape.E, k, H, device=rank)
            for key in ("MOEB_EP_MLP", *extra):
                os.environ.pop(key)
            assert other_mlp.mlp_mode == mode
            for _ in range(2):
                out = torch.full((T, H), 8.0, dtype=torch.bfloat16, device=dev)
                other_mlp.moe_forward(d.x, d.w_router, None, d.gate, d.gate_scale, d.up,
                                      d.up_scale, d.down, d.down_scale, out, shape, fused=False)
                torch.cuda.synchronize()
                mc.check_device_status()
                assert torch.equal(bits(out), bits(out_ref)), (mode, extra)
            other_mlp.close()
        pull_ctx = EPContext(T, shape.E, k, H, device=rank, transport="pull")
        for fused in (False, True, True, False, "pull", True, "pull"):   # buffers alternate by step
            out = torch.full((T, H), 9.0, dtype=torch.bfloat16, device=dev)
            if fused == "pull":     # rows fetched by the pull kernel, not fused
                pull_ctx.moe_forward(d.x, d.w_router, None, d.gate, d.gate_scale, d.up, d.up_scale,
                                     d.down, d.down_scale, out, shape, fused=False)
                assert torch.equal(pull_ctx.tokens_per_expert, staged._tokens_per_expert)
            else:                   # False: push transport; True: pull inside the GEMM
                layer(out, fused)
            torch.cuda.synchronize()
            mc.check_device_status()
            assert int(ctx.overflow.item()) == 0
            assert torch.equal(bits(out), bits(out_ref)), \
                (fused, float((out.float() - out_ref.float()).abs().max()))
        # counts, layout and expert-sorted bytes as the staged transport has them
        assert torch.equal(ctx.tokens_per_expert, staged._tokens_per_expert)
        rows = int(ctx.m_valid.item())
        assert rows % 128 == 0 and rows >= int(ctx.tokens_per_expert.sum())
        assert torch.equal(ctx.grouped_layout[:rows], staged.grouped_layout[:rows])
        assert torch.equal(ctx.source_rank[:rows], staged.source_rank[:rows])
        # oracle: a token's result does not depend on how experts are spread over ranks
        qv = lambda t: t.view(torch.uint8).numpy()  # noqa: E731
        ref = oracle.moe_layer_ref(inp.x, inp.w_router, qv(full.gate), full.gate_scale.numpy(),
                                   qv(full.up), full.up_scale.numpy(), qv(full.down),
                                   full.down_scale.numpy(), k, indices=idx.cpu().numpy(),
                                   weights=wts.cpu().numpy())
        err = (out.float().cpu() - torch.from_numpy(ref.out_f32)).abs()
        assert float(err.max() / np.abs(ref.out_f32).max()) <= 2e-2 and float(err.mean()) <= 1e-3

        # split-phase halves around the caller's own GEMMs, pre-quantised tokens in,
        # rows delivered into the caller's tensors
        xq = torch.empty((T, H), dtype=torch.float8_e4m3fn, device=dev)
        xs = torch.empty((H // 128, T), dtype=torch.float32, device=dev)
        mc.cast(d.x, xq, xs)
        M = ctx.max_recv_tokens
        ex = torch.zeros((M, H), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
        es = torch.zeros((H // 128, M), dtype=torch.float32, device=dev)
        ctx.dispatch(indices=idx, x_q=xq, x_scale_mn=xs, out_expert_x=ex, out_expert_x_scale=es,
                     do_recv=False)
        ctx.dispatch(do_send=False, do_recv=True)
        live = ctx.grouped_layout[:rows] >= 0
        torch.cuda.synchronize()
        assert torch.equal(ex.view(torch.uint8)[:rows][live], ctx.expert_x.view(torch.uint8)[:rows][live])
        inter = torch.empty((M, I), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
        inter_s = torch.empty((I // 128, M), dtype=torch.float32, device=dev)
        ey = torch.empty((M, H), dtype=torch.bfloat16, device=dev)
        mc.fp8_grouped_gemm_swiglu(ex, es, d.gate, d.gate_scale, d.up, d.up_scale, inter, inter_s,
                                   mc.GemmType.MGroupedContiguous, ctx.grouped_layout)
        mc.fp8_grouped_gemm_nt(inter, inter_s, d.down, d.down_scale, ey,
                               mc.GemmType.MGroupedContiguous, ctx.grouped_layout)
        out2 = torch.full_like(out, 4.0)
        ctx.combine(out2, wts, expert_y=ey, do_recv=False)
        ctx.combine(out2, wts, do_send=False)
        torch.cuda.synchronize()
        mc.check_device_status()
        assert torch.equal(bits(out2), bits(out_ref))
        # accumulate adds to what is there
        out3 = out_ref.clone()
        ctx.dispatch(x=d.x, indices=idx)
        ctx.combine(out3, wts, expert_y=ey, accumulate=True)
        torch.cuda.synchronize()
        assert torch.allclose(out3.float(), 2 * out_ref.float(), atol=2e-2, rtol=2e-2)

        # the two fused ops by themselves
        out4 = torch.full_like(out, 3.0)
        ctx.fused_dispatch_swiglu(d.x, idx, d.gate, d.gate_scale, d.up, d.up_scale, inter, inter_s)
        ctx.fused_gemm_combine(inter, inter_s, d.down, d.down_scale, wts, out4)
        torch.cuda.synchronize()
        mc.check_device_status()
        assert torch.equal(bits(out4), bits(out_ref))

        # the reference's module-level entry points: naive_moe_forward_dispatch with its
        # 21 positional arguments on the caller's buffers ...
        a2a = mc.All2All(T, shape.E, k, 128, H, in_dtype=torch.float8_e4m3fn,
                         out_dtype=torch.bfloat16, device=rank)
        out7 = torch.full_like(out, 7.0)
        mc.naive_moe_forward_dispatch(a2a, shape.E, k, H, mc.GemmType.MGroupedContiguous, xq, xs,
                                      d.gate, d.gate_scale, d.up, d.up_scale, d.down, d.down_scale,
                                      idx, wts, out7, ex, es, inter, inter_s, ey)
        torch.cuda.synchronize()
        mc.check_device_status()
        assert torch.equal(bits(out7), bits(out_ref))
        # ... and the 31- / 21-argument forms of the two fused ops
        tk = lambda shp, dt: mc.TKParallelTensor(shape=shp, dtype=dt, local_rank=rank,  # noqa: E731
                                                 local_world_size=world, multicast=False)
        with pytest.raises(ValueError):
            mc.TKParallelTensor((4,), torch.int32, rank, world, True)
        in_tokens, in_scales = tk((T, H), torch.float8_e4m3fn), tk([H // 128, T], torch.float32)
        in_tokens.data().view(torch.uint8).copy_(xq.view(torch.uint8))
        in_scales.data().copy_(xs)
        gnr, e2t, e2s = tk((1, shape.E), torch.int32), tk((shape.E, T), torch.int32), \
            tk((shape.E, T), torch.int32)
        barrier, out_t = tk((2 * world,), torch.int32), tk((T, H), torch.bfloat16)
        i32 = dict(dtype=torch.int32, device=dev)
        pec, nrt = torch.zeros(shape.E // world, **i32), torch.zeros(1, **i32)
        sti, sdi, ssi = (torch.full((M,), -5, **i32) for _ in range(3))
        inter.view(torch.uint8).zero_()
        mc.fused_dispatch_grouped_gemm_swiglu(
            in_tokens, in_scales, ex, es, d.gate, d.up, inter, d.gate_scale, d.up_scale, inter_s, idx,
            gnr, e2t, e2s, pec, sti, sdi, ssi, barrier, T, nrt, 0, rank, 1, 0, world, world, shape.E,
            k, 16, 116)
        mc.fused_grouped_gemm_combine(
            out_t, inter, inter_s, d.down, d.down_scale, ey, wts, pec, sti, sdi, ssi, shape.E, k, nrt,
            0, rank, 1, 0, world, 16, 116)
        torch.cuda.synchronize()
        mc.check_device_status()
        assert torch.equal(bits(out_t.data()), bits(out_ref))
        assert int(nrt.item()) == int(ctx.tokens_per_expert.sum())
        assert int(pec.sum()) == rows and bool((pec % 128 == 0).all())
        lv = ctx.grouped_layout[:rows] >= 0
        assert torch.equal(sdi[:rows][lv], ctx.source_rank[:rows][lv])
        assert torch.equal(sti[:rows][lv] * k + ssi[:rows][lv], ctx.source_pos[:rows][lv])

        # ragged ranks: odd ranks bring no tokens; the even ranks' results do not change
        n_tok = 0 if rank % 2 == 1 else T
        out5 = torch.full((n_tok, H), 5.0, dtype=torch.bfloat16, device=dev)
        for fused in (True, False):
            layer(out5, fused, d.x[:n_tok])
            torch.cuda.synchronize()
            mc.check_device_status()
            if n_tok:
                assert torch.equal(bits(out5), bits(out_ref))

        # timing of the stages inside the library
        ctx.set_timing(True)
        for _ in range(3):
            layer(out, True)
        tm = ctx.read_timing()
        assert tm["steps"] == 3 and tm["swiglu"] > 0 and tm["down"] > 0
        ctx.set_timing(False)

        # a capacity that is too small: copies are counted and dropped, nothing is
        # written out of bounds and no stale row enters a result
        small = EPContext(T, shape.E, k, H, capacity_rows=256, device=rank)
        small.home.fill_(1000.0)
        out6 = torch.full_like(out, 1.0)
        small.moe_forward(d.x, d.w_router, None, d.gate, d.gate_scale, d.up, d.up_scale, d.down,
                          d.down_scale, out6, shape, fused=True)
        torch.cuda.synchronize()
        total = torch.tensor([int(small.overflow.item())], device=dev)
        dist.all_reduce(total)
        assert int(total.item()) > 0
        assert float(out6.float().abs().max()) < 100.0
        dropped = (small.dst_row[:T] < 0).any(1)
        kept = ~dropped
        assert torch.equal(bits(out6)[kept], bits(out_ref)[kept])
        small.close()

        # one expert per rank (the Mixtral-shaped configuration at EP=8 has this form):
        # wide experts, top-2, skewed load from a router bias; all forms against the staged one
        sh1 = dataclasses.replace(wl.CONFIGS["mixtral"], T=192, H=512, I=1024, E=world,
                                  k=min(2, world))
        in1 = wl.make_layer_inputs(sh1, rank=rank, world=world)
        d1 = in1.to(dev)
        b1 = None if in1.router_bias is None else in1.router_bias.to(dev)
        st1 = All2AllStaged(sh1.T, sh1.E, sh1.k, 128, sh1.H, in_dtype=torch.float8_e4m3fn,
                            out_dtype=torch.bfloat16, device=rank)
        ref1 = torch.empty((sh1.T, sh1.H), dtype=torch.bfloat16, device=dev)
        ep_moe_forward(st1, d1.x, d1.w_router, b1, d1.gate, d1.gate_scale, d1.up, d1.up_scale,
                       d1.down, d1.down_scale, ref1, sh1)
        torch.cuda.synchronize()
        one = EPContext(sh1.T, sh1.E, sh1.k, sh1.H, device=rank)
        for fused in (False, True, False):
            o1 = torch.full_like(ref1, 2.0)
            one.moe_forward(d1.x, d1.w_router, b1, d1.gate, d1.gate_scale, d1.up, d1.up_scale,
                            d1.down, d1.down_scale, o1, sh1, fused=fused)
            torch.cuda.synchronize()
            mc.check_device_status()
            assert int(one.overflow.item()) == 0
            assert torch.equal(bits(o1), bits(ref1)), ("one expert per rank", fused)
        assert torch.equal(one.tokens_per_expert, st1._tokens_per_expert)
        one.close()
        dist.barrier()
        pull_ctx.close()
        ctx.close()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception:  # noqa: BLE001
        q.put((rank, "FAILED\n" + traceback.format_exc()))


@pytest.mark.parametrize("world", [1, 2, 4])
def test_ep_context_matches_staged_transport_and_oracle(world):
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
    for r, v in sorted(results.items()):
        if v != "ok":
            print(f"--- rank {r}\n{v}")
    assert all(v == "ok" for v in results.values()), sorted(results)


def test_ep_context_without_process_group_and_bounded_wait():
    """One GPU, no torch.distributed: the rank is its own peer. The receive half
    without a send half is refused; a row whose word never gets this step's tag
    makes the pull give up with a device-timeout status instead of hanging."""
    sys.path.insert(0, str(REPO))
    from parallel_playground_b200 import cabi
    from parallel_playground_b200 import moe_cuda as mc
    from parallel_playground_b200.ep import EPContext
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    T, E, k, H = 64, 8, 2, 256
    # the push transport first: same bytes in the same rows
    g0 = torch.Generator().manual_seed(3)
    x0 = torch.randn(T, H, generator=g0).bfloat16().to(dev)
    idx0 = torch.rand(T, E, generator=g0).argsort(1)[:, :k].int().contiguous().to(dev)
    push = EPContext(T, E, k, H, device=0, transport="push")
    push.dispatch(x=x0, indices=idx0)
    torch.cuda.synchronize()
    mc.check_device_status()
    xq0 = torch.empty((T, H), dtype=torch.float8_e4m3fn, device=dev)
    xs0 = torch.empty((T, H // 128), dtype=torch.float32, device=dev)
    mc.cast(x0, xq0, xs0)
    rows0 = push.dst_row[:T].flatten().long()
    assert torch.equal(push.expert_x.view(torch.uint8)[rows0], xq0.view(torch.uint8).repeat_interleave(k, 0))
    assert torch.equal(push.scale_mn.t()[rows0], xs0.repeat_interleave(k, 0))
    assert torch.equal(push.source_pos[rows0], torch.arange(T * k, dtype=torch.int32, device=dev))
    with pytest.raises(cabi.MoebError):       # pre-quantised tokens need the pull transport
        push.dispatch(indices=idx0, x_q=xq0, x_scale_mn=xs0.t().contiguous())
    push.close()
    ctx = EPContext(T, E, k, H, device=0, transport="pull")
    assert ctx.world_size == 1 and ctx.max_recv_tokens % 128 == 0
    with pytest.raises(cabi.MoebError):
        ctx.dispatch(do_send=False, do_recv=True)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(T, H, generator=g).bfloat16().to(dev)
    idx = torch.rand(T, E, generator=g).argsort(1)[:, :k].int().contiguous().to(dev)
    ctx.dispatch(x=x, indices=idx)
    torch.cuda.synchronize()
    mc.check_device_status()
    # every dispatched row carries the bytes of its token
    xq = torch.empty((T, H), dtype=torch.float8_e4m3fn, device=dev)
    xs = torch.empty((T, H // 128), dtype=torch.float32, device=dev)
    mc.cast(x, xq, xs)
    rows = ctx.dst_row[:T].flatten().long()
    assert torch.equal(ctx.expert_x.view(torch.uint8)[rows], xq.view(torch.uint8).repeat_interleave(k, 0))
    assert torch.equal(ctx.scale_mn.t()[rows], xs.repeat_interleave(k, 0))
    assert torch.equal(ctx.source_pos[rows], torch.arange(T * k, dtype=torch.int32, device=dev))
    # send half only, then spoil one row's word: the receive half must give up on it
    ctx.dispatch(x=x, indices=idx, do_recv=False)
    torch.cuda.synchronize()
    pos_words = ctx.sym.view(torch.int64)
    view = cabi.EpView()
    import ctypes
    # the per-row words live in the symmetric buffer right before the home rows
    n_words = ctx.max_recv_tokens
    home_off = (ctx.home.data_ptr() - ctx.sym.data_ptr()) // 8
    words = pos_words[home_off - ((n_words * 8 + 255) // 256 * 256) // 8:][:n_words]
    row = int(rows[0])
    words[row] = 0
    status = mc.status_word(dev)
    status.zero_()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    ctx.dispatch(do_send=False, do_recv=True)
    t1.record()
    torch.cuda.synchronize()
    assert status[8].item() == cabi.STATUS_DEVICE_TIMEOUT and status[9].item() == 7
    assert status[10].item() == row
    assert t0.elapsed_time(t1) < 10_000     # bounded: about two seconds, then the kernel returns
    status.zero_()
    # the context stays usable
    ctx.dispatch(x=x, indices=idx)
    torch.cuda.synchronize()
    mc.check_device_status()
    ctx.close()
    del view, ctypes
