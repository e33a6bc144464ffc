"""Expert-parallel dispatch / combine: one process per GPU, experts split in
contiguous blocks (owner(e) = e // (E/W), a2a_dispatch_send_tk.cuh:251).

Three transports, same rows in the same canonical order, bit-identical results:

`EPContext` / `All2All` — the expert-parallel context of the C ABI (moeb_ep_*):
tokens are quantised once into symmetric memory, every expert copy is announced
to its owner with one word, the owners load the rows over NVLink (inside the
gate/up GEMM in the fused form), results go home inside the down GEMM. One
library call per op, no host round trip. `All2All` is the reference's class
interface on top of it.

`All2AllStaged` — three exchanges per layer (the reference moves the same data
with peer loads/stores into symmetric buffers plus a host round trip for the
counts, csrc/all2all/all2all_tk.hpp:201-394):
  1. counts   — all-gather of the int32[E] per-expert send counts,
  2. dispatch — all-to-all-v of packed rows (H e4m3 bytes + H/128 fp32 scales),
                ordered by (destination rank, expert, token, slot),
  3. combine  — the inverse all-to-all-v of bf16 rows.
torch.distributed (NCCL on GPUs, gloo in the CPU tests) carries the bytes; the
packing, un-packing, planning and reduction are this library's CUDA kernels.
At W == 1 nothing is exchanged.

`All2AllP2P` — peer memory: this library's kernels store the quantised rows
straight into the owners' buffers over NVLink, the down GEMM's epilogue stores
the results home, and the ranks meet in a barrier kernel over flag words in
peer memory. No collective library call and no host read on the path.

The host-side helpers (`split_sizes`, `exchange_counts`, `exchange_rows`) work
on tensors of any device so that the exchange logic is testable with gloo.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import cabi
from .workloads import dispatch_row_bytes


# ------------------------------------------------------- host-side exchange --
def split_sizes(counts_all: torch.Tensor, rank: int, world: int):
    """Rows this rank sends to / receives from every peer.

    counts_all: int32 [W, E] (host), counts_all[s, e] = rows rank s routes to
    expert e. Returns (send_splits[W], recv_splits[W]) as Python lists."""
    W, E = counts_all.shape
    assert W == world and E % world == 0
    e_local = E // world
    per_dest = counts_all.view(W, world, e_local).sum(-1)       # [src, dst]
    send = per_dest[rank].tolist()
    recv = per_dest[:, rank].tolist()
    return [int(v) for v in send], [int(v) for v in recv]


def exchange_counts(send_counts: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather the per-expert send counts: int32 [E] -> int32 [W, E]."""
    world = dist.get_world_size(group)
    n = send_counts.numel()
    out = torch.empty(world * n, dtype=send_counts.dtype, device=send_counts.device)
    dist.all_gather_into_tensor(out, send_counts.contiguous().view(-1), group=group)
    return out.view(world, n)


def exchange_rows(send_buf: torch.Tensor, send_splits, recv_splits, group=None) -> torch.Tensor:
    """All-to-all-v of whole rows: send_buf [n_send, row] -> [n_recv, row]."""
    n_recv = int(sum(recv_splits))
    dtype = send_buf.dtype
    raw = send_buf.contiguous().view(torch.uint8)   # rows travel as bytes on every backend
    recv = torch.empty((n_recv,) + tuple(raw.shape[1:]), dtype=torch.uint8, device=raw.device)
    dist.all_to_all_single(recv, raw, output_split_sizes=list(recv_splits),
                           input_split_sizes=list(send_splits), group=group)
    return recv.view(dtype)


# ------------------------------------------------------------ All2AllStaged --
class All2AllStaged:
    """The reference's `moe_cuda.All2All` interface (csrc/python_api.cpp:85-166,
    477-514) over the STAGED transport: pack -> NCCL all-to-all-v -> unpack, with
    one host read of the counts. Kept as the second, independent transport that
    the peer-memory forms are compared with bit for bit (`All2All` below is the
    class the operator module exports). Same constructor keywords, `dispatch` /
    `combine` signatures and properties. Ranks come from
    torch.distributed (`group`, default world) instead of TKParallelTensor
    brokers; `max_private_tokens` is accepted and unused (no private/overflow
    split is needed); dp_group_size must be 1 (the reference's dp>1 path is
    untested, README.md:49).

    One op in flight per handle, like the reference (shared sync counter,
    all2all_tk.hpp:31-32)."""

    def __init__(self, max_num_tokens, num_experts, experts_per_token, expert_padding, hidden_dim,
                 hidden_dim_scale=None, in_dtype=torch.float8_e4m3fn, out_dtype=torch.bfloat16,
                 scale_dtype=None, max_private_tokens=None, dp_group_size=None,
                 node_group_size=None, ep_group_size=None, device=-1, stream=None, group=None):
        from . import moe_cuda as mc
        self._mc = mc
        self.group = group
        if dist.is_available() and dist.is_initialized():
            self._rank = dist.get_rank(group)
            self._world = dist.get_world_size(group)
        else:
            self._rank, self._world = 0, 1
        if node_group_size is not None and int(node_group_size) != self._world:
            raise ValueError("node_group_size must equal the process group size")
        if dp_group_size not in (None, 1):
            raise ValueError("dp_group_size must divide world size; only 1 is supported")
        if ep_group_size is not None and (ep_group_size == 0 or self._world % ep_group_size != 0):
            raise ValueError("ep_group_size must divide world size")
        if num_experts % self._world != 0:
            raise ValueError("num_experts must be a multiple of the world size")
        if out_dtype != torch.bfloat16:
            raise ValueError("combine only supports bfloat16")  # a2a_context_tk.hpp:181-182
        if hidden_dim % 128 != 0:
            raise ValueError("hidden_dim must be a multiple of 128")
        self._device = torch.device("cuda", torch.cuda.current_device() if device in (-1, None)
                                    else int(device))
        self.max_num_tokens = int(max_num_tokens)
        self.E = int(num_experts)
        self.k = int(experts_per_token)
        self.pad = int(expert_padding)
        self.H = int(hidden_dim)
        self.e_local = self.E // self._world
        self.row_bytes = dispatch_row_bytes(self.H)
        # worst case: every token of every rank routes all k slots to this rank
        self._max_recv = self.max_num_tokens * self.k * self._world
        self._m_cap = cabi.load().moeb_route_plan_rows(self.max_num_tokens * self._world, self.k,
                                                       self.e_local, self.pad)
        dev = self._device
        i32 = dict(dtype=torch.int32, device=dev)
        self._send_plan = mc.RoutePlan(self.max_num_tokens, self.k, self.E, 1, dev)
        self._send_buf = torch.empty((self.max_num_tokens * self.k, self.row_bytes),
                                     dtype=torch.uint8, device=dev)
        self._tokens_per_expert = torch.empty(self.e_local, **i32)
        self._padded_offsets = torch.empty(self.e_local + 1, **i32)
        self._recv_to_row = None
        self.grouped_layout = torch.empty(self._m_cap, **i32)
        self.source_rank = torch.empty(self._m_cap, **i32)
        self._send_splits = None
        self._recv_splits = None
        self._n_tokens = 0

    # properties of PyAll2All (python_api.cpp:156-160)
    @property
    def rank(self):
        return self._rank

    @property
    def world_size(self):
        return self._world

    @property
    def device(self):
        return self._device.index

    @property
    def max_recv_tokens(self):
        return self._m_cap

    @property
    def handle(self):
        return self

    @property
    def padded_offsets(self):
        return self._padded_offsets

    def _stream(self):
        return torch.cuda.current_stream().cuda_stream

    def _plan_and_exchange_counts(self, indices):
        T = indices.shape[0]
        if T > self.max_num_tokens:
            raise RuntimeError("num_tokens exceeds max_num_tokens")  # a2a_context_tk.hpp:150-152
        if indices.dtype != torch.int32 or indices.shape[1] != self.k:
            raise ValueError("indices must be int32 [T, experts_per_token]")
        plan = self._send_plan
        plan.T = T
        plan.run(indices)
        if self._world > 1:
            counts_all = exchange_counts(plan.expert_counts, self.group)
        else:
            counts_all = plan.expert_counts.view(1, -1)
        # the one host round trip of the op (the reference has the same one,
        # all2all_tk.hpp:309-320): the split sizes of the all-to-all-v
        host = counts_all.cpu()
        self._send_splits, self._recv_splits = split_sizes(host, self._rank, self._world)
        self._counts_all = counts_all
        self._n_tokens = T
        first = self._rank * self.e_local
        per_expert = host[:, first:first + self.e_local].sum(0)
        self._m_padded = int(((per_expert + self.pad - 1) // self.pad * self.pad).sum())
        return plan

    def _recv_plan(self, n_recv):
        self._recv_to_row = torch.empty(max(n_recv, 1), dtype=torch.int32, device=self._device)
        cabi.call("moeb_recv_plan", self._counts_all.data_ptr(), self._world, self.E,
                  self._rank * self.e_local, self.e_local, self.pad, n_recv, self._m_cap,
                  self._tokens_per_expert.data_ptr(), self._padded_offsets.data_ptr(),
                  self._recv_to_row.data_ptr(), self.grouped_layout.data_ptr(),
                  self.source_rank.data_ptr(), self._stream())

    def _finish_dispatch(self, T, out_expert_num_tokens, out_expert_x, out_expert_x_scale):
        n_send = T * self.k
        send = self._send_buf[:n_send]
        if self._world > 1:
            recv = exchange_rows(send, self._send_splits, self._recv_splits, self.group)
        else:
            recv = send
        n_recv = recv.shape[0]
        self._n_recv = n_recv
        self._recv_plan(n_recv)
        m_cap = out_expert_x.shape[0] if out_expert_x.dim() == 2 else \
            out_expert_x.shape[0] * out_expert_x.shape[1]
        if m_cap < self._m_padded or out_expert_x_scale.shape[-1] != m_cap:
            raise ValueError(f"out_expert_x needs >= {self._m_padded} rows (max_recv_tokens is "
                             "always enough) and a [H/128, rows] scale")
        cabi.call("moeb_dispatch_unpack", recv.data_ptr(), self._recv_to_row.data_ptr(), n_recv,
                  self.H, self.row_bytes, m_cap, out_expert_x.data_ptr(),
                  out_expert_x_scale.data_ptr(), self._stream())
        if out_expert_num_tokens is not None:
            out_expert_num_tokens.view(torch.int32).copy_(self._tokens_per_expert)

    def dispatch(self, out_expert_num_tokens, out_expert_x, out_expert_x_scale=None, dp_x=None,
                 dp_x_scale=None, indices=None, weights=None, bound_m=None, do_send=True,
                 do_recv=True):
        """python_api.cpp:134-143. dp_x: e4m3 [T,H]; dp_x_scale: fp32 [H/128,T]
        (MN-major); outputs: out_expert_x e4m3 [max_recv_tokens,H],
        out_expert_x_scale fp32 [H/128,max_recv_tokens], out_expert_num_tokens
        uint32/int32 [E_local] = unpadded rows per local expert. Both halves
        (do_send / do_recv) run in this call; asking for only one is rejected."""
        if not (do_send and do_recv):
            raise NotImplementedError("split-phase dispatch (do_send/do_recv) is not supported")
        if dp_x_scale is None or out_expert_x_scale is None:
            raise ValueError("dp_x_scale and out_expert_x_scale are required")  # all2all_tk.hpp:298,327
        T = dp_x.shape[0]
        plan = self._plan_and_exchange_counts(indices)
        cabi.call("moeb_dispatch_pack_q", dp_x.data_ptr(), dp_x_scale.data_ptr(),
                  plan.dst_row.data_ptr(), T, self.k, self.H, self._send_buf.data_ptr(),
                  self.row_bytes, self._stream())
        self._finish_dispatch(T, out_expert_num_tokens, out_expert_x, out_expert_x_scale)

    def dispatch_bf16(self, x, indices, out_expert_x=None, out_expert_x_scale=None,
                      out_expert_num_tokens=None):
        """Fused form: bf16 tokens are quantised (1x128) while they are packed
        for the exchange, so every token row is read once. Without output
        tensors it allocates them with exactly the padded number of received
        rows (known on the host after the count exchange) and returns
        (expert_x e4m3 [M,H], expert_x_scale fp32 [H/128,M])."""
        T = x.shape[0]
        plan = self._plan_and_exchange_counts(indices)
        if out_expert_x is None:
            M = max(self._m_padded, self.pad)
            out_expert_x = torch.empty((M, self.H), dtype=torch.uint8,
                                       device=self._device).view(torch.float8_e4m3fn)
            out_expert_x_scale = torch.empty((self.H // 128, M), dtype=torch.float32,
                                             device=self._device)
        cabi.call("moeb_dispatch_pack", x.data_ptr(), plan.dst_row.data_ptr(), T, self.k, self.H,
                  self._send_buf.data_ptr(), self.row_bytes, self._stream())
        self._finish_dispatch(T, out_expert_num_tokens, out_expert_x, out_expert_x_scale)
        return out_expert_x, out_expert_x_scale

    def combine(self, out_tokens, indices, weights, expert_y, bound_m=None, do_send=True,
                do_recv=True, accumulate=False):
        """python_api.cpp:145-150: return every expert-output row to its source
        rank and reduce out[t] = sum_j weights[t,j] * y[t,j] (bf16 in/out). Uses
        the routing of the preceding dispatch, like the reference."""
        if not (do_send and do_recv):
            raise NotImplementedError("split-phase combine (do_send/do_recv) is not supported")
        if self._recv_to_row is None:
            raise RuntimeError("combine needs a preceding dispatch")
        T = self._n_tokens
        n_recv = self._n_recv
        back = torch.empty((n_recv, self.H), dtype=torch.bfloat16, device=self._device)
        cabi.call("moeb_gather_rows_bf16", expert_y.data_ptr(), self._recv_to_row.data_ptr(),
                  n_recv, self.H, back.data_ptr(), self._stream())
        if self._world > 1:
            mine = exchange_rows(back, self._recv_splits, self._send_splits, self.group)
        else:
            mine = back
        self._mc.unpermute_combine(mine, self._send_plan.dst_row[:T], weights, out_tokens,
                                   accumulate)


# ------------------------------------------------------------- EP MoE layer --
def ep_moe_forward(a2a: "All2AllStaged", x, w_router, router_bias, gate, gate_scale, up, up_scale, down,
                   down_scale, out, shape, events=None):
    """Whole layer on W ranks: router -> fused quantise+pack -> dispatch ->
    gate/up SwiGLU GEMM -> down GEMM -> combine (src/moe_ops.cu:153-191 with the
    router in front). Weights hold this rank's E/W experts. Work buffers are
    sized by the rows actually received and come from torch's caching allocator."""
    mc = a2a._mc
    dev = x.device
    T, H = x.shape
    I = gate.shape[1]
    k, E = shape.k, shape.E
    logits = torch.empty((T, E), dtype=torch.float32, device=dev)
    idx = torch.empty((T, k), dtype=torch.int32, device=dev)
    wts = torch.empty((T, k), dtype=torch.float32, device=dev)
    mc.router_logits(x, w_router, logits, router_bias)
    mc.router_select(logits, idx, wts, shape.router_mode, shape.n_group, shape.topk_group,
                     shape.renorm, shape.route_scale)
    ex, es = a2a.dispatch_bf16(x, idx)
    M = ex.shape[0]
    inter = torch.empty((M, I), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    inter_s = torch.empty((I // 128, M), dtype=torch.float32, device=dev)
    ey = torch.empty((M, H), dtype=torch.bfloat16, device=dev)
    if events is not None:
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
    mc.fp8_grouped_gemm_swiglu(ex, es, gate, gate_scale, up, up_scale, inter, inter_s,
                               mc.GemmType.MGroupedContiguous, a2a.grouped_layout)
    if events is not None:
        e1.record()
    mc.fp8_grouped_gemm_nt(inter, inter_s, down, down_scale, ey, mc.GemmType.MGroupedContiguous,
                           a2a.grouped_layout)
    if events is not None:
        e2.record()
        events["swiglu"].append((e0, e1))
        events["down"].append((e1, e2))
    a2a.combine(out, idx, wts, ey)
    return idx, wts


def build_ep_step(mc, shape, d, bias_d, dev, rank, world):
    """Benchmark step for N > 1 ranks (used by bench.py)."""
    T, H, I, E, k = shape.T, shape.H, shape.I, shape.E, shape.k
    a2a = All2AllStaged(T, E, k, 128, H, in_dtype=torch.float8_e4m3fn, out_dtype=torch.bfloat16,
                        device=dev.index)
    out = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
    events = {"swiglu": [], "down": []}

    def step(timed: bool):
        ep_moe_forward(a2a, d.x, d.w_router, bias_d, d.gate, d.gate_scale, d.up, d.up_scale,
                       d.down, d.down_scale, out, shape, events if timed else None)

    def routed_rows():
        return int(a2a._tokens_per_expert.sum().item())

    # logits, select, plan x3, pack, recv_plan, unpack, 2 GEMMs, gather, combine (+ NCCL's own)
    def e2e_fn(x_dev, out_dev):
        ep_moe_forward(a2a, x_dev, d.w_router, bias_d, d.gate, d.gate_scale, d.up, d.up_scale,
                       d.down, d.down_scale, out_dev, shape, None)

    layer = {"kernels_per_step": 12, "out": out, "routed_rows": routed_rows, "e2e_fn": e2e_fn}
    return step, events, layer


# ------------------------------------------------------- peer-memory (P2P) EP --
class All2AllP2P:
    """Expert-parallel dispatch / combine over peer memory: every rank stores its
    quantised token rows straight into the owners' expert-sorted buffers and
    later gets the expert outputs back (stored home by the owners' down GEMM, or
    pulled), through NVLink loads/stores issued by this library's kernels
    (`moeb_ep_dispatch_p2p`, `moeb_fp8_grouped_gemm_nt_scatter`,
    `moeb_ep_combine_pull`). No host round trip: the per-expert counts travel
    with the rank barrier and are turned into destination rows by a kernel.

    Buffers come from torch's symmetric memory (CUDA VMM handles exchanged over
    the process group), the same kind of allocation the reference gets from
    ThunderKittens' TKParallelTensor (csrc/all2all/a2a_context_tk.hpp:66-71).
    Ranks exchange their counts and are fenced twice per layer (after the
    dispatch stores, after the down GEMM) by a one-CTA barrier kernel over flag
    words in peer memory, whose wait is bounded (2 s, then an error status). The
    data kernels themselves never wait on a peer, and after set-up no NCCL
    collective is on the path.

    `capacity_rows` bounds the rows a rank can receive (default: the worst case
    T*k*W plus padding; the reference bounds it the same way,
    csrc/all2all/all2all_tk.hpp:101-106). Copies that do not fit are counted in
    `overflow` and dropped, never written out of bounds."""

    def __init__(self, max_num_tokens, num_experts, experts_per_token, hidden_dim,
                 expert_padding=128, capacity_rows=None, device=None, group=None,
                 once_per_rank=None):
        import torch.distributed._symmetric_memory as symm_mem
        from . import moe_cuda as mc
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("All2AllP2P needs an initialised torch.distributed process group")
        self._mc = mc
        self.group = group if group is not None else dist.group.WORLD
        self._rank = dist.get_rank(self.group)
        self._world = dist.get_world_size(self.group)
        if num_experts % self._world != 0 or hidden_dim % 128 != 0:
            raise ValueError("num_experts % world == 0 and hidden_dim % 128 == 0 are required")
        self._device = torch.device("cuda", torch.cuda.current_device() if device is None
                                    else int(device))
        dev = self._device
        self.T, self.E, self.k, self.H = int(max_num_tokens), int(num_experts), \
            int(experts_per_token), int(hidden_dim)
        self.pad = int(expert_padding)
        self.e_local = self.E // self._world
        worst = cabi.load().moeb_route_plan_rows(self.T * self._world, self.k, self.e_local,
                                                 self.pad)
        self.m_cap = worst if capacity_rows is None else \
            (int(capacity_rows) + self.pad - 1) // self.pad * self.pad
        n_kb = self.H // 128
        # symmetric (peer-mapped) buffers: activations, scale staging, expert outputs
        self.sym_x = symm_mem.empty(self.m_cap * self.H, dtype=torch.uint8, device=dev)
        self.sym_scale = symm_mem.empty(self.m_cap * n_kb, dtype=torch.float32, device=dev)
        self.sym_y = symm_mem.empty(self.m_cap * self.H, dtype=torch.bfloat16, device=dev)
        # where each received row came from (t*k+slot at its source), and the buffer
        # that receives this rank's own tokens' expert outputs, one row per (t, slot)
        self.sym_pos = symm_mem.empty(self.m_cap, dtype=torch.int32, device=dev)
        self.sym_home = symm_mem.empty(self.T * self.k * self.H, dtype=torch.bfloat16, device=dev)
        # rank barrier flags [channels, W] and the per-expert counts of every rank [W, E]
        self.sym_flags = symm_mem.empty(self.N_CHANNELS * self._world, dtype=torch.int32,
                                        device=dev)
        self.sym_counts = symm_mem.empty(self._world * self.E, dtype=torch.int32, device=dev)
        self.sym_flags.zero_()
        self.sym_counts.zero_()
        # once-per-rank dispatch: a token crosses NVLink once per destination rank
        # (into that rank's stash, one row per (source rank, token)) instead of once
        # per expert copy; the owner fans it out locally. Pays off when a token has
        # several experts on the same rank (k > W or so); default: on for W > 1.
        self.once_per_rank = (self._world > 1) if once_per_rank is None else bool(once_per_rank)
        stash_rows = self._world * self.T if self.once_per_rank else 1
        self.sym_stash_x = symm_mem.empty(stash_rows * self.H, dtype=torch.uint8, device=dev)
        self.sym_stash_scale = symm_mem.empty(stash_rows * n_kb, dtype=torch.float32, device=dev)
        handles = [symm_mem.rendezvous(t, self.group)
                   for t in (self.sym_x, self.sym_scale, self.sym_y, self.sym_pos, self.sym_home,
                             self.sym_flags, self.sym_counts, self.sym_stash_x,
                             self.sym_stash_scale)]
        self._handles = handles  # keep the mappings alive
        mk = lambda h: torch.tensor([int(p) for p in h.buffer_ptrs], dtype=torch.int64,  # noqa: E731
                                    device=dev)
        self.peer_x, self.peer_scale, self.peer_y, self.peer_pos, self.peer_home, \
            self.peer_flags, self.peer_counts, self.peer_stash_x, self.peer_stash_scale = \
            (mk(h) for h in handles)
        self._epoch = [0] * self.N_CHANNELS
        self.home = self.sym_home.view(self.T * self.k, self.H)
        self.home_rows = torch.arange(self.T * self.k, dtype=torch.int32,
                                      device=dev).view(self.T, self.k)
        self.expert_x = self.sym_x.view(self.m_cap, self.H).view(torch.float8_e4m3fn)
        self.expert_y = self.sym_y.view(self.m_cap, self.H)
        self.scale_mn = torch.empty((n_kb, self.m_cap), dtype=torch.float32, device=dev)
        i32 = dict(dtype=torch.int32, device=dev)
        self._send_plan = mc.RoutePlan(self.T, self.k, self.E, 1, dev)
        self.counts_all = self.sym_counts.view(self._world, self.E)
        self.dest_base = torch.empty(self.E, **i32)
        self.m_valid = torch.zeros(1, **i32)
        self.dst_rank = torch.empty((self.T, self.k), **i32)
        self.dst_row = torch.empty((self.T, self.k), **i32)
        self.overflow = torch.zeros(1, **i32)
        # set to a list to collect (start, end) CUDA events around the dispatch kernel alone
        self.kernel_events = None
        self.tokens_per_expert = torch.empty(self.e_local, **i32)
        self.padded_offsets = torch.empty(self.e_local + 1, **i32)
        self.grouped_layout = torch.empty(self.m_cap, **i32)
        self.source_rank = torch.empty(self.m_cap, **i32)
        self._dummy = torch.empty(1, **i32)
        self._minus_one = torch.full((1, 1), -1, **i32)
        self._n_tokens = 0
        # nobody touches a peer buffer (the flags included) before every rank has
        # mapped and zeroed them: one NCCL barrier at set-up, none afterwards
        torch.cuda.synchronize(dev)
        dist.barrier(group=self.group)

    N_CHANNELS = 2   # flag channels: 0 = count exchange, 1 = fences

    rank = property(lambda self: self._rank)
    world_size = property(lambda self: self._world)
    max_recv_tokens = property(lambda self: self.m_cap)

    def _stream(self):
        return torch.cuda.current_stream().cuda_stream

    def _barrier(self, channel, counts=None):
        self._epoch[channel] = (self._epoch[channel] + 1) & 0xFFFFFFFF
        status = self._mc.status_word(self._device)
        cabi.call("moeb_ep_barrier", self.peer_flags.data_ptr(),
                  self.peer_counts.data_ptr() if counts is not None else 0,
                  counts.data_ptr() if counts is not None else 0, self.E if counts is not None else 0,
                  self._rank, self._world, channel, self._epoch[channel], status[8:].data_ptr(),
                  self._stream())

    def fence(self):
        """All ranks' earlier kernels on this stream are complete before any
        rank's later ones start (stream-ordered, no host wait): a bounded-wait
        barrier kernel over flag words in peer memory."""
        self._barrier(1)

    def dispatch_bf16(self, x, indices):
        """Quantise + permute + send. Afterwards `expert_x` / `scale_mn` /
        `grouped_layout` / `m_valid` describe this rank's received rows."""
        T = x.shape[0]
        if T > self.T:
            raise RuntimeError("num_tokens exceeds max_num_tokens")
        plan = self._send_plan
        plan.T = T
        plan.run(indices)                                   # counts + order inside each expert
        # every rank's counts into every rank's counts_all (peer stores + rank barrier)
        self._barrier(0, plan.expert_counts)
        st = self._stream()
        cabi.call("moeb_ep_dest_base", self.counts_all.data_ptr(), self._world, self.E, self._rank,
                  self.pad, self.dest_base.data_ptr(), self.m_valid.data_ptr(), st)
        # the count exchange above also orders this step's stores after every peer's
        # previous combine (they had to reach their own count exchange first)
        timed = self.kernel_events is not None
        if timed:
            k0, k1 = (torch.cuda.Event(enable_timing=True) for _ in range(2))
            k0.record()
        if self.once_per_rank:
            cabi.call("moeb_ep_dispatch_once", x.data_ptr(), indices.data_ptr(),
                      plan.dst_row.data_ptr(), plan.padded_offsets.data_ptr(),
                      self.dest_base.data_ptr(), T, self.T, self.k, self.H, self.E, self._world,
                      self._rank, self.m_cap, self.peer_stash_x.data_ptr(),
                      self.peer_stash_scale.data_ptr(), self.peer_pos.data_ptr(),
                      self.dst_rank.data_ptr(), self.dst_row.data_ptr(), self.overflow.data_ptr(), st)
        else:
            cabi.call("moeb_ep_dispatch_p2p", x.data_ptr(), indices.data_ptr(),
                      plan.dst_row.data_ptr(), plan.padded_offsets.data_ptr(),
                      self.dest_base.data_ptr(), T, self.k, self.H, self.E, self._world, self.m_cap,
                      self.peer_x.data_ptr(), self.peer_scale.data_ptr(), self.peer_pos.data_ptr(),
                      self.dst_rank.data_ptr(), self.dst_row.data_ptr(), self.overflow.data_ptr(), st)
        if timed:
            k1.record()
            self.kernel_events.append((k0, k1))
        self.fence()                                        # every rank's rows have landed
        cabi.call("moeb_recv_plan", self.counts_all.data_ptr(), self._world, self.E,
                  self._rank * self.e_local, self.e_local, self.pad, 0, self.m_cap,
                  self.tokens_per_expert.data_ptr(), self.padded_offsets.data_ptr(),
                  self._dummy.data_ptr(), self.grouped_layout.data_ptr(),
                  self.source_rank.data_ptr(), st)
        if self.once_per_rank:                              # fan the stash rows out to the experts
            cabi.call("moeb_ep_unstash", self.sym_stash_x.data_ptr(),
                      self.sym_stash_scale.data_ptr(), self.source_rank.data_ptr(),
                      self.sym_pos.data_ptr(), self.m_valid.data_ptr(), self.m_cap, self.k, self.T,
                      self.H, self.sym_x.data_ptr(), self.sym_scale.data_ptr(), st)
        cabi.call("moeb_ep_scale_transpose", self.sym_scale.data_ptr(), self.m_valid.data_ptr(),
                  self.m_cap, self.H // 128, self.scale_mn.data_ptr(), st)
        self._n_tokens = T

    def combine_home(self, out_tokens, weights, accumulate=False):
        """Second half of the push-style combine: the owners' down GEMM has stored
        every expert output row into this rank's `home` buffer at row t*k+slot
        (moeb_fp8_grouped_gemm_nt_scatter); reduce them locally."""
        self.fence()                                        # every rank's rows have come home
        T = self._n_tokens
        # copies the dispatch dropped (capacity overflow, expert id out of range)
        # never came home: their home rows hold stale data and stay out of the sum
        rows = torch.where(self.dst_row[:T] >= 0, self.home_rows[:T], self._minus_one)
        self._mc.unpermute_combine(self.home, rows, weights, out_tokens, accumulate)

    def combine(self, out_tokens, weights, accumulate=False):
        """Pull this rank's tokens' expert outputs from `expert_y` of their owners
        and reduce them with `weights` (bf16 out)."""
        self.fence()                                        # every rank's expert_y is complete
        T = self._n_tokens
        cabi.call("moeb_ep_combine_pull", self.peer_y.data_ptr(), self.dst_rank.data_ptr(),
                  self.dst_row.data_ptr(), weights.data_ptr(), T, self.k, self.H,
                  out_tokens.data_ptr(), int(bool(accumulate)), self._stream())


def ep_moe_forward_p2p(a2a: All2AllP2P, x, w_router, router_bias, gate, gate_scale, up, up_scale,
                       down, down_scale, out, shape, work=None, events=None, push_combine=True):
    """Whole EP layer over peer memory: router -> plan -> count exchange ->
    fused quantise + peer-store dispatch -> gate/up SwiGLU GEMM -> down GEMM ->
    combine. No host synchronisation anywhere. `work` caches the per-call scratch
    tensors. push_combine=True: the down GEMM's epilogue stores each output row
    straight into its source rank's home buffer (transport overlapped with the
    GEMM), followed by a local weighted reduce; False: the GEMM writes locally and
    every token pulls its k rows from the owners afterwards."""
    mc = a2a._mc
    dev = x.device
    T, H = x.shape
    I = gate.shape[1]
    k, E = shape.k, shape.E
    M = a2a.m_cap
    if work is None:
        work = {}
    if "logits" not in work:
        work["logits"] = torch.empty((T, E), dtype=torch.float32, device=dev)
        work["idx"] = torch.empty((T, k), dtype=torch.int32, device=dev)
        work["wts"] = torch.empty((T, k), dtype=torch.float32, device=dev)
        work["inter"] = torch.empty((M, I), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
        work["inter_s"] = torch.empty((I // 128, M), dtype=torch.float32, device=dev)
    logits, idx, wts = work["logits"], work["idx"], work["wts"]
    mc.router_logits(x, w_router, logits, router_bias)
    mc.router_select(logits, idx, wts, shape.router_mode, shape.n_group, shape.topk_group,
                     shape.renorm, shape.route_scale)
    if events is not None:
        d0, d1 = (torch.cuda.Event(enable_timing=True) for _ in range(2))
        d0.record()
    a2a.dispatch_bf16(x, idx)
    st = torch.cuda.current_stream().cuda_stream
    status = mc.status_word(dev)
    if events is not None:
        d1.record()
        events.setdefault("dispatch", []).append((d0, d1))
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
    G = gate.shape[0]
    cabi.call("moeb_fp8_grouped_gemm_swiglu_dyn", a2a.expert_x.data_ptr(), a2a.scale_mn.data_ptr(),
              gate.data_ptr(), gate_scale.data_ptr(), up.data_ptr(), up_scale.data_ptr(),
              work["inter"].data_ptr(), work["inter_s"].data_ptr(), M, a2a.m_valid.data_ptr(), I,
              H, G, cabi.GEMM_M_GROUPED_CONTIGUOUS, a2a.grouped_layout.data_ptr(), 0,
              status.data_ptr(), st)
    if events is not None:
        e1.record()
    if push_combine:
        # down GEMM whose epilogue stores every row into its source rank's home buffer
        cabi.call("moeb_fp8_grouped_gemm_nt_scatter", work["inter"].data_ptr(),
                  work["inter_s"].data_ptr(), down.data_ptr(), down_scale.data_ptr(),
                  a2a.peer_home.data_ptr(), a2a.source_rank.data_ptr(), a2a.sym_pos.data_ptr(), M,
                  a2a.m_valid.data_ptr(), H, I, G, a2a.grouped_layout.data_ptr(),
                  status[4:].data_ptr(), st)
    else:
        cabi.call("moeb_fp8_grouped_gemm_nt_dyn", work["inter"].data_ptr(),
                  work["inter_s"].data_ptr(), down.data_ptr(), down_scale.data_ptr(),
                  a2a.expert_y.data_ptr(), cabi.OUT_BF16, M, a2a.m_valid.data_ptr(), H, I, G,
                  cabi.GEMM_M_GROUPED_CONTIGUOUS, a2a.grouped_layout.data_ptr(), 0,
                  status[4:].data_ptr(), st)
    if events is not None:
        e2.record()
        events["swiglu"].append((e0, e1))
        events["down"].append((e1, e2))
    if push_combine:
        a2a.combine_home(out, wts)
    else:
        a2a.combine(out, wts)
    if events is not None:
        c1 = torch.cuda.Event(enable_timing=True)
        c1.record()
        events.setdefault("combine", []).append((e2, c1))
    return idx, wts


def build_ep_step_p2p(mc, shape, d, bias_d, dev, rank, world, push_combine=True,
                      once_per_rank=True):
    """Benchmark step for N > 1 ranks over peer memory (used by bench.py)."""
    T, H, I, E, k = shape.T, shape.H, shape.I, shape.E, shape.k
    a2a = All2AllP2P(T, E, k, H, device=dev.index, once_per_rank=once_per_rank)
    out = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
    events = {"swiglu": [], "down": []}
    work = {}

    def step(timed: bool):
        a2a.kernel_events = events.setdefault("dispatch_kernel", []) if timed else None
        ep_moe_forward_p2p(a2a, d.x, d.w_router, bias_d, d.gate, d.gate_scale, d.up, d.up_scale,
                           d.down, d.down_scale, out, shape, work, events if timed else None,
                           push_combine)
        a2a.kernel_events = None

    def routed_rows():
        return int(a2a.tokens_per_expert.sum().item())

    def e2e_fn(x_dev, out_dev):
        ep_moe_forward_p2p(a2a, x_dev, d.w_router, bias_d, d.gate, d.gate_scale, d.up, d.up_scale,
                           d.down, d.down_scale, out_dev, shape, work, None, push_combine)

    # logits, select, plan x3, count barrier, dest_base, dispatch, fence, recv_plan, scale
    # transpose, 2 GEMMs, fence, combine
    def remote_copies():
        """(token, slot) copies whose expert lives on another rank"""
        valid = a2a.dst_rank >= 0
        return int((valid & (a2a.dst_rank != rank)).sum().item())

    def dispatch_rows():
        """token rows this rank sends over NVLink in the dispatch: one per remote
        (token, slot) copy, or one per (token, remote rank) in the once-per-rank form"""
        if not a2a.once_per_rank:
            return remote_copies()
        hit = torch.zeros((T, world), dtype=torch.bool, device=dev)
        hit.scatter_(1, a2a.dst_rank.clamp(min=0).long(), a2a.dst_rank >= 0)
        hit[:, rank] = False
        return int(hit.sum().item())

    layer = {"kernels_per_step": 16 if a2a.once_per_rank else 15, "out": out,
             "routed_rows": routed_rows, "e2e_fn": e2e_fn,
             "overflow": lambda: int(a2a.overflow.item()), "remote_copies": remote_copies,
             "dispatch_rows": dispatch_rows}
    return step, events, layer


# ------------------------------------------- the C-ABI context (pull transport) --
class EPContext:
    """The expert-parallel context of the C ABI (moeb_ep_*; csrc/ep_ctx.cu) over
    torch's symmetric memory: dispatch, combine, the two fused ops and the whole
    layer are single library calls; nothing is sequenced from Python.

    Transport: push (default for bf16 tokens: every token is quantised and stored
    once per destination rank, the owners fan it out) or pull (`transport="pull"`,
    pre-quantised tokens, and `fused=True`: the owners load every copy over NVLink —
    in a kernel of their own or by a few comm CTAs inside the gate/up GEMM while its
    other CTAs compute on the row blocks that have landed, the reference's
    kernel5_1 scheme).

    With world size 1 (or without an initialised process group) the rank is its
    own and only peer and a plain device buffer serves as symmetric memory."""

    TRANSPORTS = {"auto": 0, "pull": 1, "push": 2}

    def __init__(self, max_num_tokens, num_experts, experts_per_token, hidden_dim,
                 expert_padding=128, capacity_rows=None, device=None, group=None,
                 transport="auto"):
        import ctypes
        from . import moe_cuda as mc
        self._mc = mc
        self._ctypes = ctypes
        if dist.is_available() and dist.is_initialized():
            self.group = group if group is not None else dist.group.WORLD
            self._rank = dist.get_rank(self.group)
            self._world = dist.get_world_size(self.group)
        else:
            self.group, self._rank, self._world = None, 0, 1
        self._device = torch.device("cuda", torch.cuda.current_device() if device is None
                                    else int(device))
        dev = self._device
        self.T, self.E, self.k, self.H = int(max_num_tokens), int(num_experts), \
            int(experts_per_token), int(hidden_dim)
        self.cfg = cabi.EpConfig(self.T, self.H, self.E, self.k, int(expert_padding), self._world,
                                 self._rank, int(capacity_rows or 0), self.TRANSPORTS[transport])
        lib = cabi.load()
        sym_bytes = lib.moeb_ep_symmetric_bytes(ctypes.byref(self.cfg))
        loc_bytes = lib.moeb_ep_local_bytes(ctypes.byref(self.cfg))
        if sym_bytes == 0 or loc_bytes == 0:
            raise ValueError("bad expert-parallel configuration (hidden % 128, num_experts % world, "
                             "top_k <= 32, expert_padding % 128)")
        if self._world > 1:
            import torch.distributed._symmetric_memory as symm_mem
            self.sym = symm_mem.empty(sym_bytes, dtype=torch.uint8, device=dev)
            self._handle = symm_mem.rendezvous(self.sym, self.group)
            ptrs = [int(p) for p in self._handle.buffer_ptrs]
        else:
            self.sym = torch.empty(sym_bytes, dtype=torch.uint8, device=dev)
            ptrs = [self.sym.data_ptr()]
        self.local = torch.empty(loc_bytes, dtype=torch.uint8, device=dev)
        peers = (ctypes.c_uint64 * self._world)(*ptrs)
        self._ctx = ctypes.c_void_p()
        cabi.call("moeb_ep_create", ctypes.byref(self.cfg), peers, self.local.data_ptr(), loc_bytes,
                  self._stream(), ctypes.byref(self._ctx))
        # nobody dispatches before every rank has cleared its flag words
        torch.cuda.synchronize(dev)
        if self._world > 1:
            dist.barrier(group=self.group)
        v = cabi.EpView()
        cabi.call("moeb_ep_get_view", self._ctx, ctypes.byref(v))
        self.m_cap = v.max_recv_rows
        self.e_local = v.local_experts
        n_kb = self.H // 128
        loc = lambda ptr, n, dt: self._slice(self.local, ptr, n, dt)  # noqa: E731
        self.expert_x = loc(v.expert_x, self.m_cap * self.H, torch.uint8).view(
            self.m_cap, self.H).view(torch.float8_e4m3fn)
        self.scale_mn = loc(v.expert_x_scale, n_kb * self.m_cap, torch.float32).view(n_kb, self.m_cap)
        self.grouped_layout = loc(v.grouped_layout, self.m_cap, torch.int32)
        self.m_valid = loc(v.m_valid, 1, torch.int32)
        self.tokens_per_expert = loc(v.tokens_per_expert, self.e_local, torch.int32)
        self.padded_offsets = loc(v.padded_offsets, self.e_local + 1, torch.int32)
        self.source_rank = loc(v.source_rank, self.m_cap, torch.int32)
        self._source_pos_local = loc(v.source_pos, self.m_cap, torch.int32)
        self.dst_rank = loc(v.dst_rank, self.T * self.k, torch.int32).view(self.T, self.k)
        self.dst_row = loc(v.dst_row, self.T * self.k, torch.int32).view(self.T, self.k)
        self.overflow = loc(v.overflow, 1, torch.int32)
        self.home = self._slice(self.sym, v.home, self.T * self.k * self.H,
                                torch.bfloat16).view(self.T * self.k, self.H)
        self._work = {}
        self._n_tokens = 0

    @staticmethod
    def _slice(buf, ptr, n, dtype):
        off = int(ptr) - buf.data_ptr()
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return buf[off:off + nbytes].view(dtype)

    rank = property(lambda self: self._rank)
    world_size = property(lambda self: self._world)
    max_recv_tokens = property(lambda self: self.m_cap)

    @property
    def source_pos(self):
        """token*k + slot (on its source rank) of every received row of the last
        dispatch: a local array after a pull, the senders' words after a push."""
        v = cabi.EpView()
        cabi.call("moeb_ep_get_view", self._ctx, self._ctypes.byref(v))
        buf = self.local if self.local.data_ptr() <= int(v.source_pos) < \
            self.local.data_ptr() + self.local.numel() else self.sym
        return self._slice(buf, v.source_pos, self.m_cap, torch.int32)

    def _stream(self):
        return torch.cuda.current_stream().cuda_stream

    def _status(self):
        return self._mc.status_word(self._device)

    def close(self):
        if self._ctx:
            cabi.load().moeb_ep_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001 - interpreter shutdown
            pass

    @staticmethod
    def _p(t):
        return None if t is None else t.data_ptr()

    def dispatch(self, x=None, indices=None, x_q=None, x_scale_mn=None, out_expert_x=None,
                 out_expert_x_scale=None, do_send=True, do_recv=True):
        """x bf16 [T,H] (quantised here) or x_q e4m3 [T,H] + x_scale_mn fp32 [H/128,T];
        indices int32 [T,k]. Results: `expert_x` / `scale_mn` (or the given output
        tensors) and the layout fields."""
        T = 0
        if do_send:
            src = x if x is not None else x_q
            T = src.shape[0]
            if T > self.T:
                raise RuntimeError("num_tokens exceeds max_num_tokens")  # a2a_context_tk.hpp:150-152
            self._n_tokens = T
        rows = out_expert_x.shape[0] if out_expert_x is not None else 0
        cabi.call("moeb_ep_dispatch", self._ctx, self._p(x), self._p(x_q), self._p(x_scale_mn),
                  self._p(indices), T, self._p(out_expert_x), self._p(out_expert_x_scale), rows,
                  int(bool(do_send)), int(bool(do_recv)), self._status()[8:].data_ptr(),
                  self._stream())

    def combine(self, out_tokens, weights, expert_y=None, accumulate=False, do_send=True,
                do_recv=True):
        cabi.call("moeb_ep_combine", self._ctx, self._p(expert_y), self._p(weights),
                  self._p(out_tokens), int(bool(accumulate)), int(bool(do_send)),
                  int(bool(do_recv)), self._status()[8:].data_ptr(), self._stream())

    def fused_dispatch_swiglu(self, x, indices, gate, gate_scale, up, up_scale, D, scale_d,
                              fused=True, x_q=None, x_scale_mn=None, out_expert_x=None,
                              out_expert_x_scale=None):
        src = x if x is not None else x_q
        T = src.shape[0]
        self._n_tokens = T
        rows = out_expert_x.shape[0] if out_expert_x is not None else 0
        I = gate.shape[1]
        cabi.call("moeb_ep_fused_dispatch_swiglu", self._ctx, self._p(x), self._p(x_q),
                  self._p(x_scale_mn), self._p(indices), T, self._p(out_expert_x),
                  self._p(out_expert_x_scale), rows, gate.data_ptr(), gate_scale.data_ptr(),
                  up.data_ptr(), up_scale.data_ptr(), D.data_ptr(), scale_d.data_ptr(), I,
                  int(bool(fused)), self._status().data_ptr(), self._stream())

    def fused_gemm_combine(self, A, scale_a, down, down_scale, weights, out_tokens,
                           accumulate=False):
        I = down.shape[2]
        cabi.call("moeb_ep_fused_gemm_combine", self._ctx, A.data_ptr(), scale_a.data_ptr(),
                  down.data_ptr(), down_scale.data_ptr(), I, self._p(weights), self._p(out_tokens),
                  int(bool(accumulate)), self._status()[4:].data_ptr(), self._stream())

    def moe_forward(self, x, w_router, router_bias, gate, gate_scale, up, up_scale, down,
                    down_scale, out, shape, fused=True, indices_out=None, weights_out=None):
        """The whole EP layer in one library call (moeb_ep_moe_forward)."""
        ctypes = self._ctypes
        T = x.shape[0]
        I = gate.shape[1]
        ws = self._work.get(I)
        if ws is None:
            n = cabi.load().moeb_ep_moe_forward_workspace_bytes(self._ctx, I)
            ws = self._work[I] = torch.empty(n, dtype=torch.uint8, device=self._device)
        cfg = cabi.LayerConfig(T, self.H, I, self.E, self.k, int(shape.router_mode),
                               int(shape.n_group), int(shape.topk_group), int(bool(shape.renorm)),
                               float(shape.route_scale))
        self._n_tokens = T
        cabi.call("moeb_ep_moe_forward", self._ctx, ctypes.byref(cfg), self._p(x), w_router.data_ptr(),
                  self._p(router_bias), gate.data_ptr(), gate_scale.data_ptr(), up.data_ptr(),
                  up_scale.data_ptr(), down.data_ptr(), down_scale.data_ptr(), self._p(out),
                  self._p(indices_out), self._p(weights_out), ws.data_ptr(), ws.numel(),
                  int(bool(fused)), self._status().data_ptr(), self._stream())

    @property
    def mlp_mode(self) -> str:
        """How moe_forward(fused=False) runs the two expert GEMMs: "seq" (one after the
        other) or "chunks" (row chunks, down projection of a chunk beside the gate/up
        GEMM of the next)."""
        lib = cabi.load()
        return ("seq", "chunks")[int(lib.moeb_ep_mlp_mode(self._ctx))]

    def set_timing(self, on=True):
        cabi.call("moeb_ep_set_timing", self._ctx, int(bool(on)))

    def read_timing(self):
        """Mean stage times in ms of the recorded moe_forward calls (synchronises):
        dict(router, dispatch_send, dispatch_recv, swiglu, down, combine, steps)."""
        ctypes = self._ctypes
        torch.cuda.synchronize(self._device)
        ms = (ctypes.c_float * 6)()
        n = ctypes.c_int(0)
        cabi.call("moeb_ep_read_timing", self._ctx, ms, ctypes.byref(n))
        names = ("router", "dispatch_send", "dispatch_recv", "swiglu", "down", "combine")
        out = {k: float(v) for k, v in zip(names, ms)}
        out["steps"] = n.value
        return out


class All2All:
    """Drop-in for the reference's `moe_cuda.All2All` (csrc/python_api.cpp:85-166,
    477-514) on the C-ABI context: same constructor keywords, `dispatch` /
    `combine` signatures (both halves, `do_send` / `do_recv`, as in
    csrc/all2all/all2all_tk.hpp:292-334, 376-394) and properties. Ranks come from
    torch.distributed (`group`, default world) instead of TKParallelTensor
    brokers; `max_private_tokens` is accepted and unused (no private / overflow
    split exists here); dp_group_size must be 1 (the reference's dp > 1 path is
    untested, README.md:49). One op in flight per handle, like the reference.

    After `dispatch`, `grouped_layout` (expert id per row, -1 padding) is what the
    MGroupedContiguous GEMMs take."""

    def __init__(self, max_num_tokens, num_experts, experts_per_token, expert_padding, hidden_dim,
                 hidden_dim_scale=None, in_dtype=torch.float8_e4m3fn, out_dtype=torch.bfloat16,
                 scale_dtype=None, max_private_tokens=None, dp_group_size=None,
                 node_group_size=None, ep_group_size=None, device=-1, stream=None, group=None):
        if dist.is_available() and dist.is_initialized():
            world = dist.get_world_size(group)
        else:
            world = 1
        if node_group_size is not None and int(node_group_size) != world:
            raise ValueError("node_group_size must equal the process group size")
        if dp_group_size not in (None, 1):
            raise ValueError("dp_group_size must divide world size; only 1 is supported")
        if ep_group_size is not None and (ep_group_size == 0 or world % ep_group_size != 0):
            raise ValueError("ep_group_size must divide world size")
        if num_experts % world != 0:
            raise ValueError("num_experts must be a multiple of the world size")
        if out_dtype != torch.bfloat16:
            raise ValueError("combine only supports bfloat16")  # a2a_context_tk.hpp:181-182
        if hidden_dim % 128 != 0:
            raise ValueError("hidden_dim must be a multiple of 128")
        self.ctx = EPContext(max_num_tokens, num_experts, experts_per_token, hidden_dim,
                             expert_padding, device=None if device in (-1, None) else int(device),
                             group=group)
        self.k = int(experts_per_token)

    rank = property(lambda self: self.ctx.rank)
    world_size = property(lambda self: self.ctx.world_size)
    device = property(lambda self: self.ctx._device.index)
    max_recv_tokens = property(lambda self: self.ctx.max_recv_tokens)
    handle = property(lambda self: self)
    grouped_layout = property(lambda self: self.ctx.grouped_layout)
    padded_offsets = property(lambda self: self.ctx.padded_offsets)
    tokens_per_expert = property(lambda self: self.ctx.tokens_per_expert)

    def dispatch(self, out_expert_num_tokens, out_expert_x, out_expert_x_scale=None, dp_x=None,
                 dp_x_scale=None, indices=None, weights=None, bound_m=None, do_send=True,
                 do_recv=True):
        """python_api.cpp:134-143. dp_x: e4m3 [T,H]; dp_x_scale: fp32 [H/128,T]
        (MN-major); outputs: out_expert_x e4m3 [max_recv_tokens,H],
        out_expert_x_scale fp32 [H/128,max_recv_tokens], out_expert_num_tokens
        uint32/int32 [E_local] = unpadded rows per local expert."""
        if do_send:
            if dp_x_scale is None or out_expert_x_scale is None:
                raise ValueError("dp_x_scale and out_expert_x_scale are required")  # all2all_tk.hpp:298,327
            if indices is None or indices.dtype != torch.int32 or indices.shape[1] != self.k:
                raise ValueError("indices must be int32 [T, experts_per_token]")
            if out_expert_x.shape[0] != self.max_recv_tokens or \
                    out_expert_x_scale.shape[-1] != self.max_recv_tokens:
                raise ValueError("out_expert_x needs max_recv_tokens rows and a [H/128, rows] scale")
        self.ctx.dispatch(indices=indices, x_q=dp_x, x_scale_mn=dp_x_scale,
                          out_expert_x=out_expert_x if do_send else None,
                          out_expert_x_scale=out_expert_x_scale if do_send else None,
                          do_send=do_send, do_recv=do_recv)
        if do_send and out_expert_num_tokens is not None:
            out_expert_num_tokens.view(torch.int32).copy_(self.ctx.tokens_per_expert)

    def combine(self, out_tokens, indices, weights, expert_y, bound_m=None, do_send=True,
                do_recv=True, accumulate=False):
        """python_api.cpp:145-150: return every expert-output row to its source
        rank and reduce out[t] = sum_j weights[t,j] * y[t,j] (bf16 in/out). Uses
        the routing of the preceding dispatch, like the reference."""
        if expert_y is not None and expert_y.dtype != torch.bfloat16:
            raise ValueError("combine only supports bfloat16")
        self.ctx.combine(out_tokens, weights, expert_y=expert_y, accumulate=accumulate,
                         do_send=do_send, do_recv=do_recv)
