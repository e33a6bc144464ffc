#!/usr/bin/env python
"""MoE-layer throughput benchmark (one JSON line on rank 0).

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the CPU restatement of the reference path

A step is one pass of the whole hot path over one batch of synthetic tokens:
router top-k -> routing plan -> FP8 quantise + permute (+ all-to-all dispatch at
N > 1) -> gate/up grouped GEMM with fused SwiGLU + re-quantisation -> down
grouped GEMM -> (all-to-all combine) -> weighted un-permute. Metric: tokens/s
over all ranks. Default workload: the 32-expert layer of the grouped-GEMM
configuration (T=8192/rank, H=4096, I=1536, 32 experts/rank, top-8) with a
Dirichlet(1) popularity bias so that the per-expert row counts are ragged.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import torch

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO))

from parallel_playground_b200 import workloads as wl  # noqa: E402

KERNELS_PER_STEP_1GPU = 9  # logits, select, plan x3, permute_quant, gate/up GEMM, down GEMM, combine


def router_extra_launches(mc, shape, has_bias):
    """The logits of a wide router (many tokens, more than 64 experts) take three launches
    instead of one: gate-matrix transpose, tcgen05 GEMM with split K, slice sum (the sum is
    left out when one slice without a bias writes the logits itself)."""
    if mc.router_logits_workspace_bytes(shape.T, shape.H, shape.E) == 0:
        return 0
    tiles = -(-shape.T // 128) * -(-shape.E // 256)
    return 2 if (148 // tiles > 1 or has_bias) else 1


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="gemm32", choices=sorted(wl.CONFIGS))
    ap.add_argument("--tokens", type=int, default=None, help="tokens per rank (default: workload's)")
    ap.add_argument("--cpu-sample-tokens", type=int, default=1024)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--ep-transport", default="ctx", choices=["ctx", "p2p", "nccl"],
                    help="N > 1: the C-ABI expert-parallel context (ctx: one library call per "
                         "layer, rows pulled over NVLink, inside the gate/up GEMM when fused), the "
                         "push transport sequenced from Python (p2p), or packed rows through NCCL "
                         "all-to-all (nccl)")
    ap.add_argument("--ep-fused", type=int, default=0, choices=[0, 1],
                    help="ctx transport: rows fetched by a kernel of their own before the gate/up "
                         "GEMM (0, default: measured faster) or by comm CTAs inside it (1)")
    ap.add_argument("--ep-mode", default="auto", choices=["auto", "push", "pull"],
                    help="ctx transport: senders store each token once per destination rank and "
                         "the owners fan it out (push; auto picks it unless --ep-fused 1), or the "
                         "owners load every copy (pull)")
    ap.add_argument("--targets", default=None,
                    help="comma-separated workloads for the short target runs instead of the "
                         "list of this N (e.g. the 8-GPU list on fewer GPUs)")
    ap.add_argument("--no-targets", action="store_true",
                    help="skip the short runs of the other configurations (the `targets` key)")
    ap.add_argument("--no-parity", action="store_true",
                    help="N > 1: skip the untimed parity leg (the `parity` key)")
    ap.add_argument("--profile-mode", action="store_true",
                    help="for runs under a profiler: skip the e2e leg, the FP8 peak probe and the "
                         "CPU baseline (their keys are null)")
    ap.add_argument("--ep-dispatch", default="once", choices=["once", "copy"],
                    help="peer-memory dispatch: a token crosses NVLink once per destination rank "
                         "and is fanned out by the owner (once), or once per expert copy (copy)")
    ap.add_argument("--ep-combine", default="push", choices=["push", "pull"],
                    help="p2p transport: expert outputs are stored home by the down GEMM's "
                         "epilogue (push) or loaded by the token's rank afterwards (pull)")
    return ap.parse_args()


def measured_peaks():
    p = REPO / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


def bench_shape(args, world):
    base = wl.CONFIGS[args.workload]
    shape = dataclasses.replace(base, E=base.E * world if args.workload == "gemm32" else base.E)
    if args.tokens:
        shape = dataclasses.replace(shape, T=args.tokens)
    return shape


def popularity_bias(shape, world=1):
    """log p, p ~ Dirichlet(1): the ragged expert load of the grouped-GEMM configuration.
    With W ranks the draw over one rank's experts is repeated on every rank: each
    rank's expert block has the same popularity profile (weak scaling with ranks
    balanced in expectation, as a load-balancing loss keeps them; the experts inside
    a rank stay as ragged as on one GPU, and the counts still differ by the tokens)."""
    if shape.name != "gemm32":
        return None
    g = torch.Generator().manual_seed(77)
    e_local = shape.E // world
    e = -torch.log(torch.rand(e_local, generator=g, dtype=torch.float64))  # Exp(1) = Gamma(1)
    e = e.repeat(world)
    return (e / e.sum()).log().float()


# ------------------------------------------------------------- clock sampling --
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        self.gpu = gpu_index
        self.path = Path(os.environ.get("TMPDIR", "/tmp")) / f"moeb_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.fh = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.gpu), "-lms", "20"], stdout=self.fh, stderr=subprocess.DEVNULL)
            # the first sample can take a while on a box with many GPUs: the timed
            # region must not start (and end) before the sampler is up
            t_end = time.perf_counter() + 3.0
            while time.perf_counter() < t_end and self.path.stat().st_size == 0:
                time.sleep(0.02)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.fh.close()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.path.read_text().splitlines():
            f = [c.strip() for c in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                pw.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # the sampler starts a little before the timed loop: keep the samples
        # taken under load (power well above the first, idle, reading)
        if pw:
            floor = min(pw) + 0.5 * (max(pw) - min(pw))
            loaded = [c for c, w_ in zip(sm, pw) if w_ >= floor]
            if loaded:
                sm = loaded
        try:
            self.path.unlink()
        except OSError:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm),
                "power_w_max": max(pw) if pw else None, "reasons": sorted(reasons)}


def nvlink_bytes(gpu_index):
    """Cumulative NVLink data counters of one GPU (sum over its links) as
    (tx_bytes, rx_bytes), read with `nvidia-smi nvlink -gt d`; None where the
    query is not available. Reading only: nothing is reset or configured."""
    try:
        out = subprocess.run(["nvidia-smi", "nvlink", "-gt", "d", "-i", str(gpu_index)],
                             capture_output=True, text=True, timeout=20).stdout
    except (OSError, subprocess.SubprocessError):
        return None
    tx = rx = 0
    seen = False
    for ln in out.splitlines():
        f = ln.replace(":", " ").split()
        if "Tx" in f and "KiB" in f:
            tx += int(f[f.index("KiB") - 1]) * 1024
            seen = True
        elif "Rx" in f and "KiB" in f:
            rx += int(f[f.index("KiB") - 1]) * 1024
            seen = True
    return (tx, rx) if seen else None


# ------------------------------------------------------------------ CPU arm --
def dequantised_weights_fit_host(shape):
    """fp32 copies of all experts' three matrices within half of the free host memory?"""
    need = 3.0 * shape.E * shape.H * shape.I * 4
    try:
        import psutil
        return need <= 0.5 * psutil.virtual_memory().available
    except Exception:  # noqa: BLE001 - no psutil: stay on the small side
        return shape.E <= 64


def cpu_reference_arm(shape, sample_tokens, steps, warmup, world=1):
    """Times the oracle (a CPU restatement of the reference path, fp32 on the
    de-quantised FP8 weights, torch CPU matmul on every host core) on a bounded
    sample of the workload's tokens, all `shape.E` experts present. The weights
    are de-quantised beforehand (preparation, not timed, like the GPU arm's
    pre-quantised weights) where their fp32 copies fit the host's free memory
    (19 GB for 256 experts of the default shape); otherwise each expert is
    de-quantised when its rows are processed, inside the timed region."""
    import numpy as np
    import oracle
    torch.set_num_threads(os.cpu_count() or 1)
    sub = dataclasses.replace(shape, T=sample_tokens)
    g = torch.Generator().manual_seed(shape.seed)
    x = torch.randn(sample_tokens, shape.H, generator=g).bfloat16()
    gr = torch.Generator().manual_seed(1000 + shape.seed)
    w_router = (torch.randn(shape.H, shape.E, generator=gr) * 0.02).bfloat16()
    bias = popularity_bias(shape, world)
    if bias is None and shape.zipf_bias > 0:
        bias = wl.zipf_log_bias(shape.E, shape.zipf_bias)
    q = lambda t: t.view(torch.uint8).numpy()  # noqa: E731
    keep_f32 = dequantised_weights_fit_host(shape)
    experts = []
    for e in range(shape.E):
        w = wl.make_expert_weights(shape, e)
        if keep_f32:
            experts.append(tuple(oracle.dequant_weight(q(w[n]), w[n + "_scale"].numpy())[0]
                                 for n in ("gate", "up", "down")))
        else:
            experts.append(w)

    def weights_of(e):
        if keep_f32:
            return experts[e]
        w = experts[e]
        return tuple(oracle.dequant_weight(q(w[n]), w[n + "_scale"].numpy())[0]
                     for n in ("gate", "up", "down"))

    def step():
        logits = oracle.router_logits(x, w_router, bias)
        idx, w = oracle.router_select(logits, sub.k, sub.router_mode, sub.n_group, sub.topk_group,
                                      sub.renorm, sub.route_scale)
        plan = oracle.route_plan(idx, sub.E)
        ex, es = oracle.permute_quant(x, plan.dst_row, plan.m_cap)
        a = oracle.dequant_rows(ex, es)
        y = torch.zeros((plan.m_cap, sub.H))
        for e, rows in oracle._group_rows(plan.grouped_layout, sub.E, False, 0):
            gw, uw, dw = weights_of(e)
            ar = a[rows]
            gate = ar @ gw.T
            act = (ar @ uw.T) * gate / (1.0 + torch.exp(-gate))
            dq, ds = oracle.quant_f32_1x128(act.numpy(), mn_major=True)
            y[rows] = oracle.dequant_rows(dq, ds) @ dw.T
        return oracle.unpermute_combine(y.bfloat16(), plan.dst_row, w, sub.H)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    return {"value": sample_tokens / dt, "unit": "tokens/s", "cores": torch.get_num_threads(),
            "kind": "port", "ms_per_step": dt * 1e3,
            "sample": f"{sample_tokens} tokens of the workload through all {sub.E} experts, "
                      f"{steps} timed passes, weights " +
                      ("pre-dequantised (not timed)" if keep_f32 else
                       "de-quantised per expert inside the timed pass")}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    world = max(1, args.gpus)
    shape = bench_shape(args, world)
    # K timed passes after W warm-up passes over the bounded sample (about a second each);
    # only where the weights must be de-quantised inside every pass (tens of seconds) the
    # run is cut to one pass so that it still ends within minutes
    if dequantised_weights_fit_host(shape):
        steps, warm = max(1, args.steps), max(0, args.warmup)
    else:
        steps, warm = 1, 0
    cb = cpu_reference_arm(shape, args.cpu_sample_tokens, steps, warm, world)
    line = {
        "impl": "reference", "metric": "moe_layer_tokens_per_s", "value": cb["value"],
        "unit": "tokens/s", "n_gpus": args.gpus, "steps": steps, "warmup": warm,
        "ms_per_step": cb["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 (CPU, de-quantised e4m3 inputs)", "data": "synthetic",
        "config": workload_config(shape, world, args.ep_transport, args.ep_combine, args.ep_dispatch,
                                  args.ep_fused),
        "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


def l2_note(shape, world):
    """What the timed steps mean for the 126 MB L2: the per-step inputs of every benchmark
    configuration but the tiny one are larger than it, so consecutive steps cannot feed on
    each other's cache lines and nothing is flushed."""
    weights = 3 * (shape.E // world) * shape.H * shape.I
    acts = shape.T * shape.H * 2 + shape.T * shape.k * (shape.H + shape.I + 2 * shape.H)
    if weights + acts > 126e6:
        return (f"no flush: per-step inputs (FP8 expert weights {weights / 1e6:.0f} MB + "
                f"activations {acts / 1e6:.0f} MB) exceed the 126 MB L2")
    return (f"no flush, and the per-step inputs ({(weights + acts) / 1e6:.0f} MB) fit the 126 MB L2: "
            "a launch-bound configuration timed warm")


def workload_config(shape, world, transport=None, combine=None, dispatch=None, fused=None):
    return {"workload": f"{shape.name}: MoE layer T={shape.T}/rank H={shape.H} I={shape.I} "
                        f"E={shape.E} top-{shape.k}, e4m3 1x128/128x128 scales",
            "tokens_per_rank": shape.T, "hidden": shape.H, "intermediate": shape.I,
            "experts": shape.E, "top_k": shape.k, "parallelism": f"ep{world}",
            "ep_transport": transport if world > 1 else None,
            "ep_combine": combine if (world > 1 and transport == "p2p") else None,
            "ep_dispatch": dispatch if (world > 1 and transport == "p2p") else None,
            "ep_dispatch_fused_into_gemm": bool(fused) if (world > 1 and transport == "ctx") else None,
            "expert_popularity": ("log Dirichlet(1) bias over a rank's experts, the same profile on "
                                  "every rank" if shape.name == "gemm32" else
                                  (f"log Zipf({shape.zipf_bias}) bias" if shape.zipf_bias > 0
                                   else "none (unbiased router)")),
            "l2": l2_note(shape, world)}


# ------------------------------------------------------------------ GPU arm --
def fp8_peak_tflops(dev, gpu_index=0, sustained_s=2.0):
    """Dense FP8 tensor peak of this GPU, measured like the bf16 figures in
    MEASURED_PEAKS.json: cuBLASLt e4m3 GEMM 8192^3 via torch._scaled_mm, best of
    10 (burst) and back to back for `sustained_s` seconds under the power cap
    (sustained, with the SM clock seen meanwhile). Returns a dict or None."""
    n = 8192
    try:
        a = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn).t()
        one = torch.ones((), device=dev)

        def mm():
            torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)

        for _ in range(3):
            mm()
        best = float("inf")
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            mm()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        flop = 2.0 * n ** 3
        out = {"burst": flop / (best * 1e-3) / 1e12, "sustained": None, "sustained_sm_mhz": None}
        if sustained_s > 0:
            per_batch = max(8, int(0.25 / (best * 1e-3)))   # about a quarter second per event pair
            sampler = ClockSampler(gpu_index)
            sampler.start()
            rates, t_end = [], time.perf_counter() + sustained_s
            while time.perf_counter() < t_end:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(per_batch):
                    mm()
                e1.record()
                torch.cuda.synchronize()
                rates.append(per_batch * flop / (e0.elapsed_time(e1) * 1e-3) / 1e12)
            clocks = sampler.stop()
            tail = rates[len(rates) // 2:]            # after the clocks have settled
            out["sustained"] = statistics.mean(tail)
            out["sustained_sm_mhz"] = clocks.get("sm_mhz")
        return out
    except Exception:  # noqa: BLE001 - the peak probe must never break the benchmark
        return None


# DRAM traffic of one gate/up launch of the gemm32 shape (H=4096, I=1536, 32 local
# experts), from an ncu capture of a 16 384-row launch: the FP8 weights are read
# once (2*E_local*I*H bytes) and every routed row adds 5 267 bytes
# (dram__bytes_read.sum + dram__bytes_write.sum; 489.0 MB in total for that launch).
GEMM32_GATEUP_DRAM_BYTES_PER_ROW = 5267.0


def setup_inputs(args, shape, world, rank, dev):
    inp = wl.make_layer_inputs(shape, rank=rank, world=world, weights_device=str(dev))
    d = inp.to(dev)
    bias = popularity_bias(shape, world)
    if bias is None:
        bias = inp.router_bias          # e.g. the Zipf bias of the Mixtral-shaped workload
    bias_d = None if bias is None else bias.to(dev)
    return inp, d, bias_d


def build_step(mc, args, shape, d, bias_d, dev, rank, world, fused=None):
    if world == 1:
        return build_single_gpu_step(mc, shape, d, bias_d, dev)
    if args.ep_transport == "ctx":
        return build_ep_step_ctx(mc, shape, d, bias_d, dev, rank, world,
                                 bool(args.ep_fused) if fused is None else fused, args.ep_mode)
    from parallel_playground_b200.ep import build_ep_step, build_ep_step_p2p
    if args.ep_transport == "p2p":
        return build_ep_step_p2p(mc, shape, d, bias_d, dev, rank, world,
                                 push_combine=args.ep_combine == "push",
                                 once_per_rank=args.ep_dispatch == "once")
    return build_ep_step(mc, shape, d, bias_d, dev, rank, world)


def build_ep_step_ctx(mc, shape, d, bias_d, dev, rank, world, fused, mode="auto"):
    """N > 1 ranks through the C-ABI expert-parallel context: the whole layer is
    one library call per step; stage times come from CUDA events that the library
    records around its launches."""
    from parallel_playground_b200.ep import EPContext
    T, H = shape.T, shape.H
    ctx = EPContext(T, shape.E, shape.k, H, device=dev.index, transport=mode)
    push = (mode != "pull") and not fused
    out = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
    idx = torch.empty((T, shape.k), dtype=torch.int32, device=dev)
    wts = torch.empty((T, shape.k), dtype=torch.float32, device=dev)
    state = {"timing": False}

    def run(x_dev, out_dev, want_routing=False):
        ctx.moe_forward(x_dev, d.w_router, bias_d, d.gate, d.gate_scale, d.up, d.up_scale, d.down,
                        d.down_scale, out_dev, shape, fused=fused,
                        indices_out=idx if want_routing else None,
                        weights_out=wts if want_routing else None)

    def step(timed: bool):
        if timed and not state["timing"]:
            ctx.set_timing(True)
            state["timing"] = True
        run(d.x, out)

    def stage_ms():
        tm = ctx.read_timing()
        ctx.set_timing(False)
        state["timing"] = False
        return tm

    def remote_copies():
        valid = ctx.dst_rank >= 0
        return int((valid & (ctx.dst_rank != rank)).sum().item())

    def dispatch_rows():
        """token rows that cross NVLink in the dispatch: one per remote copy (pull), or
        one per (token, remote rank) (push)"""
        if not push:
            return remote_copies()
        hit = torch.zeros((T, world), dtype=torch.bool, device=dev)
        hit.scatter_(1, ctx.dst_rank.clamp(min=0).long(), ctx.dst_rank >= 0)
        hit[:, rank] = False
        return int(hit.sum().item())

    # router x2, plan x3, exchange+plan, then push: dispatch, barrier, fan-out, transpose;
    # pull: cast, mark, announce, pull (or inside the GEMM), pos; gate/up GEMM, down GEMM,
    # barrier, reduce
    # how the library runs the two expert GEMMs of the whole-layer call: one after the
    # other, or overlapped in row chunks (see moeb_ep_mlp_mode)
    mlp_mode = "seq" if fused else ctx.mlp_mode
    overlapped = mlp_mode != "seq"
    down_sms = int(os.environ.get("MOEB_EP_DOWN_SMS", "52"))
    chunks = int(os.environ.get("MOEB_EP_MLP_CHUNKS", "4"))
    # chunked: one plan kernel and two GEMM launches per chunk instead of two launches
    extra = 2 * chunks - 1 if mlp_mode == "chunks" else 0
    extra += router_extra_launches(mc, shape, bias_d is not None)
    layer = {"kernels_per_step": (14 if push else (15 if fused else 16)) + extra, "out": out,
             "ctx": ctx, "mlp_mode": mlp_mode, "mlp_chunks": chunks if mlp_mode == "chunks" else 0,
             "mlp_overlapped": overlapped, "down_sms": down_sms if overlapped else 0,
             "run": run, "routed_rows": lambda: int(ctx.tokens_per_expert.sum().item()),
             "e2e_fn": lambda x_dev, out_dev: run(x_dev, out_dev),
             "overflow": lambda: int(ctx.overflow.item()), "remote_copies": remote_copies,
             "dispatch_rows": dispatch_rows, "stage_ms": stage_ms, "idx": idx, "wts": wts,
             "fused": fused, "push": push}
    return step, None, layer


def timed_steps(mc, step, steps, warmup, dev, world, rank, local_rank, sample_clocks):
    """W untimed steps, then exactly K steps between barrier + synchronize on both
    sides, CUDA events on the launching stream, max over ranks."""
    import torch.distributed as dist
    for _ in range(max(warmup, 3)):
        step(False)
    torch.cuda.synchronize()
    mc.check_device_status()
    sampler = ClockSampler(local_rank) if sample_clocks else None
    if sampler is not None and rank == 0:
        sampler.start()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step(True)
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms_total = e0.elapsed_time(e1)
    clocks = sampler.stop() if (sampler is not None and rank == 0) else None
    mc.check_device_status()
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    return ms_total / steps, clocks


def collect_stages(stage_events, layer):
    """Mean stage times in ms of the timed steps: from the library's own events
    (ctx transport) or from the events recorded around the Python-issued launches."""
    if "stage_ms" in layer:
        tm = layer["stage_ms"]()
        return {"swiglu": tm["swiglu"], "down": tm["down"], "dispatch": tm["dispatch_send"],
                "dispatch_recv": tm["dispatch_recv"], "combine": tm["combine"],
                "router": tm["router"], "steps_recorded": tm["steps"]}
    out = {}
    for name in ("swiglu", "down", "dispatch", "combine", "dispatch_kernel"):
        if stage_events.get(name):
            out[name] = statistics.mean(a.elapsed_time(b) for a, b in stage_events[name])
    return out


def gemm_figures(shape, world, rows, st, peaks, fp8, overlapped=False, down_sms=0):
    """TFLOP/s of the two grouped GEMMs and their roofline records. The launches
    are timed one by one with CUDA events inside a timed region of well under two
    seconds, so the denominator is the BURST rate of cuBLASLt's e4m3 GEMM measured
    in this run; the sustained rate and the nominal peak are printed beside it."""
    H, I = shape.H, shape.I
    e_local = shape.E // world
    burst = fp8["burst"] if fp8 else 2.0 * peaks["bf16_tflops"]
    burst_src = ("cuBLASLt e4m3 8192^3, best of 10 in this run (burst)" if fp8 else
                 f"2 x bf16_tflops of MEASURED_PEAKS.json ({peaks['source']})")
    sustained = fp8["sustained"] if fp8 and fp8.get("sustained") else None

    def record(kernel, flops, ms, alg_bytes):
        ach = flops / (ms * 1e-3) / 1e12
        r = {"bound": "tensor", "kernel": kernel, "achieved": ach, "peak": burst,
             "unit": "TFLOP/s", "frac": ach / burst, "peak_source": burst_src,
             "peak_sustained": sustained,
             "frac_of_sustained": ach / sustained if sustained else None,
             "peak_bf16_x2": 2.0 * peaks["bf16_tflops"], "peak_nominal": 4500.0,
             "frac_of_nominal": ach / 4500.0, "flops_per_launch": flops, "ms_per_launch": ms,
             "algorithmic_bytes": alg_bytes, "traffic": None}
        # few rows per expert (decode sizes): reading the FP8 weights takes longer than
        # the contraction, so the launch is judged against the measured HBM bandwidth
        t_tensor = flops / (burst * 1e12)
        t_hbm = alg_bytes / (peaks["hbm_gbs"] * 1e9)
        if t_hbm > t_tensor:
            gbs = alg_bytes / (ms * 1e-3) / 1e9
            r.update({"bound": "hbm", "achieved_tensor": ach, "frac_tensor": ach / burst,
                      "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                      "frac": gbs / peaks["hbm_gbs"],
                      "peak_source": f"hbm_gbs of MEASURED_PEAKS.json ({peaks['source']})"})
        return r

    if overlapped:
        # expert parallel, chunked MLP: the down projection of a row chunk runs beside the
        # gate/up GEMM of the next chunk on disjoint SMs (its rows feed NVLink meanwhile);
        # only the common span is meaningful: swiglu = up to the end of gate/up, down =
        # what is left of the down projection
        both = record("grouped_gemm_fp8_kernel: gate/up and down GEMMs overlapped "
                      f"({148 - down_sms} + {down_sms} SMs while both run)",
                      6.0 * rows * H * I, st["swiglu"] + st["down"],
                      3.0 * e_local * I * H + rows * (H + 4.0 * (H // 128) + 2.0 * I +
                                                      8.0 * (I // 128) + 2.0 * H))
        return both, None
    up = record("grouped_gemm_fp8_kernel<swiglu> (gate/up + SwiGLU + requant)",
                4.0 * rows * H * I, st["swiglu"],
                2.0 * e_local * I * H + rows * (H + 4.0 * (H // 128) + I + 4.0 * (I // 128)))
    dn = record("grouped_gemm_fp8_kernel<down> (down projection, bf16 rows out)",
                2.0 * rows * H * I, st["down"],
                1.0 * e_local * I * H + rows * (I + 4.0 * (I // 128) + 2.0 * H))
    if shape.name == "gemm32":
        up["traffic"] = 2.0 * e_local * I * H + GEMM32_GATEUP_DRAM_BYTES_PER_ROW * rows
        up["traffic_source"] = ("ncu dram__bytes_read.sum + dram__bytes_write.sum of a 16 384-row "
                                "launch of this shape: weights once + 5 267 B per routed row, "
                                "scaled to this launch's rows")
    return up, dn


def transport_figures(shape, world, layer, st, args):
    """NVLink figures of the EP transport (rank 0's view): algorithmic bytes over
    CUDA-event times, against 900 GB/s per direction."""
    H = shape.H
    row_b = wl.dispatch_row_bytes(H)
    remote = layer["remote_copies"]()
    sent = layer["dispatch_rows"]() if "dispatch_rows" in layer else remote
    out = {"remote_copies": remote, "dispatch_rows_moved": sent, "overflow_copies": layer["overflow"](),
           "nvlink_peak_gbs_per_direction": 900.0, "dispatch_ms": st.get("dispatch"),
           "combine_ms": st.get("combine"), "router_ms": st.get("router")}
    if args.ep_transport == "ctx":
        fused, push = layer["fused"], layer["push"]
        # the rows cross NVLink in the send half (push: plan, count exchange and the
        # dispatch kernel together), in the pull kernel, or inside the gate/up GEMM
        # (fused); the results go home inside the down GEMM
        xfer_ms = st["dispatch"] if push else (st["swiglu"] if fused else st["dispatch_recv"])
        comb_ms = st["down"] + (st["swiglu"] if layer.get("mlp_overlapped") else 0.0)
        out.update({"dispatch_fused_into_gemm": bool(fused),
                    "dispatch_mode": "push, once per destination rank" if push else "pull, per copy",
                    "dispatch_recv_ms": st["dispatch_recv"],
                    "dispatch_transfer_in": ("send half (plan + count exchange + dispatch kernel)"
                                             if push else ("swiglu_gemm" if fused else "pull kernel")),
                    "dispatch_nvlink_gbs": sent * row_b / (xfer_ms * 1e-3) / 1e9,
                    "dispatch_nvlink_frac": sent * row_b / (xfer_ms * 1e-3) / 1e9 / 900.0,
                    "dispatch_phase_ms": st["dispatch"] + st["dispatch_recv"],
                    "combine_transfer_in": ("down projection beside gate/up (both spans)"
                                            if layer.get("mlp_overlapped") else "down_gemm"),
                    "combine_nvlink_gbs": remote * 2.0 * H / (comb_ms * 1e-3) / 1e9,
                    "combine_nvlink_frac": remote * 2.0 * H / (comb_ms * 1e-3) / 1e9 / 900.0})
        return out
    push = args.ep_transport == "p2p" and args.ep_combine == "push"
    xfer_ms = st["down"] if push else st["combine"]
    if "dispatch_kernel" in st:
        out["dispatch_kernel_ms"] = st["dispatch_kernel"]
        out["dispatch_kernel_nvlink_gbs"] = sent * row_b / (st["dispatch_kernel"] * 1e-3) / 1e9
    out.update({"dispatch_nvlink_gbs": sent * row_b / (st["dispatch"] * 1e-3) / 1e9,
                "combine_nvlink_gbs": remote * 2.0 * H / (xfer_ms * 1e-3) / 1e9,
                "combine_transfer_in": "down_gemm" if push else "combine"})
    return out


def parity_leg(mc, args, shape, inp, d, bias_d, dev, rank, world, layer):
    """N > 1, outside the timed region. Every rank checks, for its own tokens:
      * routing: the layer's indices and weights equal the CPU oracle's selection
        on the same logits, bit for bit;
      * expert outputs: for W experts, one owned by each rank (so rows travel both
        ways over every pair of ranks), every (token, slot) copy of the first 256
        tokens routed to them is recomputed by the oracle from the same FP8 inputs
        (fp32 on de-quantised operands, intermediate re-quantised 1x128) and its
        contribution to the token's output (routing weight x expert row) is
        compared with the row that came home: max|err|/max|ref| <= 2e-2, mean|err|
        <= 1e-3;
      * the whole output equals, bit for bit, the output of the staged transport
        (pack -> NCCL all-to-all-v -> unpack), an independent second path.
    The outcome is all-reduced; the oracle is the checker here, never the timed path."""
    import numpy as np
    import torch.distributed as dist
    import oracle
    from parallel_playground_b200.ep import All2AllStaged, ep_moe_forward
    T, H, I, E, k = shape.T, shape.H, shape.I, shape.E, shape.k
    ctx = layer["ctx"]
    out = layer["out"]
    layer["run"](d.x, out, True)
    torch.cuda.synchronize()
    idx, wts = layer["idx"], layer["wts"]
    n_chk = min(T, 256)
    logits = torch.empty((T, E), dtype=torch.float32, device=dev)
    mc.router_logits(d.x, d.w_router, logits, bias_d)
    ref_idx, ref_w = oracle.router_select(logits[:n_chk].cpu().numpy(), k, shape.router_mode,
                                          shape.n_group, shape.topk_group, shape.renorm,
                                          shape.route_scale)
    routing_exact = bool(np.array_equal(idx[:n_chk].cpu().numpy(), ref_idx) and
                         np.array_equal(wts[:n_chk].cpu().numpy().view(np.uint32),
                                        ref_w.view(np.uint32)))
    e_local = E // world
    chosen = [r * e_local + (rank + r) % e_local for r in range(world)]
    # the checked experts' weights are regenerated with the seeds of their owners
    home = ctx.home.view(ctx.T, k, H)
    xq, xs = oracle.cast_1x128(inp.x[:n_chk], mn_major=True)
    max_rel = mean_abs = 0.0
    pairs = 0
    q = lambda t: t.view(torch.uint8).cpu().numpy()  # noqa: E731
    for e in chosen:
        sel = (idx[:n_chk] == e).nonzero()
        if sel.numel() == 0:
            continue
        toks, slots = sel[:, 0].cpu().numpy(), sel[:, 1].cpu().numpy()
        w = wl.make_expert_weights(shape, e, weights_device=str(dev))
        lay = np.zeros(toks.size, np.int32)
        a_q = np.ascontiguousarray(xq[toks])
        a_s = np.ascontiguousarray(xs[:, toks])
        _, d_ref, sd_ref = oracle.grouped_gemm_swiglu_ref(a_q, a_s, q(w["gate"]),
                                                          w["gate_scale"].cpu().numpy(),
                                                          q(w["up"]), w["up_scale"].cpu().numpy(), lay)
        y_ref = oracle.grouped_gemm_ref(d_ref, sd_ref, q(w["down"]), w["down_scale"].cpu().numpy(), lay)
        got = home[torch.from_numpy(toks).to(dev), torch.from_numpy(slots).to(dev)].float().cpu().numpy()
        # what the copy adds to its token's output: routing weight x expert row
        wgt = ref_w[toks, slots][:, None]
        got, y_ref = got * wgt, y_ref * wgt
        err = np.abs(got - y_ref)
        max_rel = max(max_rel, float(err.max() / max(np.abs(y_ref).max(), 1e-30)))
        mean_abs = max(mean_abs, float(err.mean()))
        pairs += int(toks.size)
    # second transport, whole batch
    staged = All2AllStaged(T, E, k, 128, H, in_dtype=torch.float8_e4m3fn, out_dtype=torch.bfloat16,
                           device=dev.index)
    out2 = torch.empty_like(out)
    ep_moe_forward(staged, d.x, d.w_router, bias_d, d.gate, d.gate_scale, d.up, d.up_scale, d.down,
                   d.down_scale, out2, shape)
    torch.cuda.synchronize()
    same = bool(torch.equal(out.view(torch.int16), out2.view(torch.int16)))
    del staged, out2
    ok = routing_exact and same and max_rel <= 2e-2 and mean_abs <= 1e-3 and pairs > 0
    t = torch.tensor([0.0 if ok else 1.0, 0.0 if routing_exact else 1.0, 0.0 if same else 1.0,
                      max_rel, mean_abs, float(pairs)], device=dev)
    worst = t.clone()
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    total = t[5:6].clone()
    dist.all_reduce(total)
    return {"ok": bool(worst[0].item() == 0.0), "routing_exact": bool(worst[1].item() == 0.0),
            "matches_staged_transport": bool(worst[2].item() == 0.0),
            "max_rel": float(worst[3].item()), "mean_abs": float(worst[4].item()),
            "sampled_pairs": int(total.item()), "ranks": world,
            "tolerance": "routing bit-exact; weighted expert rows max|err|/max|ref| <= 2e-2, "
                         "mean|err| <= 1e-3 against the CPU oracle on the same FP8 inputs; output "
                         "bit-identical to the staged NCCL transport"}


TARGET_WORKLOADS = {1: ["qwen3", "mixtral", "dsv3_rank", "dsv3_decode"], 2: ["qwen3"], 4: ["qwen3"],
                    8: ["dsv3_prefill", "dsv3_decode", "mixtral", "qwen3"]}


def run_target(mc, args, name, world, rank, local_rank, dev, peaks, fp8):
    """A short run (8 timed steps) of another benchmark configuration at this N:
    ms/step, tokens/s, both GEMMs against their rooflines and, for N > 1, the
    NVLink figures of the dispatch (fused into the GEMM, and fetched by the pull
    kernel alone) and of the combine."""
    import gc
    shape = wl.CONFIGS[name]
    inp, d, bias_d = setup_inputs(args, shape, world, rank, dev)
    res = {"workload": workload_config(shape, world, args.ep_transport)["workload"]}
    modes = [None] if (world == 1 or args.ep_transport != "ctx") else [True, False]
    for fused in modes:
        step, ev, layer = build_step(mc, args, shape, d, bias_d, dev, rank, world, fused)
        ms_step, _ = timed_steps(mc, step, 8, 3, dev, world, rank, local_rank, False)
        st = collect_stages(ev, layer)
        rows = int(layer["routed_rows"]())
        if rank == 0:
            up, dn = gemm_figures(shape, world, rows, st, peaks, fp8,
                                  layer.get("mlp_overlapped", False), layer.get("down_sms", 0))
            keys = ("kernel", "bound", "achieved", "unit", "frac", "peak", "ms_per_launch",
                    "frac_of_nominal")
            rec = {"ms_per_step": ms_step, "tokens_per_s": shape.T * world / (ms_step * 1e-3),
                   "routed_rows": rows, "gate_up": {k_: up[k_] for k_ in keys},
                   "down": None if dn is None else {k_: dn[k_] for k_ in keys},
                   "layer_tflops": 6.0 * rows * shape.H * shape.I / (ms_step * 1e-3) / 1e12}
            if world > 1:
                rec["transport"] = transport_figures(shape, world, layer, st, args)
            key = "result" if fused is None else ("fused" if fused else "unfused")
            res[key] = rec
        if "ctx" in layer:
            layer["ctx"].close()
        del step, ev, layer
        gc.collect()
        torch.cuda.empty_cache()
    del inp, d, bias_d
    gc.collect()
    torch.cuda.empty_cache()
    return res


def run_b200(args):
    import torch.distributed as dist
    from parallel_playground_b200 import moe_cuda as mc

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    shape = bench_shape(args, world)
    inp, d, bias_d = setup_inputs(args, shape, world, rank, dev)
    T, H, I, E, k = shape.T, shape.H, shape.I, shape.E, shape.k
    step, stage_events, layer = build_step(mc, args, shape, d, bias_d, dev, rank, world)

    nvl0 = nvlink_bytes(local_rank) if (rank == 0 and world > 1) else None
    ms_step, clocks = timed_steps(mc, step, args.steps, args.warmup, dev, world, rank, local_rank,
                                  True)
    nvl1 = nvlink_bytes(local_rank) if nvl0 is not None else None
    tokens_per_s = T * world / (ms_step * 1e-3)
    st = collect_stages(stage_events, layer)
    rows = int(layer["routed_rows"]())

    # e2e through the public host-buffer call (rank-local; N=1 uses the C-ABI single call)
    e2e = None if args.profile_mode else measure_e2e(mc, layer, shape, inp, dev, world, args)
    parity = None
    if world > 1 and args.ep_transport == "ctx" and not args.no_parity and not args.profile_mode:
        parity = parity_leg(mc, args, shape, inp, d, bias_d, dev, rank, world, layer)
    transport = transport_figures(shape, world, layer, st, args) \
        if (world > 1 and "remote_copies" in layer) else None

    peaks = measured_peaks()
    fp8 = None
    if rank == 0 and not args.profile_mode:
        fp8 = fp8_peak_tflops(dev, local_rank)
    targets = None
    if not args.no_targets and not args.profile_mode and args.workload == "gemm32" \
            and not args.tokens:
        if "ctx" in layer:
            layer["ctx"].close()
        del step, stage_events, d, bias_d
        layer = {"kernels_per_step": layer["kernels_per_step"],
                 "mlp_overlapped": layer.get("mlp_overlapped", False),
                 "mlp_mode": layer.get("mlp_mode", "seq"), "mlp_chunks": layer.get("mlp_chunks", 0),
                 "down_sms": layer.get("down_sms", 0)}
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        targets = [run_target(mc, args, name, world, rank, local_rank, dev, peaks, fp8)
                   for name in (args.targets.split(",") if args.targets
                                else TARGET_WORKLOADS.get(world, []))]

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return 0 if (parity is None or parity["ok"]) else 1
    overlapped = layer.get("mlp_overlapped", False)
    up, dn = gemm_figures(shape, world, rows, st, peaks, fp8, overlapped, layer.get("down_sms", 0))
    line = {
        "metric": "moe_layer_tokens_per_s", "value": tokens_per_s, "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "e4m3 x e4m3 -> f32 (bf16 in/out)", "data": "synthetic",
        "config": workload_config(shape, world, args.ep_transport, args.ep_combine, args.ep_dispatch,
                                  args.ep_fused),
        "clocks": clocks,
        "e2e": e2e,
        "gpu_launches": layer["kernels_per_step"] * args.steps,
        "roofline": up,
        "roofline_down": dn,
        "stages": {"swiglu_gemm_ms": st["swiglu"], "down_gemm_ms": st["down"],
                   "down_gemm_tflops": (None if overlapped else
                                        2.0 * rows * H * I / (st["down"] * 1e-3) / 1e12),
                   "mlp_overlapped": overlapped, "mlp_mode": layer.get("mlp_mode", "seq"),
                   "mlp_chunks": layer.get("mlp_chunks", 0), "routed_rows": rows,
                   "layer_tflops": 6.0 * rows * H * I / (ms_step * 1e-3) / 1e12},
    }
    if transport is not None:
        transport.update({
            # the hardware's own NVLink data counters over the timed steps (rank 0's GPU),
            # beside the algorithmic bytes: rows in + result rows out per step
            "nvlink_counter_tx_bytes_per_step": ((nvl1[0] - nvl0[0]) / args.steps
                                                 if nvl0 and nvl1 else None),
            "nvlink_counter_rx_bytes_per_step": ((nvl1[1] - nvl0[1]) / args.steps
                                                 if nvl0 and nvl1 else None)})
        line["stages"].update(transport)
    if parity is not None:
        line["parity"] = parity
    if targets is not None:
        line["targets"] = targets
        line["targets_note"] = ("short runs (8 timed steps) of the other benchmark configurations at "
                                "this N; north-star bars at the DeepSeek-V3 shape, EP=8: grouped GEMMs "
                                ">= 0.60 of FP8 peak, dispatch/combine >= 0.70 of 900 GB/s per direction")
    if not args.no_cpu_baseline and not args.profile_mode and world == 1:
        cb = cpu_reference_arm(shape, args.cpu_sample_tokens, 2, 1)
        line["cpu_baseline"] = {k_: cb[k_] for k_ in ("value", "unit", "cores", "kind", "sample")}
    print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0 if (parity is None or parity["ok"]) else 1


def build_single_gpu_step(mc, shape, d, bias_d, dev):
    """One rank: the stage-by-stage C-ABI calls, so that CUDA events can bracket
    the GEMM launches inside the timed region."""
    T, H, I, E, k = shape.T, shape.H, shape.I, shape.E, shape.k
    plan = mc.RoutePlan(T, k, E, 128, dev)
    M = plan.m_cap
    logits = torch.empty((T, E), dtype=torch.float32, device=dev)
    idx = torch.empty((T, k), dtype=torch.int32, device=dev)
    wts = torch.empty((T, k), dtype=torch.float32, device=dev)
    ex = torch.empty((M, H), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    es = torch.empty((H // 128, M), dtype=torch.float32, device=dev)
    inter = torch.empty((M, I), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    inter_s = torch.empty((I // 128, M), dtype=torch.float32, device=dev)
    ey = torch.empty((M, H), dtype=torch.bfloat16, device=dev)
    out = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
    events = {"swiglu": [], "down": []}

    def step(timed: bool):
        mc.router_logits(d.x, d.w_router, logits, bias_d)
        mc.router_select(logits, idx, wts, shape.router_mode, shape.n_group, shape.topk_group,
                         shape.renorm, shape.route_scale)
        plan.run(idx)
        mc.permute_quant(d.x, plan.dst_row, ex, es)
        if timed:
            a, b, c = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            a.record()
        mc.fp8_grouped_gemm_swiglu(ex, es, d.gate, d.gate_scale, d.up, d.up_scale, inter, inter_s,
                                   mc.GemmType.MGroupedContiguous, plan.grouped_layout)
        if timed:
            b.record()
        mc.fp8_grouped_gemm_nt(inter, inter_s, d.down, d.down_scale, ey,
                               mc.GemmType.MGroupedContiguous, plan.grouped_layout)
        if timed:
            c.record()
            events["swiglu"].append((a, b))
            events["down"].append((b, c))
        mc.unpermute_combine(ey, plan.dst_row, wts, out)

    layer = {"kernels_per_step": KERNELS_PER_STEP_1GPU + router_extra_launches(mc, shape,
                                                                              bias_d is not None),
             "out": out, "routed_rows": lambda: int(plan.expert_counts.sum().item())}
    return step, events, layer


def measure_e2e(mc, layer, shape, inp, dev, world, args):
    """Same metric through the public host-buffer entry point: every step copies
    the tokens from pinned host memory, runs the layer and reads the result back."""
    if world != 1:
        return measure_e2e_ep(mc, layer, shape, inp, dev, args)
    d = inp.to(dev)
    bias = popularity_bias(shape)
    if bias is None:
        bias = inp.router_bias
    ml = mc.MoELayer(shape.T, shape.H, shape.I, shape.E, shape.k, d.w_router, d.gate, d.gate_scale,
                     d.up, d.up_scale, d.down, d.down_scale, shape.router_mode, shape.n_group,
                     shape.topk_group, shape.renorm, shape.route_scale,
                     None if bias is None else bias.to(dev))
    n = e2e_batches(args)
    # two pinned host batches in, two out (alternating): consecutive steps use
    # different host buffers, as a caller feeding a stream of batches would
    xs = [inp.x.pin_memory(), inp.x.clone().pin_memory()]
    ohs = [torch.empty_like(inp.x).pin_memory() for _ in range(2)]
    x_seq = [xs[i & 1] for i in range(n)]
    o_seq = [ohs[i & 1] for i in range(n)]
    # (a) one blocking C-ABI call per batch: copy in, layer, copy out, in order
    for _ in range(3):
        ml.forward_host(xs[0], ohs[0])
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for i in range(n):
        ml.forward_host(x_seq[i], o_seq[i])
    e1.record()
    torch.cuda.synchronize()
    wall_serial = (time.perf_counter() - t0) / n
    ms_serial = max(e0.elapsed_time(e1) / n, wall_serial * 1e3)
    same = torch.equal(ohs[0].view(torch.int16), layer["out"].cpu().view(torch.int16))
    # (b) the same batches as a stream: copies of neighbouring batches overlap the layer
    ml.forward_host_batches(x_seq[:4], o_seq[:4])
    torch.cuda.synchronize()
    for o in ohs:
        o.zero_()
    t0 = time.perf_counter()
    e0.record()
    ml.forward_host_batches(x_seq, o_seq)
    e1.record()
    torch.cuda.synchronize()
    wall = (time.perf_counter() - t0) / n
    ms = max(e0.elapsed_time(e1) / n, wall * 1e3)
    mc.check_device_status()
    same = same and all(torch.equal(o.view(torch.int16), layer["out"].cpu().view(torch.int16))
                        for o in ohs)
    nbytes = shape.T * shape.H * 2
    copy_ms = copy_only_ms(tuple(inp.x.shape), dev, x_seq, o_seq)
    return {"value": shape.T / (ms * 1e-3), "unit": "tokens/s",
            "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes, "ms_per_step": ms,
            "serial_ms_per_step": ms_serial, "serial_value": shape.T / (ms_serial * 1e-3),
            "copy_only_ms_per_step": copy_ms, "copy_only_value": shape.T / (copy_ms * 1e-3),
            "batches": n, "matches_device_path": bool(same),
            "api": "MoELayer.forward_host_batches (pinned host batches, copies overlapped with the "
                   "layer over the C ABI moeb_moe_forward); serial_* = one blocking "
                   "moeb_moe_forward_host call per batch"}


def e2e_batches(args):
    """Host batches of the end-to-end stream: twice the timed steps (at least 8, at most
    60), so that filling and draining the three-stage pipeline (one copy-in before the
    first layer call, one copy-out after the last) weighs a few per cent, not ten."""
    return max(8, min(2 * args.steps, 60))


def copy_only_ms(x_shape, dev, x_seq, o_seq):
    """ms per batch of the host pipeline with the layer replaced by a device-to-device
    copy: the ceiling the H2D + D2H copies alone allow."""
    from parallel_playground_b200.hostpipe import HostPipeline
    pipe = HostPipeline(lambda x, o: o.copy_(x), x_shape, x_shape, torch.bfloat16, dev)
    pipe.process(x_seq[:4], o_seq[:4])
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    pipe.process(x_seq, o_seq)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / len(x_seq)


def measure_e2e_ep(mc, layer, shape, inp, dev, args):
    """N > 1: every rank copies its tokens from pinned host memory, runs the EP
    layer through the public ep.ep_moe_forward call and reads its result back."""
    import torch.distributed as dist
    from parallel_playground_b200.hostpipe import HostPipeline
    n = e2e_batches(args)
    xs = [inp.x.pin_memory(), inp.x.clone().pin_memory()]
    ohs = [torch.empty_like(inp.x).pin_memory() for _ in range(2)]
    x_seq = [xs[i & 1] for i in range(n)]
    o_seq = [ohs[i & 1] for i in range(n)]
    run = layer["e2e_fn"]
    pipe = HostPipeline(run, tuple(inp.x.shape), tuple(inp.x.shape), torch.bfloat16, dev)
    pipe.process(x_seq[:4], o_seq[:4])
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    pipe.process(x_seq, o_seq)
    e1.record()
    torch.cuda.synchronize()
    mc.check_device_status()
    same = all(torch.equal(o.view(torch.int16), layer["out"].cpu().view(torch.int16)) for o in ohs)
    # the same batches with the layer replaced by a device copy: what the host side of the
    # node (PCIe switches, host memory) lets N ranks move at the same time
    dist.barrier()
    copy_ms = copy_only_ms(tuple(inp.x.shape), dev, x_seq, o_seq)
    t = torch.tensor([e0.elapsed_time(e1) / n, 0.0 if same else 1.0, copy_ms], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, copy_ms = float(t[0].item()), float(t[2].item())
    nbytes = shape.T * shape.H * 2
    world = dist.get_world_size()
    return {"value": shape.T * world / (ms * 1e-3), "unit": "tokens/s",
            "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes, "ms_per_step": ms,
            "copy_only_ms_per_step": copy_ms,
            "copy_only_value": shape.T * world / (copy_ms * 1e-3),
            "batches": n, "matches_device_path": bool(t[1].item() == 0.0),
            "api": "hostpipe.HostPipeline over the expert-parallel layer call of ep.py "
                   "(pinned host batches per rank, copies overlapped with the layer)"}


def main():
    args = parse_args()
    if args.impl == "reference":
        return run_reference(args)
    return run_b200(args)


if __name__ == "__main__":
    sys.exit(main())
