#!/usr/bin/env python
"""Benchmark of the Algebraic-Transformer hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload attn|swiglu|norm|softmax|add_norm|loss_head|lm_small|lm_xl]
                    [--impl ours|reference] [--scaling strong|weak] [--no-extras]

Default workload ``attn``: causal rational attention forward+backward, bf16, B=8, H=16, S=4096, D=128 with
ALiBi.  With N ranks the 128 (batch, head) units are split into contiguous blocks of 128/N per rank (strong
scaling, no collective on the data path: the units are independent); ``--scaling weak`` gives every rank the
whole problem instead.  The line of the default workload also carries, under ``extra``, the second half of the
headline metric and the bandwidth-sweep configuration measured in the same process at the same N: the small
language model's training step (tokens/s, CUDA-graph replay and eager launches) and SwiGLU / mean-error norm /
rational softmax forward+backward in GB/s.  One JSON line is printed by rank 0.

``--impl reference`` times the CPU restatement of the reference's PyTorch path (the oracle) on the host cores
on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

L2_BYTES = 126 * 2 ** 20


# ------------------------------------------------------------------------------------------ helpers
def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a region is timed."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        return False

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def max_over_ranks(ms: float, world: int, device) -> float:
    if world == 1:
        return ms
    import torch.distributed as dist
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def launch_count() -> int:
    """Kernels launched so far by libfat_b200.so in this process (the library counts them itself)."""
    from fastalgebraictransformer_b200 import _lib
    return int(_lib.lib().fat_launch_count())


def barrier(world: int):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()


def time_steps(step, steps: int, warmup: int, world: int, device):
    """W untimed warm-ups, then exactly K steps between CUDA events on the launching stream; max over ranks."""
    for _ in range(warmup):
        step()
    torch.cuda.synchronize(device)
    barrier(world)
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize(device)
    barrier(world)
    return max_over_ranks(e0.elapsed_time(e1), world, device) / steps


def make_pipelined_e2e(device, host_inputs, compute):
    """End-to-end step over host buffers: every call uploads `host_inputs` (pinned) into one of two device buffer sets,
    runs `compute(device_inputs) -> results` (the public autograd API) and downloads the results into one of two pinned
    host sets.  The three stages run on three streams, so step i's upload, step i-1's arithmetic and step i-2's download
    overlap and share the two directions of the host link; the current stream waits for each download (the timing
    events sit there).  The first two calls also allocate the pinned result buffers: keep them in the warm-up."""
    dins = [[torch.empty_like(h, device=device) for h in host_inputs] for _ in range(2)]
    houts = [None, None]
    s_in, s_comp, s_out = (torch.cuda.Stream(device) for _ in range(3))
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_comp = [torch.cuda.Event() for _ in range(2)]       # arithmetic of the step that used buffer set i has finished
    ev_out = [torch.cuda.Event() for _ in range(2)]
    counter = [0]

    def step():
        i = counter[0] & 1
        counter[0] += 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_comp[i])                     # the step two back has read these device buffers
            for d, h in zip(dins[i], host_inputs):
                d.copy_(h, non_blocking=True)
            ev_in[i].record(s_in)
        with torch.cuda.stream(s_comp):
            s_comp.wait_event(ev_in[i])
            results = compute(dins[i])
            ev_comp[i].record(s_comp)
        if houts[i] is None:
            houts[i] = [torch.empty(r.shape, dtype=r.dtype).pin_memory() for r in results]
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_comp[i])
            s_out.wait_event(ev_out[i])                     # host set i is free again (its previous download is done)
            for h, d in zip(houts[i], results):
                h.copy_(d, non_blocking=True)
                d.record_stream(s_out)
            ev_out[i].record(s_out)
        torch.cuda.current_stream(device).wait_stream(s_out)

    return step

E2E_OVERLAP = "upload, arithmetic and download of consecutive steps on three streams, two buffer sets"


# ------------------------------------------------------------------------------------------ workloads
ATTN = dict(B=8, H=16, S=4096, D=128)


def attn_flops(B, H, S, D):
    """Causal-convention flops: forward 2 GEMMs, backward 5 GEMMs, each 2*S*S*D/2 per (b,h)."""
    fwd = 2.0 * B * H * S * S * D
    return fwd, 2.5 * fwd


def make_attn_inputs(cfg, seed, device=None, pin=False):
    g = torch.Generator().manual_seed(seed)
    shape = (cfg["B"], cfg["H"], cfg["S"], cfg["D"])
    ts = [torch.randn(*shape, generator=g, dtype=torch.float32).to(torch.bfloat16) for _ in range(4)]
    if pin:
        ts = [t.pin_memory() for t in ts]
    if device is not None:
        ts = [t.to(device) for t in ts]
    slopes = torch.tensor([2.0 ** (-8.0 * (i + 1) / cfg["H"]) for i in range(cfg["H"])], dtype=torch.float32)
    return ts, slopes


# DRAM bytes of the three backward launches of one step at B=2 (ncu, dram__bytes_read.sum + dram__bytes_write.sum):
# profiles/attention_bf16_B2_H16_S4096_D128.md, section "DRAM traffic per launch"; traffic grows in proportion to
# the (batch, head) units, so the full-size figure is this one scaled by units / 32.
ATTN_BWD_TRAFFIC_B2 = 570.6e6


def shard_batches(B: int, H: int, rank: int, world: int):
    """The block of the B*H independent (batch, head) units that `rank` owns when they are dealt out in contiguous blocks
    of B*H/world: returned as (first batch element, number of batch elements).  Blocks are whole batch elements (every rank
    keeps all heads, hence all ALiBi slopes), which needs world to divide B."""
    if B % world:
        raise SystemExit(f"splitting {B * H} (batch, head) units over {world} ranks in whole batch elements needs the "
                         f"batch ({B}) to be a multiple of the ranks")
    nb = B // world
    return rank * nb, nb


def bench_attn(args, rank, world, device):
    import fastalgebraictransformer_b200 as fat
    from fastalgebraictransformer_b200 import _lib, ops  # noqa: F401  (ops: loads the operator library)
    full = dict(ATTN, B=args.batch) if args.batch else dict(ATTN)
    strong = args.scaling == "strong" and world > 1
    lo, nb = shard_batches(full["B"], full["H"], rank, world) if strong else (0, full["B"])
    cfg = dict(full, B=nb)
    # every rank draws the whole problem from one seed and keeps its block, so the union over ranks is the 1-GPU input
    (q, k, v, go), slopes = make_attn_inputs(full, 1234 + 1 + (0 if strong else rank))
    if strong:
        q, k, v, go = (t[lo:lo + nb].contiguous() for t in (q, k, v, go))
    host_in = [t.pin_memory() for t in (q, k, v, go)]
    q, k, v, go = (t.to(device) for t in host_in)
    slopes = slopes.to(device)
    scale = 1.0 / math.sqrt(cfg["D"])
    fwd_flops, bwd_flops = attn_flops(**cfg)              # this rank's share
    total_flops = (fwd_flops + bwd_flops) * world
    path = _lib.lib().fat_attn_select_path(cfg["S"], cfg["D"], _lib.BF16, 1, 1, 1)

    state = {}

    def fwd():
        state["out"], state["L"], state["lo"] = torch.ops.algebraic.attn_fwd(q, k, v, slopes, scale, True, 1e-6, 0, False)

    def bwd():
        state["grads"] = fat.rational_attention_backward(q, k, v, state["out"], state["L"], go, slopes, scale,
                                                         output_lo=state["lo"])

    def step():
        fwd(); bwd()

    for _ in range(2):
        step()
    n0 = launch_count()
    step()
    launches_per_step = launch_count() - n0
    # The timed steps are replays of one captured step: with the units split over 8 GPUs a step lasts 0.4 ms, and eight
    # processes issuing four launches (and their allocations) per step from one host were no longer always ahead of the GPU.
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    with ClockSampler(device.index) as clocks:
        ms = time_steps(graph.replay, args.steps, args.warmup, world, device)
    fat.check_device_status()
    parts = []
    for fn in (fwd, bwd):                                 # the two halves of the step, each replayed from its own capture
        fn()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            fn()
        parts.append(time_steps(gr.replay, max(3, args.steps // 2), 1, world, device))
        del gr
    ms_fwd, ms_bwd = parts
    # the same step back to back for about a second: the regime the sustained peak is defined on
    sus_steps = max(args.steps, int(1.2e3 / max(ms, 1e-3))) if not args.batch else args.steps    # (profiling case: kept short)
    with ClockSampler(device.index) as sus_clocks:
        ms_sus = time_steps(graph.replay, sus_steps, 1, world, device)

    # end to end through the public autograd API with host buffers (pinned), copies inside the timed region
    def e2e_compute(d):
        dq, dk, dv = (t.detach().requires_grad_(True) for t in d[:3])
        out = fat.rational_attention(dq, dk, dv, slopes, scale)
        out.backward(d[3])
        return (out.detach(), dq.grad, dk.grad, dv.grad)

    e2e_step = make_pipelined_e2e(device, host_in, e2e_compute)
    e2e_steps = max(4, min(args.steps, 8))
    ms_e2e = time_steps(e2e_step, e2e_steps, 2, world, device)
    nbytes = host_in[0].numel() * host_in[0].element_size()

    peaks = measured_peaks()
    tfl = total_flops / (ms * 1e-3) / 1e12
    tfl_sus = total_flops / (ms_sus * 1e-3) / 1e12
    bwd_tfl = bwd_flops / (ms_bwd * 1e-3) / 1e12
    res = {
        "metric": "rational_attention_fwd_bwd_tflops", "value": tfl, "unit": "TFLOP/s",
        "ms_per_step": ms, "dtype": "bf16", "scaling": "strong" if strong or world == 1 else "weak",
        "config": {"workload": f"rational_attention fwd+bwd causal ALiBi bf16 B={full['B']} H=16 S=4096 D=128 "
                               + ("(headline configuration)" if full["B"] == 8 else "(REDUCED batch: profiling case, not a bench value)")
                               + (f", split over the ranks in blocks of {cfg['B'] * cfg['H']} (batch, head) units" if strong
                                  else (", the whole problem on every rank" if world > 1 else "")),
                   "units_per_gpu": cfg["B"] * cfg["H"], "shard": "batch x head, contiguous blocks, no collective",
                   "kernel_path": "tcgen05" if path == 2 else "simt", "launch": "each timed step replays one captured step (CUDA graph)", "l2": "inputs (4 x 134 MB at 128 units) exceed the 126 MB L2"
                   if cfg["B"] * cfg["H"] >= 128 else f"inputs of this rank: 4 x {nbytes / 1e6:.0f} MB (the step also writes 5 tensors of that size)",
                   "ms_fwd": ms_fwd, "ms_bwd": ms_bwd,
                   "pct_of_bf16_peak": 100.0 * tfl / world / peaks["bf16_tflops"],
                   "sustained_ms": ms_sus, "sustained_steps": sus_steps, "sustained_tflops": tfl_sus,
                   "sustained_frac_of_sustained_peak": tfl_sus / world / peaks["bf16_tflops_sustained"],
                   "sustained_clocks": sus_clocks.summary()},
        "e2e": {"value": total_flops / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s",
                "h2d_bytes_per_step": 4 * nbytes, "d2h_bytes_per_step": 4 * nbytes, "ms_per_step": ms_e2e,
                "overlap": E2E_OVERLAP},
        "gpu_launches": launches_per_step * args.steps,
        "gpu_launches_how": "fat_launch_count() of libfat_b200.so around one step, times the steps of the timed region",
        "roofline": {"bound": "tensor", "kernel": "attention backward (prepare + fused d_k/d_v/d_q + d_q convert launches)", "achieved": bwd_tfl,
                     "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": bwd_tfl / peaks["bf16_tflops"],
                     "traffic": ATTN_BWD_TRAFFIC_B2 * cfg["B"] * cfg["H"] / 32,
                     "traffic_source": "profiles/attention_bf16_B2_H16_S4096_D128.md (B=2 capture, scaled by the units)",
                     "peak_source": peaks["source"] + " (burst cuBLAS bf16)",
                     "fwd_achieved": fwd_flops / (ms_fwd * 1e-3) / 1e12,
                     "step_frac": tfl / world / peaks["bf16_tflops"]},
        "clocks": clocks.summary(),
    }
    del q, k, v, go, host_in, state, e2e_step, graph
    torch.cuda.empty_cache()
    return res


# `bytes`: algorithmic bytes of one forward+backward (2-byte elements; every tensor moved once):
#   swiglu   fwd gate, value in, out out (3) + bwd d_out, gate, value in, d_gate, d_value out (5) = 8 passes
#   norm     fwd x in, y out (2) + bwd d_out, x in, d_x out (3) = 5 passes (+ weight, means, d_weight: KBs)
#   softmax  fwd x in, p out (2) + bwd d_out, x in, d_x out (3) = 5 passes: the backward recomputes p from x instead
#            of reading the saved p (the variant that moves 3 tensors in the backward)
# `traffic`: dram__bytes_read.sum + dram__bytes_write.sum of one step's launches at these shapes, from
# profiles/fused_ops_bf16_config3.md (section "DRAM traffic per step")
FUSED = {
    "swiglu": dict(rows=16384, cols=8192, bytes=8 * 16384 * 8192 * 2, traffic=2068e6),
    "norm": dict(rows=16384, cols=4096, bytes=5 * 16384 * 4096 * 2, traffic=595e6),
    "softmax": dict(rows=4096, cols=4096, bytes=5 * 4096 * 4096 * 2, traffic=106e6),
    # residual addition fused with the norm: forward x, residual in, sum, y out; backward d_y, d_sum_in, sum in, d_sum out
    "add_norm": dict(rows=16384, cols=4096, bytes=8 * 16384 * 4096 * 2, traffic=None),
    # loss head of the small LM: logits [8, 1024, 32000] read once, their gradient written once
    "loss_head": dict(rows=8 * 1024, cols=32000, bytes=2 * 8 * 1024 * 32000 * 2, traffic=None),
    # one decode step of a key/value-cached generate(): every (batch, head) pair reads its 4096 cached key rows and value
    # rows once (the query, the appended rows and the output are KBs); shape of the headline attention configuration
    # (traffic: profiles/attention_decode_bf16_B8_H16_T4096_D128.md)
    "decode": dict(rows=8 * 16 * 4096, cols=128, bytes=2 * 8 * 16 * 4096 * 128 * 2, traffic=272.7e6, B=8, H=16, cap=4096),
}
FUSED_TRAFFIC_SOURCE = "profiles/fused_ops_bf16_config3.md"


def fused_inputs(name, gen, device=None, rows=None):
    """One input set of a fused-op workload (bf16).  `gen` is a torch.Generator on `device` (or on the CPU)."""
    cfg = FUSED[name]
    shape = (rows or cfg["rows"], cfg["cols"])
    dev = device if device is not None else "cpu"

    def rnd(std=1.0):
        return (torch.randn(*shape, generator=gen, device=dev) * std).to(torch.bfloat16)

    def weight():
        return (1 + 0.1 * torch.randn(cfg["cols"], generator=gen, device=dev)).to(torch.bfloat16)

    if name == "swiglu":
        return (rnd(), rnd(), rnd())                                          # gate, value, d_out
    if name == "norm":
        return (rnd(), weight(), rnd())                                       # x, weight, d_out
    if name == "add_norm":
        return (rnd(), weight(), rnd(), rnd(), rnd())                         # x, weight, residual, d_y, d_h
    if name == "decode":
        B, H, cap, D = cfg["B"], cfg["H"], (rows or cfg["rows"]) // (cfg["B"] * cfg["H"]), cfg["cols"]
        new = [torch.randn(B, H, D, generator=gen, device=dev).to(torch.bfloat16) for _ in range(3)]    # q, k_new, v_new
        caches = [torch.randn(B, H, cap, D, generator=gen, device=dev).to(torch.bfloat16) for _ in range(2)]
        return (*new, *caches, torch.full((B,), cap - 1, dtype=torch.int32, device=dev))
    if name == "loss_head":
        labels = torch.randint(0, cfg["cols"], (8, shape[0] // 8), generator=gen, device=dev)
        return (rnd(2.0).view(8, shape[0] // 8, cfg["cols"]), labels)
    return (rnd(math.sqrt(2.0)), rnd())                                       # softmax: scores ~ N(0, 2), d_out


def run_fused(name, steps, warmup, rank, world, device, with_e2e=True):
    import fastalgebraictransformer_b200 as fat
    from fastalgebraictransformer_b200 import ops  # noqa: F401  (loads the operator library)
    cfg = FUSED[name]
    g = torch.Generator(device=device).manual_seed(1234 + 2 + rank)
    shape = (cfg["rows"], cfg["cols"])
    nset = 1 if name != "softmax" else 6        # softmax tensors (33.5 MB) fit in L2: rotate 6 sets (> 126 MB each pass)
    sets = [fused_inputs(name, g, device) for _ in range(nset)]
    it = [0]
    alg = torch.ops.algebraic
    slopes = fat.compute_alibi_slopes(cfg["H"]).to(device) if name == "decode" else None

    def step():
        s = sets[it[0] % nset]; it[0] += 1
        if name == "swiglu":
            alg.swiglu_fwd(s[0], s[1]); alg.swiglu_bwd(s[2], s[0], s[1])
        elif name == "norm":
            y, mean = alg.norm_fwd(s[0], s[1], 1e-6)
            alg.norm_bwd(s[2], s[0], s[1], mean, 1e-6)
        elif name == "add_norm":
            h, y, mean = alg.add_norm_fwd(s[0], s[2], s[1], 1e-6)
            alg.add_norm_bwd(s[3], s[4], h, s[1], mean, 1e-6)
        elif name == "loss_head":
            alg.shifted_ce_fwd(s[0], s[1], -100)
        elif name == "decode":
            alg.attn_decode(s[0], s[1], s[2], s[3], s[4], s[5], slopes, ATTN["D"] ** -0.5, 1e-6)
        else:
            alg.softmax_fwd(s[0], 1e-6); alg.softmax_bwd(s[1], s[0], 1e-6)

    # These kernels last 10-100 us, less than the host needs to issue one, so each step is captured once in
    # a CUDA graph (one graph per rotating input set) and the timed region replays the graphs.
    side = torch.cuda.Stream(device)
    side.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(side):
        for _ in range(nset):
            step()
    torch.cuda.current_stream(device).wait_stream(side)
    graphs = []
    launches_per_step = 0
    for _ in range(nset):
        gr = torch.cuda.CUDAGraph()
        n0 = launch_count()
        with torch.cuda.graph(gr):
            step()
        launches_per_step = launch_count() - n0
        graphs.append(gr)
    gi = [0]

    def replay():
        graphs[gi[0] % nset].replay(); gi[0] += 1

    with ClockSampler(device.index) as clocks:
        ms = time_steps(replay, steps, warmup, world, device)
    peaks = measured_peaks()
    gbs = cfg["bytes"] * world / (ms * 1e-3) / 1e9
    res = {
        "metric": f"rational_{name}_fwd_bwd_gbs" if name != "decode" else "rational_attention_decode_gbs",
        "value": gbs, "unit": "GB/s", "ms_per_step": ms, "dtype": "bf16",
        "scaling": "weak",
        "config": {"workload": f"{name} fwd+bwd bf16 [{cfg['rows']},{cfg['cols']}] per GPU (bandwidth-sweep configuration)" if name != "decode" else
                   f"attention decode step bf16: {cfg['B']} x {cfg['H']} (batch, head) pairs, {cfg['cap']} cached tokens of {cfg['cols']} per GPU",
                   "algorithmic_bytes_per_step": cfg["bytes"],
                   "launch": "each step replayed from a CUDA graph",
                   "l2": "tensors exceed L2" if nset == 1 else f"{nset} rotating input sets (each pass touches > 126 MB before reuse)"},
        "gpu_launches": launches_per_step * steps,
        "gpu_launches_how": "fat_launch_count() of libfat_b200.so around the capture of one step, times the replays of the timed region",
        "roofline": {"bound": "hbm", "kernel": f"{name} fwd+bwd" if name != "decode" else "attn_decode_kernel", "achieved": gbs / world, "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": gbs / world / peaks["hbm_gbs"], "traffic": cfg["traffic"],
                     "traffic_source": (("profiles/attention_decode_bf16_B8_H16_T4096_D128.md" if name == "decode" else FUSED_TRAFFIC_SOURCE)
                                        if cfg["traffic"] else None),
                     "peak_source": peaks["source"] + " (copy bandwidth)"},
        "clocks": clocks.summary(),
    }
    if with_e2e:
        # end to end: host (pinned) -> device -> forward+backward through the autograd API -> host
        # (decode: the caches stay on the device, which is what a cache is for; the new token's rows go up, its output comes back)
        hs = [t.detach().cpu().pin_memory() for t in (sets[0][:3] if name == "decode" else sets[0])]

        def e2e_compute(dd):
            d = [t.detach() for t in dd]
            if name == "swiglu":
                a, b = d[0].requires_grad_(True), d[1].requires_grad_(True)
                o = fat.rational_swiglu(a, b); o.backward(d[2]); return (o.detach(), a.grad, b.grad)
            if name == "norm":
                a, w = d[0].requires_grad_(True), d[1].requires_grad_(True)
                o = fat.mean_error_norm(a, w); o.backward(d[2]); return (o.detach(), a.grad)
            if name == "decode":
                return (alg.attn_decode(d[0], d[1], d[2], sets[0][3], sets[0][4], sets[0][5], slopes, ATTN["D"] ** -0.5, 1e-6),)
            if name == "loss_head":
                a = d[0].requires_grad_(True)
                loss = fat.shifted_cross_entropy(a, d[1]); loss.backward(); return (loss.detach().reshape(1), a.grad)
            if name == "add_norm":
                a, w, r = d[0].requires_grad_(True), d[1].requires_grad_(True), d[2].requires_grad_(True)
                h, y = fat.add_mean_error_norm(a, r, w)
                torch.autograd.backward([h, y], [d[4], d[3]]); return (h.detach(), y.detach(), a.grad)
            a = d[0].requires_grad_(True)
            o = fat.rational_softmax(a); o.backward(d[1]); return (o.detach(), a.grad)

        e2e_step = make_pipelined_e2e(device, hs, e2e_compute)
        ms_e2e = time_steps(e2e_step, 6, 2, world, device)
        n_out = {"swiglu": 3, "norm": 2, "softmax": 2, "add_norm": 3, "loss_head": 1, "decode": 1}[name]
        out_bytes = n_out * shape[0] * shape[1] * 2 if name != "decode" else cfg["B"] * cfg["H"] * cfg["cols"] * 2
        res["e2e"] = {"value": cfg["bytes"] * world / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s",
                      "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in hs),
                      "d2h_bytes_per_step": out_bytes, "ms_per_step": ms_e2e, "overlap": E2E_OVERLAP}
    del sets, graphs
    torch.cuda.empty_cache()
    return res


LM = {
    "lm_small": dict(vocab_size=32000, d_model=768, n_head=12, n_layers=12, d_ffn=None, batch=8, seq=1024),
    "lm_xl": dict(vocab_size=50000, d_model=2048, n_head=16, n_layers=24, d_ffn=5504, batch=4, seq=2048),
}


def run_lm(name, steps, warmup, rank, world, device, graph=True, eager_steps=0, keep_logits=True):
    """One training step (forward, loss, backward with DDP's gradient all-reduce when world > 1, fused AdamW) of the
    named model.  graph: capture the step in a CUDA graph and time its replays; eager_steps > 0: also time that many
    steps issued launch by launch, as a user of the module would (reported as `eager_ms`).  keep_logits: the step is the
    reference-shaped call `model(ids, labels=labels)`, which returns the [B,T,V] logits; otherwise it asks for the loss only
    (`return_logits=False`: the head GEMM and the loss run one sequence at a time, the logits never exist)."""
    from fastalgebraictransformer_b200 import AlgebraicTransformerLM
    cfg = LM[name]
    torch.manual_seed(1234 + 3)
    model = AlgebraicTransformerLM(cfg["vocab_size"], cfg["d_model"], cfg["n_head"], cfg["n_layers"], d_ffn=cfg["d_ffn"],
                                   block_size=cfg["seq"], dropout=0.0).to(device).to(torch.bfloat16).train()
    n_params = sum(p.numel() for p in model.parameters())
    net = model
    if world > 1:
        from torch.nn.parallel import DistributedDataParallel as DDP
        ddp_stream = torch.cuda.Stream(device)            # DDP is built on a side stream so that its step can be captured
        ddp_stream.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(ddp_stream):
            net = DDP(model, device_ids=[device.index], gradient_as_bucket_view=True, bucket_cap_mb=64)
        torch.cuda.current_stream(device).wait_stream(ddp_stream)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4, fused=True, capturable=True)
    g = torch.Generator().manual_seed(1234 + 3 + rank)
    hids = torch.randint(0, cfg["vocab_size"], (cfg["batch"], cfg["seq"]), generator=g).pin_memory()
    hlab = torch.randint(0, cfg["vocab_size"], (cfg["batch"], cfg["seq"]), generator=g).pin_memory()
    ids, lab = hids.to(device), hlab.to(device)
    last = {}

    def step():
        opt.zero_grad(set_to_none=True)
        _, loss = net(ids, labels=lab, return_logits=keep_logits)
        loss.backward()
        opt.step()
        last["loss"] = loss

    def e2e_step():
        i, l = hids.to(device, non_blocking=True), hlab.to(device, non_blocking=True)
        opt.zero_grad(set_to_none=True)
        _, loss = net(i, labels=l, return_logits=keep_logits)
        loss.backward()
        opt.step()
        last["loss_host"] = loss.item()

    # The whole step (forward, loss, backward with DDP's bucketed all-reduces, AdamW) is captured once in a CUDA graph,
    # because issuing its ~1000 launches from Python takes longer than executing them.  DDP wants 11 eager steps on a
    # side stream before a capture.
    launch = "eager"
    timed = step
    side = torch.cuda.Stream(device)
    side.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(side):
        for _ in range(3 if world == 1 else 11):
            step()
    torch.cuda.current_stream(device).wait_stream(side)
    n0 = launch_count()
    step()
    launches_per_step = launch_count() - n0
    eager_ms = None
    if eager_steps > 0:
        eager_ms = time_steps(step, eager_steps, 2, world, device)
    if graph:
        try:
            graph_obj = torch.cuda.CUDAGraph()
            opt.zero_grad(set_to_none=True)
            with torch.cuda.graph(graph_obj):
                _, gloss = net(ids, labels=lab, return_logits=keep_logits)
                gloss.backward()
                opt.step()
            last["loss"] = gloss

            def timed():
                graph_obj.replay()
            launch = "cuda graph replay"
        except Exception as exc:      # noqa: BLE001 - fall back to eager launches, say so in the output
            print(f"graph capture failed ({exc!r}); timing eager launches", file=sys.stderr)
            torch.cuda.synchronize(device)
            timed, launch = step, "eager (graph capture failed)"
    with ClockSampler(device.index) as clocks:
        ms = time_steps(timed, steps, warmup, world, device)
    ms_e2e = time_steps(e2e_step, max(2, steps // 2), 1, world, device)
    tokens = cfg["batch"] * cfg["seq"] * world
    peaks = measured_peaks()
    d_head = cfg["d_model"] // cfg["n_head"]
    attn = cfg["n_layers"] * 3.5 * 2 * cfg["batch"] * cfg["n_head"] * cfg["seq"] ** 2 * d_head
    flops = 6.0 * (n_params) * cfg["batch"] * cfg["seq"] + attn
    res = {
        "metric": "lm_train_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms,
        "dtype": "bf16", "scaling": "weak",
        "config": {"workload": f"AlgebraicTransformerLM {name} training step (fwd+loss+bwd+AdamW), bf16, "
                               f"batch {cfg['batch']} x seq {cfg['seq']} per GPU", "params": n_params,
                   "parallelism": f"dp{world}", "launch": launch, "loss": float(last["loss"].item()),
                   "loss_head": "full logits kept" if keep_logits else "one sequence at a time, logits never materialised",
                   "peak_memory_gb": torch.cuda.max_memory_allocated(device) / 1e9,
                   "eager_ms": eager_ms, "eager_tokens_per_s": tokens / (eager_ms * 1e-3) if eager_ms else None},
        "e2e": {"value": tokens / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": 2 * hids.numel() * 8,
                "d2h_bytes_per_step": 4, "ms_per_step": ms_e2e, "launch": "eager"},
        "gpu_launches": launches_per_step * steps,
        "gpu_launches_how": "fat_launch_count() of libfat_b200.so around one eager step, times the steps of the timed region "
                            "(the GEMMs, AdamW and NCCL launches of the step are library kernels and not counted)",
        "roofline": {"bound": "tensor", "kernel": "whole step (GEMMs in cuBLAS + this library's kernels)",
                     "achieved": flops / (ms * 1e-3) / 1e12, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                     "frac": flops / (ms * 1e-3) / 1e12 / peaks["bf16_tflops_sustained"], "traffic": None,
                     "peak_source": peaks["source"] + " (sustained cuBLAS bf16)"},
        "clocks": clocks.summary(),
    }
    del net, model, opt
    torch.cuda.empty_cache()
    return res


def run_generate(steps, warmup, rank, world, device):
    """Decode steps of the small LM over a key/value cache: every sequence gets one new token per step.  The prompt
    (512 tokens per sequence) is run once, untimed; the timed region replays the captured decode step (all layers: norms,
    projections, cache append + attention, feed-forward, head).  Next to it: the same step issued launch by launch, and what
    the reference's generate() does for one token at this length, a full forward over the prefix (algebraic_model.py:239-265)."""
    from fastalgebraictransformer_b200 import AlgebraicTransformerLM, ops  # noqa: F401
    cfg = LM["lm_small"]
    batch, prompt = 8, 512
    capacity = prompt + warmup + 2 * steps + 64
    torch.manual_seed(1234 + 3)
    model = AlgebraicTransformerLM(cfg["vocab_size"], cfg["d_model"], cfg["n_head"], cfg["n_layers"], d_ffn=cfg["d_ffn"],
                                   block_size=capacity, dropout=0.0).to(device).to(torch.bfloat16).eval()
    g = torch.Generator(device=device).manual_seed(1234 + 3 + rank)
    ids = torch.randint(0, cfg["vocab_size"], (batch, prompt), generator=g, device=device)
    token = torch.randint(0, cfg["vocab_size"], (batch, 1), generator=g, device=device)
    with torch.no_grad():
        cache = model.new_cache(batch, capacity)
        model.forward_cached(ids, cache)
        n0 = launch_count()
        model.forward_cached(token, cache)                           # one step launch by launch (also the warm-up of the capture)
        launches_per_step = launch_count() - n0
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(device)
        e0.record()
        for _ in range(8):
            model.forward_cached(token, cache)
        e1.record()
        torch.cuda.synchronize(device)
        eager_ms = e0.elapsed_time(e1) / 8
        seen = cache.seen
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            logits = model.forward_cached(token, cache)
        cache.seen = seen

        def step():
            graph.replay()
            cache.seen += 1

        with ClockSampler(device.index) as clocks:
            ms = time_steps(step, steps, warmup, world, device)
        n_ctx = cache.seen
        # the reference's way: one forward over the whole prefix per new token
        full = torch.randint(0, cfg["vocab_size"], (batch, n_ctx), generator=g, device=device)
        ms_recompute = time_steps(lambda: model(full), 5, 2, world, device)
        # end to end: prompt up, generate(), tokens down
        host_prompt = ids.cpu().pin_memory()
        new_tokens = 64

        def e2e_step():
            out = model.generate(host_prompt.to(device, non_blocking=True), new_tokens, top_k=1)
            return out.cpu()

        ms_e2e = time_steps(e2e_step, 2, 1, world, device)
    peaks = measured_peaks()
    params = sum(p.numel() for n, p in model.named_parameters())
    kv_bytes = 2 * cfg["n_layers"] * batch * cfg["d_model"] * n_ctx * 2            # keys and values of every layer, read once
    step_bytes = params * 2 + kv_bytes                                              # plus every weight, read once
    tok_s = batch * world / (ms * 1e-3)
    gbs = step_bytes / (ms * 1e-3) / 1e9
    res = {
        "metric": "lm_generate_tokens_per_s", "value": tok_s, "unit": "tokens/s", "ms_per_step": ms, "dtype": "bf16", "scaling": "weak",
        "config": {"workload": f"lm_small decode: {batch} sequences per GPU, one new token each per step, {prompt}-token prompts, "
                               f"context {n_ctx - steps}..{n_ctx} tokens during the timed steps",
                   "params": params, "launch": "decode step replayed from a CUDA graph (cached lengths live on the device)",
                   "eager_ms": eager_ms, "reference_way_ms_per_token": ms_recompute,
                   "reference_way": "a forward over the whole prefix for every new token (what generate() does without a cache), same model and kernels",
                   "algorithmic_bytes_per_step": step_bytes},
        "e2e": {"value": batch * new_tokens * world / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": host_prompt.numel() * 8, "d2h_bytes_per_step": batch * (prompt + new_tokens) * 8,
                "what": f"model.generate(prompt from pinned host memory, {new_tokens} new tokens, greedy), prompt pass included, tokens read back"},
        "gpu_launches": launches_per_step * steps,
        "gpu_launches_how": "fat_launch_count() of libfat_b200.so around one decode step, times the replays of the timed region",
        "roofline": {"bound": "hbm", "kernel": "decode step (all launches: this library's and the cuBLAS projections)", "achieved": gbs,
                     "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"], "traffic": None,
                     "peak_source": peaks["source"] + " (copy bandwidth)"},
        "clocks": clocks.summary(),
    }
    del model, cache, graph, logits
    torch.cuda.empty_cache()
    return res


def run_extras(args, rank, world, device):
    """Compact records of the other configurations at the same N, for the default workload's line: the small LM's
    training step, the three bandwidth-sweep operators and the decode step over a key/value cache.  A failure in one is recorded, not raised."""
    extra = {}

    def compact(r):
        out = {"value": r["value"], "unit": r["unit"], "ms_per_step": r["ms_per_step"], "scaling": r["scaling"],
               "frac_of_peak": r["roofline"]["frac"], "peak": r["roofline"]["peak"], "workload": r["config"]["workload"],
               "launch": r["config"].get("launch"), "gpu_launches_per_step": r["gpu_launches"] // max(1, r["_steps"]),
               "clocks": r["clocks"]}
        for k in ("eager_ms", "eager_tokens_per_s", "params", "parallelism"):
            if r["config"].get(k) is not None:
                out[k] = r["config"][k]
        return out

    for name in ("swiglu", "norm", "softmax", "decode"):
        try:
            r = run_fused(name, 50, 5, rank, world, device, with_e2e=False)
            r["_steps"] = 50
            extra[name] = compact(r)
        except Exception as exc:      # noqa: BLE001
            extra[name] = {"error": repr(exc)[:300]}
    try:
        r = run_lm("lm_small", 20, 3, rank, world, device, graph=True, eager_steps=10)
        r["_steps"] = 20
        extra["lm_small"] = compact(r)
    except Exception as exc:      # noqa: BLE001
        extra["lm_small"] = {"error": repr(exc)[:300]}
    return extra


# ------------------------------------------------------------------------------------------ CPU arm
def use_all_host_threads():
    """torchrun exports OMP_NUM_THREADS=1; the CPU arm is meant to use every core it may run on."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def cpu_sample(workload: str):
    """A function that runs ONE bounded sample of `workload` through the oracle (the CPU restatement of the reference's
    PyTorch path, float32, autograd for the gradients), the amount of the metric's unit it stands for, and a
    description.  Returned as (run, amount, unit, what)."""
    from oracle import oracle
    if workload == "attn":
        heads = 1
        cfg = dict(ATTN, B=1, H=heads)
        (q, k, v, go), slopes = make_attn_inputs(cfg, 1234 + 1)
        q, k, v, go = (t.float() for t in (q, k, v, go))
        scale = 1.0 / math.sqrt(cfg["D"])
        f, b = attn_flops(**cfg)
        return (lambda: oracle.rational_attention_grads(q, k, v, go, slopes[:heads], scale), (f + b) / 1e12, "TFLOP/s",
                f"{heads} of the 128 (batch, head) units (S=4096, D=128), flops in the same causal convention")
    if workload in ("swiglu", "norm", "softmax", "add_norm"):
        cfg = FUSED[workload]
        rows = {"swiglu": 2048, "norm": 4096, "softmax": 4096, "add_norm": 4096}[workload]
        ins = [t.float() for t in fused_inputs(workload, torch.Generator().manual_seed(1234 + 2), rows=rows)]
        amount = cfg["bytes"] * rows / cfg["rows"] / 1e9
        what = f"rows 0..{rows - 1} of the [{cfg['rows']},{cfg['cols']}] tensors upcast to float32; bytes counted as for the bf16 kernels"
        if workload == "swiglu":
            return (lambda: oracle.autograd_grads(oracle.rational_swiglu, ins[:2], ins[2]), amount, "GB/s", what)
        if workload == "norm":
            return (lambda: oracle.autograd_grads(oracle.mean_error_norm, ins[:2], ins[2]), amount, "GB/s", what)
        if workload == "add_norm":
            def run():
                leaves = [t.detach().clone().requires_grad_(True) for t in (ins[0], ins[2], ins[1])]
                h, y = oracle.add_mean_error_norm(*leaves)
                torch.autograd.backward([h, y], [ins[4], ins[3]])
            return (run, amount, "GB/s", what)
        return (lambda: oracle.autograd_grads(oracle.rational_softmax, ins[:1], ins[1]), amount, "GB/s", what)
    if workload == "decode":
        cfg = FUSED[workload]
        q, _, _, kc, vc, _ = fused_inputs(workload, torch.Generator().manual_seed(1234 + 2))
        q, kc, vc = q.float(), kc.float(), vc.float()
        slopes = oracle.compute_alibi_slopes(cfg["H"])
        return (lambda: oracle.rational_attention_last_row(q, kc, vc, slopes, cfg["cols"] ** -0.5), cfg["bytes"] / 1e9, "GB/s",
                "the whole step (128 (batch, head) pairs x 4096 cached tokens) upcast to float32; bytes counted as for the bf16 kernel")
    if workload == "loss_head":
        cfg = FUSED[workload]
        logits, labels = fused_inputs(workload, torch.Generator().manual_seed(1234 + 2), rows=8 * 128)
        logits = logits.float()

        def run():
            x = logits.detach().clone().requires_grad_(True)
            oracle.shifted_cross_entropy(x, labels).backward()
        return (run, cfg["bytes"] / 8 / 1e9, "GB/s", "8 sequences of 128 of the 1024 positions, float32")
    if workload == "generate":
        from fastalgebraictransformer_b200 import AlgebraicTransformerLM
        cfg = LM["lm_small"]
        torch.manual_seed(1234 + 3)
        model = AlgebraicTransformerLM(cfg["vocab_size"], cfg["d_model"], cfg["n_head"], cfg["n_layers"], d_ffn=cfg["d_ffn"],
                                       block_size=1024, dropout=0.0)
        state = {k: v.detach().float() for k, v in model.state_dict().items()}
        ids = torch.randint(0, cfg["vocab_size"], (1, 512), generator=torch.Generator().manual_seed(1234 + 3))

        def run():
            with torch.no_grad():
                oracle.lm_forward(state, ids, cfg["n_head"])
        return (run, 1.0, "tokens/s", "one new token of ONE sequence the reference's way: a float32 forward over its 512-token prefix "
                "(algebraic_model.py:239-265; the GPU arm advances 8 sequences per step)")
    if workload in LM:
        from fastalgebraictransformer_b200 import AlgebraicTransformerLM
        cfg = LM[workload]
        seq = cfg["seq"] if workload == "lm_small" else 512
        torch.manual_seed(1234 + 3)
        model = AlgebraicTransformerLM(cfg["vocab_size"], cfg["d_model"], cfg["n_head"], cfg["n_layers"], d_ffn=cfg["d_ffn"],
                                       block_size=cfg["seq"], dropout=0.0)
        state = {k: v.detach().float() for k, v in model.state_dict().items()}
        g = torch.Generator().manual_seed(1234 + 3)
        ids = torch.randint(0, cfg["vocab_size"], (1, seq), generator=g)
        lab = torch.randint(0, cfg["vocab_size"], (1, seq), generator=g)
        what = (f"1 sequence of {seq} tokens (of the {cfg['batch']} x {cfg['seq']} per GPU): forward, loss and backward in float32, "
                "no optimizer step" + ("" if seq == cfg["seq"] else "; REDUCED sequence length: the full one needs ~25 GB of S x S temporaries"))
        return (lambda: oracle.lm_loss_and_grads(state, ids, lab, cfg["n_head"]), float(seq), "tokens/s", what)
    raise SystemExit(f"no CPU sample for workload {workload}")


REF_METRIC = {"attn": "rational_attention_fwd_bwd_tflops", "lm_small": "lm_train_tokens_per_s", "lm_xl": "lm_train_tokens_per_s",
              "decode": "rational_attention_decode_gbs", "generate": "lm_generate_tokens_per_s"}


def cpu_baseline(workload: str, budget_s: float = 10.0, max_passes: int = 64):
    """The oracle on all host threads on a bounded sample of the workload: mean over passes worth ~budget_s."""
    cores = use_all_host_threads()
    run, amount, unit, what = cpu_sample(workload)
    run()                                                            # warm-up / sizing pass
    total, n = 0.0, 0
    while total < budget_s and n < max_passes:
        t0 = time.perf_counter()
        run()
        total += time.perf_counter() - t0; n += 1
    sec = total / n
    return {"value": amount / sec, "unit": unit, "cores": cores, "kind": "port",
            "sample": f"oracle (plain PyTorch on the CPU, float32) on {what}; mean of {n} passes of {sec:.2f} s"}


def run_reference(args, rank, world):
    """The reference arm: the CPU restatement of the reference's PyTorch path, timed step by step on rank 0."""
    if rank != 0:
        return None
    cores = use_all_host_threads()
    run, amount, unit, what = cpu_sample(args.workload)
    run()                                                            # untimed
    for _ in range(max(0, args.warmup - 1)):
        run()
    times = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        run()
        times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    val = amount / sec
    base = {"value": val, "unit": unit, "cores": cores, "kind": "port", "sample": f"each step = {what}"}
    metric = REF_METRIC.get(args.workload, f"rational_{args.workload}_fwd_bwd_gbs")
    return {
        "impl": "reference", "metric": metric, "value": val, "unit": unit,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "strong" if args.workload == "attn" else "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: CPU restatement of the reference's PyTorch path on a bounded sample "
                               f"of the configuration the GPU arm runs ({what})"},
        "cpu_baseline": base,
        "e2e": {"value": val, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


# ------------------------------------------------------------------------------------------ main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="attn", choices=["attn", "swiglu", "norm", "softmax", "add_norm", "loss_head", "decode", "generate", "lm_small", "lm_xl"])
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="attn workload on N > 1 ranks: split the 128 (batch, head) units over the ranks (strong, default) "
                         "or give every rank all of them (weak)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="attn workload: leave out the LM / bandwidth-sweep records")
    ap.add_argument("--batch", type=int, default=0,
                    help="attn workload: override the batch size (profiling captures use a smaller case)")
    ap.add_argument("--no-graph", action="store_true", help="LM workloads: time eager launches instead of a CUDA graph")
    ap.add_argument("--no-logits", action="store_true",
                    help="LM workloads: the step asks for the loss only (return_logits=False) instead of the reference-shaped call")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank, world, local = dist_env()

    if args.impl == "reference":
        line = run_reference(args, rank, world)
        if line is not None:
            print(json.dumps(line), flush=True)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU implementation of the product path)")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    extras = args.workload == "attn" and not args.no_extras and not args.batch
    if world > 1:
        import torch.distributed as dist
        if (args.workload in LM and not args.no_graph) or extras:
            # the DDP step is captured in a CUDA graph: the watchdog must not poll work objects captured there
            os.environ.setdefault("TORCH_NCCL_ASYNC_ERROR_HANDLING", "0")
        dist.init_process_group("nccl", device_id=device)
    if world != args.gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE={world}; using WORLD_SIZE", file=sys.stderr)

    if args.workload == "attn":
        res = bench_attn(args, rank, world, device)
        if extras:
            res["extra"] = run_extras(args, rank, world, device)
    elif args.workload in FUSED:
        res = run_fused(args.workload, args.steps, args.warmup, rank, world, device)
    elif args.workload == "generate":
        res = run_generate(args.steps, args.warmup, rank, world, device)
    else:
        res = run_lm(args.workload, args.steps, args.warmup, rank, world, device, graph=not args.no_graph,
                     eager_steps=0 if args.no_graph else max(3, args.steps // 2), keep_logits=not args.no_logits)

    if rank == 0:
        line = {"metric": res["metric"], "value": res["value"], "unit": res["unit"], "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["ms_per_step"],
                "higher_is_better": True, "scaling": res["scaling"], "vs_baseline": None, "dtype": res["dtype"],
                "data": "synthetic", "config": res["config"], "e2e": res["e2e"], "gpu_launches": res["gpu_launches"],
                "gpu_launches_how": res["gpu_launches_how"], "roofline": res["roofline"], "clocks": res["clocks"]}
        if "extra" in res:
            line["extra"] = res["extra"]
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(args.workload)
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
