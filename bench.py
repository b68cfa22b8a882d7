#!/usr/bin/env python
"""Benchmark of the second backward of scaled-dot-product attention on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c4]

A "step" is one second-backward pass (Qbar, Kbar, Vbar, dObar from q, k, v, out, lse, delta, dO,
dQ and the three tangents) over one batch of seeded synthetic inputs.

Workloads
  c2  bf16 GQA B=1 Hq=32 Hkv=8 S=4096 D=64 causal on EVERY GPU (global batch = N; weak scaling).
      This is the single-GPU configuration the throughput target is quoted on.
  c4  bf16 GQA B=8 Hq=64 Hkv=8 S=8192 D=128 causal, its 64 (batch, KV head) units dealt to the N
      GPUs in contiguous blocks (strong scaling), no collective on the data path.

FLOP convention (algorithmic, matmul only): A = attending (query, key) pairs per query head,
u = 2*A*D*B*Hq; the second backward is 12 u (no credit for recomputation).

Output: one JSON line on rank 0.  `value` = whole-job TFLOP/s with inputs resident in HBM;
`e2e` = the same through the C-ABI calls with pinned host buffers holding the reference-level inputs
of the second backward (copies inside the timed region; delta and pk are regenerated on the device);
`roofline` = tensor roofline of the two-kernel second backward; `cpu_baseline` = the CPU port of
the reference's math route timed on a bounded sample.  `--impl reference` times that CPU port
alone (rank 0), as the reference arm.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "sdpa_second_backward_tflops"
UNIT = "TFLOP/s"
WORKLOADS = {
    "c2": dict(B=1, Hq=32, Hkv=8, N=4096, D=64, scaling="weak",
               name="bf16 GQA B=1/GPU Hq=32 Hkv=8 S=4096 D=64 causal"),
    "c4": dict(B=8, Hq=64, Hkv=8, N=8192, D=128, scaling="strong",
               name="bf16 GQA B=8 Hq=64 Hkv=8 S=8192 D=128 causal, (batch,kv-head) units sharded"),
    # a quarter of c2 (same tiles, fewer heads): small enough for profiler captures
    "prof": dict(B=1, Hq=8, Hkv=2, N=4096, D=64, scaling="weak",
                 name="bf16 GQA B=1 Hq=8 Hkv=2 S=4096 D=64 causal (profiling case)"),
}


# dram__bytes_read.sum + dram__bytes_write.sum of one second-backward launch pair, from the ncu capture
# summarised in profiles/bwd2_kernels_gqa_s4096_d64.md: that capture ran a quarter of the c2 workload
# (8 of 32 query heads; traffic grows with the head count), so its 51.3 MB is scaled by 4.
TRAFFIC_BYTES = {"c2": 4 * (33_890_560 + 8_960 + 17_369_088)}
TRAFFIC_NOTE = "ncu dram bytes of the row-owned + column-owned kernels on a quarter-size capture, x4; c2 only"


def causal_pairs(n: int) -> int:
    return n * (n + 1) // 2


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops, burst)"
    return 1590.0, "fallback (1590 TFLOP/s, earlier measurement on this pool)"


class ClockSampler:
    """nvidia-smi clock / throttle samples taken while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100", "-i", str(gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons, power = [], [], set(), []
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the CPU port of the reference's math route
# ------------------------------------------------------------------------------------------
def cpu_second_backward_sample(wl: dict, heads: int, steps: int, warmup: int, seed: int = 0):
    """Time the second `autograd.grad` of materialized attention on the host cores for ONE KV head
    and `heads` of its query heads (fp32).  Returns (seconds per step list, flops per step)."""
    from oracle import bob_oracle as O

    N, D = wl["N"], wl["D"]
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float32)
    q, dO, uQ = r(1, heads, N, D).requires_grad_(True), r(1, heads, N, D).requires_grad_(True), r(1, heads, N, D)
    k, v = r(1, 1, N, D).requires_grad_(True), r(1, 1, N, D).requires_grad_(True)
    uK, uV = r(1, 1, N, D), r(1, 1, N, D)
    out = O.attention_dense(q, k, v, is_causal=True)
    first = torch.autograd.grad(out, (q, k, v), dO, create_graph=True)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        torch.autograd.grad(first, (q, k, v, dO), (uQ, uK, uV), retain_graph=True)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    flops = 12 * 2 * causal_pairs(N) * D * heads
    return times, flops


def pick_cpu_heads(wl: dict, steps: int, warmup: int, budget_s: float) -> int:
    """Largest number of query heads (1..G) of one KV group whose run fits the time budget."""
    t, _ = cpu_second_backward_sample(wl, 1, 1, 0)
    G = wl["Hq"] // wl["Hkv"]
    return max(1, min(G, int(budget_s / max(1e-3, t[0] * (steps + warmup)))))


def run_reference_arm(args, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = args.steps, args.warmup
    heads = pick_cpu_heads(wl, steps, warmup, budget_s=150.0)
    times, flops = cpu_second_backward_sample(wl, heads, steps, warmup)
    sec = sum(times) / len(times)
    val = flops / sec / 1e12
    sample = (f"one KV head with {heads} of its {wl['Hq'] // wl['Hkv']} query heads of the workload "
              f"(S={wl['N']}, D={wl['D']}), fp32, second autograd.grad of materialized attention")
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": wl["scaling"], "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl["name"], "sample": sample},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=list(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile", action="store_true",
                    help="only set up and run `steps` second-backward calls (for profiler captures)")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference_arm(args, wl)
        return
    if not args.profile:
        args.warmup = max(args.warmup, 3)

    import torch.distributed as dist
    from flashbob_b200 import _lib, ops, sharding

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the kernels")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    # ---- this rank's units ---------------------------------------------------------------------
    G = wl["Hq"] // wl["Hkv"]
    N, D = wl["N"], wl["D"]
    if wl["scaling"] == "weak":
        B, Hq, Hkv = wl["B"], wl["Hq"], wl["Hkv"]
        total_heads = B * Hq * world
    else:
        units = sharding.unit_range(wl["B"] * wl["Hkv"], world, rank)
        B, Hq, Hkv = len(units), G, 1
        total_heads = wl["B"] * wl["Hq"]
    unit_flops = 2 * causal_pairs(N) * D
    flops_rank = 12 * unit_flops * B * Hq
    flops_job = 12 * unit_flops * total_heads

    gen = torch.Generator(device="cpu").manual_seed(1000 + rank)
    mk = lambda *s: torch.randn(*s, generator=gen, dtype=torch.float32).to(torch.bfloat16)
    host = {
        "q": mk(B, Hq, N, D), "k": mk(B, Hkv, N, D), "v": mk(B, Hkv, N, D), "dO": mk(B, Hq, N, D),
        "uQ": mk(B, Hq, N, D), "uK": mk(B, Hkv, N, D), "uV": mk(B, Hkv, N, D),
    }
    d = {n: t.to(dev) for n, t in host.items()}
    geom = dict(is_causal=True, window_size=0, q_offset=0, k_offset=0, scale=None)
    out, lse = ops.attention_forward(d["q"], d["k"], d["v"], **geom)
    dQ, dK, dV, delta, pk = ops.attention_first_backward(d["q"], d["k"], d["v"], out, lse, d["dO"], **geom)
    d.update(out=out, lse=lse, dQ=dQ, delta=delta, pk=pk)
    torch.cuda.synchronize()

    # ---- direct C-ABI call with preallocated results -------------------------------------------
    lib = _lib.load()
    g = ops._geom(d["q"], d["k"], **geom)
    for field, name in ((g.q_strides, "q"), (g.k_strides, "k"), (g.v_strides, "v"), (g.out_strides, "out"),
                        (g.do_strides, "dO"), (g.dq_strides, "dQ"), (g.uq_strides, "uQ"),
                        (g.uk_strides, "uK"), (g.uv_strides, "uV")):
        ops._set_strides(field, d[name])
    res = {n: torch.empty_like(d[s]) for n, s in (("Qbar", "q"), ("Kbar", "k"), ("Vbar", "k"), ("dObar", "q"))}
    ws = torch.empty(lib.bob_sm100_workspace_bytes(_lib.STAGE_BWD2, ctypes.byref(g)), dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream(dev)
    vp = lambda t: ctypes.c_void_p(t.data_ptr())

    def bwd2(src):
        rc = lib.bob_sm100_bwd2(ctypes.byref(g), vp(src["q"]), vp(src["k"]), vp(src["v"]), vp(src["out"]),
                                vp(src["lse"]), vp(src["delta"]), vp(src["pk"]), vp(src["dO"]), vp(src["dQ"]), vp(src["uQ"]),
                                vp(src["uK"]), vp(src["uV"]), vp(res["Qbar"]), vp(res["Kbar"]), vp(res["Vbar"]),
                                vp(res["dObar"]), vp(ws), ctypes.c_void_p(stream.cuda_stream))
        _lib.check(rc, "bob_sm100_bwd2")

    if args.profile:
        for _ in range(args.steps):
            bwd2(d)
        torch.cuda.synchronize()
        print(json.dumps({"profile_run": wl["name"], "second_backward_calls": args.steps}), flush=True)
        return

    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)   # > 126 MB of L2

    def timed_steps(fn, n_warm, n_steps):
        for _ in range(n_warm):
            flush.zero_(); fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        evs = []
        wall0 = time.perf_counter()
        for _ in range(n_steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream); fn(); e1.record(stream)
            evs.append((e0, e1))
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        wall = time.perf_counter() - wall0
        ms = [a.elapsed_time(b) for a, b in evs]
        return ms, wall

    sampler = ClockSampler(local_rank) if rank == 0 else None
    ms, wall = timed_steps(lambda: bwd2(d), args.warmup, args.steps)
    total_ms = torch.tensor([sum(ms)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(total_ms, op=dist.ReduceOp.MAX)
    status = lib.bob_sm100_read_status(vp(ws), ctypes.c_void_p(stream.cuda_stream))
    _lib.check(status, "bob_sm100_bwd2 (device status)")
    clocks = sampler.stop() if sampler else None
    ms_per_step = total_ms.item() / args.steps
    value = flops_job / (ms_per_step * 1e-3) / 1e12

    # ---- per-kernel split (row-owned / column-owned kernel alone) -------------------------------
    kernel_ms = {}
    for which in ("row", "col"):
        os.environ["BOB_SM100_BWD2_KERNELS"] = which
        kms, _ = timed_steps(lambda: bwd2(d), 2, min(args.steps, 10))
        kernel_ms[which] = sum(kms) / len(kms)
    os.environ.pop("BOB_SM100_BWD2_KERNELS", None)

    # ---- the other two stages of the path, same geometry, same timing rules (secondary numbers) ---
    sc = {n: torch.empty_like(d[s_]) for n, s_ in (("out", "q"), ("dQ", "q"), ("dK", "k"), ("dV", "k"))}
    sc["lse"], sc["delta"], sc["pk"] = torch.empty_like(d["lse"]), torch.empty_like(d["delta"]), torch.empty_like(d["pk"])
    ws1 = torch.empty(max(lib.bob_sm100_workspace_bytes(_lib.STAGE_FWD, ctypes.byref(g)),
                          lib.bob_sm100_workspace_bytes(_lib.STAGE_BWD1, ctypes.byref(g))), dtype=torch.uint8, device=dev)
    sp = ctypes.c_void_p(stream.cuda_stream)

    def fwd_call():
        _lib.check(lib.bob_sm100_fwd(ctypes.byref(g), vp(d["q"]), vp(d["k"]), vp(d["v"]), vp(sc["out"]),
                                     vp(sc["lse"]), vp(ws1), sp), "bob_sm100_fwd")

    def bwd1_call():
        _lib.check(lib.bob_sm100_bwd1(ctypes.byref(g), vp(d["q"]), vp(d["k"]), vp(d["v"]), vp(d["out"]),
                                      vp(d["lse"]), vp(d["dO"]), vp(sc["dQ"]), vp(sc["dK"]), vp(sc["dV"]),
                                      vp(sc["delta"]), vp(sc["pk"]), vp(ws1), sp), "bob_sm100_bwd1")

    stage_ms = {}
    for name, fn, mult in (("forward", fwd_call, 2), ("first_backward", bwd1_call, 5)):
        sms_, _ = timed_steps(fn, 2, min(args.steps, 10))
        t = sum(sms_) / len(sms_)
        stage_ms[name] = {"ms": t, "tflops": mult * unit_flops * B * Hq / (t * 1e-3) / 1e12}

    # ---- end to end: pinned host buffers -> device -> C-ABI call -> pinned host results --------
    # The host holds what the reference's second backward is called with (src/bob/sdpa.py:175-236:
    # q, k, v, out, lse, dO, dQ and the three tangents).  delta and pk are this library's own
    # by-products of the first backward; they never leave the device and are regenerated there each
    # step by bob_sm100_bwd1 (inside the timed region), which is cheaper than carrying 34 MB of
    # fp32 pk over PCIe.
    names_in = ("q", "k", "v", "out", "lse", "dO", "dQ", "uQ", "uK", "uV")
    names_dev = names_in + ("delta", "pk", "dQ1", "dK1", "dV1")
    d["dQ1"], d["dK1"], d["dV1"] = torch.empty_like(d["dQ"]), torch.empty_like(d["k"]), torch.empty_like(d["v"])
    pin = {n: d[n].cpu().pin_memory() for n in names_in}
    stage = {n: torch.empty_like(d[n]) for n in names_dev}
    ws_e2e = torch.empty(max(lib.bob_sm100_workspace_bytes(_lib.STAGE_BWD1, ctypes.byref(g)),
                             lib.bob_sm100_workspace_bytes(_lib.STAGE_BWD2, ctypes.byref(g))),
                         dtype=torch.uint8, device=dev)
    pin_out = {n: torch.empty(t.shape, dtype=t.dtype, device="cpu").pin_memory() for n, t in res.items()}
    h2d = sum(t.numel() * t.element_size() for t in pin.values())
    d2h = sum(t.numel() * t.element_size() for t in pin_out.values())

    # Steps are pipelined over three streams with two sets of device buffers: while step i computes,
    # step i+1's inputs cross PCIe and step i-1's results go back.  Every step still copies all of
    # its inputs from pinned host memory and all of its results back to pinned host memory.
    s_in, s_cmp, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    stage2 = [stage, {n: torch.empty_like(d[n]) for n in names_dev}]
    res2 = [res, {n: torch.empty_like(t) for n, t in res.items()}]
    pin_out2 = [pin_out, {n: torch.empty(t.shape, dtype=t.dtype, device="cpu").pin_memory() for n, t in res.items()}]

    def bwd2_on(src, dst, cuda_stream):
        rc = lib.bob_sm100_bwd1(ctypes.byref(g), vp(src["q"]), vp(src["k"]), vp(src["v"]), vp(src["out"]),
                                vp(src["lse"]), vp(src["dO"]), vp(src["dQ1"]), vp(src["dK1"]), vp(src["dV1"]),
                                vp(src["delta"]), vp(src["pk"]), vp(ws_e2e), ctypes.c_void_p(cuda_stream))
        _lib.check(rc, "bob_sm100_bwd1")
        rc = lib.bob_sm100_bwd2(ctypes.byref(g), vp(src["q"]), vp(src["k"]), vp(src["v"]), vp(src["out"]),
                                vp(src["lse"]), vp(src["delta"]), vp(src["pk"]), vp(src["dO"]), vp(src["dQ"]),
                                vp(src["uQ"]), vp(src["uK"]), vp(src["uV"]), vp(dst["Qbar"]), vp(dst["Kbar"]),
                                vp(dst["Vbar"]), vp(dst["dObar"]), vp(ws_e2e), ctypes.c_void_p(cuda_stream))
        _lib.check(rc, "bob_sm100_bwd2")

    def e2e_run(n_steps):
        ev_in = [None, None]; ev_cmp = [None, None]; ev_out = [None, None]
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for st_ in (s_in, s_cmp, s_out):
            st_.wait_event(start)
        for i in range(n_steps):
            s = i & 1
            with torch.cuda.stream(s_in):
                if ev_cmp[s] is not None:
                    s_in.wait_event(ev_cmp[s])           # step i-2 no longer reads this input set
                for n in names_in:
                    stage2[s][n].copy_(pin[n], non_blocking=True)
                ev_in[s] = torch.cuda.Event(); ev_in[s].record(s_in)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(ev_in[s])
                if ev_out[s] is not None:
                    s_cmp.wait_event(ev_out[s])          # step i-2's results have left this result set
                bwd2_on(stage2[s], res2[s], s_cmp.cuda_stream)
                ev_cmp[s] = torch.cuda.Event(); ev_cmp[s].record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_cmp[s])
                for n in res:
                    pin_out2[s][n].copy_(res2[s][n], non_blocking=True)
                ev_out[s] = torch.cuda.Event(); ev_out[s].record(s_out)
        for st_ in (s_in, s_cmp, s_out):
            stream.wait_stream(st_)
        end.record(stream)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        return start.elapsed_time(end)

    e2e_steps = max(4, min(args.steps, 12))
    e2e_run(3)
    e2e_total = e2e_run(e2e_steps)
    e2e_ms = torch.tensor([e2e_total], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_value = flops_job / (e2e_ms.item() / e2e_steps * 1e-3) / 1e12

    # ---- the whole two-level chain through the public operator (secondary number) --------------
    chain = None
    if wl["scaling"] == "weak":
        import bob

        def chain_step():
            q, k, v = (d[n].detach().requires_grad_(True) for n in ("q", "k", "v"))
            o = bob.sdpa_bob(q, k, v, is_causal=True)
            dq, dk, dv = torch.autograd.grad(o.float().square().mean(), (q, k, v), create_graph=True)
            L2 = dq.float().square().mean() + dk.float().square().mean() + dv.float().square().mean()
            return torch.autograd.grad(L2, (q, k, v))

        cms, _ = timed_steps(chain_step, 2, 5)
        chain_ms = sum(cms) / len(cms)
        chain = {"ms": chain_ms, "tflops_24u": 24 * unit_flops * B * Hq / (chain_ms * 1e-3) / 1e12,
                 "what": "fwd + first grads (create_graph) + second grads incl. re-entered first backward"}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_src = measured_peak()
    per_gpu = value / world
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": wl["scaling"], "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": wl["name"], "l2": "256 MiB buffer written between steps; per-step CUDA events",
                   "flops_per_step_job": flops_job, "flop_convention": "12 * 2*A*D*heads, A = S(S+1)/2"},
        "per_gpu_tflops": per_gpu, "frac_of_measured_peak": per_gpu / peak,
        "frac_of_nominal_2250": per_gpu / 2250.0,
        "roofline": {"bound": "tensor", "achieved": flops_rank / (ms_per_step * 1e-3) / 1e12, "peak": peak,
                     "unit": UNIT, "frac": flops_rank / (ms_per_step * 1e-3) / 1e12 / peak,
                     "traffic": TRAFFIC_BYTES.get(args.workload), "traffic_source": TRAFFIC_NOTE,
                     "peak_source": peak_src,
                     "kernel": "second backward = row-owned kernel + column-owned kernel",
                     "kernel_ms": kernel_ms},
        "other_stages": stage_ms,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "steps": e2e_steps, "ms_per_step": e2e_ms.item() / e2e_steps,
                "how": "pinned host (q,k,v,out,lse,dO,dQ,uQ,uK,uV) -> device -> bob_sm100_bwd1 (delta, pk) + "
                       "bob_sm100_bwd2 -> pinned host (Qbar,Kbar,Vbar,dObar) every step; steps pipelined over "
                       "copy-in / compute / copy-out streams; inputs per step exceed L2",
                "gpu_launches_per_step": lib.bob_sm100_kernel_launches(_lib.STAGE_BWD1, ctypes.byref(g)) +
                                         lib.bob_sm100_kernel_launches(_lib.STAGE_BWD2, ctypes.byref(g))},
        "gpu_launches": lib.bob_sm100_kernel_launches(_lib.STAGE_BWD2, ctypes.byref(g)) * args.steps,
        "clocks": clocks,
        "wall_s_timed_region": wall,
        "chain": chain,
    }
    if world == 1 and not args.no_cpu_baseline:
        heads = pick_cpu_heads(wl, 3, 1, budget_s=20.0)
        times, flops = cpu_second_backward_sample(wl, heads, 3, 1)
        sec = sum(times) / len(times)
        line["cpu_baseline"] = {
            "value": flops / sec / 1e12, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"one KV head with {heads} of its {G} query heads (S={N}, D={D}), fp32, 3 timed "
                      f"second-gradient passes of the CPU port of the reference's math route"}
    else:
        line["cpu_baseline"] = None
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
