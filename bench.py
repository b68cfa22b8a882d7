#!/usr/bin/env python
"""Benchmark of the second backward of scaled-dot-product attention on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c4]

A "step" is one second-backward pass (Qbar, Kbar, Vbar, dObar from q, k, v, out, lse, delta, dO,
dQ and the three tangents) over one batch of seeded synthetic inputs.

Workloads
  c2  bf16 GQA B=1 Hq=32 Hkv=8 S=4096 D=64 causal on EVERY GPU (global batch = N; weak scaling).
      This is the single-GPU configuration the throughput target is quoted on; `value` is measured
      on it.
  c4  bf16 GQA B=8 Hq=64 Hkv=8 S=8192 D=128 causal, its 64 (batch, KV head) units dealt to the N
      GPUs in contiguous blocks (strong scaling), no collective on the data path.  Every default run
      also measures this workload and reports it as `strong_c4` (at N = 1 one GPU holds all 64 units).

FLOP convention (algorithmic, matmul only): A = attending (query, key) pairs per query head,
u = 2*A*D*B*Hq; the second backward is 12 u (no credit for recomputation).

Output: one JSON line on rank 0.
  value           whole-job TFLOP/s with inputs resident in HBM (per-step CUDA events, L2 flushed)
  roofline        tensor roofline of the two-kernel second backward against the measured bf16 peak
  sustained       the same call repeated back to back for >= 2 s, against the measured sustained peak
  e2e             through the C-ABI calls from pinned host buffers, copies inside the timed region,
                  shipping what a caller of the operator owns (q, k, v, dO and the tangents) and running
                  forward, first backward and second backward on the device; `e2e_reference_level`
                  instead ships everything the reference's second backward is called with (also out,
                  lse, dQ) and skips the forward
  strong_c4       the sharded scaling workload (see above)
  reference_cuda  the unmodified reference's own CUDA route (cuDNN + Triton) from baseline/_ref on
                  this GPU: times and errors against its fp64 CPU path (N = 1 only)
  cpu_baseline    the reference's CPU route timed on the host cores on a bounded sample (N = 1 only)
`--impl reference` times the reference's CPU route alone (rank 0), as the reference arm.
"""

from __future__ import annotations

import argparse
import ctypes
import json
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
    # a quarter of c2 (same tiles, fewer heads) and one eighth of a rank's share of c4 at 8 GPUs:
    # small enough for profiler captures
    "prof": dict(B=1, Hq=8, Hkv=2, N=4096, D=64, scaling="weak",
                 name="bf16 GQA B=1 Hq=8 Hkv=2 S=4096 D=64 causal (profiling case)"),
    "prof128": dict(B=1, Hq=8, Hkv=1, N=4096, D=128, scaling="weak",
                    name="bf16 GQA B=1 Hq=8 Hkv=1 S=4096 D=128 causal (profiling case)"),
}
REF_DIR = ROOT / "baseline" / "_ref"
REF_RUNNER = ROOT / "baseline" / "run_reference.py"


# dram__bytes_read.sum + dram__bytes_write.sum of one second-backward launch pair, from the ncu capture
# summarised in profiles/bwd2_kernels_gqa_s4096_d64.md: that capture ran a quarter of the c2 workload
# (8 of 32 query heads; traffic grows with the head count), so its bytes are scaled by 4.
TRAFFIC_BYTES = {"c2": 4 * (33_890_560 + 8_960 + 17_369_088)}
TRAFFIC_NOTE = "ncu dram bytes of the row-owned + column-owned kernels on a quarter-size capture, x4; c2 only"


def causal_pairs(n: int) -> int:
    return n * (n + 1) // 2


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return (float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", 0.0)) or None,
                "measured (MEASURED_PEAKS.json bf16_tflops, burst)")
    return 1590.0, 1400.0, "fallback (1590 TFLOP/s burst / 1400 sustained, earlier measurement on this pool)"


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


class ClockSampler:
    """nvidia-smi clock / throttle samples taken while a timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, period_ms: int = 100):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", str(period_ms), "-i", str(gpu_index)],
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
        # samples under load: the upper half by power draw (the sampler also sees the idle edges)
        loaded = sm
        if len(power) >= 4:
            cut = statistics.median(power)
            loaded = [s for s, w in zip(sm, power) if w >= cut] or sm
        return {"sm_mhz": statistics.median(loaded) if loaded else None,
                "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's CPU route (or, without it, its CPU port)
# ------------------------------------------------------------------------------------------
def _run_child(argv, timeout_s):
    """Run a child python process with the thread-count variables of the launcher removed (torchrun
    sets OMP_NUM_THREADS=1 for its ranks) and return the last JSON line it printed."""
    env = {k: v for k, v in os.environ.items() if k not in ("OMP_NUM_THREADS", "MKL_NUM_THREADS")}
    res = subprocess.run([sys.executable, *argv], capture_output=True, text=True, timeout=timeout_s, env=env)
    if res.returncode != 0:
        raise RuntimeError((res.stderr or res.stdout).strip().splitlines()[-1][:300] if (res.stderr or res.stdout) else "no output")
    for line in reversed(res.stdout.strip().splitlines()):
        if line.startswith("{"):
            return json.loads(line)
    raise RuntimeError("child printed no JSON")


def cpu_port_sample(wl: dict, heads: int, steps: int, warmup: int, seed: int = 0):
    """The CPU port (oracle) of the reference's math route: second `autograd.grad` of materialized
    attention for ONE KV head and `heads` of its query heads (fp32).  Used when baseline/_ref is
    absent.  Returns (seconds per step list, flops per step)."""
    from oracle import bob_oracle as O

    torch.set_num_threads(host_threads())
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
    return times, 12 * 2 * causal_pairs(N) * D * heads


def cpu_reference_sample(wl: dict, steps: int, warmup: int, budget_s: float) -> dict:
    """Time the reference's CPU implementation of the path on the host cores, on a bounded sample
    of the workload: as many whole KV heads (each with all of its query heads) as fit the time
    budget, at least one KV head with some of its query heads."""
    G, Hkv = wl["Hq"] // wl["Hkv"], wl["Hkv"] * wl["B"]
    threads = host_threads()
    n_pass = steps + warmup
    if REF_DIR.exists() and REF_RUNNER.exists():
        base = ["--mode", "cpu", "--seq", str(wl["N"]), "--dim", str(wl["D"]), "--threads", str(threads)]
        probe = _run_child([str(REF_RUNNER), *base, "--heads", "1", "--steps", "1", "--warmup", "0"], 900)
        per_head = max(1e-3, 3.0 * probe["seconds"][0])       # a timed pass plus the untimed graph building before it
        heads = max(1, min(G, int(budget_s / (per_head * n_pass))))
        kv = max(1, min(Hkv, int(budget_s / (per_head * G * n_pass)))) if heads == G else 1
        r = _run_child([str(REF_RUNNER), *base, "--heads", str(heads), "--kv-heads", str(kv), "--steps", str(steps),
                        "--warmup", str(warmup)], 1800)
        sec, flops, kind, cores = statistics.mean(r["seconds"]), r["flops_per_step"], "reference", r["threads"]
        what = "the reference's own CPU route (bob.sdpa_bob on CPU tensors from baseline/_ref: math attention, stock autograd)"
    else:
        t, _ = cpu_port_sample(wl, 1, 1, 0)
        heads, kv = max(1, min(G, int(budget_s / max(1e-3, t[0] * (n_pass + 1))))), 1
        times, flops = cpu_port_sample(wl, heads, steps, warmup)
        sec, kind, cores = statistics.mean(times), "port", torch.get_num_threads()
        what = "the CPU port of the reference's math route (baseline/_ref not installed)"
    sample = (f"{kv} of the {Hkv} (batch, KV head) units of the workload, each with {heads} of its {G} query heads "
              f"(S={wl['N']}, D={wl['D']}), fp32, {steps} timed second-gradient passes of {what}")
    return {"value": flops / sec / 1e12, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample,
            "seconds_per_step": sec, "same_config": heads == G and kv == Hkv}


def run_reference_arm(args, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = args.steps, args.warmup
    cb = cpu_reference_sample(wl, steps, warmup, budget_s=150.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": cb["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": cb["seconds_per_step"] * 1e3, "higher_is_better": True,
        "scaling": wl["scaling"], "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl["name"], "sample": cb["sample"]},
        "cpu_baseline": cb,
        "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def reference_cuda_record(wl: dict) -> dict:
    """The unmodified reference's own CUDA route on this GPU (a child process that imports only
    baseline/_ref): warm times per stage, first-call time and errors against its fp64 CPU path."""
    if not (REF_DIR.exists() and REF_RUNNER.exists()):
        return {"unavailable": "baseline/_ref not installed (see BASELINE.md for the pip line)"}
    try:
        r = _run_child([str(REF_RUNNER), "--mode", "cuda", "--time", "--batch", str(wl["B"]), "--hq", str(wl["Hq"]),
                        "--hkv", str(wl["Hkv"]), "--seq", str(wl["N"]), "--dim", str(wl["D"])], 420)
    except Exception as e:  # noqa: BLE001 - the reference's route is outside this repository's control
        return {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}
    r["what"] = ("bob.sdpa_bob from baseline/_ref (cuDNN forward / first backward, Triton second backward) through "
                 "autograd, device-resident inputs, after warm-up (autotune excluded; first_call_s includes it); "
                 "errors of one KV group against the reference's fp64 CPU path")
    return r


# ------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------
class Problem:
    """One rank's inputs of a workload on the device, with the first-backward by-products, and the
    C-ABI call of the second backward on preallocated results."""

    def __init__(self, wl, world, rank, dev, on_device_inputs=False):
        from flashbob_b200 import _lib, ops, sharding

        self.lib, self._lib, self.ops, self.dev = _lib.load(), _lib, ops, dev
        G = wl["Hq"] // wl["Hkv"]
        N, D = wl["N"], wl["D"]
        if wl["scaling"] == "weak":
            B, Hq, Hkv = wl["B"], wl["Hq"], wl["Hkv"]
            self.total_heads = B * Hq * world
            seeds = [1000 + rank]
        else:
            units = sharding.unit_range(wl["B"] * wl["Hkv"], world, rank)
            B, Hq, Hkv = len(units), G, 1
            self.total_heads = wl["B"] * wl["Hq"]
            seeds = [4000 + u for u in units]          # one seed per (batch, KV head) unit, whatever rank owns it
        self.B, self.Hq, self.Hkv, self.N, self.D, self.G = B, Hq, Hkv, N, D, G
        self.unit_flops = 2 * causal_pairs(N) * D
        self.flops_rank = 12 * self.unit_flops * B * Hq
        self.flops_job = 12 * self.unit_flops * self.total_heads
        shapes = {"q": (Hq, N, D), "k": (Hkv, N, D), "v": (Hkv, N, D), "dO": (Hq, N, D), "uQ": (Hq, N, D),
                  "uK": (Hkv, N, D), "uV": (Hkv, N, D)}
        if on_device_inputs:
            # large sharded workload: every unit is drawn on its owning GPU from the unit's own seed
            d = {n: torch.empty((B, *s), dtype=torch.bfloat16, device=dev) for n, s in shapes.items()}
            for i, seed in enumerate(seeds):
                gen = torch.Generator(device=dev).manual_seed(seed)
                for n, s in shapes.items():
                    d[n][i] = torch.randn(s, generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
            self.host = None
        else:
            gen = torch.Generator(device="cpu").manual_seed(seeds[0])
            self.host = {n: torch.randn((B, *s), generator=gen, dtype=torch.float32).to(torch.bfloat16)
                         for n, s in shapes.items()}
            d = {n: t.to(dev) for n, t in self.host.items()}
        self.geom = dict(is_causal=True, window_size=0, q_offset=0, k_offset=0, scale=None)
        out, lse = ops.attention_forward(d["q"], d["k"], d["v"], **self.geom)
        dQ, dK, dV, delta, pk = ops.attention_first_backward(d["q"], d["k"], d["v"], out, lse, d["dO"], **self.geom)
        d.update(out=out, lse=lse, dQ=dQ, delta=delta, pk=pk)
        del dK, dV
        torch.cuda.synchronize()
        self.d = d
        g = ops._geom(d["q"], d["k"], **self.geom)
        for field, name in ((g.q_strides, "q"), (g.k_strides, "k"), (g.v_strides, "v"), (g.out_strides, "out"),
                            (g.do_strides, "dO"), (g.dq_strides, "dQ"), (g.uq_strides, "uQ"),
                            (g.uk_strides, "uK"), (g.uv_strides, "uV")):
            ops._set_strides(field, d[name])
        self.g = g
        self.res = {n: torch.empty_like(d[s]) for n, s in (("Qbar", "q"), ("Kbar", "k"), ("Vbar", "k"), ("dObar", "q"))}
        self.ws = torch.empty(self.lib.bob_sm100_workspace_bytes(_lib.STAGE_BWD2, ctypes.byref(g)), dtype=torch.uint8,
                              device=dev)
        self.stream = torch.cuda.current_stream(dev)

    @staticmethod
    def vp(t):
        return ctypes.c_void_p(t.data_ptr())

    def bwd2(self, src=None, dst=None, part=3, ws=None, cuda_stream=None):
        src, dst, vp = src or self.d, dst or self.res, self.vp
        rc = self.lib.bob_sm100_bwd2_part(
            part, ctypes.byref(self.g), vp(src["q"]), vp(src["k"]), vp(src["v"]), vp(src["out"]), vp(src["lse"]),
            vp(src["delta"]), vp(src["pk"]), vp(src["dO"]), vp(src["dQ"]), vp(src["uQ"]), vp(src["uK"]), vp(src["uV"]),
            vp(dst["Qbar"]), vp(dst["Kbar"]), vp(dst["Vbar"]), vp(dst["dObar"]), vp(ws if ws is not None else self.ws),
            ctypes.c_void_p(cuda_stream if cuda_stream is not None else self.stream.cuda_stream))
        self._lib.check(rc, "bob_sm100_bwd2")

    def check_status(self):
        st = self.lib.bob_sm100_read_status(self.vp(self.ws), ctypes.c_void_p(self.stream.cuda_stream))
        self._lib.check(st, "bob_sm100_bwd2 (device status)")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=list(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the secondary legs (strong_c4, sustained, reference_cuda, chain, e2e variants)")
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
    from flashbob_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the kernels")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    prob = Problem(wl, world, rank, dev, on_device_inputs=(wl["scaling"] == "strong"))
    lib, d, g, res, vp = prob.lib, prob.d, prob.g, prob.res, prob.vp
    stream = prob.stream
    B, Hq, N, D, G = prob.B, prob.Hq, prob.N, prob.D, prob.G
    unit_flops, flops_rank, flops_job = prob.unit_flops, prob.flops_rank, prob.flops_job

    if args.profile:
        for _ in range(args.steps):
            prob.bwd2()
        torch.cuda.synchronize()
        print(json.dumps({"profile_run": wl["name"], "second_backward_calls": args.steps}), flush=True)
        return

    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)   # > 126 MB of L2

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    def timed_steps(fn, n_warm, n_steps, do_flush=True):
        """Per-step CUDA events on the launching stream; returns (list of ms, wall seconds)."""
        for _ in range(n_warm):
            if do_flush:
                flush.zero_()
            fn()
        barrier()
        evs = []
        wall0 = time.perf_counter()
        for _ in range(n_steps):
            if do_flush:
                flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream); fn(); e1.record(stream)
            evs.append((e0, e1))
        barrier()
        wall = time.perf_counter() - wall0
        return [a.elapsed_time(b) for a, b in evs], wall

    # ---- headline: K timed steps -----------------------------------------------------------------
    sampler = ClockSampler(local_rank) if rank == 0 else None
    ms, wall = timed_steps(prob.bwd2, args.warmup, args.steps)
    ms_per_step = max_over_ranks(sum(ms)) / args.steps
    prob.check_status()
    clocks = sampler.stop() if sampler else None
    value = flops_job / (ms_per_step * 1e-3) / 1e12

    # ---- per-kernel split (row-owned / column-owned kernel alone) -------------------------------
    kernel_ms = {}
    for which, part in (("row", 1), ("col", 2)):
        kms, _ = timed_steps(lambda: prob.bwd2(part=part), 2, min(args.steps, 10))
        kernel_ms[which] = sum(kms) / len(kms)

    extras = not args.no_extras
    peak, peak_sustained, peak_src = measured_peaks()

    # ---- sustained: the same call back to back for >= 2 s, no flush (inputs + results exceed L2 anyway) ----
    sustained = None
    if extras:
        n_sus = max(50, int(2.2 / (ms_per_step * 1e-3)))
        s2 = ClockSampler(local_rank, period_ms=50) if rank == 0 else None
        for _ in range(20):
            prob.bwd2()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(n_sus):
            prob.bwd2()
        e1.record(stream)
        barrier()
        sus_ms = max_over_ranks(e0.elapsed_time(e1)) / n_sus
        sus_clocks = s2.stop() if s2 else None
        per_gpu_sus = flops_rank / (sus_ms * 1e-3) / 1e12
        sustained = {"calls": n_sus, "seconds": sus_ms * n_sus * 1e-3, "ms_per_step": sus_ms,
                     "value": flops_job / (sus_ms * 1e-3) / 1e12, "per_gpu_tflops": per_gpu_sus, "unit": UNIT,
                     "frac_of_measured_sustained_peak": per_gpu_sus / peak_sustained if peak_sustained else None,
                     "peak_sustained": peak_sustained, "clocks": sus_clocks,
                     "how": "back-to-back calls on one stream, one event pair around all of them; working set "
                            f"{sum(t.numel() * t.element_size() for t in list(d.values()) + list(res.values())) >> 20} MiB"}

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

    # ---- end to end: pinned host buffers -> device -> C-ABI calls -> pinned host results ---------
    # Variant "operator_inputs" (the headline `e2e`) ships what a caller of the operator owns (q, k, v,
    # dO and the tangents) and regenerates out, lse, dQ, delta and pk on the device (bob_sm100_fwd +
    # bob_sm100_bwd1): 67 MB in per step instead of 101 MB, and the link is the bound.  Variant
    # "reference_level" ships what the reference's second backward is called with
    # (src/bob/sdpa.py:175-236: also out, lse and dQ); delta and pk, this library's own by-products of
    # the first backward, are regenerated by bob_sm100_bwd1 (cheaper than carrying fp32 pk over PCIe).
    # Both copy every input in and every result out every step.
    e2e = e2e_alt = None
    if prob.host is not None:
        e2e_steps = max(4, min(args.steps, 12))
        s_in, s_cmp, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        names_all = ("q", "k", "v", "out", "lse", "dO", "dQ", "uQ", "uK", "uV", "delta", "pk")
        ws_e2e = torch.empty(max(lib.bob_sm100_workspace_bytes(s_, ctypes.byref(g)) for s_ in (0, 1, 2)),
                             dtype=torch.uint8, device=dev)

        def e2e_variant(names_in, with_forward):
            pin = {n: d[n].cpu().pin_memory() for n in names_in}
            stage2 = [{n: torch.empty_like(d[n]) for n in names_all} for _ in range(2)]
            for s_ in stage2:
                s_["dQ1"], s_["dK1"], s_["dV1"] = torch.empty_like(d["dQ"]), torch.empty_like(d["k"]), torch.empty_like(d["v"])
            res2 = [{n: torch.empty_like(t) for n, t in res.items()} for _ in range(2)]
            pin_out2 = [{n: torch.empty(t.shape, dtype=t.dtype, device="cpu").pin_memory() for n, t in res.items()}
                        for _ in range(2)]
            h2d = sum(t.numel() * t.element_size() for t in pin.values())
            d2h = sum(t.numel() * t.element_size() for t in pin_out2[0].values())

            def compute(src, dst, cs):
                c = ctypes.c_void_p(cs)
                if with_forward:
                    _lib.check(lib.bob_sm100_fwd(ctypes.byref(g), vp(src["q"]), vp(src["k"]), vp(src["v"]), vp(src["out"]),
                                                 vp(src["lse"]), vp(ws_e2e), c), "bob_sm100_fwd")
                dq_first = src["dQ"] if with_forward else src["dQ1"]     # shipped dQ is used when it was shipped
                _lib.check(lib.bob_sm100_bwd1(ctypes.byref(g), vp(src["q"]), vp(src["k"]), vp(src["v"]), vp(src["out"]),
                                              vp(src["lse"]), vp(src["dO"]), vp(dq_first), vp(src["dK1"]), vp(src["dV1"]),
                                              vp(src["delta"]), vp(src["pk"]), vp(ws_e2e), c), "bob_sm100_bwd1")
                prob.bwd2(src=src, dst=dst, ws=ws_e2e, cuda_stream=cs)

            def run(n_steps):
                # Steps are pipelined over three streams with two sets of device buffers: while step i
                # computes, step i+1's inputs cross PCIe and step i-1's results go back.
                ev_in, ev_cmp, ev_out = [None, None], [None, None], [None, None]
                barrier()
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
                        compute(stage2[s], res2[s], s_cmp.cuda_stream)
                        ev_cmp[s] = torch.cuda.Event(); ev_cmp[s].record(s_cmp)
                    with torch.cuda.stream(s_out):
                        s_out.wait_event(ev_cmp[s])
                        for n in res:
                            pin_out2[s][n].copy_(res2[s][n], non_blocking=True)
                        ev_out[s] = torch.cuda.Event(); ev_out[s].record(s_out)
                for st_ in (s_in, s_cmp, s_out):
                    stream.wait_stream(st_)
                end.record(stream)
                barrier()
                return start.elapsed_time(end)

            run(3)
            step_ms = max_over_ranks(run(e2e_steps)) / e2e_steps
            launches = (1 if with_forward else 0) + 4
            return {"value": flops_job / (step_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "steps": e2e_steps, "ms_per_step": step_ms,
                    "h2d_gbs_per_rank": h2d / (step_ms * 1e-3) / 1e9, "gpu_launches_per_step": launches}

        e2e = e2e_variant(("q", "k", "v", "dO", "uQ", "uK", "uV"), with_forward=True)
        e2e["how"] = ("operator_inputs: pinned host (q,k,v,dO,uQ,uK,uV: what a caller of the operator owns) -> device -> "
                      "bob_sm100_fwd (out, lse) + bob_sm100_bwd1 (dQ, delta, pk) + bob_sm100_bwd2 -> pinned host "
                      "(Qbar,Kbar,Vbar,dObar) every step; steps pipelined over copy-in / compute / copy-out streams; "
                      "inputs per step exceed L2; credited 12u per step although forward and first backward run too")
        if extras:
            e2e_alt = e2e_variant(("q", "k", "v", "out", "lse", "dO", "dQ", "uQ", "uK", "uV"), with_forward=False)
            e2e_alt["how"] = ("reference_level: pinned host (q,k,v,out,lse,dO,dQ,uQ,uK,uV: what the reference's second "
                              "backward is called with) -> device -> bob_sm100_bwd1 (delta, pk) + bob_sm100_bwd2 -> pinned "
                              "host results every step; same pipelining")

    # ---- the whole two-level chain through the public operator (secondary number) --------------
    chain = None
    if extras and wl["scaling"] == "weak":
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

    # ---- the sharded scaling workload, at every N -------------------------------------------------
    strong_c4 = None
    if extras and args.workload == "c2":
        del prob, d, res, sc
        torch.cuda.empty_cache()
        wl4 = WORKLOADS["c4"]
        p4 = Problem(wl4, world, rank, dev, on_device_inputs=True)
        c4_steps = max(20, args.steps)
        s4 = ClockSampler(local_rank, period_ms=50) if rank == 0 else None
        ms4, _ = timed_steps(p4.bwd2, 3, c4_steps)
        ms4_step = max_over_ranks(sum(ms4)) / c4_steps
        p4.check_status()
        c4_clocks = s4.stop() if s4 else None
        job = p4.flops_job / (ms4_step * 1e-3) / 1e12
        mhz = (c4_clocks or {}).get("sm_mhz")
        strong_c4 = {"workload": wl4["name"], "scaling": "strong", "n_gpus": world, "steps": c4_steps, "warmup": 3,
                     "units_per_rank": p4.B, "ms_per_step": ms4_step, "value": job, "unit": UNIT,
                     "per_gpu_tflops": job / world, "frac_of_measured_peak": job / world / peak,
                     "frac_of_measured_sustained_peak": job / world / peak_sustained if peak_sustained else None,
                     "clocks": c4_clocks, "ms_times_median_sm_mhz": ms4_step * mhz if mhz else None,
                     "flops_per_step_job": p4.flops_job,
                     "note": "per-step CUDA events, L2 flushed between steps, max over ranks; compare runs at "
                             "different N through ms_times_median_sm_mhz as well: a single GPU holding all 64 units "
                             "runs into its power cap, eight GPUs with 8 units each do not"}
        del p4
        torch.cuda.empty_cache()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

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
        "sustained": sustained,
        "other_stages": stage_ms,
        "e2e": e2e if e2e is not None else {"value": None, "unit": UNIT, "h2d_bytes_per_step": None,
                                              "d2h_bytes_per_step": None,
                                              "how": "not measured for the sharded workload (inputs are drawn on the device)"},
        "e2e_reference_level": e2e_alt,
        "gpu_launches": lib.bob_sm100_kernel_launches(_lib.STAGE_BWD2, ctypes.byref(g)) * args.steps,
        "clocks": clocks,
        "wall_s_timed_region": wall,
        "chain": chain,
        "strong_c4": strong_c4,
    }
    if world == 1 and extras:
        line["reference_cuda"] = reference_cuda_record(wl)
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_reference_sample(wl, 3, 1, budget_s=20.0)
    else:
        line["cpu_baseline"] = None
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
