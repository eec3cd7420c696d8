"""PKDA hot-path benchmark.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one forward + backward pass of the chunked PKDA operator over one
batch of synthetic input (benchmark configuration 1: B=8, T=4096, H=16,
d_k=d_v=128, chunk 64, bf16, fp32 initial state, all ten input gradients plus
the initial-state gradients).  With N > 1 (launched by torchrun) every rank runs
that same workload on its own GPU with its own seed: the operator shards by
row x head with no data-path collective, so scaling is weak and NCCL is used
only for the start/stop barriers and the max-over-ranks time.

Rank 0 prints ONE JSON line.  ``value`` is whole-job tokens/s with inputs
resident in HBM, timed as K replays of a CUDA graph of the step (the metric is
defined that way: the reference's benchmark times a captured-graph replay of
forward + backward); the same K steps launched eagerly are timed first, with a
CUDA event pair around every kernel, and reported as ``eager_ms_per_step`` and
``stages_ms_per_step``.  ``e2e`` is the same pass through the public operator with HOST
(pinned) buffers and the host<->device copies inside the timed region;
``roofline`` describes the kernel that took the largest share of the step;
``cpu_baseline`` is the CPU oracle timed on this box's host cores on a bounded
sample; ``decode`` reports the recurrent decode step (configuration 3) as
achieved HBM GB/s.  ``--impl reference`` times the CPU implementation alone.
The graph replays are repeated in rounds of K until the timed region is at least
one second long (``consistency``).  Further legs of the line: ``e2e.copy_floor_ms``
(the same pinned buffers copied with no kernels: each direction alone and both at
once), ``small_batch`` (B=2 with 16 and 8 heads: the regime with fewer (row, head)
units than SMs, where the state scans dominate), ``layer_ops`` (the operators next
to the recurrence, an HBM roofline each) and, at N > 1, ``config4`` (benchmark
configuration 4's per-GPU shape, B=16, T=8192, as max-over-ranks time).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "PKDA fwd+bwd tokens/s/GPU at T=4096; decode state-update GB/s vs HBM peak"
WORKLOADS = {
    # name: (B per GPU, T, H, D)
    "config1": (8, 4096, 16, 128),
    "config4": (16, 8192, 16, 128),
    "profile": (2, 4096, 16, 128),   # small case for ncu captures (working set still > L2)
    "profile_wide": (8, 1024, 16, 128),  # same size, 128 (row, head) units: takes the tcgen05 state scan
}
C = 64
# Algorithmic work per (token, head) for D=128, chunk 64 (dense counts).
FWD_FLOPS = 2 * C * (3 * 128 + 2 * 128) + 6 * 128 * 128 + (2 * C * C) // 3          # 182,955
FWD_BWD_FLOPS = 3 * FWD_FLOPS                                                        # 548,865
FWD_BYTES, BWD_BYTES = 1288, 2328
# Per-kernel algorithmic flops per (token, head): the dense contractions each kernel owns.
K, V = 128, 128
STAGE_FLOPS = {
    "intra_fwd": 2 * (2 * C * K) + 2 * C * K + 2 * C * V + (2 * C * C) // 3,   # M, P, Tm*Kd, Tm*V, inverse
    "scan_fwd": 2 * (2 * K * V),                                              # W*h, kg^T*F
    "out_fwd": 2 * K * V + 2 * C * V,                                         # qg*h, P*F
    "scan_bwd": 3 * (2 * K * V) + 2 * C * V,                                  # kg*dS, qg^T*dO, W^T*dE, P^T*dO
    "intra_bwd": 3 * (2 * K * V) + 3 * (2 * C * V) + 4 * (2 * C * K),         # dqg, dKd, dkg; dR, dM, dP; four gated pair products
}
# DRAM traffic per (token, head) of each kernel: dram__bytes_read.sum + dram__bytes_write.sum of one
# ncu capture on the quarter-size workload (131,072 units), divided by its units; the traffic grows
# in proportion to the units, so a launch of any size moves this many bytes per unit.
STAGE_TRAFFIC_PER_UNIT = {"intra_fwd": 2188, "scan_fwd": 1245, "out_fwd": 1280, "scan_bwd": 1655,
                          "intra_bwd": 4506}
# Bytes per (token, head) that each kernel must read and write by its own interface (its input and
# output tensors, each touched once): the HBM view of the same kernels.
STAGE_IO_BYTES = {
    "intra_fwd": 4 * 256 + (128 + 128 + 5 * 256),             # q,k,v,g -> Aqk, Akk, k_precond, w, u, kg, qg
    "scan_fwd": 3 * 256 + (512 + 256),                          # w,u,kg -> h, v_new
    "out_fwd": 512 + 256 + 256 + 128 + 256,                     # h, qg, v_new, Aqk -> o
    "scan_bwd": 4 * 256 + 128 + (512 + 256),                    # kg,w,qg,dO,Aqk -> dh, dF
    "intra_bwd": 7 * 256 + 2 * 128 + 2 * 512 + (3 * 256 + 2 * 512 + 256),  # dO,dF,E,q,k,kt,g,Akk,Aqk,h,dh -> dq,dv,dg,dk_read,dkt(+k again)
}
# The kernel behind each stage name (tcgen05 / tensor-memory build; --legacy runs the mma.sync ones).
STAGE_KERNEL = {"intra_fwd": "pkda_intra_fwd_tc_kernel", "scan_fwd": "pkda_scan_fwd_tc_kernel",
                "out_fwd": "pkda_out_fwd_tc_kernel", "scan_bwd": "pkda_scan_bwd_tc_kernel",
                "intra_bwd": "pkda_intra_bwd_tc_kernel"}
DECODE_BYTES_PER_UNIT = 2 * 4 * 128 * 128 + 2 * 4 * 128 + 4 * 2 * 128 + 8 + 2 * 128   # 133,384


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            m = json.load(f)
        return {"hbm_gbs": m["hbm_gbs"], "bf16_tflops": m["bf16_tflops"],
                "bf16_tflops_sustained": m.get("bf16_tflops_sustained", m["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, val in zip(names, r[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def _oracle_seconds(T: int, H: int, D: int) -> float:
    from delta_feedback_experiment_b200.synthetic import INPUT_NAMES, make_inputs
    from oracle.pkda_oracle import pkda_oracle_with_grads
    d = make_inputs(1, T, H, D, seed=123, dist="unit", dtype=torch.bfloat16, with_state=True)
    t0 = time.perf_counter()
    pkda_oracle_with_grads([d[n] for n in INPUT_NAMES], d["do"], initial_state=d["initial_state"],
                           initial_A_state=d["initial_A_state"], dtype=torch.float32)
    return time.perf_counter() - t0


def cpu_oracle_rate(T: int, H: int, D: int, threads: int | None = None) -> dict:
    """Times the CPU oracle (forward + autograd backward) on a bounded sample of the workload and
    converts to whole-token throughput at H heads.  The sample is ONE (row, head) unit of the full
    length T (a full row of H heads at T = 4096 needs tens of GB for the autograd tape).  The CPU
    recurrence is a per-token Python loop vectorised over the heads, so its cost does not grow in
    proportion to H: the factor between one head and all H heads is MEASURED on a short length
    (T = 256) and applied to the long unit, instead of assuming H."""
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    unit = _oracle_seconds(T, 1, D)
    short = min(T, 256)
    s1 = min(_oracle_seconds(short, 1, D) for _ in range(2))
    sh = min(_oracle_seconds(short, H, D) for _ in range(2))
    factor = max(1.0, sh / s1)
    return {"value": T / (unit * factor), "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"one (row, head) unit of the workload (T={T}, d={D}, fwd+bwd on the CPU oracle): "
                      f"{unit:.2f} s; a full row of H={H} heads costs {factor:.2f}x one head (measured at "
                      f"T={short}: {s1:.3f} s vs {sh:.3f} s), not {H}x, and the rate uses the measured factor",
            "seconds_per_unit": unit, "head_factor": factor}


def run_reference(args, rank: int, world: int) -> None:
    if rank != 0:
        return
    B, T, H, D = WORKLOADS[args.workload]
    # every step is one bounded sample: one (row, head) unit of the workload
    rates = []
    t_all = time.perf_counter()
    for i in range(args.warmup + args.steps):
        r = cpu_oracle_rate(T, H, D)
        if i >= args.warmup:
            rates.append(r)
    sec = statistics.mean(x["seconds_per_unit"] * x["head_factor"] for x in rates)
    value = T / sec
    base = rates[0]
    base["value"] = value
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": f"{args.workload}: B={B} T={T} H={H} d={D} chunk=64 fwd+bwd; each step "
                               "times one (row, head) unit of it on the host cores and the measured "
                               "cost factor of a full row of heads"},
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.perf_counter() - t_all,
    }
    print(json.dumps(line), flush=True)


def run_decode(device, steps: int, warmup: int, pk: dict) -> dict:
    """Configuration 3: B=256, H=32, d=128, fp32 state updated in place, one token per step."""
    from delta_feedback_experiment_b200 import _lib, fused_recurrent_precond_kda
    from delta_feedback_experiment_b200.synthetic import INPUT_NAMES, make_inputs
    B, H, D, NIN = 256, 32, 128, 8
    d = make_inputs(B, NIN, H, D, seed=300, dist="unit", dtype=torch.bfloat16, with_state=True)
    dev = {n: d[n].to(device) for n in INPUT_NAMES}
    S = d["initial_state"].to(device)
    A = d["initial_A_state"].to(device)
    ins = [{n: dev[n][:, t:t + 1].contiguous() for n in INPUT_NAMES[:7]} for t in range(NIN)]

    def step(i):
        fused_recurrent_precond_kda(
            **ins[i % NIN], A_log=dev["A_log"], dt_bias=dev["dt_bias"], initial_state=S,
            initial_A_state=A, output_final_state=True, log_atk_scale=dev["log_atk_scale"],
            inplace_state=True)

    for i in range(warmup):
        step(i)
    torch.cuda.synchronize(device)
    _lib.stage_timing(True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step(i)
    e1.record()
    torch.cuda.synchronize(device)
    stages = _lib.stage_timing_read()
    _lib.stage_timing(False)
    wall_ms = e0.elapsed_time(e1) / steps
    k_ms, k_n = stages["recurrent"]
    fused = run_decode_fused(device, dev, S, A, B, H, D, min(steps, 256), warmup, pk)
    bytes_per_step = DECODE_BYTES_PER_UNIT * B * H
    achieved = bytes_per_step / (k_ms / k_n * 1e-3) / 1e9
    return {
        "workload": f"config3: B={B} H={H} d={D} fp32 state in place, {steps} sequential 1-token steps",
        "ms_per_step": wall_ms, "kernel_ms": k_ms / k_n,
        "state_update_gbs_wall": bytes_per_step / (wall_ms * 1e-3) / 1e9,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "traffic": None,
                     "algorithmic_bytes_per_launch": bytes_per_step, "peak_source": pk["source"]},
        "finite": bool(torch.isfinite(S).all().item()),
        "fused_step": fused,
    }


def run_decode_fused(device, dev, S, A, B, H, D, steps, warmup, pk) -> dict:
    """The same decode step with the layer's convolution (over the cached history) and RMS-norm gate
    fused into the launch: one kernel per step, cache (histories, S, A) updated in place."""
    from delta_feedback_experiment_b200 import _lib
    from delta_feedback_experiment_b200.layer_ops import pkda_decode_step
    W, taps, NIN = H * D, 4, 8
    gen = torch.Generator().manual_seed(301)
    bf = lambda t: t.bfloat16().to(device)
    qkv = [bf(torch.randn(B, 3 * W, generator=gen)) for _ in range(NIN)]
    gate = [bf(torch.randn(B, H, D, generator=gen)) for _ in range(NIN)]
    conv = [bf(torch.randn(B, W, taps - 1, generator=gen)) for _ in range(3)]
    conv_w = (torch.randn(3 * W, taps, generator=gen) * 0.5).to(device)
    norm_w = torch.ones(D, device=device)
    ins = [{n: dev[n][:, t].contiguous() for n in ("g", "g_atk", "beta_atk", "beta")} for t in range(NIN)]

    def step(i):
        j = i % NIN
        return pkda_decode_step(qkv[j], conv, conv_w, ins[j]["g"], ins[j]["g_atk"], ins[j]["beta_atk"], ins[j]["beta"],
                                dev["A_log"], dev["dt_bias"], dev["log_atk_scale"], S, A, gate[j], norm_w, D)

    for i in range(warmup):
        step(i)
    torch.cuda.synchronize(device)
    _lib.stage_timing(True)
    out = None
    for i in range(steps):
        out = step(i)
    torch.cuda.synchronize(device)
    stages = _lib.stage_timing_read()
    _lib.stage_timing(False)
    k_ms, k_n = stages["decode_step"]
    # per (row, head): state and a_state read+write, the projection row, histories read+write, raw decay,
    # gate logits, output, four scalars
    per_unit = 2 * 4 * D * D + 2 * 4 * D + 3 * D * 2 + 2 * 3 * D * (taps - 1) * 2 + 3 * D * 2 + 12
    nbytes = per_unit * B * H
    achieved = nbytes / (k_ms / k_n * 1e-3) / 1e9
    return {"kernel_ms": k_ms / k_n, "launches_per_step": 1,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / pk["hbm_gbs"], "traffic": None,
                         "algorithmic_bytes_per_launch": nbytes, "peak_source": pk["source"]},
            "finite": bool(torch.isfinite(out.float()).all().item())}


def capture_step(device, fn):
    """Runs fn once on a side stream (allocator warm-up), then captures it into a CUDA graph."""
    side = torch.cuda.Stream(device)
    side.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream(device).wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    return graph


def time_graph(device, fn, steps: int, min_seconds: float = 0.3):
    """ms per replay of the captured fn (at least `steps` replays and `min_seconds` of them)."""
    graph = capture_step(device, fn)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize(device)
    n = max(steps, int(min_seconds * 1e3 / max(e0.elapsed_time(e1), 1e-3)) + 1)
    e0.record()
    for _ in range(n):
        graph.replay()
    e1.record()
    torch.cuda.synchronize(device)
    return e0.elapsed_time(e1) / n, n


def run_config4(device, dev, fwd_bwd, world, B, T, H, dist) -> dict:
    from delta_feedback_experiment_b200.synthetic import INPUT_NAMES
    rows = INPUT_NAMES[:7] + ("do",)
    big = {n: t.detach().clone() for n, t in dev.items()}  # fresh leaves: no autograd history from earlier steps
    for n in rows:
        x = dev[n].detach()
        big[n] = torch.cat([torch.cat([x, x], dim=1)] * 2, dim=0).contiguous()
    for n in ("initial_state", "initial_A_state"):
        big[n] = torch.cat([dev[n].detach(), dev[n].detach()], dim=0).contiguous()
    B4, T4 = big["q"].shape[0], big["q"].shape[1]
    dist.barrier()
    ms, n = time_graph(device, lambda: fwd_bwd(big), 5, 0.5)
    t = torch.tensor([ms], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    return {"workload": f"config4: B={B4}/GPU T={T4} H={H} d=128 chunk=64 bf16 fwd+bwd (rows and time of the "
                        "headline tensors repeated on the device)",
            "ms_per_step": ms, "replays": n, "value": world * B4 * T4 / (ms * 1e-3), "unit": "tokens/s",
            "timed_as": "CUDA-graph replay, max over ranks"}


def run_small_batch(device, dev, fwd_bwd, T) -> dict:
    """Rows 2, heads 16 and 8 (the defaults of the reference's operator benchmark, scripts/pkda_bench.py:288-290)."""
    from delta_feedback_experiment_b200 import _lib
    from delta_feedback_experiment_b200.synthetic import INPUT_NAMES
    out = {}
    for heads in (16, 8):
        # fresh leaves (clone of detached slices): no autograd history from the earlier steps
        small = {n: dev[n].detach()[:2, :, :heads].clone()
                 for n in ("q", "k", "v", "g", "do", "g_atk", "beta_atk", "beta")}
        small["initial_state"] = dev["initial_state"].detach()[:2, :heads].clone()
        small["initial_A_state"] = dev["initial_A_state"].detach()[:2, :heads].clone()
        small["A_log"] = dev["A_log"].detach()[:heads].clone()
        small["dt_bias"] = dev["dt_bias"].detach()[:heads * 128].clone()
        small["log_atk_scale"] = dev["log_atk_scale"].detach()[:heads].clone()
        for _ in range(3):
            fwd_bwd(small)
        torch.cuda.synchronize(device)
        _lib.stage_timing(True)
        for _ in range(5):
            fwd_bwd(small)
        torch.cuda.synchronize(device)
        stages = _lib.stage_timing_read()
        _lib.stage_timing(False)
        ms, n = time_graph(device, lambda: fwd_bwd(small), 10, 0.2)
        out[f"B2_H{heads}"] = {"units": 2 * heads, "ms_per_step": ms, "replays": n,
                              "tokens_per_s": 2 * T / (ms * 1e-3),
                              "stages_ms_per_step": {k: v / 5 for k, (v, _) in stages.items()}}
    return out


def copy_floor(device, host_in: dict, do, out_host: dict) -> dict:
    """What the host<->device copies of one end-to-end step cost by themselves: every input tensor in
    (one asynchronous copy each, from the same pinned buffers), every result out, and both directions
    at once on two streams."""
    ins = [t for t in host_in.values() if t is not None] + [do]
    dev_in = [torch.empty(t.shape, dtype=t.dtype, device=device) for t in ins]
    outs = list(out_host.values())
    dev_out = [torch.empty(t.shape, dtype=t.dtype, device=device) for t in outs]
    s1, s2 = torch.cuda.Stream(device), torch.cuda.Stream(device)

    def h2d():
        with torch.cuda.stream(s1):
            for d, h in zip(dev_in, ins):
                d.copy_(h, non_blocking=True)

    def d2h():
        with torch.cuda.stream(s2):
            for h, d in zip(outs, dev_out):
                h.copy_(d, non_blocking=True)

    def timed(fns):
        best = None
        for _ in range(3):
            torch.cuda.synchronize(device)
            t0 = time.perf_counter()
            for f in fns:
                f()
            torch.cuda.synchronize(device)
            dt = (time.perf_counter() - t0) * 1e3
            best = dt if best is None else min(best, dt)
        return best

    return {"h2d_ms": timed([h2d]), "d2h_ms": timed([d2h]), "both_ms": timed([h2d, d2h]),
            "note": "pinned host buffers of the end-to-end step, copies alone (no kernels), best of 3, wall clock "
                    "around a device synchronise"}


def bind_to_gpu_cpus(index: int):
    """Restricts this process to the CPU cores NVML reports as local to GPU `index` (same NUMA
    node / PCIe root), so that the pinned host buffers of the end-to-end leg are allocated and
    touched next to the GPU they feed.  Only this process's CPU affinity changes; returns the
    number of cores kept, or None when NVML gives no answer."""
    try:
        import pynvml
        pynvml.nvmlInit()
        try:  # match the CUDA device by its PCI address (NVML numbering can differ from CUDA's)
            pr = torch.cuda.get_device_properties(index)
            handle = pynvml.nvmlDeviceGetHandleByPciBusId(
                f"{pr.pci_domain_id:08x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0")
        except Exception:
            handle = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        allowed = os.sched_getaffinity(0)
        cpus = {64 * w + b for w, m in enumerate(mask) for b in range(64) if (m >> b) & 1} & allowed
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        pass
    return None


def run_layer_ops(device, B: int, T: int, H: int, D: int, steps: int, warmup: int, pk: dict) -> dict:
    """The two fused operators next to the recurrence on the headline shape: Q|K|V convolution
    (+SiLU +L2 norm) and RMS-norm x sigmoid gate, forward and backward, each against the HBM roofline
    with its algorithmic bytes (every input read once, every output written once)."""
    from delta_feedback_experiment_b200 import _lib, layer_ops
    W = H * D
    gen = torch.Generator().manual_seed(77)
    x = torch.randn(B, T, 3 * W, generator=gen).bfloat16().to(device)
    wconv = (torch.randn(3 * W, 4, generator=gen) * 0.5).to(device)
    dqkv = [torch.randn(B, T, W, generator=gen).bfloat16().to(device) for _ in range(3)]
    o = torch.randn(B, T, H, D, generator=gen).bfloat16().to(device)
    gate = torch.randn(B, T, H, D, generator=gen).bfloat16().to(device)
    wnorm = torch.ones(D, device=device)
    rstd_box = []

    def once():
        layer_ops.qkv_conv_forward(x, wconv, D, 2 * W, 1e-6)
        layer_ops.qkv_conv_backward(x, wconv, *dqkv, D, 2 * W, 1e-6)
        _, rstd = layer_ops.norm_gate_forward(o, gate, wnorm, 1e-6)
        layer_ops.norm_gate_backward(o, gate, wnorm, rstd, dqkv[0].view(B, T, H, D), 1e-6)

    for _ in range(warmup):
        once()
    torch.cuda.synchronize(device)
    _lib.stage_timing(True)
    for _ in range(steps):
        once()
    torch.cuda.synchronize(device)
    stages = _lib.stage_timing_read()
    _lib.stage_timing(False)
    tokens, rows = B * T, B * T * H
    algo = {  # bytes per launch
        "qkv_conv_fwd": tokens * (2 * 3 * W * 2),
        "qkv_conv_bwd": tokens * (3 * 3 * W * 2),
        "norm_gate_fwd": rows * (3 * D * 2 + 4),
        "norm_gate_bwd": rows * (5 * D * 2 + 4),
    }
    out = {"workload": f"B={B} T={T} H={H} d={D} bf16 (x [B,T,{3 * W}], 4 taps; o, gate [B,T,H,{D}]); "
                       "working sets larger than L2"}
    for name, nbytes in algo.items():
        ms, n = stages[name]
        achieved = nbytes / (ms / n * 1e-3) / 1e9
        out[name] = {"kernel_ms": ms / n, "roofline": {
            "bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
            "frac": achieved / pk["hbm_gbs"], "traffic": None, "algorithmic_bytes_per_launch": nbytes,
            "peak_source": pk["source"]}}
    for name in ("qkv_conv_dw", "norm_gate_dw"):
        ms, n = stages[name]
        out[name] = {"kernel_ms": ms / n}
    return out


def run_ours(args, rank: int, world: int, local_rank: int) -> None:
    import torch.distributed as dist
    from delta_feedback_experiment_b200 import _lib, chunk_precond_kda, ops
    from delta_feedback_experiment_b200.synthetic import INPUT_NAMES, make_inputs

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU path")
    _lib.load()
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    numa = bind_to_gpu_cpus(local_rank)  # pinned host buffers then live next to this rank's GPU
    if world > 1:
        # keep NCCL's own banner off stdout: rank 0 prints exactly one JSON line there
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=device)
    B, T, H, D = WORKLOADS[args.workload]
    pk = peaks()
    if args.only_decode:  # profiling aid: the decode legs alone
        print(json.dumps({"note": "profiling run (decode only): not a benchmark line",
                          "decode": run_decode(device, args.decode_steps, 16, pk)}), flush=True)
        return
    if args.only_layer:  # profiling aid: the convolution / norm-gate operators alone
        print(json.dumps({"note": "profiling run (layer operators only): not a benchmark line",
                          "layer_ops": run_layer_ops(device, B, T, H, D, args.steps, args.warmup, pk)}), flush=True)
        return

    for stage in filter(None, args.legacy.split(",")):  # "stage" (= the mma.sync kernel) or "stage=variant"
        name, _, variant = stage.partition("=")
        _lib.set_variant(name, int(variant) if variant else 1)
    d = make_inputs(B, T, H, D, seed=1000 + rank, dist=args.dist, dtype=torch.bfloat16, with_state=True)
    host = {n: d[n].pin_memory() for n in (*INPUT_NAMES, "do", "initial_state", "initial_A_state")}
    dev = {n: t.to(device) for n, t in host.items()}
    lean = bool(args.lean)

    def fwd_bwd(t):
        leaves = [t[n].requires_grad_(True) for n in INPUT_NAMES]
        S0 = t["initial_state"].requires_grad_(True)
        A0 = t["initial_A_state"].requires_grad_(True)
        kw = dict(zip(INPUT_NAMES, leaves))
        scale_c = kw.pop("log_atk_scale")
        o, _, _ = chunk_precond_kda(**kw, initial_state=S0, initial_A_state=A0,
                                    output_final_state=False, log_atk_scale=scale_c,
                                    disable_recompute=not lean)
        grads = torch.autograd.grad(o, leaves + [S0, A0], t["do"])
        return o, grads

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    for _ in range(args.warmup):
        fwd_bwd(dev)
    barrier()
    launches0 = ops.LAUNCHES
    _lib.stage_timing(True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    clocks = ClockSampler(local_rank)
    clocks.__enter__()  # sampled over both timed regions (device-resident steps, then end-to-end steps)
    barrier()
    e0.record()
    for _ in range(args.steps):
        fwd_bwd(dev)
    e1.record()
    barrier()
    total_ms = e0.elapsed_time(e1)
    stages = _lib.stage_timing_read()
    _lib.stage_timing(False)
    launches = ops.LAUNCHES - launches0
    if world > 1:
        tmax = torch.tensor([total_ms], device=device)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        total_ms = float(tmax.item())
        lsum = torch.tensor([launches], device=device, dtype=torch.int64)
        dist.all_reduce(lsum)
        launches = int(lsum.item())
    ms_per_step = total_ms / args.steps
    value = world * B * T / (ms_per_step * 1e-3)

    # The same step replayed from a CUDA graph (how the reference's own benchmark times this operator).
    # The K steps are replayed `rounds` times back to back so that the timed region lasts at least a
    # second (the sustained peaks the roofline divides by are measured over seconds); ms_per_step is
    # the mean over all K * rounds replays.
    graph_ms, rounds, graph_region_s = None, 1, None
    try:
        graph = capture_step(device, lambda: fwd_bwd(dev))
        graph.replay()
        torch.cuda.synchronize(device)
        rounds = max(1, -(-int(1000.0) // max(1, int(ms_per_step * args.steps))))
        if world > 1:  # the same number of replays on every rank
            rt = torch.tensor([rounds], device=device)
            dist.all_reduce(rt, op=dist.ReduceOp.MAX)
            rounds = int(rt.item())
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        g0.record()
        for _ in range(args.steps * rounds):
            graph.replay()
        g1.record()
        barrier()
        graph_region_s = g0.elapsed_time(g1) * 1e-3
        graph_ms = graph_region_s * 1e3 / (args.steps * rounds)
        del graph
    except Exception as exc:  # capture is optional: report why it was skipped
        graph_ms = f"not measured: {type(exc).__name__}"
    # Headline: the metric is defined on a captured-graph replay of forward + backward (how the
    # reference's benchmark times the operator); the eager figure (with the per-kernel events that
    # feed the roofline) is reported beside it.  If any rank could not capture, all report eager.
    eager_ms = ms_per_step
    use_graph = isinstance(graph_ms, float)
    if world > 1:
        flag = torch.tensor([1 if use_graph else 0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        use_graph = bool(flag.item())
        if use_graph:  # every rank captured: the step time is the slowest rank's
            gmax = torch.tensor([graph_ms], device=device)
            dist.all_reduce(gmax, op=dist.ReduceOp.MAX)
            graph_ms = float(gmax.item())
    if use_graph:
        ms_per_step = graph_ms
        value = world * B * T / (ms_per_step * 1e-3)

    # Multi-GPU runs also time the per-GPU shape of the eight-GPU configuration (B=16/GPU, T=8192):
    # the device tensors of the headline workload repeated along rows and time, graph replay, max over ranks.
    config4 = None
    if world > 1 and args.workload == "config1" and not args.no_config4:
        config4 = run_config4(device, dev, fwd_bwd, world, B, T, H, dist)

    # The small-batch regime the reference's own operator benchmark and trainer run at (2 rows of 16 or 8
    # heads, T=4096: 32 / 16 (row, head) units, far fewer than SMs): rank 0 only, device-resident.
    small = None
    if rank == 0 and not args.no_small and not args.no_e2e:
        small = run_small_batch(device, dev, fwd_bwd, T)

    # ---- end to end through the public operator with host buffers
    if args.no_e2e:
        clocks.__exit__(None, None, None)
        if world > 1:
            dist.destroy_process_group()
        if rank == 0:
            print(json.dumps({"note": "profiling run (no e2e leg): not a benchmark line",
                              "ms_per_step": ms_per_step, "distribution": args.dist, "legacy_stages": args.legacy,
                              "stages_ms_per_step": {n: ms / args.steps for n, (ms, _) in stages.items()}}))
        return
    # The public call for host-resident data: HostStep streams row slices so that the copy in, the
    # kernels and the copy out overlap.  Every step moves all inputs in and all results out.
    from delta_feedback_experiment_b200.host_pipeline import HostStep
    e2e_steps = max(1, min(args.steps, 5))
    e2e_plan = tuple(int(x) for x in str(args.e2e_slices).split(","))
    if len(e2e_plan) == 1:
        e2e_plan = e2e_plan[0]
    elif sum(e2e_plan) != B:
        e2e_plan = min(8, B)
    host_step = HostStep(device, slices=e2e_plan, lean=lean)
    host_in = {n: host[n] for n in (*INPUT_NAMES, "initial_state", "initial_A_state")}

    def e2e_step():
        return host_step(host_in, host["do"])

    e2e_step()
    barrier()
    e0.record()
    for _ in range(e2e_steps):
        out_host = e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    clocks.__exit__(None, None, None)
    if world > 1:
        tmax = torch.tensor([e2e_ms], device=device)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        e2e_ms = float(tmax.item())
    h2d, d2h = host_step.h2d_bytes, host_step.d2h_bytes
    e2e_finite = all(bool(torch.isfinite(t.float()).all()) for t in out_host.values())
    floor = copy_floor(device, host_in, host["do"], out_host)
    if world > 1:  # the slowest rank's copies
        ft = torch.tensor([floor["h2d_ms"], floor["d2h_ms"], floor["both_ms"]], device=device)
        dist.all_reduce(ft, op=dist.ReduceOp.MAX)
        floor["h2d_ms"], floor["d2h_ms"], floor["both_ms"] = (float(x) for x in ft.tolist())

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel (largest share of the timed step)
    units = B * T * H  # (token, head) units one launch processes
    per_launch = {name: ms / n for name, (ms, n) in stages.items()}
    step_kernel_ms = sum(ms for ms, _ in stages.values()) / args.steps
    if "out_fwd" not in stages:  # the state scan formed the output too: its products belong to that launch
        STAGE_FLOPS["scan_fwd"] += STAGE_FLOPS["out_fwd"]
        STAGE_TRAFFIC_PER_UNIT["scan_fwd"] = 1894  # (ncu, same capture: 161.0 MB read + 87.2 MB written per 131,072 units)
        STAGE_IO_BYTES["scan_fwd"] += 256 + 128 + 256  # qg, Aqk -> o
    top = max((n for n in stages if n in STAGE_FLOPS), key=lambda n: stages[n][0])
    top_ms = per_launch[top]
    achieved_tf = STAGE_FLOPS[top] * units / (top_ms * 1e-3) / 1e12
    peak_tf = pk["bf16_tflops_sustained"]
    roofline = {
        "bound": "tensor", "kernel": f"pkda_{top}_kernel" if top in args.legacy.split(",") else STAGE_KERNEL[top],
        "achieved": achieved_tf, "peak": peak_tf,
        "unit": "TFLOP/s", "frac": achieved_tf / peak_tf,
        "traffic": STAGE_TRAFFIC_PER_UNIT[top] * units if D == 128 else None,
        "traffic_source": "ncu capture of a quarter-size launch, scaled by the units processed",
        "launch_ms": top_ms, "algorithmic_flops_per_launch": STAGE_FLOPS[top] * units,
        "peak_source": pk["source"] + " (sustained bf16 GEMM; kernel timed inside a long step)",
        "share_of_step": stages[top][0] / sum(ms for ms, _ in stages.values()),
        # the same kernel against the HBM roof: its own inputs and outputs, each touched once
        "hbm_view": {"io_bytes_per_launch": STAGE_IO_BYTES[top] * units,
                     "achieved_gbs": STAGE_IO_BYTES[top] * units / (top_ms * 1e-3) / 1e9,
                     "frac": STAGE_IO_BYTES[top] * units / (top_ms * 1e-3) / 1e9 / pk["hbm_gbs"]},
        "whole_step": {
            "tensor_frac": FWD_BWD_FLOPS * units / (ms_per_step * 1e-3) / 1e12 / peak_tf,
            "hbm_frac": (FWD_BYTES + BWD_BYTES) * units / (ms_per_step * 1e-3) / 1e9 / pk["hbm_gbs"],
            "algorithmic_flops": FWD_BWD_FLOPS * units,
            "algorithmic_bytes": (FWD_BYTES + BWD_BYTES) * units,
        },
    }
    line = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {
            "workload": f"{args.workload}: B={B}/GPU T={T} H={H} d_k=d_v={D} chunk=64 bf16 fwd+bwd, "
                        "fp32 initial state, ten input gradients + initial-state gradients",
            "distribution": args.dist, "legacy_stages": args.legacy,
            "saving": "lean (recompute)" if lean else "full (retained intermediates)",
            "l2": "no flush: each of q,k,v,g,dO is larger than the 126 MB L2",
            "parallelism": f"{world} independent replica shard(s) by row x head, no collective",
            "host_cores_bound_to_gpu": numa,
        },
        "roofline": roofline,
        "e2e": {"value": world * B * T / (e2e_ms * 1e-3), "unit": "tokens/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                "steps": e2e_steps, "finite": e2e_finite, "copy_floor_ms": floor,
                "call": f"host_pipeline.HostStep(slices={args.e2e_slices}): pinned host inputs -> forward+backward -> "
                        "pinned host outputs, copies overlapped with the kernels by row slice; the kernels of a "
                        "slice replay from two CUDA graphs (forward, backward) on fixed device buffers"},
        "gpu_launches": launches,
        "clocks": clocks.summary(),
        "stages_ms_per_step": {n: ms / args.steps for n, (ms, _) in stages.items()},
        "kernel_ms_per_step": step_kernel_ms,
        "graph_replay_ms_per_step": graph_ms,
        "eager_ms_per_step": eager_ms,
        "timed_as": "CUDA-graph replay of forward+backward" if use_graph else "eager launches",
        "consistency": {"timed_region_s": graph_region_s, "replays": args.steps * rounds,
                        "rounds_of_steps": rounds},
    }
    if config4 is not None:
        line["config4"] = config4
    if small is not None:
        line["small_batch"] = small
    if not args.no_decode:
        line["decode"] = run_decode(device, args.decode_steps, 16, pk)
    if not args.no_layer:
        line["layer_ops"] = run_layer_ops(device, B, T, H, D, 10, 3, pk)
    if not args.no_cpu and world == 1:  # the CPU baseline belongs to the single-GPU line
        cb = cpu_oracle_rate(T, H, D)
        line["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--workload", choices=tuple(WORKLOADS), default="config1")
    ap.add_argument("--lean", type=int, default=0, help="1: recompute w,kg,v_new,h,qg in backward")
    ap.add_argument("--dist", choices=("unit", "production"), default="unit",
                    help="input distribution: the benchmark configurations' (unit) or the strong per-channel decay "
                         "of the reference's own operator benchmark (production)")
    ap.add_argument("--legacy", default="", help="comma-separated stages pinned to their mma.sync kernels (A/B runs)")
    ap.add_argument("--decode-steps", type=int, default=1024)
    ap.add_argument("--e2e-slices", default="8",
                    help="row slices of the host-memory step: a count of equal slices, or row counts separated by commas")
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-layer", action="store_true", help="skip the convolution / norm-gate operators")
    ap.add_argument("--no-e2e", action="store_true", help="profiling aid: device-resident leg only")
    ap.add_argument("--no-config4", action="store_true", help="multi-GPU runs: skip the B=16, T=8192 sub-measurement")
    ap.add_argument("--no-small", action="store_true", help="skip the small-batch (2 rows) sub-measurement")
    ap.add_argument("--only-layer", action="store_true", help="profiling aid: layer operators only")
    ap.add_argument("--only-decode", action="store_true", help="profiling aid: decode legs only")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        if world > 1:
            args.no_decode = True if rank != 0 else args.no_decode
            args.no_layer = True if rank != 0 else args.no_layer
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
