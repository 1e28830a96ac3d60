#!/usr/bin/env python
"""Benchmark of the GDN hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one pass of the hot path over one batch of seeded synthetic input of the shapes in
BASELINE.json.  Workloads:
  gdn_fwd_conv   config 1: causal_conv1d (W=4, SiLU) over x[8,4096,8192] bf16, then chunked GDN forward,
                 B=8 T=4096 HQK=16 HV=32 K=V=128, nonzero fp32 h0
  gdn_fwd_bwd    config 2: the same shapes, forward + backward (when the backward kernels are present)
With N > 1 every rank (one process per GPU, launched by torch.distributed.run) processes its own
batch of that shape (weak scaling, no collective on the data path); NCCL is used only for the
barrier and the max-over-ranks reduction of the measured time.  Rank 0 prints ONE JSON line.

`--impl reference` times the reference's CPU algorithm (the oracle port of its naive fp32 torch
recurrence) on the host cores for the same metric, on a bounded sample of the workload.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch
import torch.nn.functional as F

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO / "flash-linear-attention-npu_b200"))
sys.path.insert(0, str(REPO))

CFG = dict(B=8, T=4096, HK=16, HV=32, K=128, V=128, D=8192, W=4)
FWD_FLOP_PER_TOKEN_HEAD = 182955.0      # KK^T, inverse, w/u, state, output (dense 64x64 tiles, no causal credit)
BWD_FLOP_PER_TOKEN_HEAD = 524288.0
# Algorithmic FLOPs per token per value head of each kernel (dense 64x64 tiles; split-precision passes not counted):
KERNEL_FLOP_PER_TOKEN_HEAD = {
    "gdn_fwd": 182955.0 - 16384.0 - 2731.0,        # [Q;K]S, QK^T, X Z, P v_new, K^T vhat  (all but KK^T + inverse)
    "gdn_bwd_dhu": 147456.0,                        # K dS', QK^T, P^T dO, X^T dVn, [Q^T|K^T][dO~; dR]
    "gdn_bwd_par": 212992.0,                        # [dO;dZ]Vn^T, [dO;dZ]S^T, Vn dS'^T, [dP;dA]K, [dP^T|dA^T][Q;K], [Q;K]K^T / G
}
KERNEL_NAMES = {"gdn_fwd": "gdn_fwd_kernel", "gdn_bwd_dhu": "gdn_bwd_dhu_kernel", "gdn_bwd_par": "gdn_bwd_par_kernel"}
DEFAULT_WORKLOAD = "gdn_fwd_bwd"


def _peaks():
    p = REPO / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for nm, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def make_inputs(device, seed):
    """Config-1 tensors (BASELINE.json): q,k ~ N(0,1) L2-normalised; v ~ N(0,1); g = logsigmoid(N(0,1));
    beta = sigmoid(N(0,1)); h0 ~ 0.1 N(0,1) fp32; conv input x ~ N(0,1) with weights ~ N(0, 1/4)."""
    c = CFG
    g_ = torch.Generator(device=device).manual_seed(seed)
    rn = lambda *s: torch.randn(*s, device=device, generator=g_)  # noqa: E731
    d = {}
    d["q"] = F.normalize(rn(c["B"], c["T"], c["HK"], c["K"]), dim=-1).bfloat16()
    d["k"] = F.normalize(rn(c["B"], c["T"], c["HK"], c["K"]), dim=-1).bfloat16()
    d["v"] = rn(c["B"], c["T"], c["HV"], c["V"]).bfloat16()
    d["g"] = F.logsigmoid(rn(c["B"], c["T"], c["HV"])).bfloat16()
    d["beta"] = torch.sigmoid(rn(c["B"], c["T"], c["HV"])).bfloat16()
    d["h0"] = 0.1 * rn(c["B"], c["HV"], c["K"], c["V"])
    d["x"] = rn(c["B"], c["T"], c["D"]).bfloat16()
    d["w"] = (0.5 * rn(c["D"], c["W"])).bfloat16()
    d["bias"] = torch.zeros(c["D"], device=device, dtype=torch.bfloat16)
    d["do"] = rn(c["B"], c["T"], c["HV"], c["V"]).bfloat16()
    d["dht"] = 0.1 * rn(c["B"], c["HV"], c["K"], c["V"])
    return d


def step_device(d, workload):
    """One pass of the hot path with device-resident inputs.  Returns the outputs of the step."""
    import fla_b200.ops as ops
    if workload == "gdn_fwd_conv":
        y, _ = ops.causal_conv1d(d["x"], d["w"], d["bias"], activation="silu")
        o, ht = ops.chunk_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"],
                                           output_final_state=True)
        return y, o, ht
    o, ht, grads = ops.chunk_gated_delta_rule_fwd_bwd(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"],
                                                      initial_state=d["h0"], dht=d["dht"])
    return (o, ht) + tuple(grads)


def launches_per_step(workload):
    return 3 if workload == "gdn_fwd_conv" else 4      # conv + prep + fwd  |  prep + fwd + bwd_dhu + bwd_par


def kernel_time(lib, name):
    ms, n = ctypes.c_float(0), ctypes.c_int(0)
    lib.fla_b200_kernel_timing_read(name.encode(), ctypes.byref(ms), ctypes.byref(n))
    return ms.value, n.value


def cpu_reference_tokens_per_s(workload, threads, steps=1, warmup=0):
    """The reference's CPU algorithm for the same step on a bounded sample: B=1, T=1024 at full head
    count (the naive recurrence costs the same per token at any T), plus the conv reference over the
    same tokens for the conv workload.  Returns (tokens/s, description)."""
    import oracle
    torch.set_num_threads(threads)
    c = CFG
    Ts = 1024
    inp = oracle.make_gdn_inputs(1, Ts, c["HK"], c["HV"], c["K"], c["V"], seed=1001)
    xs = torch.randn(1, c["D"], Ts)
    w = 0.5 * torch.randn(c["D"], c["W"])

    def one():
        if workload == "gdn_fwd_conv":
            oracle.causal_conv1d_ref(xs, w, None, None, False, "silu")
            oracle.gdn_reference_fwd_bwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], initial_state=inp["h0"])
        else:
            oracle.gdn_reference_fwd_bwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], initial_state=inp["h0"],
                                         do=inp["do"], dht=inp["dht"])
    for _ in range(warmup):
        one()
    t0 = time.perf_counter()
    for _ in range(steps):
        one()
    dt = (time.perf_counter() - t0) / steps
    return Ts / dt, f"B=1 T={Ts} HQK={c['HK']} HV={c['HV']} K=V=128 fp32 naive recurrence, {threads} threads"


def run_reference(args, workload):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    tps, sample = cpu_reference_tokens_per_s(workload, threads, steps=max(1, args.steps), warmup=min(args.warmup, 1))
    line = {
        "impl": "reference", "metric": "GDN chunk tokens/s (%s)" % workload, "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * 1024 / tps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload, **CFG, "sample": sample},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=[None, "gdn_fwd_conv", "gdn_fwd_bwd"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()

    if args.impl == "reference":
        run_reference(args, args.workload or DEFAULT_WORKLOAD)
        return

    import torch.distributed as dist
    import fla_b200

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path for the kernels")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = fla_b200.load_library()
    workload = args.workload or DEFAULT_WORKLOAD
    K, W = args.steps, max(args.warmup, 3)

    d = make_inputs(dev, 1001 + rank)
    tokens_per_step = CFG["B"] * CFG["T"]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing: W warm-up steps, then exactly K timed steps
    for _ in range(W):
        step_device(d, workload)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(K):
        step_device(d, workload)
    e1.record()
    barrier()
    elapsed_ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(elapsed_ms, op=dist.ReduceOp.MAX)
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = elapsed_ms.item() / K
    value = world * tokens_per_step / (ms_per_step * 1e-3)

    # ---- per-kernel durations of the same step (CUDA events around each launch, on the launching stream)
    lib.fla_b200_kernel_timing_enable(1)
    for _ in range(K):
        step_device(d, workload)
    torch.cuda.synchronize()
    ktimes = {}
    for nm in ("gdn_prep", "gdn_fwd", "causal_conv1d_fwd", "gdn_bwd_dhu", "gdn_bwd_par"):
        ms, n = kernel_time(lib, nm)
        if n:
            ktimes[nm] = {"ms_per_launch": ms / n, "launches": n}
    lib.fla_b200_kernel_timing_enable(0)

    # ---- end to end through the public API with host buffers: pinned H2D of the step's inputs, D2H of its outputs
    names = ["q", "k", "v", "g", "beta", "h0"] + (["x"] if workload == "gdn_fwd_conv" else ["do", "dht"])
    host = {n: d[n].cpu().pin_memory() for n in names}
    stage = {n: torch.empty_like(d[n]) for n in names}
    h2d = sum(host[n].numel() * host[n].element_size() for n in names)
    outs = step_device(d, workload)
    outs = outs[1:] if workload == "gdn_fwd_conv" else outs          # conv output feeds the device side only
    host_out = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in outs]
    d2h = sum(o.numel() * o.element_size() for o in host_out)

    def step_e2e():
        for n in names:
            stage[n].copy_(host[n], non_blocking=True)
        dd = dict(d)
        dd.update(stage)
        res = step_device(dd, workload)
        res = res[1:] if workload == "gdn_fwd_conv" else res
        for h, o in zip(host_out, res):
            h.copy_(o, non_blocking=True)

    for _ in range(2):
        step_e2e()
    barrier()
    Ke = max(3, K // 4)
    e0.record()
    for _ in range(Ke):
        step_e2e()
    e1.record()
    barrier()
    e2e_ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_value = world * tokens_per_step / (e2e_ms.item() / Ke * 1e-3)

    if rank == 0:
        peaks = _peaks()
        token_heads = CFG["B"] * CFG["T"] * CFG["HV"]
        cands = [k for k in ktimes if k in KERNEL_FLOP_PER_TOKEN_HEAD]
        dom = max(cands, key=lambda k: ktimes[k]["ms_per_launch"]) if cands else None
        roofline = None
        if dom:
            flops = KERNEL_FLOP_PER_TOKEN_HEAD[dom] * token_heads
            achieved = flops / (ktimes[dom]["ms_per_launch"] * 1e-3) / 1e12
            roofline = {"kernel": KERNEL_NAMES[dom], "bound": "tensor", "achieved": achieved,
                        "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"],
                        "traffic": None, "peak_source": peaks["source"] + " (burst)",
                        "ms_per_launch": ktimes[dom]["ms_per_launch"]}
        step_flops = (FWD_FLOP_PER_TOKEN_HEAD + (BWD_FLOP_PER_TOKEN_HEAD if workload == "gdn_fwd_bwd" else 0.0)) * token_heads
        step_tflops = step_flops / (ms_per_step * 1e-3) / 1e12
        cpu_baseline = None
        if not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            tps, sample = cpu_reference_tokens_per_s(workload, threads)
            cpu_baseline = {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample}
        line = {
            "metric": "GDN chunk tokens/s (%s)" % workload, "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload, **CFG, "global_batch": CFG["B"] * world,
                       "parallelism": f"replicated per GPU x{world}, sharded by batch, no collective",
                       "l2": "inputs per step exceed the 126 MB L2"},
            "roofline": roofline, "kernels": ktimes,
            "step_roofline": {"algorithmic_tflops": step_tflops, "frac_of_bf16_peak": step_tflops / peaks["bf16_tflops"]},
            "cpu_baseline": cpu_baseline,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches_per_step(workload) * K, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
