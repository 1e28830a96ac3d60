#!/usr/bin/env python
"""Benchmark of the GDN / KDA hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME] [--shape B,T]

One "step" is one pass of the hot path over one batch of seeded synthetic input with the shapes and value
distributions of the benchmark specification.  Workloads (the default is the one the headline metric is quoted on):
  gdn_fwd_bwd    config 2: chunked GDN forward + backward, B=8 T=4096 HQK=16 HV=32 K=V=128, nonzero fp32 h0, dO, dht
  gdn_fwd_conv   config 1: causal_conv1d (W=4, SiLU) over x[8,4096,8192] bf16, then the chunked GDN forward
  kda_fwd        config 3 (forward half): chunked KDA, B=4 T=8192 H=32 K=V=128, g = logsigmoid/16 per channel
  kda_fwd_bwd    config 3: chunked KDA forward + backward (forward intermediates kept: disable_recompute), dO ~ N(0,1)
  decode         config 4: causal_conv1d_update + fused-recurrent GDN, 256 sequences x 1 token, fp32 state pool,
                 one CUDA graph replay per step
  conv_prefill   the conv half of config 1 alone
  conv_bwd       backward of that conv (dx, dw, db from x, dy; SiLU pre-activation recomputed)
  gdn_stage_fwd / gdn_stage_fwd_bwd   configs 1 / 2 through the stand-alone stage operators, one launch per reference operator
`value` times K steps issued round-robin on `--streams` CUDA streams (default 2): the steps are independent batches, and a
second step in flight fills the SMs that the tail of a kernel leaves idle.  `single_stream` repeats the K steps on one stream.
With N > 1 every rank (one process per GPU, launched by torch.distributed.run) processes its own batch of that
shape (weak scaling; the path has no exchange step, so there is no collective on the data path); NCCL carries only
the barrier and the max-over-ranks reduction of the measured time.  The same line then carries a `strong` block: the
named shape's ONE global batch partitioned over the ranks (batch rows, then whole GVA groups of heads) through
fla_b200.sharding, timed the same way, with speed-up and efficiency against this run's own one-GPU time of the whole
batch, and a `shard_check` (outside any timed region) that gathers a small partitioned result with NCCL and compares
it bit for bit with rank 0's single-GPU result.  At N = 1 the line also carries `workloads` (the other configurations
of the specification, each timed like the headline) and `parity` (the CUDA operators against the CPU baseline's oracle
results on that leg's sample).  Rank 0 prints ONE JSON line.

`--impl reference` times the reference's CPU algorithm (the oracle port of its naive fp32 torch goldens) on the
host cores for the same metric, each step a bounded sample of the workload.
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

DEFAULT_WORKLOAD = "gdn_fwd_bwd"
WORKLOADS = ["gdn_fwd_bwd", "gdn_fwd_conv", "kda_fwd", "kda_fwd_bwd", "decode", "conv_prefill", "conv_bwd", "gdn_stage_fwd", "gdn_stage_fwd_bwd"]
FWD_FLOP_PER_TOKEN_HEAD = 182955.0      # KK^T, inverse, w/u, state, output (dense 64x64 tiles, no causal credit)
BWD_FLOP_PER_TOKEN_HEAD = 524288.0

# Algorithmic work of each kernel per token per value head (FLOPs; dense 64x64 tiles; split-precision passes
# are overhead and not counted).
KERNEL_FLOPS = {
    "gdn_fwd": 163840.0,       # [Q;K]S, QK^T, X Z, P v_new, K^T vhat
    "gdn_bwd_dhu": 147456.0,   # K dS', QK^T, P^T dO, X^T dVn, [Q^T|K^T][dO~; dR]
    "gdn_bwd_par": 212992.0,   # [dO;dZ]Vn^T, [dO;dZ]S^T, Vn dS'^T, [dP;dA]K, [dP^T|dA^T][Q;K], [Q;K]K^T / G
    "kda_fwd": 131072.0,       # [Qp;Kp]Sa, X Z, Aqk v_new, Kn^T v_new
    "kda_prep": 32768.0,       # [Qp;Kp]Kn^T (+ the CUDA-core inverse)
    "kda_bwd_dhu": 131072.0,   # Kn dS'a, P^T dO, X^T dVn, [Qp^T|Kp^T][dO~; dR]
    "kda_bwd_par": 229376.0,   # [Qp;Kp]Kn^T, [dO;dZ]Vn^T, [dO;dZ]Sa^T, Vn dS'a^T, [dP;dM]Kn, [dP^T|dM^T][Qp;Kp]
    "gdn_prep": 16384.0,
    "tri_inverse": 8192.0,     # 2 * 64^2 FLOP per token-head of the triangular solve (CUDA cores; shown against the tensor peak)
}
# Algorithmic HBM bytes of the stand-alone stages: every input read once, every output written once
# (bf16 token tensors, fp32 A and gates, bf16 per-chunk states).
def _th(c, heads, width, es):
    return float(c["B"]) * c["T"] * c[heads] * width * es


STAGE_BYTES = {
    "chunk_local_cumsum": lambda c: _th(c, "HV", 1, 2) + _th(c, "HV", 1, 4),
    "chunk_scaled_dot_kkt": lambda c: _th(c, "HK", 128, 2) + _th(c, "HV", 1, 6) + _th(c, "HV", 64, 4),
    "solve_tri": lambda c: _th(c, "HV", 64, 4) + _th(c, "HV", 64, 2),
    "recompute_w_u_fwd": lambda c: _th(c, "HK", 128, 2) + _th(c, "HV", 128, 2) + _th(c, "HV", 64, 2) + 2 * _th(c, "HV", 128, 2),
    "chunk_fwd_h": lambda c: _th(c, "HK", 128, 2) + 2 * _th(c, "HV", 128, 2) + _th(c, "HV", 128, 2) + _th(c, "HV", 256, 2),
    "chunk_fwd_o": lambda c: 2 * _th(c, "HK", 128, 2) + _th(c, "HV", 128, 2) + _th(c, "HV", 256, 2) + _th(c, "HV", 128, 2),
    "chunk_bwd_dv_local": lambda c: 2 * _th(c, "HK", 128, 2) + 2 * _th(c, "HV", 128, 2),
    "chunk_bwd_dhu": lambda c: 2 * _th(c, "HK", 128, 2) + 4 * _th(c, "HV", 128, 2) + _th(c, "HV", 256, 2),
    # q, k, v_new, dO, dv2, h, dh in; dw and the per-value-head fp32 dq, dk rows out
    "chunk_bwd_dqkwg": lambda c: 2 * _th(c, "HK", 128, 2) + 3 * _th(c, "HV", 128, 2) + 2 * _th(c, "HV", 256, 2) + _th(c, "HV", 128, 2) +
    2 * _th(c, "HV", 128, 4),
    "chunk_bwd_dqkwg_group_sum": lambda c: 2 * _th(c, "HV", 128, 4) + 2 * _th(c, "HK", 128, 2),
    # k, v, X, dw, du in; dv and the per-value-head fp32 dk rows out
    "prepare_wy_repr_bwd": lambda c: _th(c, "HK", 128, 2) + 3 * _th(c, "HV", 128, 2) + _th(c, "HV", 64, 2) + _th(c, "HV", 128, 2) +
    _th(c, "HV", 128, 4),
    "prepare_wy_repr_bwd_group_sum": lambda c: _th(c, "HV", 128, 4) + _th(c, "HK", 128, 2),
}
KERNEL_SYMBOL = {"gdn_fwd": "gdn_scan_fwd_kernel", "gdn_bwd_dhu": "gdn_scan_bwd_kernel", "gdn_bwd_par": "gdn_bwd_par_kernel",
                 "kda_fwd": "kda_fwd_kernel", "kda_prep": "kda_prep_kernel", "kda_bwd_dhu": "kda_bwd_dhu_kernel", "kda_bwd_par": "kda_bwd_par_kernel", "gdn_prep": "gdn_prep_kernel", "tri_inverse": "tri_inverse_kernel",
                 "recurrent_gdn": "recurrent_gdn_kernel", "causal_conv1d_fwd": "conv_fwd_kernel",
                 "causal_conv1d_update": "conv_update1_kernel", "causal_conv1d_bwd": "conv_bwd_kernel",
                 "chunk_local_cumsum": "stage_cumsum_kernel", "chunk_scaled_dot_kkt": "stage_kkt_kernel",
                 "solve_tri": "stage_solve_tri_kernel", "recompute_w_u_fwd": "stage_wu_kernel",
                 "chunk_fwd_h": "stage_fwd_h_kernel", "chunk_fwd_o": "stage_fwd_o_kernel",
                 "chunk_bwd_dv_local": "stage_dv_local_kernel", "chunk_bwd_dhu": "stage_bwd_dhu_kernel",
                 "chunk_bwd_dqkwg": "stage_dqkwg_kernel", "chunk_bwd_dqkwg_group_sum": "stage_group_sum_kernel",
                 "prepare_wy_repr_bwd": "stage_wy_bwd_kernel", "prepare_wy_repr_bwd_group_sum": "stage_group_sum_kernel"}


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


# ----------------------------------------------------------------------------------------------- workloads
class Workload:
    """name, shapes, synthetic inputs, one step through the public API, and the work one step represents."""

    def __init__(self, name, shape):
        self.name = name
        self.graph = None
        if name in ("gdn_fwd_bwd", "gdn_fwd_conv", "conv_prefill", "conv_bwd", "gdn_stage_fwd", "gdn_stage_fwd_bwd"):
            self.cfg = dict(B=8, T=4096, HK=16, HV=32, K=128, V=128, D=8192, W=4)
        elif name in ("kda_fwd", "kda_fwd_bwd"):
            self.cfg = dict(B=4, T=8192, HK=32, HV=32, K=128, V=128)
        else:
            self.cfg = dict(N=256, T=1, HK=16, HV=32, K=128, V=128, D=8192, W=4)
        if shape:
            b, t = (int(x) for x in shape.split(","))
            if name == "decode":
                self.cfg["N"] = b
            else:
                self.cfg["B"], self.cfg["T"] = b, t
        c = self.cfg
        self.tokens_per_step = c["N"] if name == "decode" else c["B"] * c["T"]
        self.token_heads = self.tokens_per_step * c["HV"]

    # -- inputs (the benchmark specification's distributions): q,k ~ N(0,1) L2-normalised; v ~ N(0,1); g = logsigmoid(N(0,1))
    #    (/16 per channel for KDA); beta = sigmoid(N(0,1)); states ~ 0.1 N(0,1) fp32; conv weights ~ N(0, 1/4).
    def make_inputs(self, device, seed):
        c = self.cfg
        g_ = torch.Generator(device=device).manual_seed(seed)
        rn = lambda *s: torch.randn(*s, device=device, generator=g_)  # noqa: E731
        d = {}
        if self.name in ("gdn_fwd_bwd", "gdn_fwd_conv", "kda_fwd", "kda_fwd_bwd", "gdn_stage_fwd", "gdn_stage_fwd_bwd"):
            d["q"] = F.normalize(rn(c["B"], c["T"], c["HK"], c["K"]), dim=-1).bfloat16()
            d["k"] = F.normalize(rn(c["B"], c["T"], c["HK"], c["K"]), dim=-1).bfloat16()
            d["v"] = rn(c["B"], c["T"], c["HV"], c["V"]).bfloat16()
            d["beta"] = torch.sigmoid(rn(c["B"], c["T"], c["HV"])).bfloat16()
            if self.name in ("kda_fwd", "kda_fwd_bwd"):
                d["g"] = (F.logsigmoid(rn(c["B"], c["T"], c["HV"], c["K"])) / 16).bfloat16()
            else:
                d["g"] = F.logsigmoid(rn(c["B"], c["T"], c["HV"])).bfloat16()
                d["h0"] = 0.1 * rn(c["B"], c["HV"], c["K"], c["V"])
        if self.name in ("gdn_fwd_bwd", "gdn_stage_fwd_bwd"):
            d["do"] = rn(c["B"], c["T"], c["HV"], c["V"]).bfloat16()
            d["dht"] = 0.1 * rn(c["B"], c["HV"], c["K"], c["V"])
        if self.name == "kda_fwd_bwd":
            d["do"] = rn(c["B"], c["T"], c["HV"], c["V"]).bfloat16()
        if self.name in ("gdn_fwd_conv", "conv_prefill", "conv_bwd"):
            d["x"] = rn(c["B"], c["T"], c["D"]).bfloat16()
        if self.name == "conv_bwd":
            d["dy"] = rn(c["B"], c["T"], c["D"]).bfloat16()
        if self.name == "decode":
            d["q"] = F.normalize(rn(c["N"], 1, c["HK"], c["K"]), dim=-1).bfloat16()
            d["k"] = F.normalize(rn(c["N"], 1, c["HK"], c["K"]), dim=-1).bfloat16()
            d["v"] = rn(c["N"], 1, c["HV"], c["V"]).bfloat16()
            d["g"] = F.logsigmoid(rn(c["N"], 1, c["HV"])).bfloat16()
            d["beta"] = torch.sigmoid(rn(c["N"], 1, c["HV"])).bfloat16()
            d["state"] = 0.1 * rn(c["N"], c["HV"], c["K"], c["V"])
            d["conv_state"] = rn(c["N"], c["D"], c["W"] - 1).bfloat16()
            d["x"] = rn(c["N"], c["D"]).bfloat16()
        if "D" in c:
            d["w"] = (0.5 * rn(c["D"], c["W"])).bfloat16()
            d["bias"] = torch.zeros(c["D"], device=device, dtype=torch.bfloat16)
        return d

    def host_input_names(self):
        return {"gdn_fwd_bwd": ["q", "k", "v", "g", "beta", "h0", "do", "dht"],
                "gdn_fwd_conv": ["q", "k", "v", "g", "beta", "h0", "x"],
                "kda_fwd": ["q", "k", "v", "g", "beta"],
                "kda_fwd_bwd": ["q", "k", "v", "g", "beta", "do"],
                "decode": ["q", "k", "v", "g", "beta", "x"],
                "conv_prefill": ["x"], "conv_bwd": ["x", "dy"], "gdn_stage_fwd": ["q", "k", "v", "g", "beta", "h0"],
                "gdn_stage_fwd_bwd": ["q", "k", "v", "g", "beta", "h0", "do", "dht"]}[self.name]

    def step(self, d):
        """One pass through the public Python API.  Returns the tensors a caller reads back."""
        import fla_b200.ops as ops
        n = self.name
        if n == "gdn_fwd_bwd":
            o, ht, grads = ops.chunk_gated_delta_rule_fwd_bwd(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"],
                                                              initial_state=d["h0"], dht=d["dht"])
            return (o, ht) + tuple(grads)
        if n == "gdn_fwd_conv":
            ops.causal_conv1d(d["x"], d["w"], d["bias"], activation="silu")
            with torch.no_grad():
                return ops.chunk_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"],
                                                  output_final_state=True)
        if n == "kda_fwd":
            with torch.no_grad():
                return ops.chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], output_final_state=True)
        if n == "kda_fwd_bwd":
            o, ht, grads = ops.chunk_kda_fwd_bwd(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"],
                                                 grad_dtype=torch.bfloat16, disable_recompute=True)
            return (o, ht) + tuple(x for x in grads if x is not None)
        if n in ("gdn_stage_fwd", "gdn_stage_fwd_bwd"):
            # the reference's stage-by-stage chains (examples/flash_gated_delta_rule.py:796-881 forward, :884-1023 backward) on
            # head-first views
            hf = lambda t: t.transpose(1, 2)  # noqa: E731
            scale = self.cfg["K"] ** -0.5
            q, k, v, beta = hf(d["q"]), hf(d["k"]), hf(d["v"]), hf(d["beta"])
            gam = hf(ops.chunk_local_cumsum(d["g"], 64, head_first=False))
            A = ops.chunk_scaled_dot_kkt(k, gam, beta)
            X = ops.solve_tri(A, layout="bnsd", output_dtype=torch.bfloat16)
            w, u = ops.recompute_w_u_fwd(k, v, beta, X, 64, g=gam)
            h, v_new, ht = ops.chunk_gated_delta_rule_fwd_h(k, w, u, gam, initial_state=d["h0"], output_final_state=True)
            o = ops.chunk_fwd_o(q, k, v_new, h, scale, g=gam)
            if n == "gdn_stage_fwd":
                return o, ht
            do = hf(d["do"])
            dv = ops.chunk_bwd_dv_local(q, k, do, gam, scale, 64)
            dh, dh0, dv2 = ops.chunk_gated_delta_rule_bwd_dhu(q, k, w, do, dv, scale, 64, g=gam, h0=d["h0"], dht=d["dht"])
            dq, dk, dw, dg = ops.chunk_bwd_dqkwg(q, k, v_new, gam, h, do, dh, dv2, 64, w=w, scale=scale)
            dk2, dv_f, dbeta, dg2 = ops.prepare_wy_repr_bwd(k, v, beta, X, dw, dv2, gam, 64)
            # the reference's glue adds dk2 and dg2 with torch ops and reverse-cumsums dg (:1010-1021)
            dk = dk + dk2
            dg = ops.chunk_local_cumsum(dg + dg2, 64, reverse=True)
            return o, ht, dq, dk, dv_f, dbeta, dg, dh0
        if n == "conv_prefill":
            return ops.causal_conv1d(d["x"], d["w"], d["bias"], activation="silu")[:1]
        if n == "conv_bwd":
            return ops.causal_conv1d_bwd(d["x"], d["w"], d["dy"], d["bias"], activation="silu")[:3]
        y = ops.causal_conv1d_update(d["x"], d["conv_state"], weight=d["w"], bias=d["bias"], activation="silu")
        o, _ = ops.fused_recurrent_gated_delta_rule(d["q"], d["k"], d["v"], g=d["g"], beta=d["beta"],
                                                    initial_state=d["state"], inplace_final_state=True)
        return y, o

    def step_fast(self, d):
        """Device-resident step as timed for `value`: the decode step is replayed as one CUDA graph."""
        if self.name != "decode":
            return self.step(d)
        if self.graph is None:
            self.step(d)
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self.graph_out = self.step(d)
        self.graph.replay()
        return self.graph_out

    def launches_per_step(self):
        n = {"gdn_fwd_bwd": 5, "gdn_fwd_conv": 4, "kda_fwd": 3, "kda_fwd_bwd": 5, "decode": 2, "conv_prefill": 1, "conv_bwd": 2,
             "gdn_stage_fwd": 6, "gdn_stage_fwd_bwd": 13}[self.name]
        c = self.cfg
        if self.name in ("gdn_fwd_bwd", "kda_fwd_bwd") and c["B"] >= 2:
            # the backward launches its two kernels once per half of the batch when its scan has more chains than SMs
            chains = c["B"] * c["HV"] * (c["V"] // (128 if self.name == "gdn_fwd_bwd" else 64))
            if chains > torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count:
                n += 2
        return n

    def kernel_names(self):
        return {"gdn_fwd_bwd": ["gdn_prep", "tri_inverse", "gdn_fwd", "gdn_bwd_dhu", "gdn_bwd_par"],
                "gdn_fwd_conv": ["causal_conv1d_fwd", "gdn_prep", "tri_inverse", "gdn_fwd"],
                "kda_fwd": ["kda_prep", "tri_inverse", "kda_fwd"],
                "kda_fwd_bwd": ["kda_prep", "tri_inverse", "kda_fwd", "kda_bwd_dhu", "kda_bwd_par"], "decode": ["causal_conv1d_update", "recurrent_gdn"],
                "conv_prefill": ["causal_conv1d_fwd"], "conv_bwd": ["causal_conv1d_bwd"],
                "gdn_stage_fwd": ["chunk_local_cumsum", "chunk_scaled_dot_kkt", "solve_tri", "recompute_w_u_fwd", "chunk_fwd_h",
                                  "chunk_fwd_o"],
                "gdn_stage_fwd_bwd": ["chunk_local_cumsum", "chunk_scaled_dot_kkt", "solve_tri", "recompute_w_u_fwd", "chunk_fwd_h",
                                      "chunk_fwd_o", "chunk_bwd_dv_local", "chunk_bwd_dhu", "chunk_bwd_dqkwg",
                                      "chunk_bwd_dqkwg_group_sum", "prepare_wy_repr_bwd", "prepare_wy_repr_bwd_group_sum"]}[self.name]

    def kernel_work(self, kname):
        """(bound, algorithmic work per launch, unit) of one kernel at this workload's shape."""
        c = self.cfg
        if kname in KERNEL_FLOPS:
            return "tensor", KERNEL_FLOPS[kname] * self.token_heads, "TFLOP/s"
        if kname == "recurrent_gdn":      # state read + write, plus q,k,v,g,beta,o
            n = c["N"]
            act = n * (2 * c["HK"] * c["K"] + 2 * c["HV"] * c["V"] + 4 * c["HV"]) * 2
            return "hbm", 2.0 * n * c["HV"] * c["K"] * c["V"] * 4 + act, "GB/s"
        if kname == "causal_conv1d_fwd":  # x read + y write
            return "hbm", 2.0 * c["B"] * c["T"] * c["D"] * 2, "GB/s"
        if kname == "causal_conv1d_bwd":  # x, dy read + dx write
            return "hbm", 3.0 * c["B"] * c["T"] * c["D"] * 2, "GB/s"
        if kname in STAGE_BYTES:             # every stage streams its operands and results through HBM
            return "hbm", STAGE_BYTES[kname](c), "GB/s"
        if kname == "causal_conv1d_update":  # state read + write, x read, y write
            return "hbm", (2.0 * c["N"] * c["D"] * (c["W"] - 1) + 2.0 * c["N"] * c["D"]) * 2, "GB/s"
        raise KeyError(kname)

    def kernel_traffic(self, kname):
        """DRAM bytes (read + write) of one launch: the per-unit figure of one ncu capture of a small case of the
        same kernel (profiles/), scaled by the units this launch processes; None where no capture exists."""
        c = self.cfg
        per_chunk_head = {"gdn_fwd": 323.56e6 / 2048, "gdn_bwd_dhu": 390.73e6 / 2048, "gdn_bwd_par": 500.59e6 / 2048,
                          "kda_prep": 159.25e6 / 1024, "kda_fwd": 232.05e6 / 1024, "kda_bwd_dhu": 266.41e6 / 1024,
                          "kda_bwd_par": 396.41e6 / 1024, "recompute_w_u_fwd": 87.51e6 / 2048, "chunk_fwd_h": 144.66e6 / 2048,
                          "chunk_fwd_o": 151.88e6 / 2048}
        if kname == "gdn_fwd" and self.name == "gdn_fwd_conv":
            return None     # the capture is of the training forward (it also writes the saved images)
        if kname in per_chunk_head and "T" in c:
            return per_chunk_head[kname] * c["B"] * ((c["T"] + 63) // 64) * c["HV"]
        if kname == "recurrent_gdn":       # 541.1 MB read + 480.2 MB written for 256 sequences x 32 heads (a 537 MB pool, > 4 x L2)
            return 1021.4e6 / 256 * c["N"] * c["HV"] / 32
        if kname == "causal_conv1d_fwd":   # 229.92 MB for 2 x 4096 x 8192 elements
            return 229.92e6 / (2 * 4096 * 8192) * c["B"] * c["T"] * c["D"]
        if kname == "causal_conv1d_bwd":   # 391.52 MB for 2 x 4096 x 8192 elements
            return 391.52e6 / (2 * 4096 * 8192) * c["B"] * c["T"] * c["D"]
        return None

    def step_flops(self):
        if self.name in ("gdn_fwd_bwd", "gdn_stage_fwd_bwd"):
            return (FWD_FLOP_PER_TOKEN_HEAD + BWD_FLOP_PER_TOKEN_HEAD) * self.token_heads
        if self.name == "kda_fwd_bwd":
            return (FWD_FLOP_PER_TOKEN_HEAD + BWD_FLOP_PER_TOKEN_HEAD) * self.token_heads
        if self.name in ("gdn_fwd_conv", "kda_fwd", "gdn_stage_fwd"):
            return FWD_FLOP_PER_TOKEN_HEAD * self.token_heads
        return None


def cpu_reference(wl: Workload, threads: int, steps: int = 1, warmup: int = 0, check64: bool = False):
    """The reference's CPU algorithm for one step on a bounded sample of the workload.
    Returns (tokens/s, description of the sample, the sample's inputs, the oracle's results on it); the last two are
    None for workloads whose parity block is not built from this leg."""
    import oracle
    torch.set_num_threads(threads)
    c = wl.cfg
    inp = None
    if wl.name in ("gdn_fwd_bwd", "gdn_fwd_conv", "gdn_stage_fwd", "gdn_stage_fwd_bwd"):
        Ts = 1024
        inp = oracle.make_gdn_inputs(1, Ts, c["HK"], c["HV"], seed=1001)
        xs, w = torch.randn(1, c["D"], Ts), 0.5 * torch.randn(c["D"], c["W"])
        desc = f"B=1 T={Ts} HQK={c['HK']} HV={c['HV']} K=V=128 fp32 naive recurrence"
        if wl.name in ("gdn_fwd_bwd", "gdn_stage_fwd_bwd"):
            fn = lambda: oracle.gdn_reference_fwd_bwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"],  # noqa: E731
                                                      initial_state=inp["h0"], do=inp["do"], dht=inp["dht"])
            desc += " + autograd"
        elif wl.name == "gdn_stage_fwd":
            fn = lambda: oracle.gdn_reference_fwd_bwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"],  # noqa: E731
                                                      initial_state=inp["h0"])
        else:
            def fn():
                oracle.causal_conv1d_ref(xs, w, None, None, False, "silu")
                return oracle.gdn_reference_fwd_bwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], initial_state=inp["h0"])
            desc += " + conv1d"
        tokens = Ts
    elif wl.name in ("kda_fwd", "kda_fwd_bwd"):
        Ts = 512
        inp = oracle.make_kda_inputs(1, Ts, c["HK"], c["HV"], seed=1003, with_grad=wl.name == "kda_fwd_bwd")
        fn = lambda: oracle.kda_reference_fwd_bwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"],  # noqa: E731
                                                  do=inp.get("do"))
        tokens, desc = Ts, f"B=1 T={Ts} H={c['HV']} K=V=128 fp32 naive KDA recurrence" + (
            " + autograd" if wl.name == "kda_fwd_bwd" else "")
    elif wl.name == "conv_bwd":
        Ts = 2048
        xs, w = torch.randn(1, Ts, c["D"]), 0.5 * torch.randn(c["W"], c["D"])
        dys = torch.randn(1, Ts, c["D"])
        fn = lambda: oracle.causal_conv1d_bwd_ref(xs, w, dys, None, None, None, 1, dtype=torch.float32)  # noqa: E731
        tokens, desc = Ts, f"B=1 T={Ts} D={c['D']} W=4 autograd through the conv definition"
    elif wl.name == "conv_prefill":
        Ts = 4096
        xs, w = torch.randn(1, c["D"], Ts), 0.5 * torch.randn(c["D"], c["W"])
        fn = lambda: oracle.causal_conv1d_ref(xs, w, None, None, False, "silu")  # noqa: E731
        tokens, desc = Ts, f"B=1 T={Ts} D={c['D']} W=4 F.conv1d golden"
    else:
        Ns = 32
        dec = oracle.make_decode_inputs(Ns, c["HK"], c["HV"], seed=1004)
        asl = torch.tensor([0] + [1] * Ns, dtype=torch.int32)
        idx = torch.arange(Ns, dtype=torch.int32)
        st = dec["state"].transpose(-1, -2).contiguous()
        cs, xu, w = torch.randn(Ns, c["D"], 3), torch.randn(Ns, c["D"]), 0.5 * torch.randn(c["D"], 4)

        def fn():
            oracle.causal_conv1d_update_ref(xu, cs, w, None, "silu")
            oracle.recurrent_gated_delta_rule_golden(dec["q"], dec["k"], dec["v"], st, dec["beta"], 128 ** -0.5, asl, idx,
                                                     g=dec["g"].float(), state_out_dtype=torch.float32)
        tokens, desc = Ns, f"{Ns} sequences x 1 token, HV={c['HV']}, fp32 state golden + conv update golden"
    for _ in range(warmup):
        fn()
    t0 = time.perf_counter()
    ref = None
    for _ in range(steps):
        ref = fn()
    dt = (time.perf_counter() - t0) / steps
    if not isinstance(ref, dict):
        inp = ref = None
    elif check64:
        # The timed runs above are the reference's own fp32 arithmetic; as the CHECKER of the parity block the same
        # recurrence is evaluated once more in float64 (untimed), so that the oracle's fp32 rounding over a thousand
        # sequential steps (about 1e-3 of RMS in the gradients) is not booked as kernel error.
        if wl.name.startswith("gdn"):
            ref = oracle.gdn_reference_fwd_bwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], initial_state=inp["h0"],
                                               do=inp.get("do") if "dq" in ref else None,
                                               dht=inp.get("dht") if "dq" in ref else None, dtype=torch.float64)
        else:
            ref = oracle.kda_reference_fwd_bwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], do=inp.get("do"),
                                               dtype=torch.float64)
    return tokens / dt, f"{desc}, {threads} threads", inp, ref


def parity_block(wl: Workload, inp, ref, dev):
    """max-abs-error / RMS(oracle) per tensor of the CUDA operators on the CPU baseline's own sample (the oracle results
    of that leg are the checker): once with fp32 outputs / gradients, once as stored in bf16 (whose final rounding alone
    can reach 2^-8 |x|; `excess` is the largest error beyond 5e-3 RMS + 2^-8 |ref|, <= 0 when the bar is met)."""
    import fla_b200.ops as ops
    if inp is None or ref is None:
        return None
    d = {n: (t.to(dev) if isinstance(t, torch.Tensor) else t) for n, t in inp.items()}
    bwd = "dq" in ref

    def run(out_dtype, grad_dtype):
        if wl.name.startswith("gdn"):
            if bwd:
                o, ht, gr = ops.chunk_gated_delta_rule_fwd_bwd(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], initial_state=d["h0"],
                                                               dht=d["dht"], output_dtype=out_dtype, grad_dtype=grad_dtype)
                return dict(o=o, ht=ht, dq=gr[0], dk=gr[1], dv=gr[2], dg=gr[3], dbeta=gr[4], dh0=gr[5])
            with torch.no_grad():
                o, ht = ops.chunk_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"],
                                                   output_final_state=True, output_dtype=out_dtype)
            return dict(o=o, ht=ht)
        if bwd:
            o, ht, gr = ops.chunk_kda_fwd_bwd(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], output_dtype=out_dtype,
                                              grad_dtype=grad_dtype)
            return dict(o=o, ht=ht, dq=gr[0], dk=gr[1], dv=gr[2], dg=gr[3], dbeta=gr[4])
        with torch.no_grad():
            o, ht = ops.chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], output_final_state=True, output_dtype=out_dtype)
        return dict(o=o, ht=ht)

    out = {"sample": "the cpu_baseline sample", "oracle": "the naive recurrence (+ autograd) of the cpu_baseline leg, evaluated in float64", "tolerance": 5e-3, "fp32_out": {},
           "bf16_out": {}}
    for tag, res in (("fp32_out", run(torch.float32, torch.float32)), ("bf16_out", run(None, None))):
        for name, got in res.items():
            r = ref.get(name)
            if got is None or r is None:
                continue
            got, r = got.detach().double().cpu(), r.detach().double()
            rms = max(r.pow(2).mean().sqrt().item(), 1e-30)
            err = (got - r).abs()
            entry = {"max_abs_over_rms": err.max().item() / rms}
            if tag == "bf16_out" and res[name].dtype == torch.bfloat16:
                entry["excess_over_bar_plus_half_ulp"] = (err - (5e-3 * rms + r.abs() * 2.0 ** -8)).max().item() / rms
            out[tag][name] = entry
    out["worst_fp32_out"] = max(v["max_abs_over_rms"] for v in out["fp32_out"].values())
    return out


def run_reference(args, wl: Workload):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    threads = os.cpu_count() or 1
    tps, sample, _, _ = cpu_reference(wl, threads, steps=max(1, args.steps), warmup=min(args.warmup, 1))
    line = {
        "impl": "reference", "metric": f"GDN/KDA tokens/s ({wl.name})", "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": None,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl.name, **wl.cfg, "sample": sample},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def kernel_time(lib, name):
    ms, n = ctypes.c_float(0), ctypes.c_int(0)
    lib.fla_b200_kernel_timing_read(name.encode(), ctypes.byref(ms), ctypes.byref(n))
    return ms.value, n.value


class Bench:
    """Timing helpers shared by the headline workload, the other workloads of the `workloads` block and the
    strong-scaling partition: barrier + synchronize on both sides, CUDA events on the launching stream, max over ranks."""

    def __init__(self, dev, world, rank, lib):
        self.dev, self.world, self.rank, self.lib = dev, world, rank, lib
        self.e0, self.e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, x):
        t = torch.tensor([x], device=self.dev, dtype=torch.float64)
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    def timed(self, step, K, streams):
        """K steps; with several streams the (independent) steps are issued round-robin, so the tail of one step's
        kernels, where SMs run out of CTAs, is filled by the next step's kernels.  Device time between two events on
        the main stream, max over ranks, per step."""
        main = torch.cuda.current_stream(self.dev)
        self.barrier()
        self.e0.record()
        for st in streams:
            st.wait_stream(main)
        for i in range(K):
            if streams:
                with torch.cuda.stream(streams[i % len(streams)]):
                    step()
            else:
                step()
        for st in streams:
            main.wait_stream(st)
        self.e1.record()
        self.barrier()
        return self.max_over_ranks(self.e0.elapsed_time(self.e1)) / K

    def device_timing(self, step, K, W, n_streams):
        """W warm-up steps, then exactly K timed steps on `n_streams` streams and (when n_streams > 1) again on one.
        Returns (ms per step, single-stream ms per step or None)."""
        for _ in range(W):
            step()
        side = [torch.cuda.Stream(self.dev) for _ in range(n_streams)] if n_streams > 1 else []
        for i in range(2 * len(side)):      # warm the side streams' allocator pools
            with torch.cuda.stream(side[i % len(side)]):
                step()
        ms = self.timed(step, K, side)
        ms1 = self.timed(step, K, []) if side else None
        return ms, ms1

    def kernel_times(self, wl, d, steps):
        """Per-kernel durations of the same step (CUDA events around each launch, on the launching stream)."""
        self.lib.fla_b200_kernel_timing_enable(1)
        for _ in range(steps):
            wl.step(d)
        torch.cuda.synchronize()
        ktimes = {}
        for nm in wl.kernel_names():
            ms, n = kernel_time(self.lib, nm)
            if n:
                ktimes[nm] = {"ms_per_launch": ms / n, "launches": n}
        self.lib.fla_b200_kernel_timing_enable(0)
        return ktimes


def roofline_of(wl, ktimes, peaks):
    """Roofline entry of the kernel with the longest launch, and the per-kernel fractions (filled into `ktimes`)."""
    if not ktimes:
        return None
    dom = max(ktimes, key=lambda k: ktimes[k]["ms_per_launch"])
    bound, work, unit = wl.kernel_work(dom)
    sec = ktimes[dom]["ms_per_launch"] * 1e-3
    achieved = work / sec / (1e12 if bound == "tensor" else 1e9)
    peak = peaks["bf16_tflops"] if bound == "tensor" else peaks["hbm_gbs"]
    roofline = {"kernel": KERNEL_SYMBOL[dom], "bound": bound, "achieved": achieved, "peak": peak, "unit": unit,
                "frac": achieved / peak, "traffic": wl.kernel_traffic(dom),
                "peak_source": peaks["source"] + (" (burst)" if bound == "tensor" else ""),
                "ms_per_launch": ktimes[dom]["ms_per_launch"]}
    for k in ktimes:
        b, wk, _ = wl.kernel_work(k)
        sk = ktimes[k]["ms_per_launch"] * 1e-3
        denom = 1e12 * peaks["bf16_tflops"] if b == "tensor" else 1e9 * peaks["hbm_gbs"]
        ktimes[k]["frac_of_peak"] = wk / sk / denom
        ktimes[k]["bound"] = b
        tr = wl.kernel_traffic(k)
        if tr is not None:   # DRAM bytes of the ncu capture scaled to this launch, as a share of the copy bandwidth
            ktimes[k]["dram_gb"] = tr / 1e9
            ktimes[k]["dram_frac_of_hbm_peak"] = tr / sk / (1e9 * peaks["hbm_gbs"])
    return roofline


def other_workloads(bench, headline, local, peaks, K=10, W=3):
    """The benchmark specification's other configurations, each timed like the headline (device-resident inputs, CUDA
    events, W warm-up + K timed steps on two streams and on one, clocks sampled during its own timed region)."""
    out = {}
    for name in ("gdn_fwd_conv", "kda_fwd_bwd", "decode", "conv_prefill"):
        if name == headline:
            continue
        wl = Workload(name, None)
        d = wl.make_inputs(bench.dev, 2001)
        n_streams = 1 if name == "decode" else 2
        sampler = ClockSampler(local)
        sampler.start()
        ms, ms1 = bench.device_timing(lambda: wl.step_fast(d), K, W, n_streams)
        clocks = sampler.stop()
        ktimes = bench.kernel_times(wl, d, min(K, 5))
        roof = roofline_of(wl, ktimes, peaks)
        entry = {"config": dict(wl.cfg), "ms_per_step": ms, "value": wl.tokens_per_step / (ms * 1e-3), "unit": "tokens/s",
                 "steps": K, "warmup": W, "streams": n_streams,
                 "single_stream": None if ms1 is None else {"ms_per_step": ms1, "value": wl.tokens_per_step / (ms1 * 1e-3)},
                 "roofline": roof,
                 "kernels": {k: {"ms_per_launch": round(v["ms_per_launch"], 5), "frac_of_peak": round(v["frac_of_peak"], 4),
                                 "bound": v["bound"]} for k, v in ktimes.items()},
                 "clocks": clocks}
        if wl.step_flops():
            tf = wl.step_flops() / ((ms1 or ms) * 1e-3) / 1e12
            entry["step_roofline"] = {"algorithmic_tflops_single_stream": tf, "frac_of_bf16_peak": tf / peaks["bf16_tflops"]}
        if name == "decode":   # the whole step (conv update + recurrent kernel) against the measured copy bandwidth
            by = sum(wl.kernel_work(k)[1] for k in wl.kernel_names())
            entry["step_hbm_frac"] = by / (ms * 1e-3) / (1e9 * peaks["hbm_gbs"])
        out[name] = entry
        del d, wl
        torch.cuda.empty_cache()
    return out


def strong_partition(wl, world, rank):
    """How the named shape (global batch B) is partitioned over `world` ranks: batch rows first, then whole GVA groups of
    heads when ranks outnumber rows.  Returns (row begin, row end, q/k head begin, q/k head end, description)."""
    from fla_b200 import sharding
    c = wl.cfg
    nb = min(world, c["B"])
    while world % nb:
        nb -= 1
    nh = world // nb
    if c["HK"] % nh:
        raise SystemExit(f"cannot split {c['HK']} q/k heads over {nh} ranks")
    rb, rh = rank // nh, rank % nh
    b0, b1 = sharding.shard_range(c["B"], nb, rb)
    h0, h1 = sharding.shard_range(c["HK"], nh, rh)
    return b0, b1, h0, h1, f"{nb} batch shard(s) x {nh} head-group shard(s)"


def shard_inputs(wl, d, b0, b1, h0, h1):
    """The rank's shard of a step's inputs (contiguous copies, made once outside the timed region)."""
    c = wl.cfg
    rep = c["HV"] // c["HK"]
    out = {}
    for n, t in d.items():
        if n in ("q", "k"):
            out[n] = t[b0:b1, :, h0:h1].contiguous()
        elif n in ("v", "do", "g", "beta"):
            out[n] = t[b0:b1, :, h0 * rep:h1 * rep].contiguous()
        elif n in ("h0", "dht"):
            out[n] = t[b0:b1, h0 * rep:h1 * rep].contiguous()
        else:
            out[n] = t
    return out


def strong_scaling(bench, wl, K, W, n_streams, ms_full, ms_full_single):
    """Strong scaling of the named shape: the SAME global batch partitioned over the ranks with no exchange step.
    `ms_full` / `ms_full_single` are this run's times for the whole batch on one GPU (what every rank ran for the weak
    figure), so speed-up and efficiency come from one run on one set of GPUs."""
    world, rank = bench.world, bench.rank
    d_full = wl.make_inputs(bench.dev, 1001)           # the same global batch on every rank
    b0, b1, h0, h1, how = strong_partition(wl, world, rank)
    d = shard_inputs(wl, d_full, b0, b1, h0, h1)
    del d_full
    torch.cuda.empty_cache()
    # One batch row per GPU leaves the sequential scans with fewer chains than SMs (one CTA per (row, value head, 128
    # channels of V)); independent steps in flight on more streams fill them, so the stream count follows the shard size.
    chains = (b1 - b0) * (h1 - h0) * (wl.cfg["HV"] // wl.cfg["HK"]) * (wl.cfg["V"] // 128)
    s_streams = n_streams if n_streams == 1 else max(n_streams, min(8, -(-296 // max(chains, 1))))
    ms, ms1 = bench.device_timing(lambda: wl.step(d), K, W, s_streams)
    tokens = wl.tokens_per_step
    out = {"scaling": "strong", "global_batch": wl.cfg["B"], "partition": how, "streams": s_streams,
           "scan_chains_per_gpu": chains, "ms_per_step": ms,
           "value": tokens / (ms * 1e-3), "unit": "tokens/s", "speedup_vs_one_gpu": ms_full / ms,
           "efficiency": ms_full / ms / world}
    if ms1 is not None and ms_full_single is not None:
        out["single_stream"] = {"ms_per_step": ms1, "value": tokens / (ms1 * 1e-3), "speedup_vs_one_gpu": ms_full_single / ms1,
                                "efficiency": ms_full_single / ms1 / world}
    ktimes = bench.kernel_times(wl, d, min(K, 5))
    if ktimes:
        # the kernel that limits the partitioned step on this rank, and how much slower than linear it runs
        out["kernels_ms"] = {k: round(v["ms_per_launch"], 5) for k, v in ktimes.items()}
        out["limiting_kernel"] = KERNEL_SYMBOL[max(ktimes, key=lambda k: ktimes[k]["ms_per_launch"])]
    return out


def shard_check(bench):
    """Outside any timed region: a small GDN forward + backward partitioned like the strong-scaling run, its o / dq / dg
    gathered with NCCL, against rank 0's own single-GPU result of the whole problem, bit for bit."""
    from fla_b200 import sharding
    import fla_b200.ops as ops
    world, rank = bench.world, bench.rank
    wl = Workload("gdn_fwd_bwd", None)
    wl.cfg.update(B=max(2, min(world, 8)), T=320, HK=4, HV=8)
    d = wl.make_inputs(bench.dev, 4242)
    b0, b1, h0, h1, how = strong_partition(wl, world, rank)
    s = shard_inputs(wl, d, b0, b1, h0, h1)
    o, ht, gr = ops.chunk_gated_delta_rule_fwd_bwd(s["q"], s["k"], s["v"], s["g"], s["beta"], s["do"], initial_state=s["h0"],
                                                   dht=s["dht"])
    nb = min(world, wl.cfg["B"])
    while world % nb:
        nb -= 1
    nh = world // nb

    def gather(t):   # ranks are laid out row-major over (batch shard, head shard): gather heads inside a row shard, then rows
        parts = [torch.empty_like(t) for _ in range(world)]
        import torch.distributed as dist
        dist.all_gather(parts, t.contiguous())
        rows = [torch.cat(parts[r * nh:(r + 1) * nh], dim=2) for r in range(nb)]
        return torch.cat(rows, dim=0)
    o_all, dq_all, dg_all = gather(o), gather(gr[0]), gather(gr[3])
    ok = None
    if rank == 0:
        o1, _, g1 = ops.chunk_gated_delta_rule_fwd_bwd(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], initial_state=d["h0"],
                                                       dht=d["dht"])
        ok = bool(torch.equal(o_all, o1) and torch.equal(dq_all, g1[0]) and torch.equal(dg_all, g1[3]))
    del sharding
    return {"ok": ok, "compared": ["o", "dq", "dg"], "how": "NCCL all_gather of the shards vs rank 0's single-GPU run, bit-exact",
            "shape": {k: wl.cfg[k] for k in ("B", "T", "HK", "HV")}, "partition": how}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=WORKLOADS)
    ap.add_argument("--shape", default=None, help="B,T override (N,1 for decode) for small profiling cases")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--streams", type=int, default=2,
                    help="CUDA streams the timed steps are issued on round-robin (1 = every step waits for the one before)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-workloads", action="store_true", help="skip the `workloads` block (the other configurations)")
    args = ap.parse_args()
    wl = Workload(args.workload, args.shape)

    if args.impl == "reference":
        run_reference(args, wl)
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
    K, W = args.steps, max(args.warmup, 3)
    d = wl.make_inputs(dev, 1001 + rank)
    bench = Bench(dev, world, rank, lib)
    barrier = bench.barrier
    e0, e1 = bench.e0, bench.e1

    # ---- device-resident timing: W warm-up steps, then exactly K timed steps
    n_streams = 1 if wl.name == "decode" else max(1, args.streams)     # decode steps chain through the state pool
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_per_step, ms1 = bench.device_timing(lambda: wl.step_fast(d), K, W, n_streams)
    clocks = sampler.stop() if rank == 0 else None
    value = world * wl.tokens_per_step / (ms_per_step * 1e-3)
    single = None if ms1 is None else {"ms_per_step": ms1, "value": world * wl.tokens_per_step / (ms1 * 1e-3)}
    ktimes = bench.kernel_times(wl, d, min(K, 10))

    # ---- end to end through the public API with host buffers: pinned H2D of the step's inputs, D2H of its outputs
    e2e = None
    if not args.no_e2e:
        names = wl.host_input_names()
        host = {n: d[n].cpu().pin_memory() for n in names}
        stage = {n: torch.empty_like(d[n]) for n in names}
        h2d = sum(host[n].numel() * host[n].element_size() for n in names)
        outs = [o for o in wl.step(d) if o is not None]
        host_out = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in outs]
        d2h = sum(o.numel() * o.element_size() for o in host_out)

        # Three streams, double-buffered staging: the H2D copy of step i + 1, the kernels of step i and the D2H copy of
        # step i - 1 overlap; every step still moves all of its inputs and outputs across PCIe inside the timed region.
        s_cmp = torch.cuda.current_stream(dev)
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        stages = [stage, {n: torch.empty_like(d[n]) for n in names}]
        host_outs = [host_out, [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in outs]]
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_cmp = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]
        del outs
        # Decode: a step is two small kernels, so the Python cost of launching them would dominate.  The public-API calls of
        # a step are captured once per staging buffer as a CUDA graph and replayed; copies stay outside the graphs.
        graphs = None
        if wl.name == "decode":
            graphs = []
            for b in range(2):
                dd = dict(d)
                dd.update(stages[b])
                wl.step(dd)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    res_b = [o for o in wl.step(dd) if o is not None]
                graphs.append((g, res_b))

        def step_e2e(i):
            b = i & 1
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_cmp[b])          # the step that last read this staging buffer has run
                for n in names:
                    stages[b][n].copy_(host[n], non_blocking=True)
                ev_in[b].record(s_in)
            s_cmp.wait_event(ev_in[b])
            if graphs is not None:
                s_cmp.wait_event(ev_out[b])         # the graph's output tensors have been read back
                graphs[b][0].replay()
                res = graphs[b][1]
            else:
                dd = dict(d)
                dd.update(stages[b])
                res = [o for o in wl.step(dd) if o is not None]
            ev_cmp[b].record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_cmp[b])
                for h, o in zip(host_outs[b], res):
                    h.copy_(o, non_blocking=True)
                    if graphs is None:
                        o.record_stream(s_out)
                ev_out[b].record(s_out)

        for i in range(2):
            step_e2e(i)
        barrier()
        Ke = K      # the same K steps; the region starts with an empty pipeline and ends when the last result is on the host
        e0.record()
        for i in range(Ke):
            step_e2e(i)
        s_cmp.wait_event(ev_out[0])
        s_cmp.wait_event(ev_out[1])
        e1.record()
        barrier()
        e2e_ms = bench.max_over_ranks(e0.elapsed_time(e1))
        e2e = {"value": world * wl.tokens_per_step / (e2e_ms / Ke * 1e-3), "unit": "tokens/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               # what each rank's host link sustained in each direction while all ranks copied at once
               "per_rank_copy_gbs": {"h2d": h2d / (e2e_ms / Ke * 1e-3) / 1e9, "d2h": d2h / (e2e_ms / Ke * 1e-3) / 1e9},
               "pipeline": "3 streams (H2D, kernels, D2H), double-buffered staging" +
                           ("; the step's API calls replayed as one CUDA graph per staging buffer" if graphs is not None else "")}
        del host, stages, host_outs, graphs
        torch.cuda.empty_cache()

    # ---- the partition the path is built for: the SAME global batch split over the ranks (strong scaling) + its check
    strong = check = None
    if world > 1 and wl.name in ("gdn_fwd_bwd", "kda_fwd_bwd", "kda_fwd"):
        del d
        torch.cuda.empty_cache()
        strong = strong_scaling(bench, wl, K, W, n_streams, ms_per_step, ms1)
        check = shard_check(bench)

    if rank == 0:
        peaks = _peaks()
        roofline = roofline_of(wl, ktimes, peaks)
        step_roofline = None
        if wl.step_flops():
            tf = wl.step_flops() / (ms_per_step * 1e-3) / 1e12
            step_roofline = {"algorithmic_tflops": tf, "frac_of_bf16_peak": tf / peaks["bf16_tflops"]}
            if ms1 is not None:
                tf1 = wl.step_flops() / (ms1 * 1e-3) / 1e12
                step_roofline["single_stream"] = {"algorithmic_tflops": tf1, "frac_of_bf16_peak": tf1 / peaks["bf16_tflops"]}
        cpu_baseline = parity = None
        if not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            tps, sample, inp, ref = cpu_reference(wl, threads, steps=2, warmup=1, check64=True)   # warmed, like the --impl reference arm
            cpu_baseline = {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample}
            parity = parity_block(wl, inp, ref, dev)
        workloads = None
        if world == 1 and not args.no_workloads and not args.shape:
            workloads = other_workloads(bench, wl.name, local, peaks)
        line = {
            "metric": f"GDN/KDA tokens/s ({wl.name})", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": wl.name, **wl.cfg, "global_batch": wl.cfg.get("B", wl.cfg.get("N")) * world,
                       "parallelism": f"one replica of the batch per GPU x{world}, no collective",
                       "l2": "inputs per step exceed the 126 MB L2" if wl.name != "decode" else
                             "the 1.07 GB state pool streamed every step exceeds the 126 MB L2",
                       "cuda_graph": wl.name == "decode",
                       "streams": f"{n_streams}: the K independent steps are issued round-robin on {n_streams} CUDA streams"
                                  if n_streams > 1 else "1"},
            "single_stream": single,
            "roofline": roofline, "kernels": ktimes, "step_roofline": step_roofline, "cpu_baseline": cpu_baseline,
            "parity": parity, "e2e": e2e, "strong": strong, "shard_check": check, "workloads": workloads,
            "gpu_launches": wl.launches_per_step() * K, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
