"""Generate the committed golden fixtures by running the REFERENCE's own CPU functions.

Run once on a machine that has the reference checkout:
    FLA_REFERENCE_ROOT=<path to the reference tree> python tests/golden/make_golden.py
The reference modules import Ascend-only packages at module level, so the needed pure-torch
functions are extracted from the source text with `ast` and executed on their own.  The outputs
(inputs + reference results, float32/int32 numpy arrays) are written next to this script as .npz;
tests/test_oracle_golden.py replays them against oracle/ without needing the reference.
"""
from __future__ import annotations

import ast
import math
import os
import sys
from pathlib import Path
from typing import Any, Iterable, List, Optional, Tuple  # noqa: F401  (used by exec'd reference code)

import numpy as np
import torch
import torch.nn.functional as F

HERE = Path(__file__).resolve().parent
if "FLA_REFERENCE_ROOT" not in os.environ:
    raise SystemExit("set FLA_REFERENCE_ROOT to the reference checkout")
REF = Path(os.environ["FLA_REFERENCE_ROOT"])
sys.path.insert(0, str(HERE.parent.parent))


def extract(path: Path, names, extra=None):
    src = path.read_text()
    tree = ast.parse(src)
    ns = {"torch": torch, "F": F, "math": math, "np": np, "Optional": Optional, "Tuple": Tuple, "Iterable": Iterable, "Any": Any, "List": List}
    if extra:
        ns.update(extra)
    for node in tree.body:
        if isinstance(node, (ast.FunctionDef, ast.ClassDef)) and node.name in names:
            exec(compile(ast.Module([node], []), str(path), "exec"), ns)
    missing = [n for n in names if n not in ns]
    assert not missing, missing
    return ns


def f32(t):
    return t.detach().float().numpy()


def gdn_fixture():
    ns = extract(REF / "examples/flash_gated_delta_rule.py", ["_naive_recurrent_gated_delta_rule_cpu"])
    naive = ns["_naive_recurrent_gated_delta_rule_cpu"]
    g_ = torch.Generator().manual_seed(11)
    B, T, H, K, V = 2, 96, 3, 16, 24
    q = F.normalize(torch.randn(B, T, H, K, generator=g_), dim=-1)
    k = F.normalize(torch.randn(B, T, H, K, generator=g_), dim=-1)
    v = torch.randn(B, T, H, V, generator=g_)
    g = F.logsigmoid(torch.randn(B, T, H, generator=g_))
    beta = torch.sigmoid(torch.randn(B, T, H, generator=g_))
    do = torch.randn(B, T, H, V, generator=g_)
    leaves = [x.clone().requires_grad_(True) for x in (q, k, v, beta, g)]
    o = naive(*leaves, scale=K ** -0.5)
    (o * do).sum().backward()
    np.savez_compressed(HERE / "gdn_naive.npz", q=f32(q), k=f32(k), v=f32(v), g=f32(g), beta=f32(beta), do=f32(do),
                        o=f32(o), dq=f32(leaves[0].grad), dk=f32(leaves[1].grad), dv=f32(leaves[2].grad),
                        dbeta=f32(leaves[3].grad), dg=f32(leaves[4].grad))


def decode_fixture():
    gold_dir = REF / "fla/ops/ascendc/gdn/recurrent_gdn/recurrent_gated_delta_rule/tests/pta"
    ns = extract(gold_dir / "golden.py", ["recurrent_gated_delta_rule_golden"])
    golden = ns["recurrent_gated_delta_rule_golden"]
    torch.manual_seed(42)
    bs, mtp, nk, nv, dk, dv = 3, 2, 2, 4, 16, 8
    asl = torch.cat([torch.tensor([1], dtype=torch.int32), torch.full((bs,), mtp, dtype=torch.int32)])
    t = int(asl.sum())
    state = torch.rand((t, nv, dv, dk)).bfloat16()
    query = F.normalize(torch.rand((t, nk, dk)), p=2, dim=-1).bfloat16()
    key = F.normalize(torch.rand((t, nk, dk)), p=2, dim=-1).bfloat16()
    value = torch.rand((t, nv, dv)).bfloat16()
    beta = torch.rand((t, nv)).bfloat16()
    g = -torch.rand((t, nv))
    ssm = torch.randperm(t).to(torch.int32)
    acc = torch.tensor([1, 2, 1], dtype=torch.int32)
    out, fs = golden(query, key, value, state, beta, dk ** -0.5, asl, ssm, num_accepted_tokens=acc, g=g)
    out2, fs2 = golden(query, key, value, state, beta, dk ** -0.5, asl, ssm, num_accepted_tokens=None, g=g)
    np.savez_compressed(HERE / "decode_golden.npz", query=f32(query), key=f32(key), value=f32(value),
                        state=f32(state), beta=f32(beta), g=f32(g), actual_seq_lengths=asl.numpy(),
                        ssm_state_indices=ssm.numpy(), num_accepted_tokens=acc.numpy(), scale=np.float32(dk ** -0.5),
                        out_acc=f32(out), state_acc=f32(fs), out=f32(out2), state_out=f32(fs2))


def conv_bwd_fixture():
    ns = extract(REF / "torch_custom/fla_npu/test/test_npu_causal_conv1d_bwd.py",
                 ["causal_conv1d_preactivation_ref", "causal_conv1d_bwd_ref"])
    g_ = torch.Generator().manual_seed(23)
    B, T, D, W = 2, 19, 24, 4
    x = torch.randn(B, T, D, generator=g_)
    w = 0.5 * torch.randn(W, D, generator=g_)
    dy = torch.randn(B, T, D, generator=g_)
    init = torch.randn(B, W, D, generator=g_)
    dht = torch.randn(B, W, D, generator=g_)
    out = {}
    for name, act, i0, dh in (("plain", 0, None, None), ("silu_state", 1, init, dht)):
        pre = ns["causal_conv1d_preactivation_ref"](x, w, i0)
        dx, dw, db, dh0 = ns["causal_conv1d_bwd_ref"](x, pre, w, dy, i0, dh, act, cast_reduction_outputs=False)
        out.update({f"{name}_dx": f32(dx), f"{name}_dw": f32(dw), f"{name}_db": f32(db), f"{name}_dh0": f32(dh0)})
    np.savez_compressed(HERE / "conv_bwd_golden.npz", x=f32(x), w=f32(w), dy=f32(dy), init=f32(init), dht=f32(dht), **out)


def conv_fixture():
    ns = extract(REF / "torch_custom/fla_npu/test/test_npu_causal_conv1d.py",
                 ["causal_conv1d_ref", "causal_conv1d_update_ref", "causal_conv1d_update_spec_ref"])

    def make_tensor(shape, start=1.0):  # the reference tests' arange/128 known-answer inputs
        n = int(np.prod(shape))
        return (torch.arange(start, start + n, dtype=torch.float32).reshape(shape) / 128.0)

    x = make_tensor((2, 16, 6), 1.0)             # (batch, dim, seqlen)
    w = make_tensor((16, 4), 101.0) / 64.0
    b = make_tensor((16,), 201.0) / 64.0
    init = make_tensor((2, 16, 3), 301.0) / 64.0
    y0, fs0 = ns["causal_conv1d_ref"](x, w, b, None, True, None, "silu")
    y1, fs1 = ns["causal_conv1d_ref"](x, w, None, init, True, None, None)
    xs = make_tensor((2, 16, 2), 1.0)            # short sequence: final state is left-padded
    y2, fs2 = ns["causal_conv1d_ref"](xs, w, b, None, True, None, "silu")
    st = init.clone()
    xu = make_tensor((2, 16), 7.0)
    yu = ns["causal_conv1d_update_ref"](xu, st, w, b, "silu")
    st_spec = make_tensor((2, 16, 5), 401.0) / 64.0
    st_spec_after = st_spec.clone()
    xsp = make_tensor((2, 16, 3), 9.0)
    ysp = ns["causal_conv1d_update_spec_ref"](xsp, st_spec_after, w, b, [1, 3], "silu")
    np.savez_compressed(HERE / "conv_golden.npz", x=f32(x), w=f32(w), b=f32(b), init=f32(init), y0=f32(y0), fs0=f32(fs0),
                        y1=f32(y1), fs1=f32(fs1), xs=f32(xs), y2=f32(y2), fs2=f32(fs2), xu=f32(xu), yu=f32(yu),
                        st_after=f32(st), st_spec=f32(st_spec), st_spec_after=f32(st_spec_after), xsp=f32(xsp),
                        ysp=f32(ysp), accepted=np.array([1, 3], dtype=np.int32))


def kda_fixture():
    ns = extract(REF / "tests/atk/recurrent_kda/executor_recurrent_kda.py", ["_recurrent_kda_ref"])
    ref = ns["_recurrent_kda_ref"]
    g_ = torch.Generator().manual_seed(13)
    B, T, H, HV, K, V = 1, 40, 2, 4, 16, 8
    q = F.normalize(torch.randn(B, T, H, K, generator=g_), dim=-1)
    k = F.normalize(torch.randn(B, T, H, K, generator=g_), dim=-1)
    v = torch.randn(B, T, HV, V, generator=g_)
    g = F.logsigmoid(torch.randn(B, T, HV, K, generator=g_)) / 4
    beta = torch.sigmoid(torch.randn(B, T, HV, generator=g_))
    h0 = 0.1 * torch.randn(B, HV, V, K, generator=g_)       # reference state is V-first
    out, st = ref(dict(q=q, k=k, v=v, g=g, beta=beta, initial_state=h0, scale=K ** -0.5))
    np.savez_compressed(HERE / "kda_naive.npz", q=f32(q), k=f32(k), v=f32(v), g=f32(g), beta=f32(beta), h0=f32(h0),
                        o=f32(out), ht=f32(st))


def stages_fixture():
    """Per-operator goldens of the forward chain (cumsum -> kkt -> solve_tri -> w,u -> fwd_h -> fwd_o), each produced by the
    reference's own CPU golden for that operator, on one fixed-length and one packed variable-length case."""
    test_dir = REF / "torch_custom/fla_npu/test"
    cumsum_ref = extract(test_dir / "test_npu_chunk_local_cumsum.py", ["reference_impl"])["reference_impl"]
    kkt_ref = extract(test_dir / "test_npu_chunk_scaled_dot_kkt.py",
                      ["iter_chunk_ranges", "chunk_scaled_dot_kkt_reference"])["chunk_scaled_dot_kkt_reference"]
    tri_ref = extract(test_dir / "test_npu_solve_tri_ascend910b.py", ["solve_tril_golden"])["solve_tril_golden"]
    wu_ns = extract(test_dir / "test_npu_recompute_w_u_fwd.py", ["get_bos_eos", "compute_w_golden", "compute_u_golden"])
    common = extract(REF / "tests/atk/common/_ascendc_common_executor.py", ["_chunks", "_num_chunks"])
    h_ref = extract(REF / "tests/atk/chunk_gated_delta_rule_fwd_h/executor_chunk_gated_delta_rule_fwd_h.py",
                    ["_round_elem", "_matmul_npu_aligned", "_forward_h_ref"],
                    extra={"_chunks": common["_chunks"], "_num_chunks": common["_num_chunks"]})["_forward_h_ref"]
    o_ns = extract(REF / "fla/ops/ascendc/gdn/chunk_gdn_fwd/chunk_fwd_o/tests/pta/test_fwd_o.py",
                   ["cdiv_torch", "prepare_chunk_indices", "prepare_lens", "prepare_chunk_offsets", "forward_o_trans_cpu"])
    dv_ns = extract(REF / "fla/ops/ascendc/gdn/chunk_gdn_bwd/chunk_bwd_dv_local/tests/ATK/executor_chunk_bwd_dv_local.py",
                    ["prepare_lens", "cdiv", "prepare_chunk_indices", "chunk_bwd_dv_local_torch"])
    dhu_ref = extract(test_dir / "test_bwd_dhu.py", ["_round_elem", "_matmul_npu_aligned", "_gate_exp2", "_gate_exp",
                                                      "chunk_gated_delta_rule_bwd_dhu_cpu"],
                      extra={"_LN2": math.log(2.0)})["chunk_gated_delta_rule_bwd_dhu_cpu"]
    dqkwg_ref = extract(REF / "tests/atk/chunk_bwd_dqkwg/scripts/chunk_bwd_dqkwg_cpu.py", ["chunk_bwd_dqkwg_cpu"])["chunk_bwd_dqkwg_cpu"]
    da_ref = extract(test_dir / "test_npu_prepare_wy_repr_bwd_da.py", ["get_bos_eos", "compute_dA_cpu"])["compute_dA_cpu"]
    full_ns = extract(test_dir / "test_npu_prepare_wy_repr_bwd_full.py",
                      ["get_bos_eos", "_hv_to_hk", "compute_dv_golden_high_precision", "compute_dk_golden_high_precision",
                       "compute_dg_golden_high_precision", "compute_dbeta_golden_high_precision"])
    torch.Tensor.npu = lambda self: self   # the golden moves its CPU tensors "to the device" before computing

    C, K, V, HK, HV, T = 64, 128, 128, 1, 2, 160
    g_ = torch.Generator().manual_seed(23)
    rnd = lambda *s: torch.randn(*s, generator=g_)  # noqa: E731
    bf = lambda t: t.bfloat16().float()  # noqa: E731
    q = bf(F.normalize(rnd(1, HK, T, K), dim=-1))
    k = bf(F.normalize(rnd(1, HK, T, K), dim=-1))
    v = bf(rnd(1, HV, T, V))
    g_raw = F.logsigmoid(rnd(1, HV, T))
    beta = bf(torch.sigmoid(rnd(1, HV, T)))
    d_o = bf(rnd(1, HV, T, V))
    out = dict(q=f32(q), k=f32(k), v=f32(v), g_raw=f32(g_raw), beta=f32(beta), d_o=f32(d_o))
    for tag, cu in (("fix", None), ("var", [0, 70, 160])):
        cu_t = None if cu is None else torch.tensor(cu)
        gam = cumsum_ref(g_raw, C, False, 1.0, cu_t, torch.float32)
        rev = cumsum_ref(g_raw, C, True, 0.5, cu_t, torch.float32)
        idx = None
        if cu is not None:
            idx = [x for si, (a, b) in enumerate(zip(cu[:-1], cu[1:])) for ci in range((b - a + C - 1) // C) for x in (si, ci)]
        A = kkt_ref(k, gam, beta, C, cu, idx)
        # the inverse golden has no variable-length form: invert sequence by sequence
        if cu is None:
            X = tri_ref(A, C, layout="bnsd")
        else:
            X = torch.cat([tri_ref(A[:, :, a:b].contiguous(), C, layout="bnsd") for a, b in zip(cu[:-1], cu[1:])], dim=2)
        Xb = bf(X)
        NT = len(idx) // 2 if idx else (T + C - 1) // C
        w = wu_ns["compute_w_golden"](k, v, beta, Xb, gam, cu, idx, 1, HV, T, K, C, NT, HK)
        u = wu_ns["compute_u_golden"](v, beta, Xb, cu, idx, 1, HV, T, C, NT)
        wb, ub = bf(w), bf(u)
        if cu is None:
            h, v_new = h_ref(dict(k=k, w=wb, u=ub, g=gam, chunk_size=C), golden_mode="fp64")
            h, v_new = h.float(), v_new.float()
        else:
            parts = [h_ref(dict(k=k[:, :, a:b], w=wb[:, :, a:b], u=ub[:, :, a:b], g=gam[:, :, a:b], chunk_size=C), golden_mode="fp64")
                     for a, b in zip(cu[:-1], cu[1:])]
            h = torch.cat([p_[0] for p_ in parts], dim=2).float()
            v_new = torch.cat([p_[1] for p_ in parts], dim=2).float()
        hb, vnb = bf(h), bf(v_new)
        o = o_ns["forward_o_trans_cpu"](q, k, vnb, hb, gam, None, K ** -0.5, C, cu_t, None)
        # backward stages: intra-chunk dv, then the reverse state pass (the goldens take cu_seqlens as tensor / list)
        cu_b = cu if cu is not None else [0, T]
        dv_loc = dv_ns["chunk_bwd_dv_local_torch"](q, k, d_o, gam, K ** -0.5, torch.tensor(cu_b), C, HV // HK)
        dvb = bf(dv_loc)
        idx_b = idx if idx is not None else [x for ci in range(NT) for x in (0, ci)]
        dh, dh0, dv2 = dhu_ref(q, k, wb, d_o, dvb, cu_seqlens=cu_b, chunk_indices=idx_b, g=gam, h0=torch.zeros(1), scale=K ** -0.5,
                               chunk_size=C, golden_mode="fp64")
        first = [i for i in range(NT) if idx_b[2 * i + 1] == 0]
        # dq, dk, dw, dg from the per-chunk states (this golden is sequence-first, h / dh as [B,NT,H,K,V])
        sf = lambda t: t.transpose(1, 2).contiguous()  # noqa: E731
        dhb, dv2b = bf(dh.float()), bf(dv2.float())
        dq_, dk_, dw_, dg_ = dqkwg_ref(sf(q), sf(k), sf(vnb), sf(d_o), sf(hb), sf(dhb), torch.zeros(1), sf(gam), sf(dv2b), K ** -0.5,
                                       cu_t, C, benchmark=True)
        out.update({f"{tag}_dq": f32(sf(dq_)), f"{tag}_dk": f32(sf(dk_)), f"{tag}_dw": f32(sf(dw_)), f"{tag}_dg": f32(sf(dg_))})
        # backward of the WY representation from dw (of dqkwg) and du (= dv2), through the reference's fp32-input goldens
        dwb, dub = bf(dw_.float().transpose(1, 2)), dv2b
        k_hv = k.repeat_interleave(HV // HK, dim=1)
        dA_ = da_ref(Xb, dwb, gam, beta, k_hv, v, dub, idx, cu, 1, HV, T, K, C, NT)
        wy_dv = full_ns["compute_dv_golden_high_precision"](Xb, dub, beta, cu, idx, 1, HV, T, V, C, NT)
        wy_dk = full_ns["compute_dk_golden_high_precision"](Xb, dwb, gam, beta, dA_, k, cu, idx, 1, HK, HV, T, K, C, NT)
        wy_dg = full_ns["compute_dg_golden_high_precision"](Xb, dwb, gam, beta, dA_, k, cu, idx, 1, HK, HV, T, K, C, NT)
        wy_db = full_ns["compute_dbeta_golden_high_precision"](Xb, dwb, gam, beta, dA_, k, v, dub, cu, idx, 1, HK, HV, T, K, C, NT)
        out.update({f"{tag}_wy_dA": f32(dA_), f"{tag}_wy_dv": f32(wy_dv), f"{tag}_wy_dk": f32(wy_dk), f"{tag}_wy_dg": f32(wy_dg),
                    f"{tag}_wy_dbeta": f32(wy_db)})
        out.update({f"{tag}_dv_local": f32(dv_loc), f"{tag}_dh": f32(dh), f"{tag}_dh0": f32(dh0[0, :, first].transpose(0, 1)),
                    f"{tag}_dv2": f32(dv2)})
        out.update({f"{tag}_gam": f32(gam), f"{tag}_rev": f32(rev), f"{tag}_A": f32(A), f"{tag}_X": f32(X), f"{tag}_w": f32(w),
                    f"{tag}_u": f32(u), f"{tag}_h": f32(h), f"{tag}_v_new": f32(v_new), f"{tag}_o": f32(o)})
    del torch.Tensor.npu
    np.savez_compressed(HERE / "stages_golden.npz", **out)


def kda_bwd_intra_fixture():
    """The reference's golden of chunk_kda_bwd_intra on one dense case with a ragged last chunk."""
    ref = extract(REF / "torch_custom/fla_npu/test/test_npu_chunk_kda_bwd_intra.py",
                  ["_chunk_kda_bwd_intra_reference_bsnd"])["_chunk_kda_bwd_intra_reference_bsnd"]
    g_ = torch.Generator().manual_seed(31)
    B, T, H, K, C = 1, 88, 2, 128, 64
    rnd = lambda *s: torch.randn(*s, generator=g_)  # noqa: E731
    q = F.normalize(rnd(B, T, H, K), dim=-1).bfloat16().float()
    k = F.normalize(rnd(B, T, H, K), dim=-1).bfloat16().float()
    gate = -4.0 * torch.sigmoid(rnd(B, T, H, K))            # safe-gate range (lower bound -4)
    gk = torch.cat([gate[:, s:s + C].cumsum(1) for s in range(0, T, C)], 1) / math.log(2.0)
    beta = torch.sigmoid(rnd(B, T, H))
    d_aqk, d_akk = rnd(B, T, H, C), rnd(B, T, H, C)
    dq, dk, db, dg = rnd(B, T, H, K), rnd(B, T, H, K), rnd(B, T, H), rnd(B, T, H, K)
    out = ref(q, k, gk, beta, d_aqk, d_akk, dq, dk, db, dg, chunk_size=C)
    np.savez_compressed(HERE / "kda_bwd_intra_golden.npz", q=f32(q), k=f32(k), gk=f32(gk), beta=f32(beta), d_aqk=f32(d_aqk),
                        d_akk=f32(d_akk), dq=f32(dq), dk=f32(dk), db=f32(db), dg=f32(dg), dq_out=f32(out[0]), dk_out=f32(out[1]),
                        db_out=f32(out[2]), dg_out=f32(out[3]))


def kda_chunk_fwd_fixture():
    """The reference's chunked golden of chunk_kda_fwd (tests/atk/chunk_kda_fwd/executor_chunk_kda_fwd.py:361-530,
    `_reference_impl` with its helpers), run in float64 on bf16-valued inputs with every intermediate exported:
    one packed variable-length GVA case (HK = 1, HV = 2) with a ragged last chunk and an initial state."""
    from dataclasses import dataclass
    ns = extract(REF / "tests/atk/chunk_kda_fwd/executor_chunk_kda_fwd.py",
                 ["_PreparedInputs", "_as_bool", "_layout_to_bsnd", "_gate_cumsum", "_spans", "_stable_causal_scores",
                  "_reference_impl"], extra={"dataclass": dataclass})
    g_ = torch.Generator().manual_seed(41)
    T, H, HV, K, V, C = 136, 1, 2, 128, 128, 64
    cu = [0, 70, 136]
    rnd = lambda *s: torch.randn(*s, generator=g_)  # noqa: E731
    bf = lambda t: t.bfloat16().double()  # noqa: E731
    q, k = bf(F.normalize(rnd(1, T, H, K), dim=-1)), bf(F.normalize(rnd(1, T, H, K), dim=-1))
    v, g = bf(rnd(1, T, HV, V)), bf(F.logsigmoid(rnd(1, T, HV, K)) / 16)
    beta = bf(torch.sigmoid(rnd(1, T, HV)))
    h0 = (0.1 * rnd(len(cu) - 1, HV, K, V)).double()
    scale = K ** -0.5
    inputs = ns["_PreparedInputs"](q=q, k=k, v=v, g=g, beta=beta, A_log=None, dt_bias=None, initial_state=h0, cu_seqlens=cu,
                                   chunk_indices=None, seed=41)
    spec = dict(layout="BSND", chunk_size=C, T=T, HV=HV, K=K, scale=scale, use_gate_in_kernel=False, safe_gate=False,
                disable_recompute=True, return_intermediate_states=True, state_v_first=False, output_final_state=True)
    names = ("o", "final_state", "gk", "aqk", "akk", "w", "u", "qg", "kg", "v_new", "h")
    out = dict(zip(names, ns["_reference_impl"](inputs, spec)[:11]))
    np.savez_compressed(HERE / "kda_chunk_fwd_golden.npz", q=f32(q), k=f32(k), v=f32(v), g=f32(g), beta=f32(beta), h0=f32(h0),
                        cu=np.asarray(cu, dtype=np.int32), scale=np.float32(scale), **{n: f32(t) for n, t in out.items()})


def fast_gelu_fixture():
    """Forward golden of the reference's FastGELU test on its own input grid (fp32 and bf16 inputs)."""
    ns = extract(REF / "torch_custom/fla_npu/test/test_npu_fast_gelu_custom.py", ["fast_gelu_ref"])
    x = torch.linspace(-3, 3, steps=3 * 16 * 32, dtype=torch.float32).reshape(3, 16, 32)
    xb = (4.0 * torch.randn(5, 7, 24, generator=torch.Generator().manual_seed(7))).bfloat16()
    np.savez_compressed(HERE / "fast_gelu_golden.npz", x=f32(x), y=f32(ns["fast_gelu_ref"](x)), xb=f32(xb),
                        yb=f32(ns["fast_gelu_ref"](xb)))


if __name__ == "__main__":
    fast_gelu_fixture()
    gdn_fixture()
    decode_fixture()
    conv_fixture()
    conv_bwd_fixture()
    kda_fixture()
    stages_fixture()
    kda_bwd_intra_fixture()
    kda_chunk_fwd_fixture()
    for p in sorted(HERE.glob("*.npz")):
        print(p.name, p.stat().st_size)
