"""Parity of the chunked KDA backward with fp64 autograd through the naive per-channel-gate recurrence
(oracle/kda.py).  The reference has no complete KDA backward of its own, so autograd through its recurrence
(tests/atk/recurrent_kda/executor_recurrent_kda.py:63-83) is the pin."""
import pytest
import torch
import torch.nn.functional as F

import oracle
from _util import assert_close

pytestmark = pytest.mark.gpu
TOL = 5e-3
GRADS = ("dq", "dk", "dv", "dg", "dbeta")


def _reference(inp, cu, dht):
    if cu is None:
        return oracle.kda_reference_fwd_bwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], initial_state=inp["h0"],
                                            do=inp["do"], dht=dht, dtype=torch.float64)
    parts = []
    for i in range(len(cu) - 1):
        sl = slice(cu[i], cu[i + 1])
        parts.append(oracle.kda_reference_fwd_bwd(
            inp["q"][:, sl], inp["k"][:, sl], inp["v"][:, sl], inp["g"][:, sl], inp["beta"][:, sl],
            initial_state=None if inp["h0"] is None else inp["h0"][i:i + 1], do=inp["do"][:, sl],
            dht=None if dht is None else dht[i:i + 1], dtype=torch.float64))
    ref = {n: torch.cat([p[n] for p in parts], 1) for n in ("o",) + GRADS}
    ref["ht"] = torch.cat([p["ht"] for p in parts], 0)
    ref["dh0"] = None if inp["h0"] is None else torch.cat([p["dh0"] for p in parts], 0)
    return ref


def _run(B, T, HK, HV, seed, h0=True, with_dht=True, cu=None, gate_scale=1.0, V=128, **kw):
    from fla_b200.ops import chunk_kda
    inp = oracle.make_kda_inputs(B, T, HK, HV, V=V, seed=seed)
    inp["g"] = (inp["g"].float() * gate_scale).bfloat16()
    N = B if cu is None else len(cu) - 1
    gen = torch.Generator().manual_seed(seed + 1)
    if h0:
        inp["h0"] = (0.1 * torch.randn(N, HV, 128, V, generator=gen)).float()
    dht = (0.1 * torch.randn(N, HV, 128, V, generator=gen)).float() if with_dht else None
    ref = _reference(inp, cu, dht)
    leaves = {n: inp[n].cuda().requires_grad_(True) for n in ("q", "k", "v", "g", "beta")}
    h0_d = inp["h0"].cuda().requires_grad_(True) if h0 else None
    o, ht = chunk_kda(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"], initial_state=h0_d,
                      output_final_state=True, output_dtype=torch.float32,
                      cu_seqlens=None if cu is None else torch.tensor(cu, dtype=torch.int32), **kw)
    loss = (o * inp["do"].cuda().float()).sum()
    if with_dht:
        loss = loss + (ht * dht.cuda()).sum()
    loss.backward()
    torch.cuda.synchronize()
    got = {"o": o, "ht": ht, "dq": leaves["q"].grad, "dk": leaves["k"].grad, "dv": leaves["v"].grad,
           "dg": leaves["g"].grad, "dbeta": leaves["beta"].grad, "dh0": None if h0_d is None else h0_d.grad}
    return got, ref


def _check(got, ref, stored_bf16=True):
    assert_close("o", got["o"], ref["o"], TOL)
    assert_close("ht", got["ht"], ref["ht"], TOL)
    for n in GRADS:   # gradients come back in the dtype of their bf16 leaves
        assert_close(n, got[n], ref[n], TOL, stored_bf16=stored_bf16)
    if ref.get("dh0") is not None:
        assert_close("dh0", got["dh0"], ref["dh0"], TOL)


@pytest.mark.parametrize("B,T,HK,HV", [(1, 64, 1, 1), (1, 128, 1, 1), (2, 256, 2, 2), (1, 512, 1, 2)])
def test_kda_backward_matches_autograd(B, T, HK, HV):
    got, ref = _run(B, T, HK, HV, seed=4000 + T)
    _check(got, ref)


def test_kda_backward_fp32_gradients_through_the_c_abi():
    # the low-level entry with fp32 gradient buffers is held to the plain bar (no bf16 store allowance)
    from fla_b200.ops.kda import kda_chunk_bwd
    B, T, HK, HV = 1, 256, 2, 2
    inp = oracle.make_kda_inputs(B, T, HK, HV, seed=4100)
    gen = torch.Generator().manual_seed(4101)
    inp["h0"] = (0.1 * torch.randn(B, HV, 128, 128, generator=gen)).float()
    dht = (0.1 * torch.randn(B, HV, 128, 128, generator=gen)).float()
    ref = _reference(inp, None, dht)
    d = {n: t.cuda() for n, t in inp.items()}
    meta = (None, None, B, T, B * (T // 64))
    dq, dk, dv, dg, dbeta, dh0 = kda_chunk_bwd(d["q"], d["k"], d["v"], d["g"], d["beta"], 128 ** -0.5, d["h0"], d["do"],
                                               dht.cuda(), meta, grad_dtype=torch.float32)
    torch.cuda.synchronize()
    for n, t in (("dq", dq), ("dk", dk), ("dv", dv), ("dg", dg), ("dbeta", dbeta), ("dh0", dh0)):
        assert_close(n, t, ref[n], TOL)


@pytest.mark.parametrize("T", [1, 31, 65, 100])
def test_kda_backward_ragged_lengths(T):
    got, ref = _run(1, T, 1, 1, seed=60 + T)
    _check(got, ref)


def test_kda_backward_from_saved_intermediates():
    # disable_recompute=True: the forward keeps its operand images and the backward skips the recomputation
    got, ref = _run(2, 200, 2, 2, seed=88, disable_recompute=True)
    _check(got, ref)
    cu = [0, 70, 71, 199, 263, 300]
    got, ref = _run(1, 300, 2, 2, seed=14, cu=cu, disable_recompute=True)
    _check(got, ref)


@pytest.mark.parametrize("recompute", [True, False])
def test_kda_value_dim_256(recompute):
    """K = 128, V = 256 (the shape of the reference's published KDA forward case): four 64-column blocks of V per head."""
    got, ref = _run(2, 200, 1, 2, seed=4300, V=256, disable_recompute=not recompute)
    assert got["o"].shape[-1] == 256
    _check(got, ref)
    got, ref = _run(1, 300, 1, 2, seed=4301, V=256, cu=[0, 70, 71, 199, 300], disable_recompute=not recompute)
    _check(got, ref)


def test_kda_backward_without_states():
    got, ref = _run(1, 192, 1, 1, seed=71, h0=False, with_dht=False)
    _check(got, ref)


def test_kda_backward_strong_gates():
    got, ref = _run(1, 256, 1, 2, seed=19, gate_scale=16.0)
    _check(got, ref)


def test_kda_backward_varlen_packed():
    cu = [0, 70, 71, 199, 263, 300]
    got, ref = _run(1, 300, 2, 2, seed=13, cu=cu)
    _check(got, ref)


def test_kda_backward_through_the_gate_activation():
    from fla_b200.ops import chunk_kda
    B, T, HK, HV = 1, 128, 1, 2
    inp = oracle.make_kda_inputs(B, T, HK, HV, seed=78)
    gen = torch.Generator().manual_seed(6)
    raw = torch.randn(B, T, HV, 128, generator=gen).bfloat16()
    A_log = torch.randn(HV, generator=gen) * 0.3 - 2.0
    dt_bias = torch.randn(HV, 128, generator=gen) * 0.1
    # oracle: activation + recurrence in fp64 autograd
    raw64 = raw.double().requires_grad_(True)
    A64, b64 = A_log.double().requires_grad_(True), dt_bias.double().requires_grad_(True)
    gate = -torch.exp(A64)[None, None, :, None] * F.softplus(raw64 + b64[None, None])
    q64, k64 = inp["q"].double().repeat_interleave(HV // HK, 2), inp["k"].double().repeat_interleave(HV // HK, 2)
    o_ref, _ = oracle.naive_recurrent_kda(q64, k64, inp["v"].double(), gate, inp["beta"].double(), scale=128 ** -0.5,
                                          dtype=torch.float64)
    (o_ref * inp["do"].double()).sum().backward()
    d = {n: t.cuda() for n, t in inp.items() if t is not None}
    raw_d = raw.cuda().requires_grad_(True)
    A_d, b_d = A_log.cuda().requires_grad_(True), dt_bias.cuda().requires_grad_(True)
    o, _ = chunk_kda(d["q"], d["k"], d["v"], raw_d, d["beta"], use_gate_in_kernel=True, A_log=A_d, dt_bias=b_d,
                     output_dtype=torch.float32)
    (o * d["do"].float()).sum().backward()
    torch.cuda.synchronize()
    assert_close("o", o, o_ref, TOL)
    assert_close("d_raw_gate", raw_d.grad, raw64.grad, TOL, stored_bf16=True)
    assert_close("dA_log", A_d.grad, A64.grad, TOL)
    assert_close("d_dt_bias", b_d.grad, b64.grad, TOL)


def test_kda_beta_given_as_logits():
    """`use_beta_sigmoid_in_kernel` (kda/chunk_kda_fwd/docs/api.md): beta holds logits; output and the gradient
    with respect to the logits against fp64 autograd through sigmoid + recurrence."""
    from fla_b200.ops import chunk_kda
    B, T, HK, HV = 1, 128, 1, 2
    inp = oracle.make_kda_inputs(B, T, HK, HV, seed=79)
    logits = torch.randn(B, T, HV, generator=torch.Generator().manual_seed(9))
    l64 = logits.double().requires_grad_(True)
    q64, k64 = inp["q"].double().repeat_interleave(HV // HK, 2), inp["k"].double().repeat_interleave(HV // HK, 2)
    o_ref, _ = oracle.naive_recurrent_kda(q64, k64, inp["v"].double(), inp["g"].double(), torch.sigmoid(l64), scale=128 ** -0.5,
                                          dtype=torch.float64)
    (o_ref * inp["do"].double()).sum().backward()
    d = {n: t.cuda() for n, t in inp.items() if t is not None}
    l_d = logits.cuda().requires_grad_(True)
    o, _ = chunk_kda(d["q"], d["k"], d["v"], d["g"], l_d, use_beta_sigmoid_in_kernel=True, output_dtype=torch.float32)
    (o * d["do"].float()).sum().backward()
    torch.cuda.synchronize()
    assert_close("o", o, o_ref, TOL)
    assert_close("d_beta_logits", l_d.grad, l64.grad, TOL)


KDA_EMPTY_CASES = {
    "leading": ([0, 70, 71, 200], [0, 0, 70, 71, 200], [1, 2, 3], [0]),
    "interior": ([0, 70, 71, 200], [0, 70, 70, 71, 200], [0, 2, 3], [1]),
    "trailing": ([0, 70, 71, 200], [0, 70, 71, 200, 200], [0, 1, 2], [3]),
}


@pytest.mark.parametrize("case", list(KDA_EMPTY_CASES))
@pytest.mark.parametrize("recompute", [True, False])
def test_kda_empty_sequence_in_a_packed_batch(recompute, case):
    """A zero-length sequence (first, between two others, or last in the packed batch) changes nothing for the others; its
    final state is its initial state and the gradient of its initial state is its dht."""
    from fla_b200.ops import chunk_kda
    cu_a, cu_b, keep, empty = KDA_EMPTY_CASES[case]
    n_b = len(cu_b) - 1
    inp = oracle.make_kda_inputs(1, 200, 1, 2, seed=321)
    gen = torch.Generator().manual_seed(322)
    h0 = (0.1 * torch.randn(n_b, 2, 128, 128, generator=gen)).float()
    dht = (0.1 * torch.randn(n_b, 2, 128, 128, generator=gen)).float()

    def run(cu, h, dh):
        leaves = {n: inp[n].cuda().requires_grad_(True) for n in ("q", "k", "v", "g", "beta")}
        h_d = h.cuda().requires_grad_(True)
        o, ht = chunk_kda(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"], initial_state=h_d,
                          output_final_state=True, cu_seqlens=torch.tensor(cu, dtype=torch.int32), disable_recompute=not recompute)
        ((o.float() * inp["do"].cuda().float()).sum() + (ht * dh.cuda()).sum()).backward()
        return o.detach(), ht.detach(), [leaves[n].grad for n in ("q", "k", "v", "g", "beta")], h_d.grad
    o_a, ht_a, g_a, dh_a = run(cu_a, h0[keep], dht[keep])
    o_b, ht_b, g_b, dh_b = run(cu_b, h0, dht)
    assert torch.equal(o_a, o_b) and torch.equal(ht_a, ht_b[keep])
    for x, y in zip(g_a, g_b):
        assert torch.equal(x, y)
    assert torch.equal(dh_a, dh_b[keep])
    for e in empty:
        assert torch.equal(ht_b[e].cpu(), h0[e]) and torch.equal(dh_b[e].cpu(), dht[e])


def test_kda_qk_l2norm_in_kernel():
    """use_qk_l2norm_in_kernel normalises raw q, k rows (x * rsqrt(sum x^2 + 1e-6)) and differentiates through it."""
    from fla_b200.ops import chunk_kda
    B, T, HK, HV = 1, 150, 1, 2
    inp = oracle.make_kda_inputs(B, T, HK, HV, seed=555)
    gen = torch.Generator().manual_seed(556)
    q_raw = (2.0 * torch.randn(B, T, HK, 128, generator=gen)).bfloat16()
    k_raw = (0.5 * torch.randn(B, T, HK, 128, generator=gen)).bfloat16()

    def norm(x):
        return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + 1e-6)
    qr, kr = q_raw.double().requires_grad_(True), k_raw.double().requires_grad_(True)
    # the operator stores the normalised rows in bf16, like the reference's l2norm_fwd: the oracle sees the same rounding
    qn = norm(qr) + (norm(qr).detach().bfloat16().double() - norm(qr).detach())
    kn = norm(kr) + (norm(kr).detach().bfloat16().double() - norm(kr).detach())
    ref = oracle.naive_recurrent_kda(qn.repeat_interleave(HV // HK, 2), kn.repeat_interleave(HV // HK, 2), inp["v"].double(),
                                     inp["g"].double(), inp["beta"].double(), scale=128 ** -0.5, dtype=torch.float64)[0]
    (ref * inp["do"].double()).sum().backward()
    qd, kd = q_raw.cuda().requires_grad_(True), k_raw.cuda().requires_grad_(True)
    o, _ = chunk_kda(qd, kd, inp["v"].cuda(), inp["g"].cuda(), inp["beta"].cuda(), use_qk_l2norm_in_kernel=True,
                     output_dtype=torch.float32)
    (o * inp["do"].cuda().float()).sum().backward()
    assert_close("o", o, ref.detach(), TOL)
    assert_close("dq", qd.grad, qr.grad, TOL, stored_bf16=True)
    assert_close("dk", kd.grad, kr.grad, TOL, stored_bf16=True)


@pytest.mark.parametrize("recompute", [True, False])
def test_kda_two_half_launch_matches_single_launch(recompute):
    """More scan chains than SMs: the KDA backward launches the batch as two halves on two streams; with per-kernel
    timing on it launches it whole.  Bit-identical gradients either way (three sequences: halves of one and two)."""
    import fla_b200
    from fla_b200.ops import chunk_kda_fwd_bwd
    lib = fla_b200.load_library()
    B, T, H = 3, 200, 32          # 2 blocks of V x 32 heads x 3 sequences = 192 chains
    assert torch.cuda.get_device_properties(0).multi_processor_count < 192
    inp = oracle.make_kda_inputs(B, T, H, H, seed=41)
    d = {n: t.cuda() for n, t in inp.items() if t is not None}

    def run():
        o, ht, gr = chunk_kda_fwd_bwd(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], grad_dtype=torch.float32,
                                      disable_recompute=not recompute)
        torch.cuda.synchronize()
        return [t for t in gr if t is not None]
    split = run()
    lib.fla_b200_kernel_timing_enable(1)
    try:
        whole = run()
    finally:
        lib.fla_b200_kernel_timing_enable(0)
    assert len(split) == len(whole) >= 5
    for i, (a, b) in enumerate(zip(split, whole)):
        assert torch.equal(a, b), i


@pytest.mark.parametrize("safe_gate", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_gate_kernels_match_autograd(safe_gate, dtype):
    """The gate activation kernels (`fla_b200_kda_gate_fwd` / `_bwd`) against fp64 autograd of the documented formulas
    (kda/chunk_kda_fwd/docs/api.md:103-115), with and without dt_bias, a token count that is not a multiple of the tile."""
    from fla_b200.ops.kda import _gate_activation
    B, T, HV, K = 2, 333, 3, 128
    gen = torch.Generator().manual_seed(17)
    g = (2.0 * torch.randn(B, T, HV, K, generator=gen)).to(dtype)
    A_log = torch.randn(HV, generator=gen) * 0.5
    d_gate = torch.randn(B, T, HV, K, generator=gen)
    for bias in (torch.randn(HV * K, generator=gen) * 0.3, None):
        g64, A64 = g.double().requires_grad_(True), A_log.double().requires_grad_(True)
        b64 = None if bias is None else bias.double().requires_grad_(True)
        raw = g64 if b64 is None else g64 + b64.reshape(HV, K)
        eig = A64.exp().reshape(1, 1, HV, 1)
        ref = -5.0 * torch.sigmoid(eig * raw) if safe_gate else -eig * F.softplus(raw)
        ref.backward(d_gate.double())
        gd, Ad = g.cuda().requires_grad_(True), A_log.cuda().requires_grad_(True)
        bd = None if bias is None else bias.cuda().requires_grad_(True)
        got = _gate_activation(gd, Ad, bd, safe_gate, -5.0)
        got.backward(d_gate.cuda())
        assert got.dtype == torch.float32 and gd.grad.dtype == dtype and Ad.grad.shape == A_log.shape
        assert_close("gate", got, ref, 1e-5)
        assert_close("dg", gd.grad, g64.grad, 1e-5 if dtype == torch.float32 else TOL, stored_bf16=dtype != torch.float32)
        assert_close("dA_log", Ad.grad, A64.grad, 1e-4)
        if bias is not None:
            assert bd.grad.shape == bias.shape
            assert_close("d_dt_bias", bd.grad, b64.grad, 1e-4)


def test_kda_backward_through_the_safe_gate():
    """chunk_kda with use_gate_in_kernel and safe_gate: output and every gradient against fp64 autograd."""
    from fla_b200.ops import chunk_kda
    B, T, HK, HV = 1, 128, 1, 2
    inp = oracle.make_kda_inputs(B, T, HK, HV, seed=81)
    gen = torch.Generator().manual_seed(8)
    raw = torch.randn(B, T, HV, 128, generator=gen).bfloat16()
    A_log = torch.randn(HV, generator=gen) * 0.3
    raw64, A64 = raw.double().requires_grad_(True), A_log.double().requires_grad_(True)
    gate = -0.5 * torch.sigmoid(torch.exp(A64)[None, None, :, None] * raw64)
    q64, k64 = inp["q"].double().repeat_interleave(HV // HK, 2), inp["k"].double().repeat_interleave(HV // HK, 2)
    o_ref, _ = oracle.naive_recurrent_kda(q64, k64, inp["v"].double(), gate, inp["beta"].double(), scale=128 ** -0.5,
                                          dtype=torch.float64)
    (o_ref * inp["do"].double()).sum().backward()
    d = {n: t.cuda() for n, t in inp.items() if t is not None}
    raw_d, A_d = raw.cuda().requires_grad_(True), A_log.cuda().requires_grad_(True)
    o, _ = chunk_kda(d["q"], d["k"], d["v"], raw_d, d["beta"], use_gate_in_kernel=True, safe_gate=True, lower_bound=-0.5, A_log=A_d,
                     output_dtype=torch.float32)
    (o * d["do"].float()).sum().backward()
    assert_close("o", o, o_ref, TOL)
    assert_close("d_raw_gate", raw_d.grad, raw64.grad, TOL, stored_bf16=True)
    assert_close("dA_log", A_d.grad, A64.grad, TOL)
