"""Parity of the chunked GDN backward with fp64 autograd through the naive recurrent oracle.

Bar: max-abs-err / RMS(ref) <= 5e-3 per gradient tensor (fp32 gradient outputs; bf16 gradient outputs get the
half-ulp allowance of their final rounding on top).
"""
import pytest
import torch

import oracle
from _util import assert_close, rel_err

pytestmark = pytest.mark.gpu
TOL = 5e-3
NAMES = ("dq", "dk", "dv", "dg", "dbeta")


def _ref_and_inputs(B, T, HK, HV, seed, cu=None, h0=True, V=128):
    inp = oracle.make_gdn_inputs(B, T, HK, HV, V=V, seed=seed, h0_scale=0.1 if h0 else 0.0)
    N = B if cu is None else len(cu) - 1
    if cu is not None:
        gen = torch.Generator().manual_seed(seed + 1)
        inp["h0"] = (0.1 * torch.randn(N, HV, 128, V, generator=gen)).float() if h0 else None
        inp["dht"] = (0.1 * torch.randn(N, HV, 128, V, generator=gen)).float()
    ref = oracle.gdn_reference_fwd_bwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], initial_state=inp["h0"],
                                       do=inp["do"], dht=inp["dht"], dtype=torch.float64, cu_seqlens=cu)
    d = {n: (t.cuda() if t is not None else None) for n, t in inp.items()}
    return ref, d


@pytest.mark.parametrize("B,T,HK,HV", [(1, 64, 1, 1), (1, 128, 1, 2), (2, 256, 2, 4), (1, 512, 2, 2)])
def test_backward_fp32_grads(B, T, HK, HV):
    from fla_b200.ops import chunk_gated_delta_rule_fwd_bwd
    ref, d = _ref_and_inputs(B, T, HK, HV, seed=2000 + T)
    o, ht, grads = chunk_gated_delta_rule_fwd_bwd(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], initial_state=d["h0"],
                                                  dht=d["dht"], output_dtype=torch.float32, grad_dtype=torch.float32)
    torch.cuda.synchronize()
    assert_close("o", o, ref["o"], TOL)
    assert_close("ht", ht, ref["ht"], TOL)
    for name, got in zip(NAMES + ("dh0",), grads):
        assert_close(name, got, ref[name], TOL)


@pytest.mark.parametrize("B,T,HK,HV,cu", [(2, 256, 1, 2, None), (1, 100, 2, 2, None),
                                          (1, 300, 1, 2, [0, 70, 71, 200, 300])])
def test_value_dim_256(B, T, HK, HV, cu):
    """V = 256 (the reference's second tiling key for the value head): four 64-column blocks of V per head."""
    from fla_b200.ops import chunk_gated_delta_rule_fwd_bwd
    ref, d = _ref_and_inputs(B, T, HK, HV, seed=4100 + T, cu=cu, V=256)
    o, ht, grads = chunk_gated_delta_rule_fwd_bwd(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], initial_state=d["h0"],
                                                  dht=d["dht"], output_dtype=torch.float32, grad_dtype=torch.float32,
                                                  cu_seqlens=None if cu is None else torch.tensor(cu, dtype=torch.int32))
    torch.cuda.synchronize()
    assert o.shape[-1] == 256 and ht.shape[-1] == 256
    assert_close("o", o, ref["o"], TOL)
    assert_close("ht", ht, ref["ht"], TOL)
    for name, got in zip(NAMES + ("dh0",), grads):
        assert_close(name, got, ref[name], TOL)


@pytest.mark.parametrize("T", [1, 17, 63, 65, 130])
def test_backward_ragged_lengths(T):
    from fla_b200.ops import chunk_gated_delta_rule_fwd_bwd
    ref, d = _ref_and_inputs(1, T, 1, 2, seed=31 + T)
    _, _, grads = chunk_gated_delta_rule_fwd_bwd(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], initial_state=d["h0"],
                                                 dht=d["dht"], grad_dtype=torch.float32)
    for name, got in zip(NAMES + ("dh0",), grads):
        assert_close(name, got, ref[name], TOL)


def test_backward_varlen_packed_no_initial_state():
    from fla_b200.ops import chunk_gated_delta_rule_fwd_bwd
    cu = [0, 70, 71, 199, 263, 300]
    ref, d = _ref_and_inputs(1, 300, 2, 4, seed=77, cu=cu, h0=False)
    _, _, grads = chunk_gated_delta_rule_fwd_bwd(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], dht=d["dht"],
                                                 cu_seqlens=torch.tensor(cu, dtype=torch.int32), grad_dtype=torch.float32)
    for name, got in zip(NAMES, grads[:5]):
        assert_close(name, got, ref[name], TOL)
    assert grads[5] is None


def test_autograd_function_bf16_grads_and_determinism():
    from fla_b200.ops import chunk_gated_delta_rule
    ref, d = _ref_and_inputs(2, 192, 2, 4, seed=5)
    outs = []
    for _ in range(2):
        leaves = {n: d[n].clone().requires_grad_(True) for n in ("q", "k", "v", "g", "beta", "h0")}
        o, ht = chunk_gated_delta_rule(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"],
                                       initial_state=leaves["h0"], output_final_state=True)
        ((o.float() * d["do"].float()).sum() + (ht * d["dht"]).sum()).backward()
        outs.append({n: leaves[n].grad for n in leaves})
    g1, g2 = outs
    for n, r in (("q", "dq"), ("k", "dk"), ("v", "dv"), ("g", "dg"), ("beta", "dbeta")):
        assert g1[n].dtype == torch.bfloat16
        assert_close(r, g1[n], ref[r], TOL, stored_bf16=True)
        assert torch.equal(g1[n], g2[n]), f"{r} differs between identical runs"
    assert_close("dh0", g1["h0"], ref["dh0"], TOL)


def test_forward_only_call_saves_nothing_and_matches():
    from fla_b200.ops import chunk_gated_delta_rule
    ref, d = _ref_and_inputs(1, 128, 1, 2, seed=9)
    with torch.no_grad():
        o, ht = chunk_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"],
                                       output_final_state=True, output_dtype=torch.float32)
    assert not o.requires_grad
    assert_close("o", o, ref["o"], TOL)


# where the zero-length sequence sits in the packed batch: first (its token range starts at row 0 of every buffer), between two
# others, last (its chunk index is one past the last chunk), and two in a row
EMPTY_CASES = {
    "leading": ([0, 70, 71, 200], [0, 0, 70, 71, 200], [1, 2, 3], [0]),
    "interior": ([0, 70, 71, 200], [0, 70, 70, 71, 200], [0, 2, 3], [1]),
    "trailing": ([0, 70, 71, 200], [0, 70, 71, 200, 200], [0, 1, 2], [3]),
    "two_leading_one_trailing": ([0, 128, 200], [0, 0, 0, 128, 200, 200], [2, 3], [0, 1, 4]),
}


@pytest.mark.parametrize("case", list(EMPTY_CASES))
def test_empty_sequence_in_a_packed_batch(case):
    """Zero-length sequences change nothing for the others; their final state is their initial state and their dh0 is
    their dht."""
    from fla_b200.ops import chunk_gated_delta_rule_fwd_bwd
    cu_a, cu_b, keep, empty = EMPTY_CASES[case]
    n_b = len(cu_b) - 1
    inp = oracle.make_gdn_inputs(1, 200, 1, 2, seed=123, h0_scale=0.0)
    gen = torch.Generator().manual_seed(124)
    h0 = (0.1 * torch.randn(n_b, 2, 128, 128, generator=gen)).float()
    dht = (0.1 * torch.randn(n_b, 2, 128, 128, generator=gen)).float()
    d = {n: inp[n].cuda() for n in ("q", "k", "v", "g", "beta", "do")}

    def run(cu, h, dh):
        return chunk_gated_delta_rule_fwd_bwd(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], initial_state=h.cuda(), dht=dh.cuda(),
                                              cu_seqlens=torch.tensor(cu, dtype=torch.int32), grad_dtype=torch.float32)
    o_a, ht_a, g_a = run(cu_a, h0[keep], dht[keep])
    o_b, ht_b, g_b = run(cu_b, h0, dht)
    assert torch.equal(o_a, o_b) and torch.equal(ht_a, ht_b[keep])
    for x, y in zip(g_a[:5], g_b[:5]):
        assert torch.equal(x, y)
    assert torch.equal(g_a[5], g_b[5][keep])
    for e in empty:
        assert torch.equal(ht_b[e].cpu(), h0[e]) and torch.equal(g_b[5][e].cpu(), dht[e])


@pytest.mark.parametrize("packed", [False, True])
def test_two_half_launch_matches_single_launch(packed):
    """With more scan chains than SMs the backward launches the batch as two halves on two streams; with per-kernel
    timing on it launches it whole on one.  Same inputs, both ways: bit-identical gradients (odd number of sequences,
    one of them empty in the packed case)."""
    import fla_b200
    from fla_b200.ops import chunk_gated_delta_rule_fwd_bwd
    lib = fla_b200.load_library()
    HK, HV = 16, 32
    if packed:
        cu = [0, 70, 71, 71, 200, 264, 330, 331]        # 7 sequences x 32 heads = 224 chains
        inp = oracle.make_gdn_inputs(1, cu[-1], HK, HV, seed=31)
        N = len(cu) - 1
        gen = torch.Generator().manual_seed(32)
        inp["h0"] = 0.1 * torch.randn(N, HV, 128, 128, generator=gen)
        inp["dht"] = 0.1 * torch.randn(N, HV, 128, 128, generator=gen)
        cu_t = torch.tensor(cu, dtype=torch.int32)
    else:
        inp = oracle.make_gdn_inputs(5, 200, HK, HV, seed=33)   # 5 x 32 = 160 chains
        cu_t = None
    assert torch.cuda.get_device_properties(0).multi_processor_count < 160
    d = {n: t.cuda() for n, t in inp.items() if t is not None}

    def run():
        o, ht, gr = chunk_gated_delta_rule_fwd_bwd(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], initial_state=d["h0"],
                                                   dht=d["dht"], cu_seqlens=cu_t, grad_dtype=torch.float32)
        torch.cuda.synchronize()
        return gr
    split = run()
    lib.fla_b200_kernel_timing_enable(1)
    try:
        whole = run()
    finally:
        lib.fla_b200_kernel_timing_enable(0)
    for name, a, b in zip(NAMES + ("dh0",), split, whole):
        assert torch.equal(a, b), name
    again = run()
    for name, a, b in zip(NAMES + ("dh0",), split, again):
        assert torch.equal(a, b), name


@pytest.mark.parametrize("seed,T", [(2013, 1024), (2010, 2048), (2007, 768), (2002, 2048)])
def test_gradient_margin_over_seeds(seed, T):
    """Seeds and lengths at which dk / dg / dbeta came closest to (and once crossed) the bar while dZ travelled between the two
    backward kernels as a single bf16; with its residual every tensor stays below half the bar."""
    from fla_b200.ops import chunk_gated_delta_rule_fwd_bwd
    ref, d = _ref_and_inputs(1, T, 4, 8, seed=seed)
    o, ht, grads = chunk_gated_delta_rule_fwd_bwd(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], initial_state=d["h0"],
                                                  dht=d["dht"], output_dtype=torch.float32, grad_dtype=torch.float32)
    torch.cuda.synchronize()
    assert_close("o", o, ref["o"], TOL / 2)
    for name, got in zip(NAMES + ("dh0",), grads):
        assert_close(name, got, ref[name], TOL / 2)
