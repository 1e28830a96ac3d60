"""The reference's low-level KDA forward surface (npu_chunk_kda_fwd, 12-value return): outputs, score blocks and visibility
against the reference's chunked golden (tests/atk/chunk_kda_fwd/executor_chunk_kda_fwd.py:361-530: Aqk = scale tril(q k^T
2^{gk_i-gk_j}), Akk = (I + beta strict(k k^T 2^{gk_i-gk_j}))^-1, gk = chunk cumsum of the gate / ln 2): once replayed from the
fixture the reference's own function produced, and on further layouts through the oracle restatement pinned to that fixture."""

import pytest
import torch

import oracle
from _util import assert_close

pytestmark = pytest.mark.gpu
C = 64


def _golden_blocks(q, k, g, beta, scale, cu=None):
    """fp64 Aqk, Akk [B,HV,T,64] and base-2 gk [B,HV,T,K] per chunk: the oracle's restatement, itself pinned to the
    reference's chunked golden by tests/test_oracle_golden.py."""
    return oracle.kda_chunk_score_blocks_ref(q, k, g, beta, scale, cu, C)


def test_npu_chunk_kda_fwd_replays_the_reference_golden():
    """The fixture made by running the reference's own chunked golden (tests/atk/chunk_kda_fwd/executor_chunk_kda_fwd.py:
    402-530) on a packed GVA case with an initial state: outputs, final state, gk and both score blocks."""
    import numpy as np
    from pathlib import Path
    from fla_b200.ops import npu_chunk_kda_fwd
    f = {n: torch.from_numpy(np.asarray(a)) for n, a in np.load(Path(__file__).parent / "golden" / "kda_chunk_fwd_golden.npz").items()}
    cu = [int(x) for x in f["cu"]]
    bf = lambda n: f[n].squeeze(0).bfloat16().cuda()  # noqa: E731   (the fixture's inputs are bf16-valued)
    out = npu_chunk_kda_fwd(bf("q"), bf("k"), bf("v"), bf("g"), bf("beta"), float(f["scale"]), 64, layout="TND",
                            initial_state=f["h0"].cuda(), output_final_state=True, cu_seqlens=cu)
    o, ht, gk, aqk, akk = out[:5]
    assert_close("o", o.unsqueeze(0), f["o"], 5e-3, stored_bf16=True)
    assert_close("final_state", ht, f["final_state"], 5e-3)
    assert_close("gk", gk.unsqueeze(0), f["gk"], 1e-5)
    assert_close("Aqk", aqk.unsqueeze(0), f["aqk"], 5e-3, stored_bf16=True)
    assert_close("Akk", akk.unsqueeze(0), f["akk"], 5e-3, stored_bf16=True)


@pytest.mark.parametrize("layout,cu", [("BSND", None), ("BNSD", None), ("TND", [0, 70, 71, 200])])
def test_npu_chunk_kda_fwd_matches_golden(layout, cu):
    from fla_b200.ops import npu_chunk_kda_fwd
    B, T, HK, HV = (1, 200, 2, 4) if cu else (2, 150, 2, 4)
    inp = oracle.make_kda_inputs(B, T, HK, HV, seed=31, with_grad=False)
    scale = 128 ** -0.5
    N = B if cu is None else len(cu) - 1
    h0 = 0.1 * torch.randn(N, HV, 128, 128, generator=torch.Generator().manual_seed(3))
    ref = oracle.kda_reference_fwd_bwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], scale=scale, initial_state=h0) if cu is None else None
    aqk_r, akk_r, gk_r = _golden_blocks(inp["q"], inp["k"], inp["g"], inp["beta"], scale, cu)

    def lay(t):
        t = t.cuda()
        if layout == "BNSD":
            return t.transpose(1, 2).contiguous()
        return t.squeeze(0).contiguous() if layout == "TND" else t

    out = npu_chunk_kda_fwd(lay(inp["q"]), lay(inp["k"]), lay(inp["v"]), lay(inp["g"]), lay(inp["beta"]), scale, 64, layout=layout,
                            initial_state=h0.cuda(), output_final_state=True, cu_seqlens=cu)
    assert len(out) == 12 and all(x is None for x in out[5:11]) and out[11] is not None
    o, ht, gk, aqk, akk = out[:5]
    if layout == "TND":
        o, gk, aqk, akk = o.unsqueeze(0), gk.unsqueeze(0), aqk.unsqueeze(0), akk.unsqueeze(0)
    elif layout == "BNSD":
        o = o.transpose(1, 2)
    assert aqk.dtype == torch.bfloat16 and gk.dtype == torch.float32 and tuple(aqk.shape) == (B, HV, T, C)
    assert_close("gk", gk, gk_r, 1e-5)
    assert_close("Aqk", aqk, aqk_r, 5e-3, stored_bf16=True)
    assert_close("Akk", akk, akk_r, 5e-3, stored_bf16=True)
    if ref is not None:
        assert_close("o", o, ref["o"], 5e-3, stored_bf16=True)
        assert_close("ht", ht, ref["ht"], 5e-3)


def test_visibility_and_refusals():
    from fla_b200.ops import npu_chunk_kda_fwd
    inp = oracle.make_kda_inputs(1, 64, 1, 1, seed=5, with_grad=False)
    args = [inp[n].cuda() for n in ("q", "k", "v", "g", "beta")]
    out = npu_chunk_kda_fwd(*args, 128 ** -0.5, 64)
    assert out[1] is None and out[2] is not None and out[11] is None          # no final state asked, gk visible
    A_log = torch.zeros(1).cuda()
    out = npu_chunk_kda_fwd(*args, 128 ** -0.5, 64, use_gate_in_kernel=True, A_log=A_log)
    assert out[2] is None                                                      # gate activated in the kernel: gk hidden
    out = npu_chunk_kda_fwd(*args, 128 ** -0.5, 64, return_intermediate_states=True)
    assert all(x is None for x in out[5:10]) and tuple(out[10].shape) == (1, 1, 1, 128, 128)   # h alone
    out = npu_chunk_kda_fwd(*args, 128 ** -0.5, 64, use_gate_in_kernel=True, A_log=A_log, disable_recompute=True)
    assert out[2] is not None and all(x is not None for x in out[5:11])       # disable_recompute shows gk and all six
    with pytest.raises(RuntimeError, match="chunk_size must be 64 or 128"):
        npu_chunk_kda_fwd(*args, 128 ** -0.5, 32)
    with pytest.raises(RuntimeError, match="layout must be uppercase"):
        npu_chunk_kda_fwd(*args, 128 ** -0.5, 64, layout="bsnd")


def test_state_v_first_and_value_dim_256():
    """`state_v_first=True` takes / returns `[N,HV,V,K]` states; V = 256 flows through the same surface."""
    from fla_b200.ops import npu_chunk_kda_fwd
    B, T, HK, HV, V = 2, 130, 1, 2, 256
    inp = oracle.make_kda_inputs(B, T, HK, HV, V=V, seed=37, with_grad=False)
    scale = 128 ** -0.5
    h0 = 0.1 * torch.randn(B, HV, 128, V, generator=torch.Generator().manual_seed(4))
    ref = oracle.kda_reference_fwd_bwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], scale=scale, initial_state=h0)
    args = [inp[n].cuda() for n in ("q", "k", "v", "g", "beta")]
    a = npu_chunk_kda_fwd(*args, scale, 64, initial_state=h0.cuda(), output_final_state=True)
    b = npu_chunk_kda_fwd(*args, scale, 64, initial_state=h0.transpose(-1, -2).contiguous().cuda(), output_final_state=True,
                          state_v_first=True)
    assert tuple(b[1].shape) == (B, HV, V, 128) and b[1].is_contiguous()
    assert torch.equal(b[1].transpose(-1, -2), a[1]) and torch.equal(a[0], b[0])
    assert_close("o", a[0], ref["o"], 5e-3, stored_bf16=True)
    assert_close("ht", a[1], ref["ht"], 5e-3)
    with pytest.raises(RuntimeError, match="state_v_first"):
        npu_chunk_kda_fwd(*args, scale, 64, initial_state=h0.cuda(), state_v_first=True)


def test_intermediates_replay_the_reference_golden():
    """disable_recompute=True: w, u, qg, kg, v_new, h against the fixture the reference's own chunked golden produced
    (tests/atk/chunk_kda_fwd/executor_chunk_kda_fwd.py:447-492) on a packed GVA case with a ragged last chunk and an initial
    state; the other outputs must not change when the intermediates are asked for."""
    import numpy as np
    from pathlib import Path
    from fla_b200.ops import npu_chunk_kda_fwd
    f = {n: torch.from_numpy(np.asarray(a)) for n, a in np.load(Path(__file__).parent / "golden" / "kda_chunk_fwd_golden.npz").items()}
    cu = [int(x) for x in f["cu"]]
    bf = lambda n: f[n].squeeze(0).bfloat16().cuda()  # noqa: E731   (the fixture's inputs are bf16-valued)
    args = (bf("q"), bf("k"), bf("v"), bf("g"), bf("beta"), float(f["scale"]), 64)
    kw = dict(layout="TND", initial_state=f["h0"].cuda(), output_final_state=True, cu_seqlens=cu)
    plain = npu_chunk_kda_fwd(*args, **kw)
    out = npu_chunk_kda_fwd(*args, disable_recompute=True, **kw)
    for i in range(5):
        assert torch.equal(out[i], plain[i])
    names = ("w", "u", "qg", "kg", "v_new")
    for name, got in zip(names, out[5:10]):
        assert got.dtype == torch.bfloat16 and tuple(got.shape) == tuple(f[name].shape[1:])
        assert_close(name, got.unsqueeze(0), f[name], 5e-3, stored_bf16=True)
    assert tuple(out[10].shape) == tuple(f["h"].shape[1:])
    assert_close("h", out[10].unsqueeze(0), f["h"], 5e-3, stored_bf16=True)
    only_h = npu_chunk_kda_fwd(*args, return_intermediate_states=True, **kw)
    assert all(x is None for x in only_h[5:10]) and torch.equal(only_h[10], out[10])


@pytest.mark.parametrize("layout", ["BSND", "BNSD"])
def test_intermediates_fixed_length_layouts_and_v_first(layout):
    """Fixed-length batches in both rank-4 layouts, V = 256 and `state_v_first`: the intermediates satisfy the relations that
    define them, v_new = u - w S and S_next = 2^{gk_last} S + kg^T v_new, checked in fp64 on what the call returned (every
    returned tensor is rounded to bf16, and u - w S cancels: 5e-2 of the RMS covers that rounding, a wrong layout or a
    missing factor misses it by orders of magnitude; the values themselves are pinned by the golden replay above)."""
    from fla_b200.ops import npu_chunk_kda_fwd
    B, T, HK, HV, V = 2, 192, 1, 2, 256
    inp = oracle.make_kda_inputs(B, T, HK, HV, V=V, seed=53, with_grad=False)
    h0 = 0.1 * torch.randn(B, HV, 128, V, generator=torch.Generator().manual_seed(6))

    def lay(t):
        return t.cuda().transpose(1, 2).contiguous() if layout == "BNSD" else t.cuda()

    args = [lay(inp[n]) for n in ("q", "k", "v", "g", "beta")]
    out = npu_chunk_kda_fwd(*args, 128 ** -0.5, 64, layout=layout, initial_state=h0.cuda(), output_final_state=True,
                            disable_recompute=True)
    outv = npu_chunk_kda_fwd(*args, 128 ** -0.5, 64, layout=layout, initial_state=h0.transpose(-1, -2).contiguous().cuda(),
                             output_final_state=True, disable_recompute=True, state_v_first=True)
    gk, w, u, qg, kg, v_new, h = (out[i].double().cpu() for i in (2, 5, 6, 7, 8, 9, 10))
    assert tuple(h.shape) == (B, T // 64, HV, 128, V) and tuple(w.shape) == (B, HV, T, 128) and tuple(u.shape) == (B, HV, T, V)
    assert torch.equal(outv[10].transpose(-1, -2), out[10])
    for c in range(T // 64):
        sl = slice(c * 64, (c + 1) * 64)
        S = h[:, c]                                                    # [B,HV,K,V]
        assert_close(f"v_new chunk {c}", v_new[:, :, sl], u[:, :, sl] - w[:, :, sl] @ S, 5e-2)
        nxt = h[:, c + 1] if c + 1 < T // 64 else out[1].double().cpu()
        upd = torch.exp2(gk[:, :, sl][:, :, -1]).unsqueeze(-1) * S + kg[:, :, sl].transpose(-1, -2) @ v_new[:, :, sl]
        assert_close(f"state after chunk {c}", nxt, upd, 5e-2)
    q64 = inp["q"].double().repeat_interleave(HV // HK, 2).permute(0, 2, 1, 3)
    assert_close("qg", qg, q64 * torch.exp2(gk), 5e-3, stored_bf16=True)


@pytest.mark.parametrize("layout,cu", [("BSND", None), ("TND", [0, 70, 71, 200, 392]), ("BNSD", None)])
def test_chunk_size_128(layout, cu):
    """chunk_size = 128 (two of the reference's four published KDA cases, KDA_FORWARD_VALIDATION_REPORT.md:83-84): gk, Aqk and Akk
    of 128-token chunks against the oracle's restatement of the reference golden run with that chunk size (ragged chunks with
    fewer than 65 and with 65..127 tokens included); o and the final state do not depend on the blocking; h holds the state at
    the start of every 128-token chunk."""
    from fla_b200.ops import npu_chunk_kda_fwd
    B, T, HK, HV = (1, 392, 1, 2) if cu else (2, 330, 2, 4)
    inp = oracle.make_kda_inputs(B, T, HK, HV, seed=47, with_grad=False)
    scale = 128 ** -0.5
    aqk_r, akk_r, gk_r = oracle.kda_chunk_score_blocks_ref(inp["q"], inp["k"], inp["g"], inp["beta"], scale, cu, 128)

    def lay(t):
        t = t.cuda()
        if layout == "BNSD":
            return t.transpose(1, 2).contiguous()
        return t.squeeze(0).contiguous() if layout == "TND" else t

    args = [lay(inp[n]) for n in ("q", "k", "v", "g", "beta")]
    ref64 = npu_chunk_kda_fwd(*args, scale, 64, layout=layout, output_final_state=True, cu_seqlens=cu, return_intermediate_states=True)
    out = npu_chunk_kda_fwd(*args, scale, 128, layout=layout, output_final_state=True, cu_seqlens=cu, return_intermediate_states=True)
    assert torch.equal(out[0], ref64[0]) and torch.equal(out[1], ref64[1])
    gk, aqk, akk, h = out[2], out[3], out[4], out[10]
    if layout == "TND":
        gk, aqk, akk = gk.unsqueeze(0), aqk.unsqueeze(0), akk.unsqueeze(0)
    assert tuple(aqk.shape) == (B, HV, T, 128) and aqk.dtype == torch.bfloat16
    assert_close("gk", gk, gk_r, 1e-5)
    assert_close("Aqk", aqk, aqk_r, 5e-3, stored_bf16=True)
    assert_close("Akk", akk, akk_r, 5e-3, stored_bf16=True)
    # h: every second 64-token state of each sequence
    h64 = ref64[10]
    if cu is None:
        n64 = (T + 63) // 64
        assert torch.equal(h, h64[:, 0:n64:2])
    else:
        starts, first = [], 0
        for bos, eos in zip(cu[:-1], cu[1:]):
            n64 = (eos - bos + 63) // 64
            starts += list(range(first, first + n64, 2))
            first += n64
        assert torch.equal(h, h64[starts])
    # disable_recompute at chunk size 128: every intermediate against the oracle's restatement of the reference's chunk loop
    # (pinned to the reference fixture at chunk size 64 by tests/test_oracle_golden.py) run with chunk size 128
    full = npu_chunk_kda_fwd(*args, scale, 128, layout=layout, output_final_state=True, cu_seqlens=cu, disable_recompute=True)
    ref = oracle.kda_chunk_intermediates_ref(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], scale, cu_seqlens=cu, chunk_size=128)
    assert torch.equal(full[0], out[0]) and torch.equal(full[3], out[3]) and torch.equal(full[4], out[4])
    for name, got in zip(("w", "u", "qg", "kg", "v_new"), full[5:10]):
        got = got.unsqueeze(0) if layout == "TND" else got
        assert got.dtype == torch.bfloat16
        assert_close(name, got, ref[name], 5e-3, stored_bf16=True)
    hh = full[10] if layout == "TND" else full[10].reshape(-1, *full[10].shape[2:])
    assert_close("h", hh, ref["h"], 5e-3, stored_bf16=True)


@pytest.mark.parametrize("chunk", [64, 128])
def test_intermediates_edge_cases(chunk):
    """A packed batch with an empty sequence, a one-token sequence and ragged chunks, V = 256, GVA, fp16 tensors and an initial
    state: every one of the twelve values against the oracle's chunk loop on the bf16-rounded tensors, at both chunk sizes."""
    from fla_b200.ops import npu_chunk_kda_fwd
    cu = [0, 0, 1, 130, 131, 330]
    T, HK, HV, V = 330, 1, 2, 256
    inp = oracle.make_kda_inputs(1, T, HK, HV, V=V, seed=71, dtype=torch.float16, with_grad=False)
    h0 = 0.1 * torch.randn(len(cu) - 1, HV, 128, V, generator=torch.Generator().manual_seed(12))
    scale = 128 ** -0.5
    rq, rk, rv = (inp[n].bfloat16() for n in ("q", "k", "v"))
    ref = oracle.kda_chunk_intermediates_ref(rq, rk, rv, inp["g"], inp["beta"], scale, initial_state=h0, cu_seqlens=cu, chunk_size=chunk)
    args = [inp[n].squeeze(0).cuda() for n in ("q", "k", "v")] + [inp["g"].squeeze(0).cuda().float(), inp["beta"].squeeze(0).cuda().float()]
    out = npu_chunk_kda_fwd(*args, scale, chunk, layout="TND", initial_state=h0.cuda(), output_final_state=True, cu_seqlens=cu,
                            disable_recompute=True)
    names = ("o", "final_state", "gk", "aqk", "akk", "w", "u", "qg", "kg", "v_new", "h")
    for name, got in zip(names, out[:11]):
        r = ref[name]
        if name == "o":
            r = r.permute(0, 2, 1, 3)
        if name not in ("final_state", "h"):
            got = got.unsqueeze(0)
        assert got.dtype == (torch.float32 if name in ("final_state", "gk") else torch.float16), name
        assert_close(name, got, r, 1e-5 if name == "gk" else 5e-3, stored_bf16=name not in ("final_state", "gk"))
