"""Randomised parity cases (seeded, so every run sees the same ones): ragged lengths, packed batches, GVA ratios, both value
head dims, optional initial state / final-state cotangent, recomputing and saving backward, conv widths 2-4 with odd channel
counts.  Every output and gradient is held to the bars of the dedicated test files (an absolute 1e-6 is added so that
gradients whose reference is identically zero, e.g. dg of a one-token sequence without initial state, do not divide by 0)."""
import random

import pytest
import torch

import oracle
from _util import rms

pytestmark = pytest.mark.gpu


def _check(tag, got, ref, tol, bf=False):
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    assert got.shape == ref.shape, tag
    r = max(rms(ref), 1e-30)
    err = (got - ref).abs()
    allowed = tol * r + (ref.abs() * 2.0 ** -8 if bf else 0) + 1e-6
    worst = (err - allowed).max().item()
    assert worst <= 0, f"{tag}: max err/RMS {err.max().item() / r:.3e}"


def _lens(rng, n_max, longest):
    return [rng.choice([1, 2, 63, 64, 65, rng.randint(1, longest)]) for _ in range(rng.randint(1, n_max))]


@pytest.mark.parametrize("seed", [1, 2])
def test_gdn_forward_backward_random_cases(seed):
    from fla_b200.ops import chunk_gated_delta_rule_fwd_bwd
    rng = random.Random(seed)
    for it in range(16):
        V, HK, G = rng.choice([128, 128, 256]), rng.choice([1, 2]), rng.choice([1, 2, 4])
        HV = HK * G
        if rng.random() < 0.5:
            cu = [0]
            for L in _lens(rng, 5, 200):
                cu.append(cu[-1] + L)
            B, T = 1, cu[-1]
        else:
            cu, B, T = None, rng.choice([1, 2, 3]), rng.choice([1, 7, 64, 65, 128, 130, rng.randint(1, 260)])
        N = B if cu is None else len(cu) - 1
        inp = oracle.make_gdn_inputs(B, T, HK, HV, V=V, seed=1000 * seed + it, h0_scale=0.0)
        gen = torch.Generator().manual_seed(1000 * seed + it + 7)
        h0 = (0.1 * torch.randn(N, HV, 128, V, generator=gen)).float() if rng.random() < 0.7 else None
        dht = (0.1 * torch.randn(N, HV, 128, V, generator=gen)).float() if rng.random() < 0.7 else None
        ref = oracle.gdn_reference_fwd_bwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], initial_state=h0, do=inp["do"],
                                           dht=dht, dtype=torch.float64, cu_seqlens=cu)
        d = {n: t.cuda() for n, t in inp.items() if t is not None}
        o, ht, grads = chunk_gated_delta_rule_fwd_bwd(
            d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], initial_state=None if h0 is None else h0.cuda(),
            dht=None if dht is None else dht.cuda(), cu_seqlens=None if cu is None else torch.tensor(cu, dtype=torch.int32),
            output_dtype=torch.float32, grad_dtype=torch.float32)
        tag = f"case {it}: B={B} T={T} HK={HK} HV={HV} V={V} cu={cu} h0={h0 is not None} dht={dht is not None}"
        _check(tag + " o", o, ref["o"], 5e-3)
        _check(tag + " ht", ht, ref["ht"], 5e-3)
        for name, got in zip(("dq", "dk", "dv", "dg", "dbeta", "dh0"), grads):
            if got is not None and ref.get(name) is not None:
                _check(f"{tag} {name}", got, ref[name], 5e-3)


@pytest.mark.parametrize("seed", [1, 2])
def test_kda_forward_backward_random_cases(seed):
    from fla_b200.ops import chunk_kda
    rng = random.Random(seed)
    for it in range(10):
        V, HK, G = rng.choice([128, 128, 256]), rng.choice([1, 2]), rng.choice([1, 2])
        HV = HK * G
        if rng.random() < 0.5:
            cu = [0]
            for L in _lens(rng, 4, 150):
                cu.append(cu[-1] + L)
            B, T = 1, cu[-1]
        else:
            cu, B, T = None, rng.choice([1, 2]), rng.choice([1, 7, 64, 65, 128, 130, rng.randint(1, 200)])
        N = B if cu is None else len(cu) - 1
        inp = oracle.make_kda_inputs(B, T, HK, HV, V=V, seed=3000 * seed + it)
        gen = torch.Generator().manual_seed(3000 * seed + it + 7)
        h0 = (0.1 * torch.randn(N, HV, 128, V, generator=gen)).float() if rng.random() < 0.7 else None
        dht = (0.1 * torch.randn(N, HV, 128, V, generator=gen)).float() if rng.random() < 0.7 else None
        recompute = rng.random() < 0.5
        bounds = [0, T] if cu is None else cu
        parts = []
        for i in range(len(bounds) - 1):
            if cu is None:
                parts.append(oracle.kda_reference_fwd_bwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], initial_state=h0,
                                                          do=inp["do"], dht=dht, dtype=torch.float64))
                break
            sl = slice(bounds[i], bounds[i + 1])
            parts.append(oracle.kda_reference_fwd_bwd(
                inp["q"][:, sl], inp["k"][:, sl], inp["v"][:, sl], inp["g"][:, sl], inp["beta"][:, sl],
                initial_state=None if h0 is None else h0[i:i + 1], do=inp["do"][:, sl],
                dht=None if dht is None else dht[i:i + 1], dtype=torch.float64))
        ref = {n: torch.cat([p[n] for p in parts], 1) for n in ("o", "dq", "dk", "dv", "dg", "dbeta")}
        ref["ht"] = torch.cat([p["ht"] for p in parts], 0)
        leaves = {n: inp[n].cuda().requires_grad_(True) for n in ("q", "k", "v", "g", "beta")}
        h0d = None if h0 is None else h0.cuda().requires_grad_(True)
        o, ht = chunk_kda(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"], initial_state=h0d,
                          output_final_state=True, output_dtype=torch.float32,
                          cu_seqlens=None if cu is None else torch.tensor(cu, dtype=torch.int32), disable_recompute=not recompute)
        loss = (o * inp["do"].cuda().float()).sum()
        if dht is not None:
            loss = loss + (ht * dht.cuda()).sum()
        loss.backward()
        tag = f"case {it}: B={B} T={T} HK={HK} HV={HV} V={V} cu={cu} h0={h0 is not None} dht={dht is not None} recompute={recompute}"
        _check(tag + " o", o, ref["o"], 5e-3)
        _check(tag + " ht", ht, ref["ht"], 5e-3)
        for name, leaf in (("dq", "q"), ("dk", "k"), ("dv", "v"), ("dg", "g"), ("dbeta", "beta")):
            _check(f"{tag} {name}", leaves[leaf].grad, ref[name], 5e-3, bf=True)
        if h0 is not None:
            _check(tag + " dh0", h0d.grad, torch.cat([p["dh0"] for p in parts], 0), 5e-3)


def _conv_reference(x, w, b, init, res, act):
    """One sequence in fp64: x [T,D], w [D,W], init [D,W-1] | None -> (y [T,D], final state [D,W-1])."""
    T, W = x.shape[0], w.shape[1]
    pad = torch.zeros(W - 1, x.shape[1], dtype=x.dtype) if init is None else init.t()
    xe = torch.cat([pad, x], 0)
    pre = sum(w[:, j] * xe[j:j + T] for j in range(W))
    if b is not None:
        pre = pre + b
    y = torch.nn.functional.silu(pre) if act else pre
    if res is not None:
        y = y + res
    return y, xe[-(W - 1):].t()


@pytest.mark.parametrize("seed", [1, 2])
def test_conv_forward_backward_random_cases(seed):
    from fla_b200.ops import causal_conv1d
    rng = random.Random(seed)
    for it in range(16):
        W, D, act = rng.choice([2, 3, 4]), rng.choice([8, 64, 1032, 2048]), rng.random() < 0.6
        if rng.random() < 0.5:
            lens = [max(L, W - 1) for L in (rng.choice([1, 2, 3, 4, 5, 63, 64, 65, 129, rng.randint(3, 300)])
                                            for _ in range(rng.randint(1, 5)))]
            cu = [0]
            for L in lens:
                cu.append(cu[-1] + L)
            B, T = 1, cu[-1]
        else:
            cu, B, T = None, rng.choice([1, 2]), rng.choice([W - 1, 5, 64, 65, 128, 200, rng.randint(W - 1, 400)])
        N = B if cu is None else len(cu) - 1
        g = torch.Generator().manual_seed(5000 * seed + it)
        x = torch.randn(B, T, D, generator=g).bfloat16()
        w = (0.5 * torch.randn(D, W, generator=g)).bfloat16()
        b = torch.randn(D, generator=g).bfloat16() if rng.random() < 0.5 else None
        init = torch.randn(N, D, W - 1, generator=g).bfloat16() if rng.random() < 0.6 else None
        res = torch.randn(B, T, D, generator=g).bfloat16() if rng.random() < 0.3 else None
        dy = torch.randn(B, T, D, generator=g).bfloat16()
        dfin = torch.randn(N, D, W - 1, generator=g).bfloat16()
        xr, wr = x.double().requires_grad_(True), w.double().requires_grad_(True)
        br = None if b is None else b.double().requires_grad_(True)
        ir = None if init is None else init.double().requires_grad_(True)
        rr = None if res is None else res.double().requires_grad_(True)
        ys, fins = [], []
        for n in range(N):
            sl = slice(None) if cu is None else slice(cu[n], cu[n + 1])
            row = n if cu is None else 0
            y, f = _conv_reference(xr[row, sl], wr, br, None if ir is None else ir[n], None if rr is None else rr[row, sl], act)
            ys.append(y)
            fins.append(f)
        yref = torch.stack(ys) if cu is None else torch.cat(ys)[None]
        fref = torch.stack(fins)
        ((yref * dy.double()).sum() + (fref * dfin.double()).sum()).backward()
        xd, wd = x.cuda().requires_grad_(True), w.cuda().requires_grad_(True)
        bd = None if b is None else b.cuda().requires_grad_(True)
        idd = None if init is None else init.cuda().requires_grad_(True)
        rd = None if res is None else res.cuda().requires_grad_(True)
        y, fin = causal_conv1d(xd, wd, bd, rd, idd, True, "silu" if act else None,
                               None if cu is None else torch.tensor(cu, dtype=torch.int32).cuda())
        ((y.float() * dy.cuda().float()).sum() + (fin.float() * dfin.cuda().float()).sum()).backward()
        tag = f"case {it}: B={B} T={T} D={D} W={W} silu={act} cu={cu} bias={b is not None} init={init is not None} res={res is not None}"
        _check(tag + " y", y, yref, 2e-3, bf=True)
        _check(tag + " final state", fin, fref, 1e-6, bf=True)
        _check(tag + " dx", xd.grad, xr.grad, 3e-3, bf=True)
        _check(tag + " dw", wd.grad, wr.grad, 3e-3, bf=True)
        if b is not None:
            _check(tag + " db", bd.grad, br.grad, 3e-3, bf=True)
        if init is not None:
            _check(tag + " dh0", idd.grad, ir.grad, 3e-3, bf=True)
        if res is not None:
            _check(tag + " dres", rd.grad, rr.grad, 1e-6, bf=True)
