"""Parity of the stand-alone chunk_kda_bwd_intra operator with the CPU oracle (pinned to the reference's golden by
tests/test_oracle_golden.py) and with the committed vectors the reference's golden produced, through the C ABI.
All of its arithmetic is fp32: the bar is max-abs-err / RMS(ref) <= 1e-5."""
import math
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
from _util import assert_close

pytestmark = pytest.mark.gpu
G = Path(__file__).resolve().parent / "golden"
TOL = 1e-5
NAMES = ("q", "k", "gk", "beta", "d_aqk", "d_akk", "dq", "dk", "db", "dg")


def _inputs(B, T, H, seed, cu=None, beta_dtype=torch.float32, lower=-4.0):
    g_ = torch.Generator().manual_seed(seed)
    rnd = lambda *s: torch.randn(*s, generator=g_)  # noqa: E731
    K, C = 128, 64
    q = torch.nn.functional.normalize(rnd(B, T, H, K), dim=-1).bfloat16()
    k = torch.nn.functional.normalize(rnd(B, T, H, K), dim=-1).bfloat16()
    gate = lower * torch.sigmoid(rnd(B, T, H, K))
    bounds = [0, T] if cu is None else cu
    gk = torch.cat([gate[:, s:min(s + C, e)].cumsum(1) for a, e in zip(bounds[:-1], bounds[1:]) for s in range(a, e, C)], 1) / math.log(2.0)
    beta = torch.sigmoid(rnd(B, T, H)).to(beta_dtype)
    return dict(q=q, k=k, gk=gk, beta=beta, d_aqk=rnd(B, T, H, C), d_akk=rnd(B, T, H, C), dq=rnd(B, T, H, K), dk=rnd(B, T, H, K),
                db=rnd(B, T, H), dg=rnd(B, T, H, K))


def _check(d, cu=None, layout="BSND"):
    from fla_b200.ops import chunk_kda_bwd_intra
    ref = oracle.chunk_kda_bwd_intra_ref(*(d[n] for n in NAMES), cu_seqlens=cu)

    def to_layout(t):
        if layout == "BNSD":
            return t.transpose(1, 2).contiguous()
        return t.squeeze(0).contiguous() if layout == "TND" else t.contiguous()

    dev = [to_layout(d[n]).cuda() for n in NAMES]
    out = chunk_kda_bwd_intra(*dev, cu_seqlens=cu, layout=layout)
    assert all(o.data_ptr() == t.data_ptr() for o, t in zip(out, dev[6:]))      # in place
    for name, got, want in zip(("dq", "dk", "db", "dg"), out, ref):
        got = got.transpose(1, 2) if layout == "BNSD" else (got.unsqueeze(0) if layout == "TND" else got)
        assert_close(name, got, want, TOL)


@pytest.mark.parametrize("B,T,H", [(1, 88, 2), (2, 256, 3), (1, 64, 1), (3, 17, 2)])
def test_dense_bsnd(B, T, H):
    _check(_inputs(B, T, H, seed=3 + T))


def test_dense_bnsd_and_bf16_beta():
    _check(_inputs(2, 130, 2, seed=9, beta_dtype=torch.bfloat16), layout="BNSD")


def test_steepest_safe_gate():
    """Gates at the safe-gate lower bound (-5 per token): 2^(gk differences) spans hundreds of binades across a chunk."""
    d = _inputs(1, 128, 2, seed=11, lower=-5.0)
    gate = torch.full_like(d["gk"], -5.0)
    d["gk"] = torch.cat([gate[:, s:s + 64].cumsum(1) for s in range(0, 128, 64)], 1) / math.log(2.0)
    _check(d)


@pytest.mark.parametrize("layout", ["TND", "BSND"])
def test_varlen(layout):
    cu = [0, 70, 70, 71, 200, 300]      # an empty and a one-token sequence among ragged ones
    _check(_inputs(1, 300, 2, seed=21, cu=cu), cu=cu, layout=layout)


def test_reference_golden_vectors():
    from fla_b200.ops import chunk_kda_bwd_intra
    f = {k: torch.from_numpy(v) for k, v in np.load(G / "kda_bwd_intra_golden.npz").items()}
    dev = [f[n].bfloat16().cuda() if n in ("q", "k") else f[n].cuda() for n in NAMES]
    out = chunk_kda_bwd_intra(*dev)
    for name, got in zip(("dq_out", "dk_out", "db_out", "dg_out"), out):
        assert_close(name, got, f[name], 2e-5)


def test_argument_checks():
    from fla_b200.ops import chunk_kda_bwd_intra
    d = _inputs(1, 64, 1, seed=1)
    dev = [d[n].cuda() for n in NAMES]
    with pytest.raises(RuntimeError, match="chunk_size must be 64"):
        chunk_kda_bwd_intra(*dev, chunk_size=128)
    with pytest.raises(RuntimeError, match="safe_gate=False"):
        chunk_kda_bwd_intra(*dev, safe_gate=False)
    with pytest.raises(RuntimeError, match="TND requires cu_seqlens"):
        chunk_kda_bwd_intra(*dev, layout="TND")
    bad = list(dev)
    bad[2] = bad[2].bfloat16()
    with pytest.raises(RuntimeError, match="gk must be torch.float32"):
        chunk_kda_bwd_intra(*bad)
