"""fp16 tensors through the operators that take them in the reference (examples/flash_gated_delta_rule.py:1161-1162 rejects
only fp32; the published KDA 4-stage case is fp16, fla/ops/ascendc/kda/KDA_FORWARD_VALIDATION_REPORT.md:133-146).

* the conversion kernel: bit-exact against `Tensor.to` for every pair of f32 / bf16 / f16, dense, strided and odd rows;
* decode (`fused_recurrent_gated_delta_rule`, `recurrent_gated_delta_rule`, `recurrent_kda`): fp16 values are read exactly
  and the arithmetic is fp32, so the fp32-oracle bar of the bf16 tests holds unchanged;
* chunk operators: q, k, v are rounded to the bf16 operands of the tensor-core products.  Two comparisons, both with the
  tolerance written here: against the fp64 oracle fed the SAME rounded operands at the plain 5e-3 bar (the kernels add
  nothing beyond what they add for bf16 callers), and against the fp64 oracle fed the original fp16 tensors at
  FP16_INPUT_TOL = 6e-2: rounding q, k, v, dO from 11 to 8 significant bits alone moves o, the final state and the
  gradients by 1e-2..4e-2 of their RMS in the worst element (the same distance a bf16 caller's tensors are from their
  fp32 originals), so fp16 callers get bf16-operand accuracy, not fp16-operand accuracy.
"""
import pytest
import torch

import oracle
from _util import assert_close, rel_err

pytestmark = pytest.mark.gpu
TOL = 5e-3
FP16_INPUT_TOL = 6e-2
DTYPES = (torch.float32, torch.bfloat16, torch.float16)


@pytest.mark.parametrize("src", DTYPES)
@pytest.mark.parametrize("dst", DTYPES)
def test_convert_matches_torch_bit_exact(src, dst):
    from fla_b200.ops._convert import convert
    gen = torch.Generator().manual_seed(7)
    x = (torch.randn(3, 50, 4, 128, generator=gen) * torch.logspace(-6, 3, 128)).to(src).cuda()
    assert torch.equal(convert(x, dst), x.to(dst))
    xt = x.transpose(1, 2)                       # head-first view: strided rows, dense result
    got = convert(xt, dst)
    assert got.is_contiguous() and torch.equal(got, xt.to(dst))
    odd = x[0, :, 0, :37]                        # rows of 37 elements at unaligned addresses: the scalar path
    assert torch.equal(convert(odd, dst), odd.to(dst))
    flat = x.reshape(-1)[: 8 * 1000]
    assert torch.equal(convert(flat, dst), flat.to(dst))


def test_convert_is_differentiable():
    from fla_b200.ops._convert import to_dtype
    x = torch.randn(2, 16, 2, 64, device="cuda", dtype=torch.float16, requires_grad=True)
    y = to_dtype(x, torch.bfloat16)
    assert y.dtype == torch.bfloat16 and to_dtype(y, torch.bfloat16) is y
    y.float().sum().backward()
    assert x.grad.dtype == torch.float16 and torch.equal(x.grad, torch.ones_like(x))


def _bf16_rounded(inp):
    return {n: (t.to(torch.bfloat16) if (t is not None and n in ("q", "k", "v", "do")) else t) for n, t in inp.items()}


@pytest.mark.parametrize("B,T,HK,HV", [(1, 200, 1, 2), (2, 256, 2, 4)])
def test_chunk_gated_delta_rule_fp16(B, T, HK, HV):
    from fla_b200.ops import chunk_gated_delta_rule
    inp = oracle.make_gdn_inputs(B, T, HK, HV, seed=900 + T, dtype=torch.float16)
    refs = {}
    for tag, src in (("exact", inp), ("rounded", _bf16_rounded(inp))):
        refs[tag] = oracle.gdn_reference_fwd_bwd(src["q"], src["k"], src["v"], src["g"], src["beta"], initial_state=src["h0"],
                                                 do=src["do"], dht=src["dht"], dtype=torch.float64)
    d = {n: (t.cuda() if t is not None else None) for n, t in inp.items()}
    leaves = [d[n].requires_grad_() for n in ("q", "k", "v", "g", "beta", "h0")]
    o, ht = chunk_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"], output_final_state=True)
    assert o.dtype == torch.float16 and ht.dtype == torch.float32
    torch.autograd.backward([o, ht], [d["do"], d["dht"]])
    for t in leaves[:5]:
        assert t.grad.dtype == torch.float16
    got = dict(o=o, ht=ht, dq=d["q"].grad, dk=d["k"].grad, dv=d["v"].grad, dg=d["g"].grad, dbeta=d["beta"].grad, dh0=d["h0"].grad)
    half_stored = {"o", "dq", "dk", "dv", "dg", "dbeta"}     # rounded to bf16 / fp16 on the way out: half-ulp allowance
    for name, val in got.items():
        assert_close(f"{name} vs oracle on the rounded operands", val, refs["rounded"][name], TOL, stored_bf16=name in half_stored)
        assert_close(f"{name} vs oracle on the fp16 tensors", val, refs["exact"][name], FP16_INPUT_TOL,
                     stored_bf16=name in half_stored)


def test_flash_gated_delta_rule_fp16_head_first():
    """The reference's composed entry with fp16 `[B,H,T,D]` tensors: same result as the bf16 call on the rounded tensors."""
    from fla_b200.ops import flash_gated_delta_rule
    inp = oracle.make_gdn_inputs(2, 192, 2, 2, seed=77, dtype=torch.float16, with_grad=False)
    q, k, v = (inp[n].cuda().transpose(1, 2).contiguous() for n in ("q", "k", "v"))       # [B,H,T,D]
    g, beta = inp["g"].cuda(), inp["beta"].cuda()
    o16, ht16 = flash_gated_delta_rule(q, k, v, g, beta, output_final_state=True)
    ob, htb = flash_gated_delta_rule(q.bfloat16(), k.bfloat16(), v.bfloat16(), g.float(), beta.float(), output_final_state=True)
    assert o16.dtype == torch.float16 and o16.shape == ob.shape
    assert torch.equal(ht16, htb)
    # the same fp32 result stored once as fp16 and once as bf16: half an ulp of each apart at most
    diff = (o16.double() - ob.double()).abs()
    assert (diff <= ob.double().abs() * (2.0 ** -8 + 2.0 ** -11) + 2.0 ** -24).all()   # 2^-24: fp16 subnormal spacing, rel_err(o16, ob)


@pytest.mark.parametrize("T", [128, 200])
def test_chunk_kda_fp16(T):
    from fla_b200.ops import chunk_kda
    inp = oracle.make_kda_inputs(1, T, 2, 2, seed=300 + T, dtype=torch.float16)
    refs = {}
    for tag, src in (("exact", inp), ("rounded", _bf16_rounded(inp))):
        refs[tag] = oracle.kda_reference_fwd_bwd(src["q"], src["k"], src["v"], src["g"], src["beta"], do=src["do"],
                                                 dtype=torch.float64)
    d = {n: (t.cuda() if t is not None else None) for n, t in inp.items()}
    for n in ("q", "k", "v", "g", "beta"):
        d[n].requires_grad_()
    o, _ = chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"])
    assert o.dtype == torch.float16
    o.backward(d["do"])
    got = dict(o=o, dq=d["q"].grad, dk=d["k"].grad, dv=d["v"].grad, dg=d["g"].grad, dbeta=d["beta"].grad)
    for name, val in got.items():
        assert val.dtype == torch.float16
        assert_close(f"{name} vs oracle on the rounded operands", val, refs["rounded"][name], TOL, stored_bf16=True)
        assert_close(f"{name} vs oracle on the fp16 tensors", val, refs["exact"][name], FP16_INPUT_TOL, stored_bf16=True)


def test_decode_reads_fp16_exactly():
    from fla_b200.ops import fused_recurrent_gated_delta_rule
    N, HK, HV = 6, 2, 4
    inp = oracle.make_decode_inputs(N, HK, HV, seed=41, tokens_per_seq=3, dtype=torch.float16)
    T = 3
    q, k, v = (inp[n].view(N, T, *inp[n].shape[1:]) for n in ("q", "k", "v"))
    g, beta = (inp[n].view(N, T, HV) for n in ("g", "beta"))
    rep = HV // HK
    ref_o, ref_s = oracle.naive_recurrent_gated_delta_rule(q.repeat_interleave(rep, 2), k.repeat_interleave(rep, 2), v, beta, g,
                                                           scale=128 ** -0.5, initial_state=inp["state"], dtype=torch.float64)
    o, s = fused_recurrent_gated_delta_rule(q.cuda(), k.cuda(), v.cuda(), g.cuda(), beta.cuda(), initial_state=inp["state"].cuda(),
                                            output_final_state=True)
    assert o.dtype == torch.float16
    assert_close("final state", s, ref_s, 1e-5)
    # the fp16 store may move a value by half an fp16 ulp (2^-11 |x|) on top of the fp32 bar
    err = (o.double().cpu() - ref_o).abs()
    rms = ref_o.pow(2).mean().sqrt()
    assert (err <= 1e-5 * rms + ref_o.abs() * 2.0 ** -11).all(), (err.max() / rms).item()


def test_decode_rejects_mixed_activation_dtypes():
    from fla_b200.ops import fused_recurrent_gated_delta_rule
    inp = oracle.make_decode_inputs(2, 1, 1, seed=5)
    q, k, v = (inp[n].unsqueeze(1).cuda() for n in ("q", "k", "v"))
    with pytest.raises(TypeError, match="share one dtype"):
        fused_recurrent_gated_delta_rule(q.half(), k, v, inp["g"].unsqueeze(1).cuda(), inp["beta"].unsqueeze(1).cuda())


def test_npu_chunk_kda_fwd_fp16():
    """The reference's low-level KDA forward takes fp16 q, k, v (_aclnn_ctypes.py:1143-1144): all twelve values come back, the
    fp16 ones equal to the bf16 call on the rounded tensors up to the two storage roundings."""
    from fla_b200.ops import npu_chunk_kda_fwd
    inp = oracle.make_kda_inputs(1, 130, 1, 2, seed=61, dtype=torch.float16, with_grad=False)
    h, b = ([inp[n].cuda().to(dt) for n in ("q", "k", "v")] for dt in (torch.float16, torch.bfloat16))
    g, beta = inp["g"].cuda().float(), inp["beta"].cuda().float()
    o16 = npu_chunk_kda_fwd(*h, g, beta, 128 ** -0.5, 64, output_final_state=True, disable_recompute=True)
    ob = npu_chunk_kda_fwd(*b, g, beta, 128 ** -0.5, 64, output_final_state=True, disable_recompute=True)
    assert torch.equal(o16[1], ob[1]) and torch.equal(o16[2], ob[2])            # final state and gk are fp32 in both
    for i in (0, 3, 4, 5, 6, 7, 8, 9, 10):
        assert o16[i].dtype == torch.float16 and o16[i].shape == ob[i].shape
        diff = (o16[i].double() - ob[i].double()).abs()
        assert (diff <= ob[i].double().abs() * (2.0 ** -8 + 2.0 ** -11) + 2.0 ** -24).all(), i


def _bf16_valued_half(t):
    """fp16 tensor holding values that are exactly representable in bf16 as well (so both dtypes carry the same numbers)."""
    return t.bfloat16().half()


def test_decode_surfaces_fp16_equal_bf16_on_shared_values():
    """recurrent_gated_delta_rule and recurrent_kda with fp16 tensors whose values are bf16-representable: the kernel's
    arithmetic is fp32 on the same numbers, so the updated state pools are bit-identical to the bf16 calls."""
    from fla_b200.ops import recurrent_gated_delta_rule, recurrent_kda
    torch.manual_seed(3)
    bs, mtp, nk, nv, dk, dv = 3, 2, 2, 4, 128, 128
    asl = torch.cat([torch.tensor([1], dtype=torch.int32), torch.full((bs,), mtp, dtype=torch.int32)])
    t = int(asl.sum())
    state = torch.rand((t, nv, dv, dk))
    q = _bf16_valued_half(torch.nn.functional.normalize(torch.rand((t, nk, dk)), p=2, dim=-1)).cuda()
    k = _bf16_valued_half(torch.nn.functional.normalize(torch.rand((t, nk, dk)), p=2, dim=-1)).cuda()
    v = _bf16_valued_half(torch.rand((t, nv, dv))).cuda()
    beta = _bf16_valued_half(torch.rand((t, nv))).cuda()
    g = (-torch.rand((t, nv))).cuda()
    ssm = torch.randperm(t).to(torch.int32).cuda()
    pools, outs = [], []
    for dt in (torch.float16, torch.bfloat16):
        pool = state.clone().cuda()
        outs.append(recurrent_gated_delta_rule(q.to(dt), k.to(dt), v.to(dt), pool, beta=beta.to(dt), scale=dk ** -0.5,
                                               actual_seq_lengths=asl.cuda(), ssm_state_indices=ssm, g=g))
        pools.append(pool)
    assert outs[0].dtype == torch.float16 and torch.equal(pools[0], pools[1])
    a16, ab = outs[0][1:].double(), outs[1][1:].double()          # token 0 is the skipped prefix: its output row is never written
    assert ((a16 - ab).abs() <= ab.abs() * (2.0 ** -8 + 2.0 ** -11) + 2.0 ** -24).all()

    B, T, H, HV = 2, 3, 2, 4
    gen = torch.Generator().manual_seed(5)
    qk = [_bf16_valued_half(torch.nn.functional.normalize(torch.randn(B, T, H, 128, generator=gen), dim=-1)).cuda() for _ in range(2)]
    vv = _bf16_valued_half(torch.randn(B, T, HV, 128, generator=gen)).cuda()
    gg = _bf16_valued_half(torch.nn.functional.logsigmoid(torch.randn(B, T, HV, 128, generator=gen)) / 4).cuda()
    bb = _bf16_valued_half(torch.sigmoid(torch.randn(B, T, HV, generator=gen))).cuda()
    st = (0.1 * torch.randn(B, HV, 128, 128, generator=gen))
    res = []
    for dt in (torch.float16, torch.bfloat16):
        pool = st.clone().cuda()
        o, ht = recurrent_kda(qk[0].to(dt), qk[1].to(dt), vv.to(dt), gg.to(dt), bb.to(dt), pool, output_final_state=True,
                              inplace_final_state=True)
        res.append((o, pool))
    assert res[0][0].dtype == torch.float16 and torch.equal(res[0][1], res[1][1])


def test_flash_gated_delta_rule_fp16_varlen_backward():
    """The composed entry with fp16 head-first tensors, packed sequences and in-kernel l2norm, forward and backward: equal to
    the bf16 call on the rounded tensors up to the storage roundings of o and of the gradients."""
    from fla_b200.ops import flash_gated_delta_rule
    cu = torch.tensor([0, 70, 71, 200], dtype=torch.int32)
    inp = oracle.make_gdn_inputs(1, 200, 2, 4, seed=83, dtype=torch.float16)
    res = {}
    for dt in (torch.float16, torch.bfloat16):
        q, k, v = (inp[n].cuda().to(dt).transpose(1, 2).contiguous().requires_grad_() for n in ("q", "k", "v"))   # [B,H,T,D]
        g, beta = inp["g"].cuda().float().requires_grad_(), inp["beta"].cuda().float().requires_grad_()
        o, ht = flash_gated_delta_rule(q, k, v, g, beta, output_final_state=True, cu_seqlens=cu.cuda(), use_qk_l2norm_in_kernel=True)
        (o.float() * inp["do"].cuda().to(dt).float()).sum().backward()
        res[dt] = (o, ht, q.grad, k.grad, v.grad, g.grad, beta.grad)
    a, b = res[torch.float16], res[torch.bfloat16]
    assert a[0].dtype == torch.float16 and a[2].dtype == torch.float16 and a[4].dtype == torch.float16
    assert torch.equal(a[1], b[1])
    for i, name in ((0, "o"), (2, "dq"), (3, "dk"), (4, "dv"), (5, "dg"), (6, "dbeta")):
        x, y = a[i].double(), b[i].double()                                # the same fp32 values behind two storage roundings
        assert ((x - y).abs() <= y.abs() * (2.0 ** -8 + 2.0 ** -11) + 2.0 ** -24).all(), (name, rel_err(a[i], b[i]))


def test_chunk_kda_fp16_with_gate_in_kernel_backward():
    """fp16 q, k, v and an fp16 raw gate with `use_gate_in_kernel`: same result and gradients (incl. A_log, dt_bias) as the bf16 /
    fp32 call on the rounded tensors, up to the storage roundings."""
    from fla_b200.ops import chunk_kda
    B, T, HK, HV = 1, 130, 1, 2
    inp = oracle.make_kda_inputs(B, T, HK, HV, seed=91, dtype=torch.float16)
    gen = torch.Generator().manual_seed(2)
    raw = torch.randn(B, T, HV, 128, generator=gen).half()
    A_log, dt_bias = torch.randn(HV, generator=gen) * 0.3 - 2.0, torch.randn(HV, 128, generator=gen) * 0.1
    res = {}
    for dt in (torch.float16, torch.bfloat16):
        q, k, v = (inp[n].cuda().to(dt).requires_grad_() for n in ("q", "k", "v"))
        g = (raw.cuda() if dt == torch.float16 else raw.cuda().float()).requires_grad_()
        A, b = A_log.cuda().requires_grad_(), dt_bias.cuda().requires_grad_()
        o, _ = chunk_kda(q, k, v, g, inp["beta"].cuda().float(), use_gate_in_kernel=True, A_log=A, dt_bias=b)
        (o.float() * inp["do"].cuda().to(dt).float()).sum().backward()
        res[dt] = (o, q.grad, k.grad, v.grad, g.grad, A.grad, b.grad)
    a, c = res[torch.float16], res[torch.bfloat16]
    assert a[0].dtype == torch.float16 and a[4].dtype == torch.float16
    assert torch.allclose(a[5], c[5], rtol=1e-5, atol=1e-7) and torch.allclose(a[6], c[6], rtol=1e-5, atol=1e-7)
    for i, name in ((0, "o"), (1, "dq"), (2, "dk"), (3, "dv"), (4, "dg")):
        assert rel_err(a[i], c[i]) < 3e-2, (name, rel_err(a[i], c[i]))
