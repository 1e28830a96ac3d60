"""The allocation-free backward entry point, called straight through the C ABI.

Some callers cannot allocate device memory when they reach the backward (a runtime with a frozen
device arena, a plugin inside another framework's callback, a fixed-budget loop), so
`fla_b200_gdn_chunk_bwd_noalloc` keeps its scratch in a fixed array inside the library.  This test
checks that it returns exactly what the workspace-taking entry point returns, twice in a row (the
second call meets the first call's leftovers in the shared scratch), and that it refuses problems
that do not fit.  It lives in a file pytest collects last so that a failure here cannot hide others.
"""
import ctypes

import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def _forward(d, scale):
    from fla_b200.ops.gdn import gdn_chunk_fwd
    return gdn_chunk_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], scale, d["h0"], True, None, save_for_backward=True)


def _bwd_args(d, saved, scale, outs):
    from fla_b200 import _runtime as rt
    from fla_b200.ops._structs import GdnChunkBwdArgs
    a = GdnChunkBwdArgs()
    a.q, a.k, a.v, a.beta = rt.desc(d["q"]), rt.desc(d["k"]), rt.desc(d["v"]), rt.desc(d["beta"])
    a.gam, a.x_inv, a.s_img, a.vn_img, a.p_img = (rt.desc(saved[n]) for n in ("gam", "x_inv", "s_img", "vn_img", "p_img"))
    a.d_o, a.dht = rt.desc(d["do"]), rt.desc(d["dht"])
    a.dq, a.dk, a.dv, a.dg, a.dbeta, a.dh0 = (rt.desc(t) for t in outs)
    a.scale, a.chunk_size, a.max_seqlen, a.total_chunks = scale, 64, saved["max_len"], saved["total_chunks"]
    return a


def _alloc_outs(d):
    B, T, HK, K = d["q"].shape
    HV, V = d["v"].shape[2], d["v"].shape[3]
    f = dict(dtype=torch.float32, device="cuda")
    return [torch.full((B, T, HK, K), float("nan"), **f), torch.full((B, T, HK, K), float("nan"), **f),
            torch.full((B, T, HV, V), float("nan"), **f), torch.full((B, T, HV), float("nan"), **f),
            torch.full((B, T, HV), float("nan"), **f), torch.full((B, HV, K, V), float("nan"), **f)]


def test_noalloc_backward_matches_workspace_entry_point_twice(lib):
    scale = 128 ** -0.5
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, seed in enumerate((41, 42)):              # two calls in a row on different data
        inp = oracle.make_gdn_inputs(1, 256 - 64 * call + 7, 2, 4, seed=seed)
        d = {n: t.cuda() for n, t in inp.items()}
        _, _, saved = _forward(d, scale)
        ref_outs, new_outs = _alloc_outs(d), _alloc_outs(d)
        a_ref = _bwd_args(d, saved, scale, ref_outs)
        n = ctypes.c_uint64(0)
        assert lib.fla_b200_gdn_chunk_bwd_workspace_size(ctypes.byref(a_ref), ctypes.byref(n)) == 0
        ws = torch.empty(n.value, dtype=torch.uint8, device="cuda")
        assert lib.fla_b200_gdn_chunk_bwd(ctypes.byref(a_ref), ctypes.c_void_p(ws.data_ptr()), n, stream) == 0
        a_new = _bwd_args(d, saved, scale, new_outs)
        if call == 1:
            # The first call above may have loaded the library's device code and placed the built-in array; from the
            # second call on nothing may change the device's free memory.  mem_get_info asks the driver, so it also
            # sees allocations that bypass torch's caching allocator (a cudaMalloc inside the library).
            torch.cuda.synchronize()
            free_before, _ = torch.cuda.mem_get_info()
        assert lib.fla_b200_gdn_chunk_bwd_noalloc(ctypes.byref(a_new), stream) == 0
        torch.cuda.synchronize()
        if call == 1:
            free_after, _ = torch.cuda.mem_get_info()
            assert free_after == free_before, f"device free memory changed by {free_before - free_after} bytes"
        word = ctypes.c_int32(-1)
        assert lib.fla_b200_gdn_chunk_bwd_noalloc_status(stream, ctypes.byref(word)) == 0
        assert word.value == 0, f"device status {word.value} after the allocation-free call"
        for name, r, o in zip(("dq", "dk", "dv", "dg", "dbeta", "dh0"), ref_outs, new_outs):
            assert torch.isfinite(o).all(), name
            # same kernels, same inputs, deterministic reductions: the results agree to the last bit,
            # well inside the 5e-3 * RMS bar the other backward tests use
            assert torch.equal(r, o), f"{name}: max diff {(r - o).abs().max().item():.3e}"


def test_noalloc_backward_rejects_problems_beyond_its_scratch(lib):
    cap = ctypes.c_uint64(0)
    assert lib.fla_b200_gdn_chunk_bwd_static_scratch_bytes(ctypes.byref(cap)) == 0
    assert cap.value == 32 << 20
    scale = 128 ** -0.5
    inp = oracle.make_gdn_inputs(1, 1024, 16, 32, seed=43)     # 16 chunks x 32 heads: needs ~57 MiB of scratch
    d = {n: t.cuda() for n, t in inp.items()}
    _, _, saved = _forward(d, scale)
    outs = _alloc_outs(d)
    a = _bwd_args(d, saved, scale, outs)
    need = ctypes.c_uint64(0)
    assert lib.fla_b200_gdn_chunk_bwd_workspace_size(ctypes.byref(a), ctypes.byref(need)) == 0
    assert need.value > cap.value
    status = lib.fla_b200_gdn_chunk_bwd_noalloc(ctypes.byref(a), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert status == 9                                        # FLA_ERR_TOO_LARGE, nothing launched
    torch.cuda.synchronize()
    assert torch.isnan(outs[0]).all()
