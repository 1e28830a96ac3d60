"""Device-side failures are observable from the host.

The reference turns every non-zero aclnnStatus into a RuntimeError
(torch_custom/fla_npu/fla_npu/ops/ascendc/_runtime.py:410-411,427-428).  Here launches are asynchronous, so a
kernel reports through the int32 status word at the head of its workspace.  These tests make a bounded wait
run out on purpose - a barrier nobody arrives at, a few thousand polls, no trap and no unbounded loop - and
check that the word, the read-back entry point and the Python runtime all report FLA_ERR_TIMEOUT, that the
context stays usable afterwards, and that healthy calls leave the word at zero.
"""
import ctypes

import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

FLA_ERR_TIMEOUT = 8


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def test_wait_that_runs_out_sets_the_status_word_and_returns(lib):
    ws = torch.zeros(256, dtype=torch.uint8, device="cuda")
    assert lib.fla_b200_selftest_wait_timeout(ctypes.c_uint32(4096), ctypes.c_void_p(ws.data_ptr()), _stream()) == 0
    word = ctypes.c_int32(0)
    assert lib.fla_b200_read_status_word(ctypes.c_void_p(ws.data_ptr()), _stream(), ctypes.byref(word)) == 0
    assert word.value == FLA_ERR_TIMEOUT
    assert int(ws[:4].view(torch.int32).item()) == FLA_ERR_TIMEOUT
    # the kernel returned and released its TMEM: a tensor-core kernel runs right after it on the same context
    from fla_b200.ops import chunk_gated_delta_rule
    inp = oracle.make_gdn_inputs(1, 64, 1, 1, seed=5, with_grad=False)
    o, _ = chunk_gated_delta_rule(*(inp[n].cuda() for n in ("q", "k", "v", "g", "beta")))
    assert torch.isfinite(o).all()


def test_selftest_wait_rejects_long_limits(lib):
    ws = torch.zeros(256, dtype=torch.uint8, device="cuda")
    assert lib.fla_b200_selftest_wait_timeout(ctypes.c_uint32(0), ctypes.c_void_p(ws.data_ptr()), _stream()) == 7
    assert lib.fla_b200_selftest_wait_timeout(ctypes.c_uint32((1 << 20) + 1), ctypes.c_void_p(ws.data_ptr()), _stream()) == 7
    assert lib.fla_b200_selftest_wait_timeout(ctypes.c_uint32(16), None, _stream()) == 1


def test_runtime_raises_on_a_recorded_timeout(lib):
    from fla_b200 import _runtime as rt
    ws = torch.zeros(256, dtype=torch.uint8, device="cuda")
    rt.read_device_status(ws, "selftest")                     # a clean word passes
    assert lib.fla_b200_selftest_wait_timeout(ctypes.c_uint32(1024), ctypes.c_void_p(ws.data_ptr()), _stream()) == 0
    with pytest.raises(RuntimeError, match="FLA_ERR_TIMEOUT"):
        rt.read_device_status(ws, "selftest")


def test_checked_mode_reads_the_word_after_every_chunk_operator():
    """With the check on, every chunk operator synchronises and inspects its status word; healthy calls pass."""
    from fla_b200 import _runtime as rt
    from fla_b200.ops import chunk_gated_delta_rule_fwd_bwd, chunk_kda
    seen = []
    real = rt.read_device_status

    def spy(ws, op="operator"):
        seen.append(op)
        return real(ws, op)
    prev = rt.set_device_status_check(True)
    rt.read_device_status = spy
    try:
        inp = oracle.make_gdn_inputs(1, 130, 1, 2, seed=6)
        d = {n: inp[n].cuda() for n in ("q", "k", "v", "g", "beta", "do")}
        chunk_gated_delta_rule_fwd_bwd(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"])
        kin = oracle.make_kda_inputs(1, 130, 1, 2, seed=7)
        chunk_kda(*(kin[n].cuda() for n in ("q", "k", "v", "g", "beta")))
    finally:
        rt.read_device_status = real
        rt.set_device_status_check(prev)
    assert seen == ["gdn_chunk_fwd", "gdn_chunk_bwd", "kda_chunk_fwd"]
