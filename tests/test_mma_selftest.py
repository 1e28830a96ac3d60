"""Hardware check of the tcgen05 tile-GEMM building block through the C ABI.

Every chunk kernel stages its tensor-core operands with the same panel layout and descriptors,
so a wrong swizzle, operand-major bit or accumulator lane map would silently corrupt all of
them; this test pins each combination against a float64 matmul of the same bf16 inputs.
"""
import ctypes
import itertools

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(lib, M, N, K, a_mn, b_mn, lane_off=0, prefill=0, seed=0):
    g = torch.Generator().manual_seed(seed)
    A = torch.randn(M, K, generator=g).to(torch.bfloat16)
    B = torch.randn(N, K, generator=g).to(torch.bfloat16)
    a_dev = (A.t().contiguous() if a_mn else A.contiguous()).cuda()
    b_dev = (B.t().contiguous() if b_mn else B.contiguous()).cuda()
    d = torch.full((128, N), float("nan"), device="cuda", dtype=torch.float32)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    st = lib.fla_b200_selftest_mma(
        ctypes.c_void_p(a_dev.data_ptr()), ctypes.c_void_p(b_dev.data_ptr()), ctypes.c_void_p(d.data_ptr()),
        M, N, K, a_mn, b_mn, lane_off, prefill, ctypes.c_void_p(err.data_ptr()),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == 0, f"status {st}"
    torch.cuda.synchronize()
    assert int(err.item()) == 0, "device-side wait timed out"
    ref = A.double() @ B.double().t()
    rows = torch.arange(M)
    lanes = rows if M == 128 else (rows % 16) + 32 * (rows // 16) + lane_off
    got = d.cpu()[lanes].double()
    if prefill:
        ref = ref + lanes.double()[:, None] + torch.arange(N).double()[None, :] * 0.001
    return got, ref


CASES = [
    (128, 64, 128, 0, 0), (128, 64, 64, 0, 0), (64, 64, 128, 0, 0),
    (128, 64, 64, 1, 1), (128, 128, 64, 1, 1), (64, 64, 64, 1, 1),
    (128, 64, 128, 0, 1), (64, 64, 64, 0, 1), (64, 128, 64, 0, 1),
    (64, 64, 64, 1, 0), (128, 128, 128, 0, 0), (128, 256, 64, 0, 1),
]


@pytest.mark.parametrize("M,N,K,a_mn,b_mn", CASES)
def test_tile_gemm(lib, M, N, K, a_mn, b_mn):
    got, ref = _run(lib, M, N, K, a_mn, b_mn)
    err = (got - ref).abs().max().item()
    assert err < 1e-3 * max(1.0, ref.abs().max().item()), f"max err {err}"


def test_m64_lane_offset_16(lib):
    got, ref = _run(lib, 64, 64, 64, 0, 0, lane_off=16)
    assert (got - ref).abs().max().item() < 1e-2


def test_accumulate_on_tmem_store(lib):
    got, ref = _run(lib, 128, 64, 64, 0, 0, prefill=1)
    assert (got - ref).abs().max().item() < 1e-2



@pytest.mark.parametrize("N,K,b_mn,a_col", [(128, 128, 0, 0), (64, 64, 0, 64), (128, 64, 1, 8), (64, 64, 1, 0), (256, 64, 1, 128)])
def test_tile_gemm_with_a_from_tensor_memory(lib, N, K, b_mn, a_col):
    """A operand packed into TMEM by the kernel (two bf16 per 32-bit column, 8 columns per K = 16 step), B from panels."""
    g = torch.Generator().manual_seed(100 + N + K + b_mn)
    A = torch.randn(128, K, generator=g).to(torch.bfloat16)
    B = torch.randn(N, K, generator=g).to(torch.bfloat16)
    b_dev = (B.t().contiguous() if b_mn else B.contiguous()).cuda()
    a_dev = A.contiguous().cuda()
    d = torch.full((128, N), float("nan"), device="cuda", dtype=torch.float32)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    st = lib.fla_b200_selftest_mma_ts(ctypes.c_void_p(a_dev.data_ptr()), ctypes.c_void_p(b_dev.data_ptr()), ctypes.c_void_p(d.data_ptr()),
                                      N, K, b_mn, a_col, ctypes.c_void_p(err.data_ptr()),
                                      ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == 0, f"status {st}"
    torch.cuda.synchronize()
    assert int(err.item()) == 0, "device-side wait timed out"
    ref = A.double() @ B.double().t()
    e = (d.cpu().double() - ref).abs().max().item()
    assert e < 1e-3 * max(1.0, ref.abs().max().item()), f"max err {e}"


@pytest.mark.parametrize("N,K", [(64, 64), (128, 64), (128, 128), (64, 32)])
@pytest.mark.parametrize("variant", [0, 1, 2])
def test_tile_gemm_with_strip_layout_operands(lib, N, K, variant):
    """Operands in the un-swizzled strip layout ([N / 8][K rows][16 bytes], reduction dim along rows) that the scan kernels save
    for the chunk-parallel backward: B always, A from tensor memory (variant 0) or in strips too (variant 1).  Variant 2 reads
    strips laid along the reduction dim ([K / 8][N rows][16 bytes]): how the reverse scan reads the chunk inverse transposed."""
    g = torch.Generator().manual_seed(300 + N + K)
    A = torch.randn(128, K, generator=g).to(torch.bfloat16)
    B = torch.randn(N, K, generator=g).to(torch.bfloat16)
    a_dev, b_dev = A.contiguous().cuda(), (B.contiguous() if variant == 2 else B.t().contiguous()).cuda()
    d = torch.full((128, N), float("nan"), device="cuda", dtype=torch.float32)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    st = lib.fla_b200_selftest_mma_nosw(ctypes.c_void_p(a_dev.data_ptr()), ctypes.c_void_p(b_dev.data_ptr()), ctypes.c_void_p(d.data_ptr()),
                                        N, K, variant, ctypes.c_void_p(err.data_ptr()),
                                        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == 0, f"status {st}"
    torch.cuda.synchronize()
    assert int(err.item()) == 0, "device-side wait timed out"
    ref = A.double() @ B.double().t()
    e = (d.cpu().double() - ref).abs().max().item()
    assert e < 1e-3 * max(1.0, ref.abs().max().item()), f"max err {e}"
