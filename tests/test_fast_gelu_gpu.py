"""Parity of the FastGELU operators with the CPU oracle and the reference's golden grid
(torch_custom/fla_npu/test/test_npu_fast_gelu_custom.py:22-45), through the C ABI."""
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).parent / "golden" / "fast_gelu_golden.npz"


def test_reference_grid_fp32():
    from fla_b200.ops import npu_fast_gelu_custom
    f = np.load(GOLDEN)
    x = torch.from_numpy(f["x"]).cuda()
    y = npu_fast_gelu_custom(x)
    assert y.shape == x.shape and y.dtype == torch.float32
    # the reference's own pass rule
    assert torch.allclose(y.cpu(), torch.from_numpy(f["y"]), rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(y.cpu().double(), oracle.fast_gelu_ref(x.cpu()), rtol=2e-6, atol=2e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(3, 16, 32), (5, 7, 13), (1,), (2, 4099)])
def test_forward_backward_match_oracle(dtype, shape):
    from fla_b200.ops import npu_fast_gelu_custom, npu_fast_gelu_custom_backward
    g_ = torch.Generator().manual_seed(sum(shape))
    x = (3 * torch.randn(shape, generator=g_)).to(dtype)
    dy = torch.randn(shape, generator=g_).to(dtype)
    y = npu_fast_gelu_custom(x.cuda())
    dx = npu_fast_gelu_custom_backward(dy.cuda(), x.cuda())
    assert y.dtype == dtype and dx.dtype == dtype and y.shape == x.shape
    # one rounding to the storage dtype on top of fp32 arithmetic with fast exp
    tol = {torch.float32: 3e-6, torch.bfloat16: 2 ** -8, torch.float16: 2 ** -10}[dtype]
    ref_y, ref_dx = oracle.fast_gelu_ref(x), oracle.fast_gelu_bwd_ref(dy, x)
    torch.testing.assert_close(y.cpu().double(), ref_y, rtol=tol, atol=tol)
    torch.testing.assert_close(dx.cpu().double(), ref_dx, rtol=tol, atol=tol)


def test_autograd_binding_and_non_contiguous_input():
    from fla_b200.ops import fast_gelu_custom
    base = torch.randn(6, 40, generator=torch.Generator().manual_seed(1)).cuda()
    x = base.t().requires_grad_(True)          # non-contiguous view
    y = fast_gelu_custom(x)
    dy = torch.randn(y.shape, generator=torch.Generator().manual_seed(2)).cuda()
    (y * dy).sum().backward()
    torch.testing.assert_close(y.detach().cpu().double(), oracle.fast_gelu_ref(x.detach().cpu()), rtol=3e-6, atol=3e-6)
    torch.testing.assert_close(x.grad.cpu().double(), oracle.fast_gelu_bwd_ref(dy.cpu(), x.detach().cpu()), rtol=3e-6, atol=3e-6)
    assert fast_gelu_custom(torch.empty(0, 4, device="cuda")).shape == (0, 4)
