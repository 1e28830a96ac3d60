"""CPU restatement of FastGELU (test infrastructure: only tests, the smoke check and the bench's CPU baseline import it).

Forward golden of the reference: torch_custom/fla_npu/test/test_npu_fast_gelu_custom.py:22-24
(`x / (1 + exp(-1.702 x))` in fp32, cast back to the input dtype).  The reference's backward operator is a vendor
library call (aclnnFastGeluBackward, torch_custom/fla_npu/fla_npu/ops/ascendc/_aclnn_ctypes.py:233-239) with no golden in
the repository: it is pinned here as the exact derivative of the forward formula, checked against autograd in
tests/test_oracle_golden.py.
"""
from __future__ import annotations

import torch

ALPHA = 1.702


def fast_gelu_ref(x: torch.Tensor, dtype=torch.float64) -> torch.Tensor:
    xf = x.to(dtype)
    return xf / (1 + torch.exp(-ALPHA * xf))


def fast_gelu_bwd_ref(dy: torch.Tensor, x: torch.Tensor, dtype=torch.float64) -> torch.Tensor:
    xf, gf = x.to(dtype), dy.to(dtype)
    s = torch.sigmoid(ALPHA * xf)
    return gf * (s + ALPHA * xf * s * (1 - s))
