"""Operator surface.  Every function launches hand-written sm_100a kernels through the C ABI; nothing here computes on
the CPU.  The gate activation of `chunk_kda(use_gate_in_kernel=True)` is a mode of the prep kernel in inference and the
library's gate kernels (`fla_b200_kda_gate_fwd` / `_bwd`) when gradients are required; fp16 tensors enter and leave through
the library's conversion kernel.  What remains PyTorch: the sigmoid of `use_beta_sigmoid_in_kernel` on the `[B,T,HV]`
logits, and layout glue (views, the re-laying of `[B,T,H]` gates)."""
from .conv import (causal_conv1d, causal_conv1d_bwd, causal_conv1d_update, npu_causal_conv1d,  # noqa: F401
                   npu_causal_conv1d_bwd)
from .gdn import (chunk_gated_delta_rule, chunk_gated_delta_rule_bwd, chunk_gated_delta_rule_fwd_bwd,  # noqa: F401
                  ChunkGatedDeltaRuleFunction, flash_gated_delta_rule)
from .kda import chunk_kda, chunk_kda_fwd_bwd, kda_chunk_bwd, npu_chunk_kda_fwd  # noqa: F401
from .gelu import fast_gelu_custom, npu_fast_gelu_custom, npu_fast_gelu_custom_backward  # noqa: F401
from .l2norm import l2norm_bwd, l2norm_fwd  # noqa: F401
from .recurrent import fused_recurrent_gated_delta_rule, recurrent_gated_delta_rule, recurrent_kda  # noqa: F401

npu_recurrent_gated_delta_rule = recurrent_gated_delta_rule
npu_recurrent_kda = recurrent_kda
from .stages import chunk_bwd_dqkwg, chunk_kda_bwd_intra, npu_chunk_bwd_dqkwg, npu_chunk_kda_bwd_intra  # noqa: F401,E402
from .stages import (npu_prepare_wy_repr_bwd, npu_prepare_wy_repr_bwd_da, npu_prepare_wy_repr_bwd_full,  # noqa: F401,E402
                     prepare_wy_repr_bwd, prepare_wy_repr_bwd_da, prepare_wy_repr_bwd_full)
from .stages import (chunk_bwd_dv_local, chunk_gated_delta_rule_bwd_dhu, kda_gate_cumsum, npu_chunk_bwd_dv_local,  # noqa: F401,E402
                     npu_kda_gate_cumsum,
                     npu_chunk_gated_delta_rule_bwd_dhu)
from .stages import (chunk_fwd_o, chunk_gated_delta_rule_fwd_h, chunk_local_cumsum, chunk_scaled_dot_kkt,  # noqa: F401,E402
                     npu_chunk_fwd_o, npu_chunk_gated_delta_rule_fwd_h, npu_chunk_local_cumsum, npu_chunk_scaled_dot_kkt,
                     npu_recompute_w_u_fwd, npu_solve_tri, recompute_w_u_fwd, solve_tri)
