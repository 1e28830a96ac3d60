"""CPU oracle: TEST INFRASTRUCTURE ONLY.

Restates, in plain CPU torch, the reference's own CPU goldens for the GDN / KDA hot path so that
the CUDA kernels can be checked against them on machines where the reference is not present.
Nothing in the shipped package imports this directory; only tests, the smoke check and the
benchmark's CPU-baseline legs do.  Each function cites the reference file:line it follows.

Pinning: every function here is compared against the reference's own function (loaded from the
reference tree by tests/golden/make_golden.py) on seeded inputs; the resulting vectors are the
committed fixtures under tests/golden/, and tests/test_oracle_golden.py replays them.
"""
from .gdn import naive_recurrent_gated_delta_rule, gdn_reference_fwd_bwd, chunk_gated_delta_rule_restated  # noqa: F401
from .kda import (chunk_kda_bwd_intra_ref, kda_chunk_intermediates_ref, kda_chunk_score_blocks_ref, kda_reference_fwd_bwd,  # noqa: F401
                  naive_recurrent_kda)
from .recurrent import recurrent_gated_delta_rule_golden  # noqa: F401
from .conv import (causal_conv1d_bwd_ref, causal_conv1d_ref, causal_conv1d_update_ref,  # noqa: F401
                   causal_conv1d_update_spec_ref)
from .inputs import make_gdn_inputs, make_kda_inputs, make_decode_inputs, make_conv_inputs  # noqa: F401
from . import stages  # noqa: F401
from .gelu import fast_gelu_bwd_ref, fast_gelu_ref  # noqa: F401
