"""Deprecated alias module: the old ``*_tail`` names of the LIF -> avgpool -> linear backend
(reference runtime/triton_temporal_lif_tail_backend.py:3-12)."""
from .triton_temporal_lif_avgpool_linear_backend import (  # noqa: F401
    TritonTemporalLIFTailResult,
    check_temporal_lif_tail_support,
    run_triton_fused_temporal_lif_tail,
    strict_temporal_lif_tail_enabled,
)
