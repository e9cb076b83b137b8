"""Backend of the LIF -> global avgpool -> linear tail (sum of logits over T).

Mirrors the public names of the reference module of the same name
(runtime/triton_temporal_lif_avgpool_linear_backend.py:8-115 in
pengjh0111/triton-snn-fusion). One ``snnb_lif_avgpool_linear`` call: a single
cluster kernel instead of the reference's two kernels and pooled[T,N,C] round trip.
``use_autotune`` (passed by the op layer, runtime/snn_custom_ops.py:1706) is accepted.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from .. import _lib
from ._common import Gate, is_nhwc_dense, lif_scalars, raise_reasons, state_or_none


@dataclass
class TritonTemporalLIFAvgPoolLinearResult:
    out_sum: torch.Tensor
    v_next: torch.Tensor
    used_triton: bool
    kernel_key: str = "temporal_lif_avgpool_linear"
    fallback_reason: str = ""
    kernel_diagnostics: Optional[Dict] = None


def strict_temporal_lif_avgpool_linear_enabled(strict: bool = False) -> bool:
    return bool(strict) or os.environ.get("CHRONOS_STRICT_TEMPORAL_LIF_AVGPOOL_LINEAR_TRITON", "0") == "1"


def check_temporal_lif_avgpool_linear_support(x_seq, v_init, fc_weight, fc_bias, tau) -> List[str]:
    """Reasons why the tail kernel cannot take this call (empty = it can). Same role as the reference's function
    of this name (runtime/triton_temporal_lif_avgpool_linear_backend.py:22-55); any T >= 1 passes here."""
    g = Gate("x_seq", x_seq)
    if not g:
        return g.why
    g.lead_is(rank=5)
    g.state(v_init, tuple(x_seq.shape[1:]) if x_seq.dim() == 5 else None)
    classes = None
    if g.companion("fc_weight", fc_weight, rank=2, code="unsupported_linear"):
        classes = int(fc_weight.shape[0])
        if x_seq.dim() == 5 and int(fc_weight.shape[1]) != int(x_seq.shape[2]):
            g.add("unsupported_linear", f"fc_weight reads {int(fc_weight.shape[1])} features, the pooled map has "
                                        f"{int(x_seq.shape[2])} channels")
    if isinstance(fc_bias, torch.Tensor) and fc_bias.numel() > 0:
        if classes is not None and fc_bias.numel() != classes:
            g.add("unsupported_linear", f"fc_bias holds {fc_bias.numel()} values for {classes} classes")
        g.companion("fc_bias", fc_bias)
    g.tau(tau)
    return g.why


def run_triton_fused_temporal_lif_avgpool_linear(x_seq, v_init, fc_weight, fc_bias, v_threshold, v_reset, tau,
                                                 detach_reset, strict=False, verbose=False, use_autotune=True):
    """x_seq [T,N,C,H,W] -> (sum_t logits [N,classes], last membrane [N,C,H,W])."""
    reasons = check_temporal_lif_avgpool_linear_support(x_seq, v_init, fc_weight, fc_bias, tau)
    raise_reasons("temporal_lif_avgpool_linear", reasons, strict_temporal_lif_avgpool_linear_enabled(strict), verbose)
    T, N, C, H, W = (int(d) for d in x_seq.shape)
    v0 = state_or_none(v_init)
    nhwc = is_nhwc_dense(x_seq) and (v0 is None or is_nhwc_dense(v0)) and not x_seq.is_contiguous()
    if not nhwc:
        x_seq = x_seq.contiguous()
        v0 = v0.contiguous() if v0 is not None else None
    layout = _lib.NHWC if nhwc else _lib.NCHW
    K = int(fc_weight.shape[0])
    b = fc_bias if isinstance(fc_bias, torch.Tensor) and fc_bias.numel() > 0 else None
    out_sum = torch.empty((N, K), dtype=x_seq.dtype, device=x_seq.device)
    v_next = torch.empty_strided(x_seq.shape[1:], x_seq.stride()[1:], dtype=x_seq.dtype, device=x_seq.device)
    th, vr, ta = lif_scalars(v_threshold, v_reset, tau)
    dt = _lib.dtype_code(x_seq.dtype)
    fc_w = fc_weight.contiguous()  # named so the buffer outlives the launch call
    _lib.check(
        _lib.lib.snnb_lif_avgpool_linear(
            _lib.ptr(x_seq), _lib.ptr(v0), _lib.ptr(fc_w), _lib.ptr(b), _lib.ptr(out_sum),
            _lib.ptr(v_next), T, N, C, H * W, K, layout, dt, dt, th, vr, ta, _lib.current_stream(x_seq.device)),
        "snnb_lif_avgpool_linear")
    diagnostics = {
        "kernel_kind": "standalone_temporal_lif_avgpool_linear",
        "implementation": "sm_100a CUDA (snnb_lif_avgpool_linear)",
        "fuse_organization": "single_cluster_kernel",
        "intermediate_materialization": "none (spike counts in shared memory)",
        "layout": "NHWC" if nhwc else "NCHW",
        "T": T,
        "shape": tuple(x_seq.shape),
        "classes": K,
    }
    return TritonTemporalLIFAvgPoolLinearResult(out_sum, v_next, True, kernel_diagnostics=diagnostics)


# Deprecated aliases kept by the reference (:111-115).
TritonTemporalLIFTailResult = TritonTemporalLIFAvgPoolLinearResult
strict_temporal_lif_tail_enabled = strict_temporal_lif_avgpool_linear_enabled
check_temporal_lif_tail_support = check_temporal_lif_avgpool_linear_support
run_triton_fused_temporal_lif_tail = run_triton_fused_temporal_lif_avgpool_linear
