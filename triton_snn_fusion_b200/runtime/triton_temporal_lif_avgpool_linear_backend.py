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
from ._common import ACT_DTYPES, is_nhwc_dense, lif_scalars, raise_reasons, state_or_none


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
    reasons: List[str] = []
    if not isinstance(x_seq, torch.Tensor):
        return ["x_seq must be a tensor"]
    if not x_seq.is_cuda:
        reasons.append("unsupported_device: x_seq is not CUDA")
    if x_seq.dim() != 5:
        reasons.append(f"unsupported_rank: x_seq.dim must be 5, got {x_seq.dim()}")
    if x_seq.dtype not in ACT_DTYPES:
        reasons.append(f"unsupported_dtype: x_seq dtype must be float32, bfloat16 or float16, got {x_seq.dtype}")
    if not isinstance(v_init, torch.Tensor):
        reasons.append("v_init must be a tensor")
    elif v_init.dim() != 0:
        if x_seq.dim() == 5 and tuple(v_init.shape) != tuple(x_seq.shape[1:]):
            reasons.append(
                f"unsupported_membrane_state: v_init shape {tuple(v_init.shape)} does not match {tuple(x_seq.shape[1:])}")
        if v_init.device != x_seq.device or v_init.dtype != x_seq.dtype:
            reasons.append("unsupported_dtype: v_init device/dtype must match x_seq")
    if not isinstance(fc_weight, torch.Tensor) or fc_weight.dim() != 2:
        reasons.append("fc_weight must be a 2D tensor")
    elif x_seq.dim() == 5:
        if int(fc_weight.shape[1]) != int(x_seq.shape[2]):
            reasons.append(f"unsupported_linear: fc in_features {fc_weight.shape[1]} must match channels {x_seq.shape[2]}")
        if fc_weight.device != x_seq.device or fc_weight.dtype != x_seq.dtype:
            reasons.append("unsupported_dtype: fc_weight device/dtype must match x_seq")
    if isinstance(fc_bias, torch.Tensor) and fc_bias.numel() > 0:
        if isinstance(fc_weight, torch.Tensor) and fc_bias.numel() != fc_weight.shape[0]:
            reasons.append("unsupported_linear: fc_bias shape does not match out_features")
        if fc_bias.device != x_seq.device or fc_bias.dtype != x_seq.dtype:
            reasons.append("unsupported_dtype: fc_bias device/dtype must match x_seq")
    if float(tau) == 0.0:
        reasons.append("unsupported_tau: tau must be nonzero")
    return reasons


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
