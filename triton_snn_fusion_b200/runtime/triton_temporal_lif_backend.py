"""Backend of the standalone temporal LIF op.

Same entry point and result type as the reference module of this name
(runtime/triton_temporal_lif_backend.py:8-117 in pengjh0111/triton-snn-fusion); the
work is done by ``snnb_lif_scan`` (one coalesced pass, membrane in registers).
Differences from the reference, all widening: bf16 is accepted, T is arbitrary,
``use_autotune`` (passed by the op layer, runtime/snn_custom_ops.py:1632) is
accepted and ignored, and there is no fallback of any kind.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from .. import _lib
from ._common import Gate, lif_scalars, raise_reasons, state_or_none


@dataclass
class TritonTemporalLIFResult:
    spikes: torch.Tensor
    v_next: torch.Tensor
    used_triton: bool
    kernel_key: str = "temporal_lif"
    fallback_reason: str = ""
    kernel_temporal_config: Optional[Dict] = None
    kernel_diagnostics: Optional[Dict] = None


def strict_temporal_lif_enabled(strict: bool = False) -> bool:
    return bool(strict) or os.environ.get("CHRONOS_STRICT_TEMPORAL_LIF_TRITON", "0") == "1"


def check_temporal_lif_support(x_seq, v_init, v_threshold, v_reset, tau, detach_reset) -> List[str]:
    """Reasons why the scan cannot take this call (empty = it can). Same role as the reference's function of
    this name (runtime/triton_temporal_lif_backend.py:23-54); bf16 and any T >= 1 pass here."""
    g = Gate("x_seq", x_seq)
    if not g:
        return g.why
    g.lead_is(rank=5)
    if x_seq.dim() >= 1 and int(x_seq.shape[0]) < 1:
        g.add("unsupported_temporal_length", "x_seq holds no timestep")
    g.state(v_init, tuple(x_seq.shape[1:]) if x_seq.dim() == 5 else None)
    g.tau(tau)
    return g.why


def _same_dense_layout(x_seq: torch.Tensor, v: Optional[torch.Tensor]) -> bool:
    """x_seq[t] frames densely packed, T outermost, and v (if any) laid out like one frame."""
    T = int(x_seq.shape[0])
    frame = x_seq[0]
    n = frame.numel()
    if T > 1 and x_seq.stride(0) != n:
        return False
    # dense and non-overlapping within a frame: sorted strides must tile the frame exactly
    dims = sorted(((s, d) for s, d in zip(frame.stride(), frame.shape) if d > 1))
    expect = 1
    for s, d in dims:
        if s != expect:
            return False
        expect *= d
    if v is not None:
        return all(sv == sf for sv, sf, d in zip(v.stride(), frame.stride(), frame.shape) if d > 1)
    return True


def run_triton_fused_temporal_lif_state(
    x_seq,
    v_init,
    v_threshold: float,
    v_reset: float,
    tau: float,
    detach_reset: bool,
    strict: bool = False,
    verbose: bool = False,
    use_autotune: bool = True,
    spike_dtype: Optional[torch.dtype] = None,
    v_dtype: Optional[torch.dtype] = None,
) -> TritonTemporalLIFResult:
    """LIF over x_seq [T,N,C,H,W]; returns spikes [T,N,C,H,W] and the last membrane [N,C,H,W].

    ``spike_dtype=torch.uint8`` and ``v_dtype=torch.float32`` select the compact spike
    format / full-precision state; by default both follow x_seq's dtype as the op schema
    promises (runtime/snn_custom_ops.py:799 in the reference).
    """
    reasons = check_temporal_lif_support(x_seq, v_init, v_threshold, v_reset, tau, detach_reset)
    strict = strict_temporal_lif_enabled(strict)
    raise_reasons("temporal_lif", reasons, strict, verbose)

    v0 = state_or_none(v_init)
    if v_dtype is not None and v0 is not None and v0.dtype != v_dtype:
        v0 = v0.to(v_dtype)
    if not _same_dense_layout(x_seq, v0):
        x_seq = x_seq.contiguous()
        v0 = v0.contiguous() if v0 is not None else None
    T = int(x_seq.shape[0])
    n = x_seq[0].numel()
    s_dt = spike_dtype or x_seq.dtype
    v_dt = v_dtype or x_seq.dtype
    spikes = torch.empty_strided(x_seq.shape, x_seq.stride(), dtype=s_dt, device=x_seq.device)
    v_next = torch.empty_strided(x_seq.shape[1:], x_seq.stride()[1:], dtype=v_dt, device=x_seq.device)
    th, vr, ta = lif_scalars(v_threshold, v_reset, tau)
    _lib.check(
        _lib.lib.snnb_lif_scan(
            _lib.ptr(x_seq), _lib.ptr(v0), _lib.ptr(spikes), _lib.ptr(v_next), T, n,
            _lib.dtype_code(x_seq.dtype), _lib.dtype_code(s_dt), _lib.dtype_code(v_dt),
            th, vr, ta, _lib.current_stream(x_seq.device)),
        "snnb_lif_scan")
    config = {"BLOCK_SIZE": 256 * (16 // x_seq.element_size()), "num_warps": 8}
    diagnostics = {
        "kernel_kind": "standalone_temporal_lif",
        "implementation": "sm_100a CUDA (snnb_lif_scan)",
        "compute_dtype": "float32",
        "membrane_dtype": str(v_dt),
        "spike_dtype": str(s_dt),
        "T": T,
        "numel_per_step": int(n),
        "kernel_temporal_config": config,
    }
    return TritonTemporalLIFResult(
        spikes=spikes, v_next=v_next, used_triton=True, kernel_key="temporal_lif",
        kernel_temporal_config=config, kernel_diagnostics=diagnostics)
