"""Backend of the temporal linear + LIF ops (list, packed and caller-owned-output forms).

Mirrors the public names of the reference module of the same name
(runtime/triton_temporal_linear_lif_backend.py:8-274 in pengjh0111/triton-snn-fusion).
The work is one ``snnb_linear_lif`` call: a tcgen05 GEMM with the LIF recurrence in the
epilogue for 16-bit inputs with K % 64 == 0, a CUDA-core GEMM otherwise. bf16 is
accepted, T is arbitrary, and there is no fallback.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from .. import _lib
from ._common import Gate, lif_scalars, raise_reasons, state_or_none
from .triton_convlif_backend import _PATH
from . import triton_convlif_backend as _conv


@dataclass
class TritonTemporalLinearLIFResult:
    spikes: torch.Tensor
    v_next: torch.Tensor
    used_triton: bool
    kernel_key: str = "temporal_linear_lif"
    fallback_reason: str = ""
    kernel_temporal_config: Optional[Dict] = None
    kernel_diagnostics: Optional[Dict] = None


def strict_temporal_linear_lif_enabled(strict: bool = False) -> bool:
    return bool(strict) or os.environ.get("CHRONOS_STRICT_TEMPORAL_LINEAR_LIF_TRITON", "0") == "1"


def check_temporal_linear_lif_support(x_seq, weight, bias, v_init, v_threshold, v_reset, tau, detach_reset) -> List[str]:
    """Reasons why the linear + LIF kernel cannot take this call (empty = it can). Same role as the reference's
    function of this name (runtime/triton_temporal_linear_lif_backend.py:23-71)."""
    g = Gate("x_seq", x_seq)
    if not g:
        return g.why
    g.lead_is(rank=3)
    n_out = None
    if g.companion("weight", weight, rank=2, code="unsupported_weight_rank"):
        n_out = int(weight.shape[0])
        if x_seq.dim() == 3 and int(weight.shape[1]) != int(x_seq.shape[2]):
            g.add("unsupported_shape", f"weight reads {int(weight.shape[1])} features per token, x_seq has "
                                       f"{int(x_seq.shape[2])}")
    if isinstance(bias, torch.Tensor) and bias.numel() > 0:
        if n_out is not None and tuple(bias.shape) != (n_out,):
            g.add("unsupported_bias", f"bias is {tuple(bias.shape)}, one value per output feature would be ({n_out},)")
        g.companion("bias", bias)
    g.state(v_init, (int(x_seq.shape[1]), n_out) if (x_seq.dim() == 3 and n_out is not None) else None, fp32_ok=True)
    g.tau(tau)
    return g.why


def _impl(x_seq, weight, bias, v_init, v_threshold, v_reset, tau, detach_reset, strict, verbose,
          stack_materialized=False, spike_out=None, v_out=None) -> TritonTemporalLinearLIFResult:
    spike_shape = v_shape = None
    if isinstance(x_seq, torch.Tensor) and x_seq.dim() > 3:
        if not isinstance(weight, torch.Tensor) or weight.dim() != 2:
            raise RuntimeError("temporal Linear+LIF flatten path requires rank-2 weight")
        n_out = int(weight.shape[0])
        spike_shape = tuple(x_seq.shape[:-1]) + (n_out,)
        v_shape = tuple(x_seq.shape[1:-1]) + (n_out,)
        x_seq = x_seq.contiguous().reshape(int(x_seq.shape[0]), -1, int(x_seq.shape[-1]))
        if isinstance(v_init, torch.Tensor) and v_init.dim() > 0:
            v_init = v_init.contiguous().reshape(-1, n_out)
    reasons = check_temporal_linear_lif_support(x_seq, weight, bias, v_init, v_threshold, v_reset, tau, detach_reset)
    raise_reasons("temporal_linear_lif", reasons, strict_temporal_linear_lif_enabled(strict), verbose)

    T, M, K = (int(d) for d in x_seq.shape)
    N = int(weight.shape[0])
    if x_seq.stride(2) != 1 or x_seq.stride(1) != K or (T > 1 and x_seq.stride(0) < M * K):
        x_seq = x_seq.contiguous()
    x_stride = x_seq.stride(0) if T > 1 else 0
    weight = weight.contiguous()
    b = bias if isinstance(bias, torch.Tensor) and bias.numel() > 0 else None
    v0 = state_or_none(v_init)
    v_dtype = x_seq.dtype if v0 is None else v0.dtype
    if v0 is not None:
        v0 = v0.contiguous()
    use_out = (isinstance(spike_out, torch.Tensor) and isinstance(v_out, torch.Tensor)
               and spike_out.is_contiguous() and v_out.is_contiguous()
               and spike_out.dtype == x_seq.dtype and v_out.dtype == v_dtype
               and spike_out.numel() == T * M * N and v_out.numel() == M * N)
    spikes = spike_out.view(T, M, N) if use_out else torch.empty((T, M, N), dtype=x_seq.dtype, device=x_seq.device)
    v_next = v_out.view(M, N) if use_out else torch.empty((M, N), dtype=v_dtype, device=x_seq.device)
    th, vr, ta = lif_scalars(v_threshold, v_reset, tau)
    dt = _lib.dtype_code(x_seq.dtype)
    stream = _lib.current_stream(x_seq.device)

    def call(t0, steps, v_in, v_to, v_dt):
        _lib.check(
            _lib.lib.snnb_linear_lif(
                _lib.ptr(x_seq) + t0 * x_stride * x_seq.element_size(), x_stride, _lib.ptr(weight), _lib.ptr(b),
                _lib.ptr(v_in), _lib.ptr(spikes) + t0 * M * N * spikes.element_size(), _lib.ptr(v_to),
                steps, M, K, N, dt, dt, _lib.dtype_code(v_dt), th, vr, ta, _PATH[_conv._conv_path], stream),
            "snnb_linear_lif")

    # Sequences beyond what one launch of the GEMM kernel takes run as windows of four timesteps with the membrane
    # handed over in fp32: the arithmetic of a single pass.
    windowed = (T > _conv.MAX_STEPS and T % _conv.WINDOW == 0 and _conv._conv_path != "simt"
                and x_seq.dtype in (torch.bfloat16, torch.float16))
    if windowed:
        carry = [torch.empty((M, N), dtype=torch.float32, device=x_seq.device) for _ in range(2)]
        v_in = None
        if v0 is not None:
            carry[1].copy_(v0)
            v_in = carry[1]
        for w in range(T // _conv.WINDOW):
            call(w * _conv.WINDOW, _conv.WINDOW, v_in, carry[w % 2], torch.float32)
            v_in = carry[w % 2]
        v_next.copy_(v_in)
    else:
        call(0, T, v0, v_next, v_dtype)
    if isinstance(spike_out, torch.Tensor) and not use_out:
        spike_out.copy_(spikes.reshape(spike_out.shape))
        v_out.copy_(v_next.reshape(v_out.shape))
        spikes, v_next = spike_out, v_out
    if spike_shape is not None:
        spikes = spikes.reshape(spike_shape)
        v_next = v_next.reshape(v_shape)
    diagnostics = {
        "kernel_kind": "temporal_linear_lif",
        "implementation": "sm_100a CUDA (snnb_linear_lif)",
        "membrane_dtype": str(v_dtype),
        "spike_dtype": str(x_seq.dtype),
        "stack_materialized": stack_materialized,
        "flattened_leading_dims": spike_shape is not None,
        "T": T, "M": M, "K": K, "N": N,
        "kernel_temporal_window": _conv.WINDOW if windowed else T,
    }
    return TritonTemporalLinearLIFResult(
        spikes=spikes, v_next=v_next, used_triton=True, kernel_key="temporal_linear_lif",
        kernel_temporal_config=diagnostics, kernel_diagnostics=diagnostics)


def run_triton_fused_temporal_linear_lif_state(xs, weight, bias, v_init, v_threshold, v_reset, tau, detach_reset,
                                               strict=False, verbose=False, use_autotune=True):
    """List-of-T form (reference :74-116). Equally spaced views of one buffer are used in place."""
    if isinstance(xs, torch.Tensor):
        return run_triton_fused_temporal_linear_lif_state_packed(
            xs, weight, bias, v_init, v_threshold, v_reset, tau, detach_reset, strict=strict, verbose=verbose)
    if not isinstance(xs, (tuple, list)) or len(xs) == 0:
        raise RuntimeError("fused temporal linear LIF requires a non-empty Tensor list or [T,N,F] tensor")
    x_seq = torch.stack(list(xs), dim=0)
    return _impl(x_seq, weight, bias, v_init, v_threshold, v_reset, tau, detach_reset, strict, verbose,
                 stack_materialized=True)


def run_triton_fused_temporal_linear_lif_state_packed(x_seq, weight, bias, v_init, v_threshold, v_reset, tau,
                                                      detach_reset, strict=False, verbose=False, use_autotune=True):
    """Packed [T,...,K] form (reference :119-149)."""
    return _impl(x_seq, weight, bias, v_init, v_threshold, v_reset, tau, detach_reset, strict, verbose)


def run_triton_fused_temporal_linear_lif_state_packed_out(x_seq, weight, bias, v_init, v_threshold, v_reset, tau,
                                                          detach_reset, spike_out, v_out, strict=False, verbose=False,
                                                          use_autotune=True):
    """Packed form writing into caller-owned spike_out / v_out (reference :152-182)."""
    return _impl(x_seq, weight, bias, v_init, v_threshold, v_reset, tau, detach_reset, strict, verbose,
                 spike_out=spike_out, v_out=v_out)
