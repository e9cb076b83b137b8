"""CPU oracle for the fused temporal SNN ops — TEST INFRASTRUCTURE ONLY.

A restatement, on CPU tensors, of the arithmetic the reference's own checks
compare its kernels against: the un-fused per-timestep loops of
``runtime/snn_custom_ops.py`` in pengjh0111/triton-snn-fusion. Only tests, the
smoke check and the benchmark's CPU-baseline leg may import this module; the
product (``triton_snn_fusion_b200``) never does and has no CPU path.

Parity pin: ``tests/golden/make_golden.py`` runs every function here against
the reference's ``*_torch`` functions (imported from the reference checkout) on
seeded inputs, requires bit-identical results, and stores the vectors under
``tests/golden/``; ``tests/test_oracle_golden.py`` replays them.

Where the reference leaves the arithmetic to PyTorch (``F.conv2d``,
``F.linear``, ``F.adaptive_avg_pool2d``) so does this file, with the same
torch build, so the oracle and the reference agree to the last bit.

dtype policy for 16-bit inputs: the reference's fast path has no bf16 mode, so
the bf16/fp16 oracle is defined as this fp32 arithmetic applied to the 16-bit
values widened to fp32 (see ``widen``) — the same convention the reference's
conv benchmark uses for its half-precision comparison
(kernels/benchmark_conv_lif_temporal_general.py:388-389).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.nn.functional as F


def widen(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """16-bit float tensor -> fp32 copy on CPU (values unchanged); others pass through on CPU."""
    if t is None:
        return None
    t = t.detach().cpu()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.float()
    return t


def _initial_v(x: torch.Tensor, v_prev: Optional[torch.Tensor]) -> torch.Tensor:
    # A 0-dim or mismatching state means "start from zero"
    # (runtime/snn_custom_ops.py:378-381).
    if v_prev is None or v_prev.dim() == 0 or tuple(v_prev.shape) != tuple(x.shape) or v_prev.dtype != x.dtype:
        return torch.zeros_like(x)
    return v_prev


def lif_step(x, v_prev, v_th: float, v_reset: float, tau: float):
    """One LIF update; follows runtime/snn_custom_ops.py:384-409.

    charge: h = v + x (tau <= 1) or v + (x - v) / tau; fire: s = h >= v_th;
    reset: hard to v_reset when v_reset >= 0, else soft (h - s * v_th).
    """
    v = _initial_v(x, v_prev)
    if float(tau) <= 1.0:
        h = v + x
    else:
        h = v + (x - v) / float(tau)
    s = (h >= float(v_th)).to(x.dtype)
    if float(v_reset) < 0:
        v_next = h - s * float(v_th)
    else:
        v_next = torch.where(s.bool(), torch.full_like(h, float(v_reset)), h)
    return s, v_next


def temporal_lif(x_seq, v_init, v_th, v_reset, tau):
    """LIF scan over x_seq[t]; follows runtime/snn_custom_ops.py:521-536."""
    v = v_init
    out = []
    for t in range(int(x_seq.shape[0])):
        s, v = lif_step(x_seq[t], v, v_th, v_reset, tau)
        out.append(s)
    return torch.stack(out, 0), v


def temporal_conv_lif(xs: Sequence[torch.Tensor], weight, bias, v_init, stride, padding, dilation, groups,
                      v_th, v_reset, tau, residuals: Optional[Sequence[torch.Tensor]] = None):
    """conv2d (+ residual[t]) then LIF per timestep.

    Follows runtime/snn_custom_ops.py:430-453 (plain; also the pointwise and
    depthwise ops, which share the body) and :491-518 (residual add).
    """
    if len(xs) == 0:
        raise RuntimeError("temporal conv+LIF needs at least one timestep")
    if residuals is not None and len(residuals) != len(xs):
        raise RuntimeError("xs and residuals must have the same temporal length")
    v = v_init
    out = []
    for t, x in enumerate(xs):
        y = F.conv2d(x, weight, bias, stride, padding, dilation, groups)
        if residuals is not None:
            y = y + residuals[t]
        s, v = lif_step(y, v, v_th, v_reset, tau)
        out.append(s)
    return torch.stack(out, 0), v


def temporal_conv_only(xs: Sequence[torch.Tensor], weight, bias, stride, padding, dilation=1, groups=1):
    """conv2d per timestep without LIF (the BN-folded shortcut conv of a residual block)."""
    return torch.stack([F.conv2d(x, weight, bias, stride, padding, dilation, groups) for x in xs], 0)


def temporal_linear_lif(x_seq, weight, bias, v_init, v_th, v_reset, tau):
    """linear then LIF per timestep; follows runtime/snn_custom_ops.py:583-611."""
    b = bias if isinstance(bias, torch.Tensor) and bias.numel() > 0 else None
    v = v_init
    out = []
    for t in range(int(x_seq.shape[0])):
        s, v = lif_step(F.linear(x_seq[t], weight, b), v, v_th, v_reset, tau)
        out.append(s)
    return torch.stack(out, 0), v


def temporal_lif_avgpool_linear(x_seq, v_init, fc_weight, fc_bias, v_th, v_reset, tau):
    """LIF -> global average pool -> linear, logits summed over T.

    Follows runtime/snn_custom_ops.py:539-558. Returns (sum_t logits_t, v_last).
    """
    b = fc_bias if isinstance(fc_bias, torch.Tensor) and fc_bias.numel() > 0 else None
    v = v_init
    total = None
    for t in range(int(x_seq.shape[0])):
        s, v = lif_step(x_seq[t], v, v_th, v_reset, tau)
        logits = F.linear(F.adaptive_avg_pool2d(s, (1, 1)).flatten(1), fc_weight, b)
        total = logits if total is None else total + logits
    return total, v


def fold_bn(conv_weight, conv_bias, running_mean, running_var, gamma, beta, eps: float):
    """Inference BatchNorm folded into the preceding conv.

    Follows compiler/fx_lif_rewrite.py:340-353: scale = gamma / sqrt(var + eps),
    W' = W * scale, b' = (b - mean) * scale + beta, in the statistics' dtype.
    """
    if conv_bias is None:
        conv_bias = torch.zeros_like(running_mean)
    if gamma is None:
        gamma = torch.ones_like(running_mean)
    if beta is None:
        beta = torch.zeros_like(running_mean)
    w = conv_weight.to(running_mean.dtype)
    b = conv_bias.to(running_mean.dtype)
    scale = gamma / torch.sqrt(running_var + float(eps))
    return w * scale.reshape(-1, 1, 1, 1), (b - running_mean) * scale + beta


def compare(spikes, spikes_ref, v, v_ref):
    """The reference's three correctness numbers
    (kernels/benchmark_conv_lif_temporal_general.py:392-402): fraction of differing
    spikes, max and mean absolute membrane error; plus the max relative error."""
    s = spikes.detach().cpu().float()
    sr = spikes_ref.detach().cpu().float()
    vv = v.detach().cpu().float()
    vr = v_ref.detach().cpu().float()
    dv = (vv - vr).abs()
    return {
        "flip_rate": float((s != sr).float().mean()) if s.numel() else 0.0,
        "v_max_abs": float(dv.max()) if dv.numel() else 0.0,
        "v_mean_abs": float(dv.mean()) if dv.numel() else 0.0,
        "v_max_rel": float((dv / vr.abs().clamp_min(1e-3)).max()) if dv.numel() else 0.0,
    }
