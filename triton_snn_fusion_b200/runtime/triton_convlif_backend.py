"""Backend of the conv (+ folded BN) + LIF ops: single step, temporal, pointwise,
depthwise, residual-add and caller-owned-output variants.

Mirrors the public names of the reference module of the same name
(runtime/triton_convlif_backend.py in pengjh0111/triton-snn-fusion: result type :7-15,
classify_conv_lif_config :50-82, check_triton_support :118-211, the run_* entry points
:331-817), so the reference's op layer binds to it unchanged. Behind the names:
``snnb_conv_lif`` (tcgen05 implicit GEMM for 16-bit activations with Cin % 64 == 0,
CUDA-core implicit GEMM otherwise) and ``snnb_dwconv3x3_lif``.

Deliberate differences from the reference backend:
  * bf16 is accepted next to fp32 / fp16; v_threshold, v_reset (incl. soft reset) and
    tau are run-time values, detach_reset is accepted (it does not change forward values);
  * activations are processed channels-last. Inputs that already are channels-last views
    (what this backend returns, and what ``x.contiguous(memory_format=channels_last)``
    gives) are used in place; anything else is converted once. Outputs are logical
    [T,B,C,H,W] / [B,C,H,W] tensors with channels-last memory;
  * T inputs that are one tensor (direct encoding) are convolved once, and equally spaced
    views of one spike stack are consumed without the ``torch.stack`` copy the reference
    makes (:579);
  * no fallback: an unsupported request raises.
"""
from __future__ import annotations

import weakref
from collections import OrderedDict
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .. import _lib
from ._common import (Gate, as_pair, empty_nhwc, is_nhwc_dense, lif_scalars, raise_reasons, stack_frames,
                      state_or_none, to_nhwc)


@dataclass
class TritonConvLIFResult:
    spikes: torch.Tensor
    v_next: torch.Tensor
    used_triton: bool
    kernel_key: str = "unsupported"
    fallback_reason: str = ""
    kernel_temporal_config: Optional[Dict] = None
    kernel_diagnostics: Optional[Dict] = None


_as_pair = as_pair

# Implementation choice forwarded to the C ABI: "auto", "simt", "tcgen05" or "tcgen05_taps".
_PATH = {"auto": _lib.PATH_AUTO, "simt": _lib.PATH_SIMT, "tcgen05": _lib.PATH_TCGEN05,
         "tcgen05_taps": _lib.PATH_TCGEN05_TAPS, "tcgen05_halo": _lib.PATH_TCGEN05_HALO}
_conv_path = "auto"


def set_conv_path(path: str) -> str:
    """Select the dense-conv implementation ("auto" | "simt" | "tcgen05" | "tcgen05_taps"); returns the previous one."""
    global _conv_path
    if path not in _PATH:
        raise ValueError(f"path must be one of {sorted(_PATH)}, got {path!r}")
    prev, _conv_path = _conv_path, path
    return prev


def _conv2d_output_shape(x, weight, stride, padding, dilation) -> Tuple[int, int, int, int]:
    sh, sw = as_pair(stride)
    ph, pw = as_pair(padding)
    dh, dw = as_pair(dilation)
    kh, kw = int(weight.shape[2]), int(weight.shape[3])
    ho = (int(x.shape[2]) + 2 * ph - dh * (kh - 1) - 1) // sh + 1
    wo = (int(x.shape[3]) + 2 * pw - dw * (kw - 1) - 1) // sw + 1
    return int(x.shape[0]), int(weight.shape[0]), ho, wo


# kernel -> {(stride, padding[, "depthwise"]): key}; same table as the reference (:96-115)
SUPPORTED_CONV_LIF_CONFIGS = {
    (1, 1): {((1, 1), (0, 0)): "k1_s1_p0"},
    (3, 3): {
        ((1, 1), (1, 1)): "k3_s1_p1",
        ((2, 2), (1, 1)): "k3_s2_p1",
        ((1, 1), (1, 1), "depthwise"): "depthwise_k3_s1_p1",
        ((2, 2), (1, 1), "depthwise"): "depthwise_k3_s2_p1",
    },
    (5, 5): {((1, 1), (2, 2)): "k5_s1_p2"},
    (7, 7): {((2, 2), (3, 3)): "k7_s2_p3"},
    (11, 11): {((4, 4), (2, 2)): "k11_s4_p2"},
}


def classify_conv_lif_config(weight, stride, padding, dilation, groups) -> str:
    """Kernel key of a conv (same keys as the reference, :50-82) or "unsupported"."""
    if weight is None or not isinstance(weight, torch.Tensor) or weight.dim() != 4:
        return "unsupported"
    if tuple(as_pair(dilation)) != (1, 1):
        return "unsupported"
    s, p, k = tuple(as_pair(stride)), tuple(as_pair(padding)), tuple(int(d) for d in weight.shape[-2:])
    table = SUPPORTED_CONV_LIF_CONFIGS.get(k, {})
    if int(groups) == int(weight.shape[0]) and int(weight.shape[1]) == 1:
        return table.get((s, p, "depthwise"), "unsupported")
    if int(groups) != 1:
        return "unsupported"
    return table.get((s, p), "unsupported")


def classify_conv_lif_runtime_kind(weight, stride, padding, dilation, groups) -> str:
    key = classify_conv_lif_config(weight, stride, padding, dilation, groups)
    if key.startswith("depthwise_"):
        return "depthwise"
    if key == "k1_s1_p0":
        return "pointwise"
    return "regular" if key != "unsupported" else "unsupported"


def check_triton_support(x, weight, bias, v_prev, stride, padding, dilation, groups,
                         v_threshold, v_reset, tau, detach_reset) -> List[str]:
    """Reasons why this backend cannot take the call (empty list = supported). Same role as the reference's
    function of this name (runtime/triton_convlif_backend.py:118-211); here bf16 passes and the LIF constants
    are free."""
    g = Gate("x", x)
    if not g:
        return g.why
    g.lead_is(rank=4)
    if bias is None:
        g.add("missing_or_unsupported_bias", "the conv carries no bias tensor (a folded BatchNorm always yields one)")
    else:
        g.companion("bias", bias)
    if not g.companion("weight", weight, rank=4):
        return g.why
    if g.why:
        return g.why
    groups = int(groups)
    cin, cout, wcin = int(x.shape[1]), int(weight.shape[0]), int(weight.shape[1])
    depthwise = wcin == 1 and groups == cin == cout and groups > 1
    if groups != 1 and not depthwise:
        g.add("unsupported_groups", f"groups = {groups}: only dense (1) and depthwise (= channels) convs have kernels")
    if groups == 1 and wcin != cin:
        g.add("unsupported_shape", f"weight reads {wcin} channels, x has {cin}")
    if tuple(as_pair(dilation)) != (1, 1):
        g.add("unsupported_dilation", f"dilation {tuple(as_pair(dilation))}: only undilated convs have kernels")
    s, p, k = tuple(as_pair(stride)), tuple(as_pair(padding)), tuple(int(d) for d in weight.shape[-2:])
    table = SUPPORTED_CONV_LIF_CONFIGS.get(k)
    if table is None:
        g.add("unsupported_kernel", f"{k[0]}x{k[1]} window; kernels exist for "
                                    f"{', '.join(f'{a}x{b}' for a, b in SUPPORTED_CONV_LIF_CONFIGS)}")
    elif ((s, p, "depthwise") if depthwise else (s, p)) not in table:
        same_kind = [c for c in table if (len(c) == 3) == depthwise]
        if not any(c[0] == s for c in same_kind):
            g.add("unsupported_stride", f"{k[0]}x{k[1]} window with stride {s}; implemented: "
                                        f"{sorted({c[0] for c in same_kind})}")
        else:
            g.add("unsupported_padding", f"{k[0]}x{k[1]} window, stride {s}, padding {p}; implemented: "
                                         f"{sorted({c[1] for c in same_kind if c[0] == s})}")
    g.tau(tau)
    if not g.why:
        g.state(v_prev, _conv2d_output_shape(x, weight, stride, padding, dilation), fp32_ok=True)
    return g.why


# ------------------------------------------------------------------ weights ----
# id(weight) -> (weak reference to the weight, its version counter, channels-last copy). The weak
# reference is what makes the entry safe: a dead tensor's id or address may be handed to a new one.
_PACKED: "OrderedDict[int, tuple]" = OrderedDict()
_PACKED_MAX = 512


def _packed_weight(weight: torch.Tensor) -> torch.Tensor:
    """Dense-conv weight as [Cout][KH][KW][Cin] memory (channels_last); converted once per tensor version."""
    if is_nhwc_dense(weight):
        return weight
    hit = _PACKED.get(id(weight))
    if hit is not None and hit[0]() is weight and hit[1] == weight._version:
        _PACKED.move_to_end(id(weight))
        return hit[2]
    packed = weight.permute(0, 2, 3, 1).contiguous().permute(0, 3, 1, 2)
    _PACKED[id(weight)] = (weakref.ref(weight), weight._version, packed)
    while len(_PACKED) > _PACKED_MAX:
        _PACKED.popitem(last=False)
    for k in [k for k, v in list(_PACKED.items())[:8] if v[0]() is None]:
        del _PACKED[k]
    return packed


_STEM: "OrderedDict[int, tuple]" = OrderedDict()


def _stem_weight(weight: torch.Tensor, dt: int) -> torch.Tensor:
    """[Cout,3,7,7] weight re-packed for snnb_stem7x7_lif ([Cout][4][4][16]); once per tensor version."""
    hit = _STEM.get(id(weight))
    if hit is not None and hit[0]() is weight and hit[1] == weight._version:
        return hit[2]
    w = _packed_weight(weight).permute(0, 2, 3, 1).contiguous()  # [Cout][7][7][3] memory
    wp = torch.empty((int(weight.shape[0]), 256), dtype=weight.dtype, device=weight.device)
    _lib.check(_lib.lib.snnb_stem7x7_pack_weight(_lib.ptr(w), _lib.ptr(wp), int(weight.shape[0]), dt,
                                                 _lib.current_stream(weight.device)), "snnb_stem7x7_pack_weight")
    _STEM[id(weight)] = (weakref.ref(weight), weight._version, wp)
    while len(_STEM) > 64:
        _STEM.popitem(last=False)
    return wp


def _validate_kind(kind: str, key: str) -> None:
    """An op that names its conv kind (regular / pointwise / depthwise) must be handed a conv of that kind."""
    actual = "depthwise" if key.startswith("depthwise_") else ("pointwise" if key == "k1_s1_p0" else "regular")
    if kind != actual:
        raise RuntimeError(f"the {kind} conv + LIF op was called with a {actual} conv (kernel key {key})")


def _launch(x_base, x_t_stride, T, weight, bias, residual, v_init, stride, padding, groups, v_threshold, v_reset, tau,
            spikes, v_next, lif=True, spike_dtype=None, v_dtype=None, t0=0):
    """One C-ABI call over timesteps t0 .. t0 + T - 1. x_base: [B,Cin,H,W] channels-last frame 0; ``residual`` and
    ``spikes`` are dense channels-last stacks whose frame t0 is where this call starts."""
    B, Cin, H, W = (int(d) for d in x_base.shape)
    Cout, _, KH, KW = (int(d) for d in weight.shape)
    s = as_pair(stride)[0]
    p = as_pair(padding)[0]
    th, vr, ta = lif_scalars(v_threshold, v_reset, tau)
    dt = _lib.dtype_code(x_base.dtype)
    sdt = _lib.dtype_code(spike_dtype or x_base.dtype)
    vdt = _lib.dtype_code(v_dtype or x_base.dtype)
    stream = _lib.current_stream(x_base.device)
    x_ptr = _lib.ptr(x_base) + t0 * x_t_stride * x_base.element_size()
    s_ptr = _lib.ptr(spikes) + t0 * spikes.stride(0) * spikes.element_size() if t0 else _lib.ptr(spikes)
    r_ptr = _lib.ptr(residual)
    if residual is not None and t0:
        r_ptr += t0 * residual.numel() * residual.element_size()
    if (groups == 1 and lif and residual is None and Cin == 3 and KH == 7 and KW == 7 and s == 2 and p == 3
            and x_base.dtype in (torch.bfloat16, torch.float16) and H % 2 == 0 and W % 2 == 0 and Cout % 16 == 0
            and _conv_path != "simt"):
        # 7x7/s2 three-channel stem: tensor-core path over a re-laid copy of the input held in scratch
        wp = _stem_weight(weight, dt)
        frames = B if x_t_stride == 0 else T * B
        nbytes = int(_lib.lib.snnb_stem7x7_scratch_bytes(frames, H, W))
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=x_base.device)
        _lib.check(
            _lib.lib.snnb_stem7x7_lif(
                x_ptr, x_t_stride, _lib.ptr(wp), _lib.ptr(bias), _lib.ptr(v_init), s_ptr,
                _lib.ptr(v_next), _lib.ptr(scratch), nbytes, T, B, H, W, Cout, dt, sdt, vdt, th, vr, ta, stream),
            "snnb_stem7x7_lif")
        return
    if groups == 1:
        w = _packed_weight(weight)
        _lib.check(
            _lib.lib.snnb_conv_lif(
                x_ptr, x_t_stride, _lib.ptr(w), _lib.ptr(bias), r_ptr, _lib.ptr(v_init),
                s_ptr, _lib.ptr(v_next), T, B, Cin, H, W, Cout, KH, KW, s, p, 1 if lif else 0,
                dt, sdt, vdt, th, vr, ta, _PATH[_conv_path], stream),
            "snnb_conv_lif")
    else:
        w = weight.contiguous()
        _lib.check(
            _lib.lib.snnb_dwconv3x3_lif(
                x_ptr, x_t_stride, _lib.ptr(w), _lib.ptr(bias), r_ptr, _lib.ptr(v_init),
                s_ptr, _lib.ptr(v_next), T, B, Cin, H, W, s, dt, sdt, vdt, th, vr, ta, stream),
            "snnb_dwconv3x3_lif")


# The fastest dense-conv kernel loops over timestep pairs inside one launch, as the reference loops its windows
# inside its kernel (kernels/benchmark_conv_lif_temporal_general.py:649), for any even T up to MAX_STEPS (what every tensor-core kernel of the library accepts). Longer
# (or odd, multiple-of-WINDOW) sequences run as windows of WINDOW steps with the membrane handed over in fp32: the
# same arithmetic as one pass over all T, since the membrane is fp32 inside a kernel too.
WINDOW = 4
MAX_STEPS = 32


def _windowed(T, x_t_stride, groups, dtype) -> bool:
    return (T > MAX_STEPS and T % WINDOW == 0 and x_t_stride != 0 and groups == 1 and _conv_path != "simt"
            and dtype in (torch.bfloat16, torch.float16))


def _launch_windows(x_base, x_t_stride, T, weight, bias, residual, v_init, stride, padding, v_threshold, v_reset, tau,
                    spikes, v_next):
    """T = n * WINDOW timesteps as n chained calls; v_init / v_next keep the dtype the caller gave them."""
    shape = v_next.permute(0, 2, 3, 1).shape   # channels-last memory order
    carry = [torch.empty(shape, dtype=torch.float32, device=x_base.device).permute(0, 3, 1, 2) for _ in range(2)]
    v_in = None
    if v_init is not None:
        carry[1].copy_(v_init)
        v_in = carry[1]
    for w in range(T // WINDOW):
        _launch(x_base, x_t_stride, WINDOW, weight, bias, residual, v_in, stride, padding, 1, v_threshold, v_reset, tau,
                spikes, carry[w % 2], v_dtype=torch.float32, t0=w * WINDOW)
        v_in = carry[w % 2]
    v_next.copy_(v_in)   # one rounding to the membrane dtype, as at the end of a single pass


def _diagnostics(dtype, key, copied, residual=False):
    return {
        "implementation": "sm_100a CUDA (libsnnb200)",
        "kernel_key": key,
        "compute_dtype": "float32 accumulate",
        "membrane_dtype": str(dtype),
        "spike_dtype": str(dtype),
        "residual_add": residual,
        "stack_materialized": bool(copied),
    }


def _check_list(xs, what, reasons):
    if not isinstance(xs, (list, tuple)) or len(xs) == 0:
        reasons.append(f"{what} must be a non-empty list/tuple of tensors")
        return
    first = xs[0]
    for i, x in enumerate(xs):
        if not isinstance(x, torch.Tensor):
            reasons.append(f"{what}[{i}] is not a tensor")
            continue
        if tuple(x.shape) != tuple(first.shape):
            reasons.append(f"{what}[{i}] shape {tuple(x.shape)} differs from first shape {tuple(first.shape)}")
        if x.device != first.device or x.dtype != first.dtype:
            reasons.append(f"{what}[{i}] device/dtype differs from first tensor")


def _run_temporal(kind, xs, residuals, weight, bias, v_init, stride, padding, dilation, groups,
                  v_threshold, v_reset, tau, detach_reset, strict, verbose, compute_dtype,
                  spike_out=None, v_out=None, x_seq=None) -> TritonConvLIFResult:
    reasons: List[str] = []
    if x_seq is None:
        _check_list(xs, "xs", reasons)
    if residuals is not None:
        _check_list(residuals, "residuals", reasons)
        if not reasons and len(xs) != len(residuals):
            reasons.append(f"xs and residuals length mismatch: {len(xs)} vs {len(residuals)}")
    raise_reasons("temporal_conv", reasons, strict, verbose)
    first = x_seq[0] if x_seq is not None else xs[0]
    reasons = check_triton_support(first, weight, bias, v_init, stride, padding, dilation, groups,
                                   v_threshold, v_reset, tau, detach_reset)
    raise_reasons("temporal_conv", reasons, strict, verbose)
    if compute_dtype is not None and compute_dtype not in ("float32", "float16", "bfloat16"):
        raise RuntimeError(f"compute_dtype={compute_dtype} is not a known dtype path")
    key = classify_conv_lif_config(weight, stride, padding, dilation, groups)
    if key == "unsupported":
        raise RuntimeError("unsupported dispatch key after support check")
    if kind is not None:
        _validate_kind(kind, key)
    if verbose:
        print(f"[SNNB200][DISPATCH] kind={kind} key={key} x={tuple(first.shape)} w={tuple(weight.shape)}")

    if x_seq is not None:
        T = int(x_seq.shape[0])
        xq = to_nhwc(x_seq)
        copied = xq is not x_seq
        x_base, x_stride = xq[0], (xq.stride(0) if T > 1 else 0)
    else:
        T = len(xs)
        x_base, x_stride, copied = stack_frames(list(xs))
    _, cout, ho, wo = _conv2d_output_shape(first, weight, stride, padding, dilation)
    B = int(first.shape[0])
    res_base = None
    if residuals is not None:
        if tuple(residuals[0].shape) != (B, cout, ho, wo):
            raise RuntimeError(f"residual shape {tuple(residuals[0].shape)} does not match conv output {(B, cout, ho, wo)}")
        r_base, r_stride, r_copied = stack_frames(list(residuals))
        if T > 1 and r_stride != r_base.numel():
            stacked = empty_nhwc([T, B, cout, ho, wo], first.dtype, first.device)
            for t, r in enumerate(residuals):
                stacked[t].copy_(r)
            r_base, r_copied = stacked[0], True
        res_base = r_base
        copied = copied or r_copied
    v0 = state_or_none(v_init)
    v_dtype = first.dtype
    if v0 is not None:
        v_dtype = v0.dtype
        v0 = to_nhwc(v0)

    direct_out = (spike_out is not None and v_out is not None and is_nhwc_dense(spike_out) and is_nhwc_dense(v_out)
                  and spike_out.dtype == first.dtype and v_out.dtype == v_dtype)
    if direct_out:
        spikes, v_next = spike_out, v_out
    else:
        spikes = empty_nhwc([T, B, cout, ho, wo], first.dtype, first.device)
        v_next = empty_nhwc([B, cout, ho, wo], v_dtype, first.device)
    windowed = _windowed(T, x_stride, int(groups), first.dtype)
    if windowed:
        _launch_windows(x_base, x_stride, T, weight, bias, res_base, v0, stride, padding, v_threshold, v_reset, tau,
                        spikes, v_next)
    else:
        _launch(x_base, x_stride, T, weight, bias, res_base, v0, stride, padding, int(groups), v_threshold, v_reset,
                tau, spikes, v_next, v_dtype=v_dtype)
    if spike_out is not None and not direct_out:
        spike_out.copy_(spikes)
        v_out.copy_(v_next)
        spikes, v_next = spike_out, v_out
    return TritonConvLIFResult(
        spikes, v_next, True, kernel_key=key,
        kernel_temporal_config={"BTILE_T": WINDOW if windowed else T, "REUSE_GROUPS": 1,
                                "kernel_temporal_window": WINDOW if windowed else T, "implementation": "snnb200"},
        kernel_diagnostics=_diagnostics(first.dtype, key, copied, residuals is not None))


def run_triton_fused_conv_lif_state(x, weight, bias, v_prev, stride, padding, dilation, groups,
                                    v_threshold, v_reset, tau, detach_reset, strict=False, verbose=False,
                                    use_autotune=True, compute_dtype=None) -> TritonConvLIFResult:
    """Single-step conv + LIF (reference :331-390): the temporal kernel with T = 1."""
    res = _run_temporal(None, [x], None, weight, bias, v_prev, stride, padding, dilation, groups,
                        v_threshold, v_reset, tau, detach_reset, strict, verbose, compute_dtype)
    res.spikes = res.spikes[0]
    return res


def run_triton_fused_temporal_conv_lif_state(xs, weight, bias, v_init, stride, padding, dilation, groups,
                                             v_threshold, v_reset, tau, detach_reset, strict=False, verbose=False,
                                             use_autotune=True, compute_dtype=None) -> TritonConvLIFResult:
    """Regular conv + LIF over T (reference :393-430)."""
    return _run_temporal("regular", xs, None, weight, bias, v_init, stride, padding, dilation, groups,
                         v_threshold, v_reset, tau, detach_reset, strict, verbose, compute_dtype)


def run_triton_fused_temporal_pointwise_conv_lif_state(xs, weight, bias, v_init, stride, padding, dilation, groups,
                                                       v_threshold, v_reset, tau, detach_reset, strict=False,
                                                       verbose=False, use_autotune=True,
                                                       compute_dtype=None) -> TritonConvLIFResult:
    """1x1 conv + LIF over T (reference :433-470)."""
    return _run_temporal("pointwise", xs, None, weight, bias, v_init, stride, padding, dilation, groups,
                         v_threshold, v_reset, tau, detach_reset, strict, verbose, compute_dtype)


def run_triton_fused_temporal_depthwise_conv_lif_state(xs, weight, bias, v_init, stride, padding, dilation, groups,
                                                       v_threshold, v_reset, tau, detach_reset, strict=False,
                                                       verbose=False, use_autotune=True,
                                                       compute_dtype=None) -> TritonConvLIFResult:
    """3x3 depthwise conv + LIF over T (reference :473-510)."""
    return _run_temporal("depthwise", xs, None, weight, bias, v_init, stride, padding, dilation, groups,
                         v_threshold, v_reset, tau, detach_reset, strict, verbose, compute_dtype)


def run_triton_fused_temporal_conv_add_lif_state(xs, residuals, weight, bias, v_init, stride, padding, dilation,
                                                 groups, v_threshold, v_reset, tau, detach_reset, strict=False,
                                                 verbose=False, use_autotune=True,
                                                 compute_dtype=None) -> TritonConvLIFResult:
    """conv + residual[t] + LIF over T (reference :689-817); dense and depthwise convs."""
    return _run_temporal(None, xs, residuals, weight, bias, v_init, stride, padding, dilation, groups,
                         v_threshold, v_reset, tau, detach_reset, strict, verbose, compute_dtype)


def run_triton_fused_temporal_conv_lif_state_packed_out(x_seq, weight, bias, v_init, stride, padding, dilation,
                                                        groups, v_threshold, v_reset, tau, detach_reset,
                                                        spike_out, v_out, strict=False, verbose=False,
                                                        use_autotune=True, compute_dtype=None) -> TritonConvLIFResult:
    """Pre-stacked input [T,B,C,H,W] and caller-owned outputs (reference :601-686)."""
    reasons: List[str] = []
    if not isinstance(x_seq, torch.Tensor):
        reasons.append("x_seq must be a tensor")
    elif x_seq.dim() != 5:
        reasons.append(f"x_seq must have rank 5 [T,N,C,H,W], got {x_seq.dim()}")
    if not isinstance(spike_out, torch.Tensor) or not isinstance(v_out, torch.Tensor):
        reasons.append("spike_out and v_out must be tensors")
    raise_reasons("temporal_conv_out", reasons, strict, verbose)
    res = _run_temporal(None, None, None, weight, bias, v_init, stride, padding, dilation, groups,
                        v_threshold, v_reset, tau, detach_reset, strict, verbose, compute_dtype,
                        spike_out=spike_out, v_out=v_out, x_seq=x_seq)
    expect = (int(x_seq.shape[0]),) + tuple(_conv2d_output_shape(x_seq[0], weight, stride, padding, dilation))
    if tuple(spike_out.shape) != expect or tuple(v_out.shape) != expect[1:]:
        raise RuntimeError(f"spike_out/v_out shapes {tuple(spike_out.shape)}/{tuple(v_out.shape)} do not match {expect}")
    return res


def conv_bias_only(xs, weight, bias, stride, padding, residuals=None) -> torch.Tensor:
    """conv + bias (+ residual) for every t WITHOUT the LIF: [T,B,Cout,Ho,Wo] in the input dtype.

    No counterpart among the reference's fused ops: it is the BN-folded shortcut conv of a
    residual block, which the reference leaves to an ordinary aten conv on flatten(0,1) of the
    spike stack (compiler/fx_spatial_batching.py:799-879).
    """
    x_base, x_stride, _ = stack_frames(list(xs))
    T = len(xs)
    first = xs[0]
    _, cout, ho, wo = _conv2d_output_shape(first, weight, stride, padding, (1, 1))
    out = empty_nhwc([T, int(first.shape[0]), cout, ho, wo], first.dtype, first.device)
    res_base = None
    if residuals is not None:
        res_base, r_stride, _ = stack_frames(list(residuals))
        if T > 1 and r_stride != res_base.numel():
            raise RuntimeError("conv_bias_only: residuals must be one dense stack")
    _launch(x_base, x_stride, T, weight, bias, res_base, None, stride, padding, 1, 1.0, 0.0, 2.0, out, None, lif=False)
    return out
