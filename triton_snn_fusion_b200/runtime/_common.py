"""Helpers shared by the backend modules: layout handling and argument marshalling."""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch

from .. import _lib

ACT_DTYPES = (torch.float32, torch.bfloat16, torch.float16)


def as_pair(value) -> Tuple[int, int]:
    if isinstance(value, int):
        return value, value
    return int(value[0]), int(value[1])


def raise_reasons(tag: str, reasons, strict: bool, verbose: bool):
    """Error convention of the reference backends: print when verbose, always raise."""
    if not reasons:
        return
    text = "; ".join(reasons)
    if verbose:
        print(f"[SNNB200][REJECT][{tag}] {text}")
    if strict:
        raise RuntimeError(f"[TRITON][STRICT][{tag}] {text}")
    raise RuntimeError(text)


class Gate:
    """Collects the reasons why a call cannot be taken, as "<code>: <detail>" strings.

    The codes (``unsupported_dtype``, ``unsupported_rank`` ...) are the keys under which the reference's op
    layer files a rejected call in its statistics (it splits the reason at the first colon,
    runtime/snn_custom_ops.py:161-169 in pengjh0111/triton-snn-fusion); the detail text is free.
    """

    def __init__(self, lead_name: str, lead):
        self.why: list = []
        self.lead_name = lead_name
        self.lead = lead if isinstance(lead, torch.Tensor) else None
        if self.lead is None:
            self.why.append(f"{lead_name} is {type(lead).__name__}, expected a Tensor")

    def __bool__(self) -> bool:     # True while the leading tensor can be inspected at all
        return self.lead is not None

    def add(self, code: str, detail: str) -> None:
        self.why.append(f"{code}: {detail}" if code else detail)

    def lead_is(self, rank: int) -> None:
        """The leading tensor: on a GPU, of the given rank, in an activation dtype."""
        x = self.lead
        if not x.is_cuda:
            self.add("unsupported_device", f"{self.lead_name} lives on {x.device}; this backend has GPU kernels only")
        if x.dim() != rank:
            self.add("unsupported_rank", f"{self.lead_name} has {x.dim()} dimensions, the op is defined for {rank}")
        if x.dtype not in ACT_DTYPES:
            self.add("unsupported_dtype", f"{self.lead_name} is {x.dtype}; float32, bfloat16 and float16 are implemented")

    def companion(self, name: str, t, rank=None, fp32_ok: bool = False, code: str = "") -> bool:
        """A tensor that has to sit beside the leading one: same device, same dtype (optionally fp32)."""
        if not isinstance(t, torch.Tensor):
            self.add(code, f"{name} is {type(t).__name__}, expected a Tensor")
            return False
        if rank is not None and t.dim() != rank:
            self.add(code or "unsupported_rank", f"{name} has {t.dim()} dimensions, expected {rank}")
            return False
        ok_dtypes = (self.lead.dtype, torch.float32) if fp32_ok else (self.lead.dtype,)
        if t.device != self.lead.device or t.dtype not in ok_dtypes:
            self.add("unsupported_dtype", f"{name} is {t.dtype} on {t.device} while {self.lead_name} is "
                                          f"{self.lead.dtype} on {self.lead.device}")
        return True

    def state(self, v_init, expected_shape, fp32_ok: bool = False) -> None:
        """Initial membrane: a 0-dim tensor (start from rest) or one value per output neuron."""
        if not isinstance(v_init, torch.Tensor):
            self.add("", f"v_init is {type(v_init).__name__}, expected a Tensor (0-dim for a zero state)")
            return
        if v_init.dim() == 0:
            return
        if expected_shape is not None and tuple(v_init.shape) != tuple(expected_shape):
            self.add("unsupported_membrane_state",
                     f"v_init is {tuple(v_init.shape)}, one value per output neuron would be {tuple(expected_shape)}")
        self.companion("v_init", v_init, fp32_ok=fp32_ok)

    def tau(self, tau) -> None:
        if float(tau) == 0.0:
            self.add("unsupported_tau", "tau = 0 (the charge step divides by tau)")


def is_nhwc_dense(t: torch.Tensor) -> bool:
    """True if a [..., C, H, W] tensor is stored densely with C innermost ([..., H, W, C] memory)."""
    if t.dim() < 4:
        return False
    perm = list(range(t.dim() - 3)) + [t.dim() - 2, t.dim() - 1, t.dim() - 3]
    return t.permute(perm).is_contiguous()


def to_nhwc(t: torch.Tensor) -> torch.Tensor:
    """[..., C, H, W] tensor -> same logical tensor with dense channels-last memory (copy only if needed)."""
    if is_nhwc_dense(t):
        return t
    lead = t.dim() - 3
    perm = list(range(lead)) + [lead + 1, lead + 2, lead]
    inv = list(range(lead)) + [lead + 2, lead, lead + 1]
    return t.permute(perm).contiguous().permute(inv)


def empty_nhwc(shape: Sequence[int], dtype, device) -> torch.Tensor:
    """Uninitialised logical [..., C, H, W] tensor with channels-last memory."""
    shape = list(shape)
    lead = len(shape) - 3
    c, h, w = shape[lead:]
    base = torch.empty(shape[:lead] + [h, w, c], dtype=dtype, device=device)
    inv = list(range(lead)) + [lead + 2, lead, lead + 1]
    return base.permute(inv)


def state_or_none(v_init: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """The reference passes a 0-dim tensor for 'start from zero' (runtime/snn_custom_ops.py:378-381)."""
    if v_init is None or not isinstance(v_init, torch.Tensor) or v_init.dim() == 0:
        return None
    return v_init


def stack_frames(xs: Sequence[torch.Tensor]) -> Tuple[torch.Tensor, int, bool]:
    """T frames [B,C,H,W] -> (base tensor, element stride between frames, whether a copy was made).

    Zero-copy cases: every entry is the same tensor (direct encoding: stride 0), or the
    entries are equally spaced channels-last views of one buffer (what indexing a fused
    op's spike stack yields). Anything else is copied into one channels-last stack.
    """
    first = xs[0]
    T = len(xs)
    if all(x.data_ptr() == first.data_ptr() for x in xs) and is_nhwc_dense(first):
        return first, 0, False
    if all(is_nhwc_dense(x) for x in xs):
        if T == 1:
            return first, 0, False
        esz = first.element_size()
        step = xs[1].data_ptr() - first.data_ptr()
        if step > 0 and step % esz == 0 and all(
            xs[t].data_ptr() - first.data_ptr() == t * step for t in range(T)
        ) and step // esz >= first.numel():
            return first, step // esz, False
    if all(x.data_ptr() == first.data_ptr() for x in xs):
        return to_nhwc(first), 0, True
    out = empty_nhwc([T] + list(first.shape), first.dtype, first.device)
    for t, x in enumerate(xs):
        out[t].copy_(x)
    return out[0], out.stride(0), True


def lif_scalars(v_threshold, v_reset, tau):
    return float(v_threshold), float(v_reset), float(tau)
