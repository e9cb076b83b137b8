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
