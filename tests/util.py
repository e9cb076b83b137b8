"""Parity checks shared by the GPU tests."""
import torch

# Bounds from the build's statement of parity for conv/linear-fused layers: membrane within
# rtol 1e-4 in fp32 (1e-2 with 16-bit inputs) and a spike-flip rate of at most 1e-4.
FLIP_RATE_MAX = 1e-4
# A tensor with fewer than 1e5 elements cannot resolve a rate of 1e-4 (one flip is already 1e-5 or
# more of it): there the bound is a count.
FLIP_COUNT_SMALL = 2
TOL = {torch.float32: (1e-4, 2e-5), torch.bfloat16: (1e-2, 1e-2), torch.float16: (1e-2, 1e-2)}


def check_parity(spikes, v, ref_spikes, ref_v, dtype, flip_max=FLIP_RATE_MAX, what=""):
    """spikes [T,...], v [...] from the device against the oracle's. Returns the flip rate.

    A flipped spike resets (or fails to reset) its neuron, so the membrane is compared on
    the neurons whose whole spike history agrees; the flips themselves are bounded by rate.
    """
    s = spikes.detach().cpu().float()
    rs = ref_spikes.detach().cpu().float()
    vv = v.detach().cpu().float()
    rv = ref_v.detach().cpu().float()
    assert s.shape == rs.shape and vv.shape == rv.shape, (what, s.shape, rs.shape, vv.shape, rv.shape)
    assert bool(((s == 0) | (s == 1)).all()), f"{what}: spikes must be 0/1"
    flips = (s != rs)
    n_flips = int(flips.sum())
    rate = n_flips / s.numel() if s.numel() else 0.0
    allowed = max(int(flip_max * s.numel()), FLIP_COUNT_SMALL if s.numel() < 100000 else 0)
    assert n_flips <= allowed, (f"{what}: {n_flips} flipped spikes of {s.numel()} (rate {rate:.3e}); "
                                f"allowed {allowed} (rate {flip_max:.1e})")
    same = ~flips.any(dim=0)
    rtol, atol = TOL[dtype]
    if same.any():
        torch.testing.assert_close(vv[same], rv[same], rtol=rtol, atol=atol, msg=lambda m: f"{what}: membrane: {m}")
    return rate
