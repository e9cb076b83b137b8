"""Dense / depthwise conv + LIF through the reference-shaped backend against the oracle."""
import pytest
import torch

from conftest import golden_cases, load_golden
from oracle import snn_oracle as orc
from util import check_parity

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _be():
    from triton_snn_fusion_b200.runtime import triton_convlif_backend as be
    return be


def _run(xs, w, b, v0, stride, pad, groups, lif, residuals=None):
    be = _be()
    xs_d = [x.to(DEV) for x in xs]
    v0_d = v0.to(DEV) if v0 is not None and v0.dim() else torch.tensor(0.0, device=DEV, dtype=xs[0].dtype)
    args = (w.to(DEV), b.to(DEV), v0_d, [stride] * 2, [pad] * 2, [1, 1], groups, lif[0], lif[1], lif[2], False)
    if residuals is not None:
        res = be.run_triton_fused_temporal_conv_add_lif_state(xs_d, [r.to(DEV) for r in residuals], *args, strict=True)
    elif groups > 1:
        res = be.run_triton_fused_temporal_depthwise_conv_lif_state(xs_d, *args, strict=True)
    elif w.shape[-1] == 1:
        res = be.run_triton_fused_temporal_pointwise_conv_lif_state(xs_d, *args, strict=True)
    else:
        res = be.run_triton_fused_temporal_conv_lif_state(xs_d, *args, strict=True)
    torch.cuda.synchronize()
    return res


@pytest.mark.parametrize("name", golden_cases("conv"))
def test_golden(name):
    a, z = load_golden(name)
    res_in = list(z["residual"]) if "residual" in z else None
    r = _run(list(z["x"]), z["w"], z["b"], z["v_init"], a["stride"], a["padding"], a["groups"],
             (a["v_th"], a["v_reset"], a["tau"]), residuals=res_in)
    assert r.kernel_key == name.split("conv_")[1].split("_res")[0].split("_plain")[0].replace("_odd", "")
    check_parity(r.spikes, r.v_next, z["spikes"], z["v"], torch.float32, flip_max=2e-3, what=name)


CASES = [
    # cin, cout, k, stride, pad, groups, H, W
    (3, 64, 3, 1, 1, 1, 32, 32),     # CNN-small layer 1
    (64, 128, 3, 2, 1, 1, 32, 32),   # CNN-small layer 2
    (128, 256, 3, 2, 1, 1, 16, 16),  # CNN-small layer 3
    (3, 64, 7, 2, 3, 1, 64, 64),     # ResNet stem
    (64, 64, 1, 1, 0, 1, 14, 14),    # pointwise
    (24, 40, 5, 1, 2, 1, 13, 11),    # k5 key, ragged channels
    (3, 16, 11, 4, 2, 1, 35, 35),    # k11 key
    (32, 32, 3, 1, 1, 32, 28, 28),   # depthwise s1
    (64, 64, 3, 2, 1, 64, 29, 31),   # depthwise s2, odd
    (6, 6, 3, 1, 1, 6, 9, 9),        # depthwise, channels not a multiple of 4
]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("residual", [False, True])
def test_seeded_vs_oracle(case, dtype, residual):
    cin, cout, k, s, p, g, H, W = case
    T, B = 4, 3
    torch.manual_seed(2026 + cin + cout + k)
    xs = [torch.randn(B, cin, H, W).to(dtype) for _ in range(T)]
    w = (torch.randn(cout, cin // g, k, k) * (2.0 / (cin // g * k * k)) ** 0.5).to(dtype)
    b = (torch.randn(cout) * 0.1).to(dtype)
    ho, wo = (H + 2 * p - k) // s + 1, (W + 2 * p - k) // s + 1
    v0 = (torch.randn(B, cout, ho, wo) * 0.3).to(dtype)
    res = [(torch.rand(B, cout, ho, wo) < 0.2).to(dtype) for _ in range(T)] if residual else None
    rs, rv = orc.temporal_conv_lif([orc.widen(x) for x in xs], orc.widen(w), orc.widen(b), orc.widen(v0),
                                   [s, s], [p, p], [1, 1], g, 1.0, 0.0, 2.0,
                                   residuals=[orc.widen(r) for r in res] if res else None)
    r = _run(xs, w, b, v0, s, p, g, (1.0, 0.0, 2.0), residuals=res)
    assert r.spikes.dtype == dtype and r.v_next.dtype == dtype
    check_parity(r.spikes, r.v_next, rs, rv, dtype, what=str(case))
    assert 0.02 < float(rs.mean()) < 0.6


def test_direct_encoding_alias_convolves_once():
    """All T inputs are the same tensor: result equals the stacked evaluation."""
    torch.manual_seed(1)
    x = torch.randn(2, 3, 16, 16)
    w = torch.randn(8, 3, 3, 3) * 0.3
    b = torch.randn(8) * 0.1
    rs, rv = orc.temporal_conv_lif([x] * 4, w, b, None, [1, 1], [1, 1], [1, 1], 1, 1.0, 0.0, 2.0)
    xd = x.to(DEV)
    r = _be().run_triton_fused_temporal_conv_lif_state(
        [xd] * 4, w.to(DEV), b.to(DEV), torch.tensor(0.0, device=DEV), [1, 1], [1, 1], [1, 1], 1, 1.0, 0.0, 2.0, False)
    check_parity(r.spikes, r.v_next, rs, rv, torch.float32)


def test_views_of_a_spike_stack_are_used_in_place():
    be = _be()
    torch.manual_seed(2)
    T, B, C, H, W = 4, 2, 8, 10, 10
    stack = be.empty_nhwc([T, B, C, H, W], torch.float32, DEV)
    stack.copy_((torch.rand(T, B, C, H, W) < 0.3).float())
    w = torch.randn(16, C, 3, 3) * 0.3
    b = torch.randn(16) * 0.1
    r = be.run_triton_fused_temporal_conv_lif_state(
        [stack[t] for t in range(T)], w.to(DEV), b.to(DEV), torch.tensor(0.0, device=DEV),
        [1, 1], [1, 1], [1, 1], 1, 1.0, 0.0, 2.0, False)
    assert r.kernel_diagnostics["stack_materialized"] is False
    rs, rv = orc.temporal_conv_lif(list(stack.cpu()), w, b, None, [1, 1], [1, 1], [1, 1], 1, 1.0, 0.0, 2.0)
    check_parity(r.spikes, r.v_next, rs, rv, torch.float32)


def test_packed_out_and_single_step():
    be = _be()
    torch.manual_seed(3)
    T, B, C, H, W = 2, 2, 4, 8, 8
    x_seq = torch.randn(T, B, C, H, W)
    w = torch.randn(8, C, 3, 3) * 0.4
    b = torch.randn(8) * 0.1
    rs, rv = orc.temporal_conv_lif(list(x_seq), w, b, None, [1, 1], [1, 1], [1, 1], 1, 1.0, 0.0, 2.0)
    spike_out = torch.empty(T, B, 8, H, W, device=DEV)
    v_out = torch.empty(B, 8, H, W, device=DEV)
    be.run_triton_fused_temporal_conv_lif_state_packed_out(
        x_seq.to(DEV), w.to(DEV), b.to(DEV), torch.tensor(0.0, device=DEV), [1, 1], [1, 1], [1, 1], 1,
        1.0, 0.0, 2.0, False, spike_out, v_out)
    check_parity(spike_out, v_out, rs, rv, torch.float32)
    one = be.run_triton_fused_conv_lif_state(
        x_seq[0].to(DEV), w.to(DEV), b.to(DEV), torch.tensor(0.0, device=DEV), [1, 1], [1, 1], [1, 1], 1,
        1.0, 0.0, 2.0, False)
    s1, v1 = orc.temporal_conv_lif([x_seq[0]], w, b, None, [1, 1], [1, 1], [1, 1], 1, 1.0, 0.0, 2.0)
    check_parity(one.spikes.unsqueeze(0), one.v_next, s1, v1, torch.float32)


def test_conv_without_lif():
    be = _be()
    torch.manual_seed(4)
    xs = [(torch.rand(2, 16, 12, 12) < 0.3).float() for _ in range(3)]
    w = torch.randn(32, 16, 1, 1) * 0.3
    b = torch.randn(32) * 0.1
    ref = orc.temporal_conv_only(xs, w, b, [2, 2], [0, 0])
    out = be.conv_bias_only([x.to(DEV) for x in xs], w.to(DEV), b.to(DEV), [2, 2], [0, 0])
    torch.testing.assert_close(out.cpu(), ref, rtol=1e-4, atol=1e-5)


def test_rejections():
    be = _be()
    x = torch.randn(1, 4, 8, 8, device=DEV)
    z = torch.tensor(0.0, device=DEV)
    w = torch.randn(4, 4, 3, 3, device=DEV)
    b = torch.zeros(4, device=DEV)
    with pytest.raises(RuntimeError, match="unsupported_stride"):
        be.run_triton_fused_temporal_conv_lif_state([x], w, b, z, [3, 3], [1, 1], [1, 1], 1, 1.0, 0.0, 2.0, False)
    with pytest.raises(RuntimeError, match="unsupported_dilation"):
        be.run_triton_fused_temporal_conv_lif_state([x], w, b, z, [1, 1], [1, 1], [2, 2], 1, 1.0, 0.0, 2.0, False)
    with pytest.raises(RuntimeError, match="unsupported_groups"):
        be.run_triton_fused_temporal_conv_lif_state([x], w[:, :2], b, z, [1, 1], [1, 1], [1, 1], 2, 1.0, 0.0, 2.0, False)
    with pytest.raises(RuntimeError, match="missing_or_unsupported_bias"):
        be.run_triton_fused_temporal_conv_lif_state([x], w, None, z, [1, 1], [1, 1], [1, 1], 1, 1.0, 0.0, 2.0, False)
    with pytest.raises(RuntimeError, match="was called with a pointwise conv"):
        be.run_triton_fused_temporal_conv_lif_state([x], w[:, :, :1, :1], b, z, [1, 1], [0, 0], [1, 1], 1, 1.0, 0.0, 2.0, False)
    with pytest.raises(RuntimeError, match="non-empty"):
        be.run_triton_fused_temporal_conv_lif_state([], w, b, z, [1, 1], [1, 1], [1, 1], 1, 1.0, 0.0, 2.0, False)
    assert be.classify_conv_lif_config(w, 1, 1, 1, 1) == "k3_s1_p1"
    assert be.classify_conv_lif_config(torch.empty(8, 1, 3, 3), 2, 1, 1, 8) == "depthwise_k3_s2_p1"
    assert be.classify_conv_lif_config(torch.empty(8, 4, 2, 2), 1, 0, 1, 1) == "unsupported"
