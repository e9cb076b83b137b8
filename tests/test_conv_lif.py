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
    check_parity(r.spikes, r.v_next, z["spikes"], z["v"], torch.float32, what=name)


CASES = [
    # cin, cout, k, stride, pad, groups, H, W
    (3, 64, 3, 1, 1, 1, 32, 32),     # CNN-small layer 1
    (64, 128, 3, 2, 1, 1, 32, 32),   # CNN-small layer 2
    (128, 256, 3, 2, 1, 1, 16, 16),  # CNN-small layer 3
    (3, 32, 3, 2, 1, 1, 30, 34),     # MobileNet stem (direct kernel for few input channels)
    (3, 64, 7, 2, 3, 1, 64, 64),     # ResNet stem
    (64, 64, 1, 1, 0, 1, 14, 14),    # pointwise
    (24, 40, 5, 1, 2, 1, 13, 11),    # k5 key, ragged channels
    (3, 16, 11, 4, 2, 1, 35, 35),    # k11 key
    (32, 32, 3, 1, 1, 32, 28, 28),   # depthwise s1
    (64, 64, 3, 2, 1, 64, 29, 31),   # depthwise s2, odd
    (6, 6, 3, 1, 1, 6, 9, 9),        # depthwise, channels not a multiple of 4
    (64, 64, 3, 1, 1, 64, 56, 56),   # depthwise on the shared-memory tile kernel: 64-channel blocks, strips of 7
    (128, 128, 3, 2, 1, 128, 28, 28),  # tile kernel, stride 2
    (96, 96, 3, 1, 1, 96, 14, 14),   # tile kernel, 32-channel blocks
    (64, 64, 3, 1, 1, 64, 7, 7),     # tile kernel, map narrower than one strip
    (64, 64, 3, 1, 1, 64, 33, 20),   # tile kernel, ragged rows and columns
    (32, 32, 3, 2, 1, 32, 15, 17),   # tile kernel, stride 2 on odd sizes
    (64, 64, 3, 1, 1, 64, 16, 32),   # tile kernel, strips of 8
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


@pytest.mark.parametrize("C", [64, 96])
@pytest.mark.parametrize("stride", [1, 2])
def test_depthwise_tile_kernel_variants(C, stride):
    """The depthwise tile kernel through the C ABI with 64- and 32-channel blocks, one-byte spikes, an fp32
    membrane updated in place over two chained calls (T = 3 + 2), f16 data and a residual."""
    from triton_snn_fusion_b200 import _lib as L
    strip = C
    dtype, B, H, W, T = torch.float16, 3, 22, 19, 5
    Ho, Wo = (H - 1) // stride + 1, (W - 1) // stride + 1
    g = torch.Generator().manual_seed(C * 10 + stride)
    x = torch.randn(T, B, H, W, C, generator=g).to(dtype)
    w = (torch.randn(C, 3, 3, generator=g) * 0.4).to(dtype)
    b = (torch.randn(C, generator=g) * 0.1).to(dtype)
    res = (torch.rand(T, B, Ho, Wo, C, generator=g) < 0.2).to(dtype)
    nchw = lambda t: orc.widen(t).permute(0, 3, 1, 2)
    rs, rv = orc.temporal_conv_lif([nchw(x[t]) for t in range(T)], orc.widen(w).unsqueeze(1), orc.widen(b), None,
                                   [stride] * 2, [1, 1], [1, 1], C, 1.0, 0.0, 2.0, residuals=[nchw(res[t]) for t in range(T)])
    xd, wd, bd, rd = x.to(DEV), w.to(DEV), b.to(DEV), res.to(DEV)
    sp = torch.empty(T, B, Ho, Wo, C, dtype=torch.uint8, device=DEV)
    v = torch.empty(B, Ho, Wo, C, dtype=torch.float32, device=DEV)
    for t0, n in ((0, 3), (3, 2)):
        L.check(L.lib.snnb_dwconv3x3_lif(xd[t0].data_ptr(), xd.stride(0), wd.data_ptr(), bd.data_ptr(), rd[t0].data_ptr(),
                                         v.data_ptr() if t0 else None, sp[t0].data_ptr(), v.data_ptr(), n, B, C, H, W, stride,
                                         L.F16, L.U8, L.F32, 1.0, 0.0, 2.0, None), "snnb_dwconv3x3_lif")
    torch.cuda.synchronize()
    assert L.device_status() == 0
    check_parity(sp.permute(0, 1, 4, 2, 3), v.permute(0, 3, 1, 2), rs, rv, torch.float32, what=f"C {C} stride {stride}")
    assert 0.02 < float(rs.mean()) < 0.6


def test_depthwise_tile_kernel_one_frame_for_all_steps_and_soft_reset():
    from triton_snn_fusion_b200 import _lib as L
    dtype, B, C, H, W, T = torch.bfloat16, 2, 32, 12, 12, 4
    g = torch.Generator().manual_seed(9)
    x = torch.randn(B, H, W, C, generator=g).to(dtype)
    w = (torch.randn(C, 3, 3, generator=g) * 0.5).to(dtype)
    b = (torch.randn(C, generator=g) * 0.1).to(dtype)
    rs, rv = orc.temporal_conv_lif([orc.widen(x).permute(0, 3, 1, 2)] * T, orc.widen(w).unsqueeze(1), orc.widen(b), None,
                                   [1, 1], [1, 1], [1, 1], C, 0.8, -1.0, 3.0)
    xd, wd, bd = x.to(DEV), w.to(DEV), b.to(DEV)
    sp = torch.empty(T, B, H, W, C, dtype=dtype, device=DEV)
    v = torch.empty(B, H, W, C, dtype=dtype, device=DEV)
    L.check(L.lib.snnb_dwconv3x3_lif(xd.data_ptr(), 0, wd.data_ptr(), bd.data_ptr(), None, None, sp.data_ptr(), v.data_ptr(),
                                     T, B, C, H, W, 1, L.BF16, L.BF16, L.BF16, 0.8, -1.0, 3.0, None), "snnb_dwconv3x3_lif")
    torch.cuda.synchronize()
    check_parity(sp.permute(0, 1, 4, 2, 3), v.permute(0, 3, 1, 2), rs, rv, dtype, what="soft reset, tau 3")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_packed_out_writes_channels_last_buffers_in_place(dtype):
    """Caller-owned outputs that already are channels-last (what this backend's own outputs and the graph executor's
    buffers are): the kernel writes straight into them - the result object holds the caller's tensors, poisoned
    buffers come back fully overwritten, and a pre-stacked channels-last input is read without a copy."""
    be = _be()
    torch.manual_seed(5)
    T, B, cin, cout, H, W = 4, 2, 64, 128, 12, 9
    x = (torch.rand(T, B, cin, H, W) < 0.2).to(dtype)
    w = (torch.randn(cout, cin, 3, 3) * 0.15).to(dtype)
    b = (torch.randn(cout) * 0.1).to(dtype)
    v0 = (torch.randn(B, cout, H, W) * 0.3).to(dtype)
    rs, rv = orc.temporal_conv_lif([orc.widen(x[t]) for t in range(T)], orc.widen(w), orc.widen(b), orc.widen(v0),
                                   [1, 1], [1, 1], [1, 1], 1, 1.0, 0.0, 2.0)
    x_seq = be.empty_nhwc([T, B, cin, H, W], dtype, DEV)
    x_seq.copy_(x)
    spike_out = be.empty_nhwc([T, B, cout, H, W], dtype, DEV)
    v_out = be.empty_nhwc([B, cout, H, W], dtype, DEV)
    spike_out.fill_(7.0)
    v_out.fill_(7.0)
    r = be.run_triton_fused_temporal_conv_lif_state_packed_out(
        x_seq, w.to(DEV), b.to(DEV), be.to_nhwc(v0.to(DEV)), [1, 1], [1, 1], [1, 1], 1, 1.0, 0.0, 2.0, False,
        spike_out, v_out, strict=True)
    assert r.spikes.data_ptr() == spike_out.data_ptr() and r.v_next.data_ptr() == v_out.data_ptr()
    assert r.kernel_diagnostics["stack_materialized"] is False
    check_parity(spike_out, v_out, rs, rv, dtype, what="packed_out, channels-last buffers")
