"""Temporal linear + LIF and the LIF -> avgpool -> linear tail against the oracle."""
import pytest
import torch

from conftest import golden_cases, load_golden
from oracle import snn_oracle as orc
from util import check_parity

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _lin():
    from triton_snn_fusion_b200.runtime import triton_temporal_linear_lif_backend as be
    return be


def _tail():
    from triton_snn_fusion_b200.runtime import triton_temporal_lif_avgpool_linear_backend as be
    return be


def _z(dtype=torch.float32):
    return torch.tensor(0.0, device=DEV, dtype=dtype)


@pytest.mark.parametrize("name", golden_cases("linear"))
def test_linear_golden(name):
    a, z = load_golden(name)
    v0 = z["v_init"].to(DEV) if z["v_init"].dim() else _z()
    b = z["b"].to(DEV) if "b" in z else torch.empty(0, device=DEV)
    r = _lin().run_triton_fused_temporal_linear_lif_state_packed(
        z["x"].to(DEV), z["w"].to(DEV), b, v0, a["v_th"], a["v_reset"], a["tau"], False, strict=True)
    check_parity(r.spikes, r.v_next, z["spikes"], z["v"], torch.float32, what=name)


@pytest.mark.parametrize("shape", [(4, 64, 512, 512), (4, 16, 1024, 512), (2, 33, 100, 70), (1, 4, 4096, 1000)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_linear_seeded(shape, dtype):
    T, M, K, N = shape
    torch.manual_seed(2026 + T + M + K + N)
    x = (torch.rand(T, M, K) < 0.15).to(dtype)  # spikes from a previous layer
    w = (torch.randn(N, K) * (1.0 / K) ** 0.5 * 3.0).to(dtype)
    b = (torch.randn(N) * 0.1).to(dtype)
    v0 = (torch.randn(M, N) * 0.3).to(dtype)
    rs, rv = orc.temporal_linear_lif(orc.widen(x), orc.widen(w), orc.widen(b), orc.widen(v0), 1.0, 0.0, 2.0)
    be = _lin()
    r = be.run_triton_fused_temporal_linear_lif_state_packed(
        x.to(DEV), w.to(DEV), b.to(DEV), v0.to(DEV), 1.0, 0.0, 2.0, False, strict=True)
    check_parity(r.spikes, r.v_next, rs, rv, dtype, what=str(shape))
    # list form and caller-owned outputs give the same tensors
    r2 = be.run_triton_fused_temporal_linear_lif_state(
        [x[t].to(DEV) for t in range(T)], w.to(DEV), b.to(DEV), v0.to(DEV), 1.0, 0.0, 2.0, False)
    assert torch.equal(r2.spikes, r.spikes) and torch.equal(r2.v_next, r.v_next)
    so = torch.empty(T, M, N, device=DEV, dtype=dtype)
    vo = torch.empty(M, N, device=DEV, dtype=dtype)
    be.run_triton_fused_temporal_linear_lif_state_packed_out(
        x.to(DEV), w.to(DEV), b.to(DEV), v0.to(DEV), 1.0, 0.0, 2.0, False, so, vo)
    assert torch.equal(so, r.spikes) and torch.equal(vo, r.v_next)


def test_linear_flattens_leading_dims():
    torch.manual_seed(9)
    x = torch.randn(3, 2, 5, 32) * 0.5
    w = torch.randn(16, 32) * 0.2
    rs, rv = orc.temporal_linear_lif(x, w, None, None, 1.0, 0.0, 2.0)
    r = _lin().run_triton_fused_temporal_linear_lif_state_packed(
        x.to(DEV), w.to(DEV), None, _z(), 1.0, 0.0, 2.0, False)
    assert tuple(r.spikes.shape) == (3, 2, 5, 16) and tuple(r.v_next.shape) == (2, 5, 16)
    check_parity(r.spikes, r.v_next, rs, rv, torch.float32)


@pytest.mark.parametrize("name", golden_cases("tail"))
def test_tail_golden(name):
    a, z = load_golden(name)
    v0 = z["v_init"].to(DEV) if z["v_init"].dim() else _z()
    r = _tail().run_triton_fused_temporal_lif_avgpool_linear(
        z["x"].to(DEV), v0, z["w"].to(DEV), z["b"].to(DEV), a["v_th"], a["v_reset"], a["tau"], False, strict=True)
    torch.testing.assert_close(r.out_sum.cpu(), z["out_sum"], rtol=1e-4, atol=1e-5)
    assert torch.equal(r.v_next.cpu(), z["v"])  # the LIF part is bit-exact


@pytest.mark.parametrize("shape", [(4, 16, 256, 8, 8, 10), (4, 64, 1024, 7, 7, 1000), (4, 5, 512, 7, 7, 1000),
                                   (2, 3, 20, 3, 5, 7), (5, 9, 128, 4, 4, 33), (9, 2, 64, 2, 2, 5), (4, 40, 2048, 2, 2, 100),
                                   (4, 300, 512, 7, 7, 100),    # eight samples per cluster, last group partial
                                   (8, 6, 512, 7, 7, 100)])     # 392 spikes per channel at most: counts kept as two 16-bit parts
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nhwc", [False, True])
def test_tail_seeded(shape, dtype, nhwc):
    T, N, C, H, W, K = shape
    torch.manual_seed(2026 + N + C + K)
    x = (torch.randn(T, N, C, H, W) * 0.75 + 0.15).to(dtype)
    v0 = (torch.randn(N, C, H, W) * 0.3).to(dtype)
    w = (torch.randn(K, C) * 0.05).to(dtype)
    b = (torch.randn(K) * 0.05).to(dtype)
    ro, rv = orc.temporal_lif_avgpool_linear(orc.widen(x), orc.widen(v0), orc.widen(w), orc.widen(b), 1.0, 0.0, 2.0)
    xd, vd = x.to(DEV), v0.to(DEV)
    if nhwc:
        xd = xd.permute(0, 1, 3, 4, 2).contiguous().permute(0, 1, 4, 2, 3)
        vd = vd.permute(0, 2, 3, 1).contiguous().permute(0, 3, 1, 2)
    r = _tail().run_triton_fused_temporal_lif_avgpool_linear(xd, vd, w.to(DEV), b.to(DEV), 1.0, 0.0, 2.0, False)
    assert r.kernel_diagnostics["layout"] == ("NHWC" if nhwc else "NCHW")
    rtol, atol = (1e-4, 1e-5) if dtype == torch.float32 else (1e-2, 1e-2)
    torch.testing.assert_close(r.out_sum.cpu().float(), ro, rtol=rtol, atol=atol)
    assert torch.equal(r.v_next.cpu(), rv.to(dtype))
    # deterministic: integer spike counts, no floating-point atomics
    r2 = _tail().run_triton_fused_temporal_lif_avgpool_linear(xd, vd, w.to(DEV), b.to(DEV), 1.0, 0.0, 2.0, False)
    assert torch.equal(r.out_sum, r2.out_sum)


def test_tail_alias_module():
    from triton_snn_fusion_b200.runtime import triton_temporal_lif_tail_backend as old
    assert old.run_triton_fused_temporal_lif_tail is _tail().run_triton_fused_temporal_lif_avgpool_linear
