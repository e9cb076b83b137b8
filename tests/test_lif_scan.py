"""snnb_lif_scan (through the reference-shaped backend entry) against the oracle: bit-exact."""
import pytest
import torch

from conftest import golden_cases, load_golden
from oracle import snn_oracle as orc

pytestmark = pytest.mark.gpu


def _backend():
    from triton_snn_fusion_b200.runtime.triton_temporal_lif_backend import run_triton_fused_temporal_lif_state
    return run_triton_fused_temporal_lif_state


def _run(x, v0, v_th, v_reset, tau, **kw):
    dev = torch.device("cuda")
    v0d = v0.to(dev) if v0 is not None else torch.tensor(0.0, device=dev, dtype=x.dtype)
    res = _backend()(x.to(dev), v0d, v_th, v_reset, tau, False, strict=True, **kw)
    torch.cuda.synchronize()
    return res.spikes.cpu(), res.v_next.cpu()


@pytest.mark.parametrize("name", golden_cases("lif"))
def test_golden(name):
    a, z = load_golden(name)
    v0 = z["v_init"] if z["v_init"].dim() else None
    s, v = _run(z["x"], v0, a["v_th"], a["v_reset"], a["tau"])
    assert torch.equal(s, z["spikes"])
    assert torch.equal(v, z["v"])


@pytest.mark.parametrize("T", [1, 2, 3, 4, 8, 16])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_seeded_vs_oracle(T, dtype):
    # input distribution of the standalone-scan benchmark: N(0.6, 0.8)
    torch.manual_seed(2026 + T)
    shape = (4, 32, 32, 32)  # 2^17 neurons
    x = (torch.randn((T,) + shape) * 0.8 + 0.6).to(dtype)
    v0 = (torch.randn(shape) * 0.3).to(dtype)
    rs, rv = orc.temporal_lif(orc.widen(x), orc.widen(v0), 1.0, 0.0, 2.0)
    s, v = _run(x, v0, 1.0, 0.0, 2.0)
    assert s.dtype == dtype and v.dtype == dtype
    assert torch.equal(s.float(), rs), "spikes must be bit-exact"
    # membrane is kept in fp32 in the kernel and rounded once on the way out
    assert torch.equal(v, rv.to(dtype))
    if T >= 4:
        assert 0.05 < float(rs.mean()) < 0.5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_u8_spikes_fp32_state(dtype):
    torch.manual_seed(7)
    x = (torch.randn(4, 2, 16, 8, 8) * 0.8 + 0.6).to(dtype)
    rs, rv = orc.temporal_lif(orc.widen(x), None, 1.0, 0.0, 2.0)
    s, v = _run(x, None, 1.0, 0.0, 2.0, spike_dtype=torch.uint8, v_dtype=torch.float32)
    assert s.dtype == torch.uint8 and v.dtype == torch.float32
    assert torch.equal(s.float(), rs) and torch.equal(v, rv)


@pytest.mark.parametrize("n_shape", [(1, 1, 1, 1), (1, 3, 5, 7), (2, 1, 1, 9), (1, 1, 3, 11)])
def test_ragged_sizes_take_scalar_path(n_shape):
    torch.manual_seed(11)
    x = torch.randn((5,) + n_shape) * 0.8 + 0.6
    v0 = torch.randn(n_shape)
    for v_th, v_reset, tau in ((1.0, 0.0, 2.0), (1.0, -1.0, 2.0), (0.7, 0.2, 3.0), (1.0, 0.0, 0.5)):
        rs, rv = orc.temporal_lif(x, v0, v_th, v_reset, tau)
        s, v = _run(x, v0, v_th, v_reset, tau)
        assert torch.equal(s, rs) and torch.equal(v, rv)


def test_channels_last_frames_keep_layout():
    torch.manual_seed(3)
    x = (torch.randn(4, 2, 6, 6, 16) * 0.8 + 0.6).permute(0, 1, 4, 2, 3)  # logical NCHW, NHWC memory
    v0 = torch.randn(2, 6, 6, 16).permute(0, 3, 1, 2)
    rs, rv = orc.temporal_lif(x, v0, 1.0, 0.0, 2.0)
    dev = torch.device("cuda")
    res = _backend()(x.to(dev), v0.to(dev), 1.0, 0.0, 2.0, False, strict=True)
    assert res.spikes.stride() == x.stride()
    assert torch.equal(res.spikes.cpu(), rs) and torch.equal(res.v_next.cpu(), rv)


def test_window_chaining_full_size():
    """Size-independent property at benchmark size (T=8, 2^24 neurons): one scan over T=8 equals
    two chained scans over T=4 with the membrane handed over."""
    torch.manual_seed(5)
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(5)
    x = torch.randn((8, 16, 64, 128, 128), device=dev, generator=g) * 0.8 + 0.6
    z = torch.tensor(0.0, device=dev)
    f = _backend()
    full = f(x, z, 1.0, 0.0, 2.0, False)
    a = f(x[:4], z, 1.0, 0.0, 2.0, False)
    b = f(x[4:], a.v_next, 1.0, 0.0, 2.0, False)
    assert torch.equal(full.spikes[:4], a.spikes) and torch.equal(full.spikes[4:], b.spikes)
    assert torch.equal(full.v_next, b.v_next)
    rate = float(full.spikes.mean())
    assert 0.05 < rate < 0.5


def test_rejects_bad_arguments():
    dev = torch.device("cuda")
    f = _backend()
    x = torch.randn(4, 2, 3, 4, 4, device=dev)
    with pytest.raises(RuntimeError, match="unsupported_rank"):
        f(x[0], torch.tensor(0.0, device=dev), 1.0, 0.0, 2.0, False)
    with pytest.raises(RuntimeError, match="unsupported_membrane_state"):
        f(x, torch.zeros(2, 3, 4, 5, device=dev), 1.0, 0.0, 2.0, False)
    with pytest.raises(RuntimeError, match="unsupported_tau"):
        f(x, torch.tensor(0.0, device=dev), 1.0, 0.0, 0.0, False)
    with pytest.raises(RuntimeError, match="unsupported_device"):
        f(x.cpu(), torch.tensor(0.0), 1.0, 0.0, 2.0, False)
