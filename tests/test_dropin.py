"""The drop-in claim, tested through the reference's own layers.

The reference's op layer (runtime/snn_custom_ops.py) and FX passes (compiler/*.py) are used exactly as they
are (staged byte for byte under oracle/_ref); only the five backend modules beneath them are this library's
(``runtime.install.install``). CPU part: the binding itself - every name the op layer imports resolves to
this library and accepts the arguments the op layer passes. GPU part: ``torch.ops.snn_custom.*`` with
``configure_fused_op(backend="triton", strict_triton=True)`` against the oracle, with the reference's own
call statistics showing that nothing fell back, and whole models through the reference's pass pipeline.
"""
import ast
import contextlib
import hashlib
import inspect
import io
import json

import pytest
import torch

from conftest import REF_STAGE, ROOT
from oracle import snn_oracle as orc
from util import check_parity

BACKENDS = ("triton_convlif_backend", "triton_temporal_lif_backend", "triton_temporal_lif_avgpool_linear_backend",
            "triton_temporal_linear_lif_backend")


def _op_layer_ast():
    return ast.parse((REF_STAGE / "runtime" / "snn_custom_ops.py").read_text())


def test_staged_files_are_the_reference_unmodified(ref_ops):
    manifest = json.loads((REF_STAGE / "MANIFEST.json").read_text())["files"]
    assert "runtime/snn_custom_ops.py" in manifest and any(k.startswith("compiler/") for k in manifest)
    for rel, digest in manifest.items():
        assert hashlib.sha256((REF_STAGE / rel).read_bytes()).hexdigest() == digest, rel
    # where the checkout itself is present (the build container), the staged copy equals it
    origin = ROOT.parent / "reference"
    if (origin / "runtime").is_dir():
        for rel in manifest:
            assert (origin / rel).read_bytes() == (REF_STAGE / rel).read_bytes(), rel


def test_every_name_the_op_layer_imports_is_bound_to_this_library(ref_ops):
    import triton_snn_fusion_b200.runtime as ours
    imported = {}
    for node in _op_layer_ast().body:
        if isinstance(node, ast.ImportFrom) and node.module and node.module.startswith("runtime.triton_"):
            imported[node.module.split(".")[1]] = [a.name for a in node.names]
    assert sorted(imported) == sorted(BACKENDS)
    total = 0
    for mod, names in imported.items():
        mine = __import__(f"{ours.__name__}.{mod}", fromlist=["x"])
        for name in names:
            assert getattr(ref_ops, name) is getattr(mine, name), f"{mod}.{name} is not this library's function"
            total += 1
    assert total == 13   # 8 conv entry points / helpers, 1 scan, 1 tail, 3 linear


def test_backends_accept_the_arguments_the_op_layer_passes(ref_ops):
    """Every call site of a backend function inside the reference's op layer: the positional count and the
    keyword names (strict=, verbose=, use_autotune=, compute_dtype= ...) bind to this library's signature."""
    tree = _op_layer_ast()
    bound = {a.name for n in tree.body if isinstance(n, ast.ImportFrom) and n.module and n.module.startswith("runtime.triton_")
             for a in n.names}
    sites = 0
    for node in ast.walk(tree):
        if isinstance(node, ast.Call) and isinstance(node.func, ast.Name) and node.func.id in bound:
            fn = getattr(ref_ops, node.func.id)
            kwargs = {k.arg: None for k in node.keywords if k.arg}
            inspect.signature(fn).bind(*([None] * len(node.args)), **kwargs)   # raises TypeError on a mismatch
            sites += 1
    assert sites >= 10


def test_result_objects_carry_what_the_op_layer_reads():
    from triton_snn_fusion_b200.runtime import (triton_convlif_backend, triton_temporal_lif_avgpool_linear_backend,
                                                triton_temporal_lif_backend, triton_temporal_linear_lif_backend)
    for cls, fields in ((triton_convlif_backend.TritonConvLIFResult, ("spikes", "v_next")),
                        (triton_temporal_lif_backend.TritonTemporalLIFResult, ("spikes", "v_next")),
                        (triton_temporal_linear_lif_backend.TritonTemporalLinearLIFResult, ("spikes", "v_next")),
                        (triton_temporal_lif_avgpool_linear_backend.TritonTemporalLIFAvgPoolLinearResult, ("out_sum", "v_next"))):
        names = {f for f in cls.__dataclass_fields__}
        assert set(fields) <= names and {"kernel_key", "kernel_diagnostics"} <= names, cls


def _pipeline(ref_ops, name, T, hw, B, dtype, device, mode, gain=1.0, classes=10, **executor_options):
    from oracle import torch_models as tm
    from triton_snn_fusion_b200 import chronos, specs
    spec = specs.NETS[name](classes)
    params = specs.make_params(spec, seed=2026, gain=gain)
    model = tm.build(spec, params, T).to(device=device, dtype=dtype)
    report = chronos.RewriteReport()
    executors = []

    def backend(gm, example_inputs, **kw):
        with contextlib.redirect_stdout(io.StringIO()):   # the reference's passes print their statistics
            chronos.rewrite_graph(gm, example_inputs, T, report=report)
        if mode == "eager":
            return gm.forward
        from triton_snn_fusion_b200.fx_executor import build_fx_standalone_backend
        ex = build_fx_standalone_backend(gm, use_cuda_graph=(device != "cpu"), example_inputs=tuple(example_inputs),
                                         **executor_options)
        executors.append(ex)
        return ex

    torch._dynamo.reset()
    compiled = torch.compile(model, backend=backend)
    xs = [torch.randn(B, 3, hw, hw, generator=torch.Generator().manual_seed(7 + i)).to(device=device, dtype=dtype)
          for i in range(2)]
    outs = []
    with torch.no_grad():
        for x in xs:
            model.layer.reset()
            outs.append(compiled(x).float().cpu().clone())
    return outs, report, executors, (spec, params, xs)


def test_pass_pipeline_on_cpu_keeps_the_eager_result(ref_ops):
    """CNN-small (fp32, T=4) through the reference's passes in the reference's order, on CPU, where the fused
    ops run the reference's eager loops: same logits as the un-rewritten model, through both hand-offs."""
    from oracle import torch_models as tm
    ref_ops.configure_fused_op(backend="torch")
    for mode in ("eager", "executor"):
        outs, report, executors, (spec, params, xs) = _pipeline(ref_ops, "cnn_small", 4, 32, 4, torch.float32, "cpu", mode)
        assert report.fused_nodes == {"fused_temporal_conv_lif_state": 3, "fused_temporal_lif_avgpool_linear": 1}
        assert report.lif_nodes_left == 0
        plain = tm.build(spec, params, 4)
        with torch.no_grad():
            for x, got in zip(xs, outs):
                plain.layer.reset()
                torch.testing.assert_close(got, plain(x), rtol=0, atol=0)
        if mode == "executor":
            assert executors and executors[0].stats["fused_via_op_layer"] == 4 and not executors[0].stats["cuda_graph"]


def test_resnet18_graph_on_cpu_lowers_the_neighbours(ref_ops):
    ref_ops.configure_fused_op(backend="torch")
    outs, report, executors, _ = _pipeline(ref_ops, "resnet18", 4, 64, 2, torch.float32, "cpu", "executor", gain=4.0)
    assert report.fused_nodes == {"fused_temporal_conv_lif_state": 9, "fused_temporal_conv_add_lif_state": 8}
    st = executors[0].stats
    assert st["lowered_maxpool"] == 1 and st["lowered_conv_bn"] == 3 and st["fused_via_op_layer"] == 17
    assert all(torch.isfinite(o).all() for o in outs)


# ------------------------------------------------------------------------------------------- GPU ----
def _strict(ref_ops):
    ref_ops.configure_fused_op(backend="triton", strict_triton=True)
    ref_ops.reset_fused_op_call_stats()


def _no_fallback(ref_ops, calls):
    st = ref_ops.get_fused_op_call_stats()
    assert st["fallback"] == 0 and st["temporal_fallback"] == 0 and not st["fallback_reasons"], st["fallback_reasons"]
    assert st["temporal_lif_fallback"] == 0 and st["temporal_linear_lif_fallback"] == 0
    assert st["temporal_lif_avgpool_linear_fallback"] == 0 and st["temporal_residual_fallback"] == 0
    assert st["total"] >= calls


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_conv_ops_through_the_reference_op_layer(ref_ops, dtype):
    """regular / pointwise / depthwise / residual temporal conv ops and the single-step op, called as
    torch.ops.snn_custom.* (dtypes the reference's Meta functions and support gate accept)."""
    ops = torch.ops.snn_custom
    dev, T, B = "cuda", 4, 2
    g = torch.Generator().manual_seed(11)
    z = torch.tensor(0.0, dtype=dtype, device=dev)
    lif = (1.0, 0.0, 2.0, False)
    cases = [
        ("regular", ops.fused_temporal_conv_lif_state.default, 64, 64, 3, 1, 1, 1),
        ("regular_s2", ops.fused_temporal_conv_lif_state.default, 64, 128, 3, 2, 1, 1),
        ("pointwise", ops.fused_temporal_pointwise_conv_lif_state.default, 64, 128, 1, 1, 0, 1),
        ("depthwise", ops.fused_temporal_depthwise_conv_lif_state.default, 64, 64, 3, 1, 1, 64),
        ("depthwise_alias", ops.fused_temporal_conv_lif_state_depthwise.default, 32, 32, 3, 2, 1, 32),
    ]
    _strict(ref_ops)
    n = 0
    for tag, op, cin, cout, k, s, p, groups in cases:
        xs = [(torch.rand(B, cin, 16, 16, generator=g) < 0.25).to(dtype) for _ in range(T)]
        w = (torch.randn(cout, cin // groups, k, k, generator=g) * (2.0 / (cin // groups * k * k)) ** 0.5 * 2).to(dtype)
        b = (torch.randn(cout, generator=g) * 0.1).to(dtype)
        rs, rv = orc.temporal_conv_lif([orc.widen(x) for x in xs], orc.widen(w), orc.widen(b), None,
                                       [s, s], [p, p], [1, 1], groups, 1.0, 0.0, 2.0)
        sp, v = op([x.to(dev) for x in xs], w.to(dev), b.to(dev), z, [s, s], [p, p], [1, 1], groups, *lif)
        assert sp.dtype == dtype and v.dtype == dtype and tuple(sp.shape) == tuple(rs.shape)
        check_parity(sp, v, rs, rv, dtype, what=tag)
        n += 1
    # residual form
    xs = [(torch.rand(B, 64, 16, 16, generator=g) < 0.25).to(dtype) for _ in range(T)]
    res = [(torch.rand(B, 64, 16, 16, generator=g) < 0.2).to(dtype) for _ in range(T)]
    w = (torch.randn(64, 64, 3, 3, generator=g) * 0.1).to(dtype)
    b = (torch.randn(64, generator=g) * 0.1).to(dtype)
    rs, rv = orc.temporal_conv_lif([orc.widen(x) for x in xs], orc.widen(w), orc.widen(b), None, [1, 1], [1, 1], [1, 1], 1,
                                   1.0, 0.0, 2.0, residuals=[orc.widen(r) for r in res])
    sp, v = ops.fused_temporal_conv_add_lif_state.default([x.to(dev) for x in xs], [r.to(dev) for r in res], w.to(dev),
                                                          b.to(dev), z, [1, 1], [1, 1], [1, 1], 1, *lif)
    check_parity(sp, v, rs, rv, dtype, what="residual")
    # single step
    rs1, rv1 = orc.temporal_conv_lif([orc.widen(xs[0])], orc.widen(w), orc.widen(b), None, [1, 1], [1, 1], [1, 1], 1, 1.0, 0.0, 2.0)
    s1, v1 = ops.fused_conv_lif_state.default(xs[0].to(dev), w.to(dev), b.to(dev), z, [1, 1], [1, 1], [1, 1], 1, *lif)
    check_parity(s1.unsqueeze(0), v1, rs1, rv1, dtype, what="single step")
    _no_fallback(ref_ops, n + 2)
    st = ref_ops.get_fused_op_call_stats()
    assert st["temporal_k3_s1_p1"] >= 1 and st["temporal_k1_s1_p0"] == 1 and st["temporal_depthwise_k3_s1_p1"] == 1


@pytest.mark.gpu
def test_scan_linear_and_tail_ops_through_the_reference_op_layer(ref_ops):
    ops = torch.ops.snn_custom
    dev, dtype = "cuda", torch.float32
    g = torch.Generator().manual_seed(5)
    z = torch.tensor(0.0, device=dev)
    _strict(ref_ops)
    # standalone scan: bit-exact
    x = torch.randn(4, 2, 8, 12, 12, generator=g) * 0.8 + 0.6
    rs, rv = orc.temporal_lif(x, None, 1.0, 0.0, 2.0)
    sp, v = ops.fused_temporal_lif_state.default(x.to(dev), z, 1.0, 0.0, 2.0, False)
    assert torch.equal(sp.cpu(), rs) and torch.equal(v.cpu(), rv)
    # linear + LIF, caller-owned outputs (the form the compiler emits)
    xl = (torch.rand(4, 96, 64, generator=g) < 0.2).float()
    w = torch.randn(48, 64, generator=g) * 0.3
    b = torch.randn(48, generator=g) * 0.1
    rls, rlv = orc.temporal_linear_lif(xl, w, b, None, 1.0, 0.0, 2.0)
    so = torch.empty(4, 96, 48, device=dev)
    vo = torch.empty(96, 48, device=dev)
    ops.fused_temporal_linear_lif_state_packed_out.default(xl.to(dev), w.to(dev), b.to(dev), z, 1.0, 0.0, 2.0, False, so, vo)
    check_parity(so, vo, rls, rlv, dtype, what="linear packed_out")
    # tail
    xt = torch.randn(4, 3, 32, 7, 7, generator=g) * 0.8 + 0.5
    fw = torch.randn(10, 32, generator=g) * 0.2
    fb = torch.randn(10, generator=g) * 0.1
    ro, rtv = orc.temporal_lif_avgpool_linear(xt, None, fw, fb, 1.0, 0.0, 2.0)
    out, tv = ops.fused_temporal_lif_avgpool_linear.default(xt.to(dev), z, fw.to(dev), fb.to(dev), 1.0, 0.0, 2.0, False)
    torch.testing.assert_close(out.cpu(), ro, rtol=1e-4, atol=1e-5)
    assert torch.equal(tv.cpu(), rtv)
    _no_fallback(ref_ops, 3)
    st = ref_ops.get_fused_op_call_stats()
    assert st["temporal_lif_triton"] == 1 and st["temporal_lif_avgpool_linear_triton"] == 1


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["eager", "executor"])
def test_cnn_small_fp32_through_the_reference_passes(ref_ops, mode):
    """CNN-small (fp32, T=4, batch 16, 3x32x32) compiled by the reference's passes: logits on the GPU (this
    library beneath the op layer, strict, no fallbacks) within 1e-4 of the same pipeline on the CPU, where the
    ops run the reference's eager loops."""
    ref_ops.configure_fused_op(backend="torch")
    cpu_outs, _, _, _ = _pipeline(ref_ops, "cnn_small", 4, 32, 16, torch.float32, "cpu", "eager")
    _strict(ref_ops)
    outs, report, executors, _ = _pipeline(ref_ops, "cnn_small", 4, 32, 16, torch.float32, "cuda", mode)
    for got, want in zip(outs, cpu_outs):
        torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-4)
    assert report.fused_nodes == {"fused_temporal_conv_lif_state": 3, "fused_temporal_lif_avgpool_linear": 1}
    if mode == "eager":
        _no_fallback(ref_ops, 8)   # 4 fused ops per forward, two forwards
    else:
        st = executors[0].stats
        assert st["fused_direct"] == 4 and st["fused_via_op_layer"] == 0 and st["cuda_graph"] and st["graph_replays"] == 2


@pytest.mark.gpu
def test_resnet18_bf16_executor_matches_the_op_layer_route(ref_ops):
    """Spiking ResNet-18 (bf16, T=4) through the reference's passes: this library's graph executor (direct
    backend calls, one CUDA graph, two different batches through the same captured graph) against the plain
    hand-off in which every fused op goes through the reference's op layer. With the neighbours left to ATen the
    two routes run the same kernels on the same values: identical logits. With pooling and the shortcut conv +
    BatchNorm lowered to this library's kernels the shortcut is folded in fp32 instead of two 16-bit ops, so
    spikes may differ from there on; that form is checked op by op below."""
    _strict(ref_ops)
    eager, _, _, _ = _pipeline(ref_ops, "resnet18", 4, 64, 2, torch.bfloat16, "cuda", "eager", gain=4.0, classes=100)
    _no_fallback(ref_ops, 34)
    plain, report, executors, _ = _pipeline(ref_ops, "resnet18", 4, 64, 2, torch.bfloat16, "cuda", "executor", gain=4.0,
                                            classes=100, lower_neighbours=False)
    st = executors[0].stats
    assert st["fused_direct"] == 17 and st["fused_via_op_layer"] == 0 and st["cuda_graph"] and st["graph_replays"] == 2
    assert not torch.equal(plain[0], plain[1])
    for a, b in zip(plain, eager):
        assert torch.equal(a, b)
    lowered, _, executors, _ = _pipeline(ref_ops, "resnet18", 4, 64, 2, torch.bfloat16, "cuda", "executor", gain=4.0,
                                         classes=100)
    st = executors[0].stats
    assert st["fused_direct"] == 17 and st["lowered_maxpool"] == 1 and st["lowered_conv_bn"] == 3 and st["cuda_graph"]
    assert all(torch.isfinite(o).all() for o in lowered) and not torch.equal(lowered[0], lowered[1])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_lowered_neighbours_match_aten(dtype):
    """The two lowerings of the graph executor on their own: max_pool2d(3, 2, 1) is exact; the shortcut conv +
    inference BatchNorm agrees with the two ATen ops to the rounding of the activation dtype."""
    import torch.nn.functional as F
    from triton_snn_fusion_b200 import fx_executor as fx
    g = torch.Generator().manual_seed(3)
    x = (torch.rand(8, 64, 28, 28, generator=g) < 0.3).to(dtype).cuda().contiguous(memory_format=torch.channels_last)
    assert torch.equal(fx._maxpool_3_2_1(x), F.max_pool2d(x, 3, 2, 1))
    w = (torch.randn(128, 64, 1, 1, generator=g) * 0.2).to(dtype).cuda()
    mean, var = (torch.randn(128, generator=g) * 0.1).to(dtype).cuda(), (torch.rand(128, generator=g) + 0.5).to(dtype).cuda()
    gamma, beta = (torch.rand(128, generator=g) + 0.5).to(dtype).cuda(), (torch.randn(128, generator=g) * 0.1).to(dtype).cuda()
    got = fx._guarded_shortcut(fx._FoldedShortcut())(x, w, [2, 2], [0, 0], mean, var, gamma, beta, 1e-5)
    cpu = lambda t: t.float().cpu()   # on the CPU: cuDNN would run the fp32 conv in TF32
    want = F.batch_norm(torch.conv2d(cpu(x), cpu(w), None, 2, 0), cpu(mean), cpu(var), cpu(gamma), cpu(beta), False, 0.0, 1e-5)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    torch.testing.assert_close(got.float().cpu(), want, rtol=tol, atol=tol)
    assert tuple(got.shape) == (8, 128, 14, 14)
