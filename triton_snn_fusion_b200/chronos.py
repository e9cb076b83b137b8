"""Drives the reference's own FX rewrite passes and hands the rewritten graph to this package.

The reference compiles a single-step spiking model looped T times by letting Dynamo capture the
unrolled graph and running its passes over it inside a custom ``torch.compile`` backend
(``make_rewrite_backend``, benchmarks/validate_chronos_baselines.py:868-1261 in
pengjh0111/triton-snn-fusion). That driver lives in a benchmark script which cannot be imported
outside the reference's own environment (it needs SpikingJelly and a ``test`` package), so this
module applies the same passes in the same order:

    annotate -> collect conv-BN-LIF patterns -> temporal schedule -> temporal rewrites
    (conv-BN-LIF, conv-BN-add-LIF, linear-LIF, LIF-avgpool-linear, standalone LIF) -> single-step
    rewrites -> spatial batching -> canonicalisation

Every pass is the reference's, imported from the user's checkout of its ``compiler`` package; nothing
of it is reimplemented here. The rewritten ``GraphModule`` calls ``torch.ops.snn_custom.*``; with
``runtime.install.install()`` in effect those ops run this package's kernels. Hand-off modes:

    "eager"     the rewritten ``gm.forward`` (every fused op goes through the reference's op layer)
    "executor"  ``fx_executor.GraphExecutor``: this package's static executor (one CUDA graph)
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch

SPATIAL_OPS = ("conv", "bn", "add", "maxpool", "avgpool", "flatten", "linear")


@dataclass
class RewriteReport:
    """What the passes did to one captured graph."""
    graphs: int = 0
    fused_nodes: Dict[str, int] = field(default_factory=dict)   # op name -> number of call sites
    lif_nodes_left: int = 0
    log: List[str] = field(default_factory=list)


def count_snn_ops(gm: torch.fx.GraphModule) -> Dict[str, int]:
    out: Dict[str, int] = {}
    for n in gm.graph.nodes:
        if n.op == "call_function" and str(n.target).startswith("snn_custom."):
            name = str(n.target).split(".")[1]
            out[name] = out.get(name, 0) + 1
    return out


def rewrite_graph(gm: torch.fx.GraphModule, example_inputs: Sequence, T: int, window: Optional[int] = None,
                  spatial_batching: bool = True, max_patterns: int = 1_000_000,
                  report: Optional[RewriteReport] = None) -> torch.fx.GraphModule:
    """Applies the reference's passes to ``gm`` in place, in the reference's order, with the options of its
    full validation run (run_full_validation.sh:142-166: temporal rewrite, temporal schedule and spatial
    batching on, window = T unless given)."""
    from compiler import fx_lif_rewrite as single
    from compiler import fx_lif_temporal_rewrite as tr
    from compiler.fx_spatial_batching import apply_spatial_batching
    from compiler.fx_temporal_annotation import annotate_temporal_metadata
    from compiler.fx_temporal_scheduler import reorder_fx_graph_by_temporal_windows
    from compiler.fx_temporal_spatial_canonicalize import canonicalize_temporal_spatial_ir

    W = int(window or T)
    placeholders = [n for n in gm.graph.nodes if n.op == "placeholder"]
    values = dict(zip(placeholders, example_inputs))
    log: List[str] = []
    annotate_temporal_metadata(gm, W, T, strict=False)
    patterns = tr.collect_conv_bn_lif_state_patterns(gm)
    if patterns:
        sched = reorder_fx_graph_by_temporal_windows(gm, T, W, patterns, dump_dir=None, strict=False)
        if sched.ok:
            patterns = tr.collect_conv_bn_lif_state_patterns(gm)
        else:
            log.append(f"schedule: {sched.reason}")
    done = 0
    if W > 1:
        windows = tr.make_temporal_windows(tr.group_temporal_patterns(patterns), W, False)
        st = tr.rewrite_temporal_conv_bn_lif_state_to_fused(gm, windows, values, max_patterns)
        done += st.temporal_replaced_patterns
        log.extend(st.log)
        res = tr.collect_conv_bn_add_lif_state_patterns(gm)
        res_windows = tr.make_temporal_residual_windows(tr.group_temporal_residual_patterns(res), W, False)
        if res_windows:
            st = tr.rewrite_temporal_conv_bn_add_lif_state_to_fused(gm, res_windows, values, max(0, max_patterns - done))
            done += st.temporal_residual_replaced_patterns
            log.extend(st.log)
        lin = tr.collect_temporal_linear_lif_state_patterns(gm)
        lin_windows = tr.make_temporal_linear_lif_windows(tr.group_temporal_linear_lif_patterns(lin), W, False)
        if lin_windows:
            st = tr.rewrite_temporal_linear_lif_state_to_fused(gm, lin_windows, max(0, max_patterns - done))
            done += st.temporal_linear_lif_replaced_patterns
            log.extend(st.log)
        tail = tr.collect_temporal_lif_avgpool_linear_patterns(gm)
        tail_windows = tr.make_temporal_lif_avgpool_linear_windows(tr.group_temporal_lif_avgpool_linear_patterns(tail), W, False)
        if tail_windows:
            st = tr.rewrite_temporal_lif_avgpool_linear_to_fused(gm, tail_windows, max(0, max_patterns - done))
            done += st.temporal_lif_avgpool_linear_replaced_patterns
            log.extend(st.log)
        lif = tr.collect_standalone_lif_state_patterns(gm)
        lif_windows = tr.make_temporal_lif_windows(tr.group_temporal_lif_patterns(lif), W, False)
        if lif_windows:
            st = tr.rewrite_temporal_lif_state_to_fused(gm, lif_windows, max(0, max_patterns - done))
            done += st.temporal_lif_replaced_patterns
            log.extend(st.log)
    direct = single.match_conv_lif_state(gm)
    conv_bn = single.match_conv_bn_lif_state(gm)
    remaining = max(0, max_patterns - done)
    n_bn = single.rewrite_conv_bn_lif_state_to_fused(gm, conv_bn, values, remaining)
    single.rewrite_conv_lif_state_to_fused(gm, direct, values, max(0, remaining - n_bn))
    if spatial_batching:
        try:
            apply_spatial_batching(gm, W, list(SPATIAL_OPS), dump_dir=None, strict=False, enable_chain=False)
        except Exception as exc:   # the reference continues with the graph as it is (its :1174-1176)
            log.append(f"spatial batching skipped: {type(exc).__name__}: {exc}")
    canonicalize_temporal_spatial_ir(gm, dump_dir=None, strict=False, rewrite_temporal_mean=False,
                                     drop_intermediate_states=False)
    gm.graph.lint()
    gm.recompile()
    if report is not None:
        report.graphs += 1
        for k, v in count_snn_ops(gm).items():
            report.fused_nodes[k] = report.fused_nodes.get(k, 0) + v
        report.lif_nodes_left += single.count_lif_state_nodes(gm)
        report.log.extend(log)
    return gm


def make_backend(T: int, window: Optional[int] = None, mode: str = "executor", spatial_batching: bool = True,
                 use_cuda_graph: bool = True, report: Optional[RewriteReport] = None) -> Callable:
    """A ``torch.compile`` backend: the reference's passes, then ``mode`` ("eager" | "executor")."""
    if mode not in ("eager", "executor"):
        raise ValueError(f"mode must be 'eager' or 'executor', got {mode!r}")

    def backend(gm: torch.fx.GraphModule, example_inputs, **_kwargs):
        rewrite_graph(gm, example_inputs, T, window, spatial_batching, report=report)
        if mode == "eager":
            return gm.forward
        from .fx_executor import build_fx_standalone_backend
        return build_fx_standalone_backend(gm, use_cuda_graph=use_cuda_graph, example_inputs=tuple(example_inputs))

    return backend
