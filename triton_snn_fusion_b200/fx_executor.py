"""Static executor for a rewritten FX graph: the role of the reference's
``runtime/fx_standalone_executor.py`` (:301-1260 in pengjh0111/triton-snn-fusion), built for this library.

Input is the ``GraphModule`` the reference's passes leave behind (``chronos.rewrite_graph``): calls of
``torch.ops.snn_custom.fused_temporal_*`` joined by ``getitem`` / ``flatten`` / ``chunk`` views and the few
ordinary ops the passes batch over time (max-pool, the strided 1x1 shortcut conv + BatchNorm of a residual
block, avgpool / flatten / linear of the head). The executor compiles the node list once into a flat plan:

  * every ``snn_custom`` fused op is bound straight to the backend function behind it (the same functions
    the op layer calls, runtime/snn_custom_ops.py:9-25), skipping the dispatcher and the op layer's
    bookkeeping on the hot path. Activations stay channels-last from layer to layer: the backends return
    channels-last stacks, ``stack[t]`` and ``flatten(0, 1)`` are views of them, and the next backend call
    recognises equally spaced views and reads them in place;
  * neighbours with a kernel in this library are lowered to it: ``max_pool2d(3, 2, 1)`` on a channels-last
    activation -> ``snnb_maxpool3x3s2``; a bias-free ``conv2d`` whose only user is an inference
    ``batch_norm`` -> one conv + bias launch with the BatchNorm folded the way the reference's own rewrite
    folds it (compiler/fx_lif_rewrite.py:340-353);
  * everything else runs as the node's own target;
  * the whole plan is captured into ONE CUDA graph over static input buffers (tensors that arrive at the
    same address on every call, i.e. the parameters Dynamo passes as graph inputs, are used in place; the
    others are copied into a static clone), so a forward pass is a copy of the batch plus one graph launch.
    Buffers come from the graph's private pool: the memory plan is fixed at capture.

Same calling convention as the reference's ``build_fx_standalone_backend`` (its :1263-1280): the returned
object is called with the graph's flat inputs and returns the graph's outputs; the returned tensors are
the executor's static buffers and are overwritten by the next call.
"""
from __future__ import annotations

import operator
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


def _map_nodes(value: Any, fn: Callable[[torch.fx.Node], Any]) -> Any:
    if isinstance(value, torch.fx.Node):
        return fn(value)
    if isinstance(value, (list, tuple)):
        out = [_map_nodes(v, fn) for v in value]
        return type(value)(out) if not hasattr(value, "_fields") else type(value)(*out)
    if isinstance(value, dict):
        return {k: _map_nodes(v, fn) for k, v in value.items()}
    if isinstance(value, slice):
        return slice(_map_nodes(value.start, fn), _map_nodes(value.stop, fn), _map_nodes(value.step, fn))
    return value


def _backend_table() -> Dict[str, Callable]:
    """op name -> callable(*op_args) -> op result, bound to this package's backend functions."""
    from .runtime import triton_convlif_backend as conv
    from .runtime import triton_temporal_lif_avgpool_linear_backend as tail
    from .runtime import triton_temporal_lif_backend as lif
    from .runtime import triton_temporal_linear_lif_backend as lin

    def pair(fn):
        def call(*a):
            r = fn(*a, strict=True)
            return r.spikes, r.v_next
        return call

    def tail_call(*a):
        r = tail.run_triton_fused_temporal_lif_avgpool_linear(*a, strict=True)
        return r.out_sum, r.v_next

    def conv_out(x_seq, w, b, v, s, p, d, g, th, vr, tau, det, spike_out, v_out):
        conv.run_triton_fused_temporal_conv_lif_state_packed_out(x_seq, w, b, v, s, p, d, g, th, vr, tau, det,
                                                                 spike_out, v_out, strict=True)
        return ()

    def lin_out(x_seq, w, b, v, th, vr, tau, det, spike_out, v_out):
        lin.run_triton_fused_temporal_linear_lif_state_packed_out(x_seq, w, b, v, th, vr, tau, det, spike_out, v_out,
                                                                  strict=True)
        return ()

    def batched_tn(fn):
        def call(*a):
            s, v = fn(*a)
            return torch.flatten(s, 0, 1), v
        return call

    t = {
        "fused_conv_lif_state": pair(conv.run_triton_fused_conv_lif_state),
        "fused_temporal_conv_lif_state": pair(conv.run_triton_fused_temporal_conv_lif_state),
        "fused_temporal_pointwise_conv_lif_state": pair(conv.run_triton_fused_temporal_pointwise_conv_lif_state),
        "fused_temporal_depthwise_conv_lif_state": pair(conv.run_triton_fused_temporal_depthwise_conv_lif_state),
        "fused_temporal_conv_lif_state_depthwise": pair(conv.run_triton_fused_temporal_depthwise_conv_lif_state),
        "fused_temporal_conv_add_lif_state": pair(conv.run_triton_fused_temporal_conv_add_lif_state),
        "fused_temporal_conv_add_lif_state_depthwise": pair(conv.run_triton_fused_temporal_conv_add_lif_state),
        "fused_temporal_conv_lif_state_packed_out": conv_out,
        "fused_temporal_lif_state": pair(lif.run_triton_fused_temporal_lif_state),
        "fused_temporal_lif_avgpool_linear": tail_call,
        "fused_temporal_lif_tail": tail_call,
        "fused_temporal_linear_lif_state": pair(lin.run_triton_fused_temporal_linear_lif_state),
        "fused_temporal_linear_lif_state_packed": pair(lin.run_triton_fused_temporal_linear_lif_state_packed),
        "fused_temporal_linear_lif_state_packed_out": lin_out,
    }
    t["fused_temporal_conv_lif_state_batched_tn"] = batched_tn(t["fused_temporal_conv_lif_state"])
    t["fused_temporal_conv_add_lif_state_batched_tn"] = batched_tn(t["fused_temporal_conv_add_lif_state"])
    return t


def _snn_op_name(node: torch.fx.Node) -> Optional[str]:
    if node.op != "call_function":
        return None
    text = str(node.target)
    if not text.startswith("snn_custom."):
        return None
    return text.split(".")[1]


def _is_target(node: torch.fx.Node, *fns) -> bool:
    return node.op == "call_function" and any(node.target is f for f in fns)


class _FoldedShortcut:
    """conv2d (no bias) + inference batch_norm as one conv + bias launch; the fold is redone when a parameter
    tensor is replaced or modified in place."""

    def __init__(self):
        self.key = None
        self.w = self.b = None

    def __call__(self, x, w, stride, padding, mean, var, gamma, beta, eps):
        from .runtime import triton_convlif_backend as conv
        key = tuple((t.data_ptr(), t._version) for t in (w, mean, var, gamma, beta))
        if key != self.key:
            scale = gamma.float() / torch.sqrt(var.float() + float(eps))
            self.w = (w.float() * scale.reshape(-1, 1, 1, 1)).to(w.dtype).contiguous(memory_format=torch.channels_last)
            self.b = ((torch.zeros_like(mean, dtype=torch.float32) - mean.float()) * scale + beta.float()).to(w.dtype)
            self.key = key
        # the passes hand over flatten(0, 1) of a spike stack: its T*B frames are one large batch here
        return conv.conv_bias_only([x], self.w, self.b, stride, padding)[0]


class GraphExecutor:
    """Compiled plan of one rewritten ``GraphModule`` (see the module docstring).

    ``direct_backends`` / ``lower_neighbours`` / ``use_cuda_graph`` can be switched off one by one: with all
    three off the executor is a plain interpreter of the graph (usable on CPU tensors, where the fused ops
    fall through the reference's op layer to its eager loops). ``stats`` says what the plan contains.
    """

    def __init__(self, gm: torch.fx.GraphModule, *, use_cuda_graph: bool = True, example_inputs: Optional[Sequence] = None,
                 direct_backends: Optional[bool] = None, lower_neighbours: bool = True, warmup: int = 2):
        self.gm = gm
        self.use_cuda_graph = bool(use_cuda_graph)
        self.warmup = int(warmup)
        self.nodes = list(gm.graph.nodes)
        self.placeholders = [n for n in self.nodes if n.op == "placeholder"]
        self.output_node = next(n for n in self.nodes if n.op == "output")
        self.stats = {"fused_direct": 0, "fused_via_op_layer": 0, "lowered_maxpool": 0, "lowered_conv_bn": 0,
                      "generic": 0, "cuda_graph": False, "graph_replays": 0, "static_inputs_copied": 0}
        self._steps: List[Tuple[int, Callable, Any, Any]] = []   # (slot, fn, args, kwargs) with nodes replaced by slots
        self._slot: Dict[torch.fx.Node, int] = {}
        self._const: Dict[int, Any] = {}
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self._static_in: Optional[List[Any]] = None
        self._static_out: Any = None
        if direct_backends is None:   # the backends are GPU code: bind them when the graph is going to see GPU tensors
            direct_backends = example_inputs is None or any(isinstance(v, torch.Tensor) and v.is_cuda
                                                            for v in example_inputs)
        self._compile(bool(direct_backends), lower_neighbours)
        if example_inputs is not None and self.use_cuda_graph and any(
                isinstance(v, torch.Tensor) and v.is_cuda for v in example_inputs):
            self._capture(tuple(example_inputs))

    # ------------------------------------------------------------------ plan ----
    def _compile(self, direct: bool, lower: bool) -> None:
        table = _backend_table() if direct else {}
        for i, n in enumerate(self.nodes):
            self._slot[n] = i
        skip = set()
        for n in self.nodes:
            if n in skip or n.op in ("placeholder", "output"):
                continue
            if n.op == "get_attr":
                obj = self.gm
                for part in str(n.target).split("."):
                    obj = getattr(obj, part)
                self._const[self._slot[n]] = obj
                continue
            name = _snn_op_name(n)
            if name is not None:
                if name in table:
                    self._add(n, table[name], n.args, n.kwargs)
                    self.stats["fused_direct"] += 1
                else:
                    self._add(n, n.target, n.args, n.kwargs)
                    self.stats["fused_via_op_layer"] += 1
                continue
            if lower and self._try_lower(n, skip):
                continue
            if n.op == "call_function":
                self._add(n, n.target, n.args, n.kwargs)
            elif n.op == "call_method":
                self._add(n, _method(str(n.target)), n.args, n.kwargs)
            elif n.op == "call_module":
                self._add(n, self.gm.get_submodule(str(n.target)), n.args, n.kwargs)
            else:
                raise RuntimeError(f"GraphExecutor: unsupported node kind {n.op}")
            if n.target is not operator.getitem:
                self.stats["generic"] += 1

    def _add(self, node, fn, args, kwargs) -> None:
        ref = lambda m: _SlotRef(self._slot[m])   # noqa: E731
        self._steps.append((self._slot[node], fn, _map_nodes(tuple(args), ref), _map_nodes(dict(kwargs), ref)))

    def _try_lower(self, n: torch.fx.Node, skip: set) -> bool:
        # max_pool2d(x, 3, 2, 1): this library's channels-last pooling kernel
        if _is_target(n, F.max_pool2d, torch.max_pool2d):
            if _pool_args(n) is not None:
                self._add(n, _maxpool_3_2_1, (n.args[0],), {})
                self.stats["lowered_maxpool"] += 1
                return True
        # conv2d(x, w, None, stride, padding, (1,1), 1) -> batch_norm(eval), conv used by nothing else
        if _is_target(n, torch.conv2d, F.conv2d) and len(n.users) == 1:
            bn = next(iter(n.users))
            if _is_target(bn, F.batch_norm, torch.batch_norm) and bn.args and bn.args[0] is n:
                ca = _conv_args(n)
                ba = _bn_args(bn)
                # the fused step is emitted where the conv stands and stored as the batch_norm node's value, so
                # the BatchNorm's other inputs have to be known by then (they are parameters: graph inputs)
                early = ba is not None and all(not isinstance(v, torch.fx.Node) or self._slot[v] < self._slot[n]
                                               for v in ba)
                if ca is not None and early:
                    x, w, stride, padding = ca
                    mean, var, gamma, beta, eps = ba
                    self._add(bn, _guarded_shortcut(_FoldedShortcut()), (x, w, stride, padding, mean, var, gamma, beta, eps), {})
                    skip.add(bn)
                    self.stats["lowered_conv_bn"] += 1
                    return True
        return False

    # ------------------------------------------------------------------- run ----
    def _run_plan(self, inputs: Sequence[Any]) -> Any:
        env: List[Any] = [None] * len(self.nodes)
        for slot, v in self._const.items():
            env[slot] = v
        for n, v in zip(self.placeholders, inputs):
            env[self._slot[n]] = v
        get = lambda r: env[r.slot]   # noqa: E731
        for slot, fn, args, kwargs in self._steps:
            env[slot] = fn(*_map_refs(args, get), **_map_refs(kwargs, get))
        return _map_nodes(self.output_node.args[0], lambda m: env[self._slot[m]])

    def _capture(self, example_inputs: Tuple[Any, ...]) -> None:
        dev = next(v.device for v in example_inputs if isinstance(v, torch.Tensor) and v.is_cuda)
        # parameters and buffers arrive at the same address on every call and are used where they are; the rest
        # (the batch) gets a static clone that every call copies into
        self._static_in = [v.clone() if (isinstance(v, torch.Tensor) and not isinstance(v, torch.nn.Parameter)
                                         and not _looks_persistent(n)) else v
                           for n, v in zip(self.placeholders, example_inputs)]
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(max(1, self.warmup)):   # fills the weight caches of the backends before capture
                self._run_plan(self._static_in)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        g = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(g):
            self._static_out = self._run_plan(self._static_in)
        self._graph = g
        self.stats["cuda_graph"] = True

    def __call__(self, *inputs: Any) -> Any:
        if self._graph is None:
            if self.use_cuda_graph and any(isinstance(v, torch.Tensor) and v.is_cuda for v in inputs):
                self._capture(tuple(inputs))
            else:
                with torch.no_grad():
                    return self._run_plan(inputs)
        for dst, src in zip(self._static_in, inputs):
            if isinstance(dst, torch.Tensor) and isinstance(src, torch.Tensor) and dst.data_ptr() != src.data_ptr():
                dst.copy_(src, non_blocking=True)
                self.stats["static_inputs_copied"] += 1
        self._graph.replay()
        self.stats["graph_replays"] += 1
        return self._static_out


class _SlotRef:
    __slots__ = ("slot",)

    def __init__(self, slot: int):
        self.slot = slot


def _map_refs(value: Any, get: Callable) -> Any:
    if isinstance(value, _SlotRef):
        return get(value)
    if isinstance(value, tuple):
        return tuple(_map_refs(v, get) for v in value)
    if isinstance(value, list):
        return [_map_refs(v, get) for v in value]
    if isinstance(value, dict):
        return {k: _map_refs(v, get) for k, v in value.items()}
    if isinstance(value, slice):
        return slice(_map_refs(value.start, get), _map_refs(value.stop, get), _map_refs(value.step, get))
    return value


def _method(name: str) -> Callable:
    def call(self_, *a, **k):
        return getattr(self_, name)(*a, **k)
    return call


def _looks_persistent(node: torch.fx.Node) -> bool:
    """Dynamo names the graph inputs that are module parameters / buffers after their attribute path."""
    text = node.name.lower()
    return "parameters" in text or "buffers" in text or text.startswith("l_self_") or text.startswith("_fx_")


def _pool_args(n: torch.fx.Node):
    a = list(n.args) + [None] * 6
    kw = n.kwargs
    k = kw.get("kernel_size", a[1])
    s = kw.get("stride", a[2])
    p = kw.get("padding", a[3])
    d = kw.get("dilation", a[4])
    ceil = kw.get("ceil_mode", a[5])
    ret_idx = kw.get("return_indices", a[6] if len(n.args) > 6 else False)
    norm = lambda v: tuple(v) if isinstance(v, (list, tuple)) else (v, v)   # noqa: E731
    if norm(k) != (3, 3) or norm(s) != (2, 2) or norm(p) != (1, 1):
        return None
    if d not in (None, 1, (1, 1), [1, 1]) or ceil or ret_idx:
        return None
    return True


def _maxpool_3_2_1(x: torch.Tensor) -> torch.Tensor:
    from . import _lib
    from .runtime._common import empty_nhwc, is_nhwc_dense
    if not (x.is_cuda and x.dim() == 4 and x.dtype in (torch.float32, torch.bfloat16, torch.float16) and is_nhwc_dense(x)):
        return F.max_pool2d(x, 3, 2, 1)
    n, c, h, w = (int(d) for d in x.shape)
    out = empty_nhwc([n, c, (h - 1) // 2 + 1, (w - 1) // 2 + 1], x.dtype, x.device)
    _lib.check(_lib.lib.snnb_maxpool3x3s2(_lib.ptr(x), _lib.ptr(out), n, h, w, c, _lib.dtype_code(x.dtype),
                                          _lib.current_stream(x.device)), "snnb_maxpool3x3s2")
    return out


def _conv_args(n: torch.fx.Node):
    a = list(n.args) + [None] * 7
    kw = n.kwargs
    x, w = a[0], a[1]
    bias = kw.get("bias", a[2])
    stride = kw.get("stride", a[3] if a[3] is not None else 1)
    padding = kw.get("padding", a[4] if a[4] is not None else 0)
    dilation = kw.get("dilation", a[5] if a[5] is not None else 1)
    groups = kw.get("groups", a[6] if a[6] is not None else 1)
    norm = lambda v: tuple(v) if isinstance(v, (list, tuple)) else (v, v)   # noqa: E731
    if bias is not None or groups != 1 or norm(dilation) != (1, 1) or isinstance(padding, str):
        return None
    if norm(stride)[0] != norm(stride)[1] or norm(padding)[0] != norm(padding)[1]:
        return None
    return x, w, list(norm(stride)), list(norm(padding))


def _bn_args(n: torch.fx.Node):
    # F.batch_norm(input, running_mean, running_var, weight, bias, training, momentum, eps)
    a = list(n.args) + [None] * 8
    kw = n.kwargs
    mean, var = a[1], a[2]
    gamma = kw.get("weight", a[3])
    beta = kw.get("bias", a[4])
    training = kw.get("training", a[5] if a[5] is not None else False)
    eps = kw.get("eps", a[7] if a[7] is not None else 1e-5)
    if training or any(v is None for v in (mean, var, gamma, beta)):
        return None
    return mean, var, gamma, beta, eps


def _guarded_shortcut(folded: _FoldedShortcut) -> Callable:
    def call(x, w, stride, padding, mean, var, gamma, beta, eps):
        from .runtime._common import is_nhwc_dense
        ok = (x.is_cuda and x.dim() == 4 and x.dtype in (torch.float32, torch.bfloat16, torch.float16)
              and w.dtype == x.dtype and is_nhwc_dense(x))
        if not ok:
            return F.batch_norm(torch.conv2d(x, w, None, stride, padding), mean, var, gamma, beta, False, 0.0, eps)
        return folded(x, w, stride, padding, mean, var, gamma, beta, eps)
    return call


def build_fx_standalone_backend(gm: torch.fx.GraphModule, *, num_streams: int = 1, use_cuda_graph: bool = False,
                                example_inputs: Optional[Tuple[Any, ...]] = None, debug: bool = False,
                                schedule_policy: str = "topo", **options) -> GraphExecutor:
    """Same signature as the reference's function of this name (runtime/fx_standalone_executor.py:1263-1280).
    ``num_streams`` and ``schedule_policy`` are accepted for compatibility: inside one CUDA graph the kernels of
    this library each fill the GPU, so the plan is a single stream in graph order."""
    ex = GraphExecutor(gm, use_cuda_graph=use_cuda_graph, example_inputs=example_inputs, **options)
    if debug:
        print(f"[SNNB200][FX_EXECUTOR] {ex.stats}")
    return ex


def make_fx_standalone_torch_compile_backend(*, num_streams: int = 1, use_cuda_graph: bool = False, debug: bool = False,
                                             schedule_policy: str = "topo", **options) -> Callable:
    """``torch.compile`` backend that hands Dynamo's graph to a ``GraphExecutor`` as it is (reference :1283-1300)."""
    def backend(gm: torch.fx.GraphModule, example_inputs, **_kwargs):
        return build_fx_standalone_backend(gm, num_streams=num_streams, use_cuda_graph=use_cuda_graph,
                                           example_inputs=tuple(example_inputs), debug=debug,
                                           schedule_policy=schedule_policy, **options)
    return backend
