"""Binds this package beneath the reference's unchanged custom-op layer.

The reference's ``runtime/snn_custom_ops.py`` imports its five backend modules by name
(:9-25). ``install()`` registers this package's modules under those names in
``sys.modules`` before that file is imported, so the reference's op layer and FX rewrite
passes drive the sm_100a kernels with no change to their source:

    from triton_snn_fusion_b200.runtime.install import install
    install()                                   # before importing the reference
    import runtime.snn_custom_ops as ops        # the reference's own file
    ops.configure_fused_op(backend="triton", strict_triton=True)

The string "triton" is the reference's switch for "use the backend modules"
(runtime/snn_custom_ops.py:185); with ``strict_triton=True`` nothing falls back to its
eager loops.
"""
from __future__ import annotations

import importlib
import sys
import types

_NAMES = (
    "triton_convlif_backend",
    "triton_temporal_lif_backend",
    "triton_temporal_linear_lif_backend",
    "triton_temporal_lif_avgpool_linear_backend",
    "triton_temporal_lif_tail_backend",
)


def install(package: str = "runtime") -> None:
    """Register the backend modules as ``<package>.<name>``; the reference's own files keep
    resolving from its checkout for every other submodule of ``<package>``."""
    if "runtime.snn_custom_ops" in sys.modules and package == "runtime":
        raise RuntimeError("install() must run before the reference's runtime.snn_custom_ops is imported")
    for name in _NAMES:
        mod = importlib.import_module(f"{__package__}.{name}")
        sys.modules[f"{package}.{name}"] = mod
        parent = sys.modules.get(package)
        if isinstance(parent, types.ModuleType):
            setattr(parent, name, mod)
