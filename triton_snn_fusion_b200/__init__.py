"""B200 (sm_100a) fused temporal kernels for spiking neural networks.

A from-scratch CUDA implementation of the fused temporal hot path of
pengjh0111/triton-snn-fusion: LIF scan, conv/linear + folded BN + LIF over all T
timesteps, depthwise conv + LIF and the LIF -> avgpool -> linear tail, behind the C ABI
of ``include/snnb200.h`` and a Python mirror of the reference's backend modules
(``triton_snn_fusion_b200.runtime``). There is no CPU path: every backend module loads
``libsnnb200.so`` through ``_lib`` and raises if it has not been built
(``python -m triton_snn_fusion_b200.build``).
"""
import importlib

__version__ = "0.1.0"


def __getattr__(name):
    # ``_lib`` is resolved on first use so that the build module can be run before the
    # shared library exists.
    if name == "_lib":
        return importlib.import_module(__name__ + "._lib")
    raise AttributeError(name)
