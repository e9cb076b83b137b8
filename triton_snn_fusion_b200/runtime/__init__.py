"""Host-side mirror of the reference's backend modules.

The module and function names are the ones the reference's custom-op layer
imports (runtime/snn_custom_ops.py:9-25 in pengjh0111/triton-snn-fusion), so that
layer can bind to this package unchanged (see ``install``); behind them are the
sm_100a CUDA kernels of libsnnb200.so, reached through its C ABI.
"""
