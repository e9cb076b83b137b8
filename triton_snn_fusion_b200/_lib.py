"""ctypes binding of libsnnb200.so (the C ABI declared in include/snnb200.h).

There is no CPU implementation behind these calls and no fallback: if the
library has not been built the import of this module raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p, POINTER
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "libsnnb200.so"

SNNB_OK = 0
F32, BF16, F16, U8, B1 = 0, 1, 2, 3, 4   # B1: spikes packed one bit each along the channel axis
NCHW, NHWC = 0, 1
PATH_AUTO, PATH_SIMT, PATH_TCGEN05, PATH_TCGEN05_TAPS, PATH_TCGEN05_HALO = 0, 1, 2, 3, 4

_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16, torch.uint8: U8}

# name -> (restype, argtypes); every symbol declared in include/snnb200.h
SIGNATURES = {
    "snnb_version": (c_int, []),
    "snnb_last_error": (c_char_p, []),
    "snnb_device_status": (c_int, [POINTER(c_int)]),
    "snnb_selftest_arm_wait_timeout": (c_int, [c_int64]),
    "snnb_probe_mma_cycles": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "snnb_lif_scan": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_int,
                              c_float, c_float, c_float, c_void_p]),
    "snnb_lif_avgpool_linear": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                        c_float, c_float, c_float, c_void_p]),
    "snnb_dwconv3x3_lif": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                   c_float, c_float, c_float, c_void_p]),
    "snnb_conv_lif": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                              c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                              c_int, c_int, c_int, c_float, c_float, c_float, c_int, c_void_p]),
    "snnb_conv_lif_which": (c_int, [c_int] * 15 + [c_char_p, c_int]),
    "snnb_linear_lif": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                c_float, c_float, c_float, c_int, c_void_p]),
    "snnb_stem7x7_scratch_bytes": (c_int64, [c_int, c_int, c_int]),
    "snnb_stem7x7_pack_weight": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "snnb_stem7x7_lif": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                 c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                 c_float, c_float, c_float, c_void_p]),
    "snnb_stem7x7_static_scratch_bytes": (c_int64, []),
    "snnb_stem7x7_lif_static": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                        c_float, c_float, c_float, c_void_p]),
    "snnb_nchw_to_nhwc": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]),
    "snnb_nhwc_to_nchw": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]),
    "snnb_maxpool3x3s2": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p]),
    "snnb_conv3x3_shortcut_lif": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
                                          c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                          c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                          c_float, c_float, c_float, c_void_p]),
    "snnb_maxpool3x3s2_u8": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p]),
    "snnb_maxpool3x3s2_bits": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p]),
    "snnb_avgpool_linear_mean": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
}


def _load() -> ctypes.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m triton_snn_fusion_b200.build` "
            "(there is no CPU fallback for the fused kernels)"
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the build lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


class SnnbError(RuntimeError):
    pass


def check(status: int, what: str) -> None:
    if status != SNNB_OK:
        msg = lib.snnb_last_error().decode("utf-8", "replace")
        raise SnnbError(f"{what} failed (status {status}): {msg}")


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dt]
    except KeyError:
        raise SnnbError(f"unsupported dtype {dt}") from None


def ptr(t) -> int | None:
    """Device address of a tensor (None -> NULL)."""
    if t is None:
        return None
    return t.data_ptr()


def current_stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def conv_kernel_name(T, B, Cin, H, W, Cout, k, stride, pad, dtype, lif=True, one_frame=False, residual=False,
                     path=PATH_AUTO) -> str:
    """Which kernel snnb_conv_lif would run for this shape (no launch)."""
    buf = ctypes.create_string_buffer(64)
    check(lib.snnb_conv_lif_which(T, B, Cin, H, W, Cout, k, k, stride, pad, int(lif), dtype_code(dtype), int(one_frame),
                                  int(residual), path, buf, 64), "snnb_conv_lif_which")
    return buf.value.decode()


def device_status() -> int:
    out = c_int(0)
    check(lib.snnb_device_status(ctypes.byref(out)), "snnb_device_status")
    return out.value
