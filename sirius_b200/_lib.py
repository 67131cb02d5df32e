"""ctypes binding of libsirius_b200.so (the C ABI declared in include/sirius_b200.h).

There is no fallback: if the shared library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_PKG = Path(__file__).resolve().parent
# SIRIUS_B200_LIB selects another build of the same sources, e.g. the ThreadSanitizer build of the host runtime
# (`python -m sirius_b200._build --tsan`); unset, the in-tree library is the only one ever loaded.
LIB_PATH = Path(os.environ.get("SIRIUS_B200_LIB") or _PKG / "libsirius_b200.so")

SRT_F32, SRT_BF16 = 0, 1
IMPL_AUTO, IMPL_SIMT, IMPL_TCGEN05 = 0, 1, 2


class SrtError(RuntimeError):
    pass


class ConvDesc(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("N", "H", "W", "C", "K", "R", "S", "stride", "pad", "P", "Q")]

    @classmethod
    def make(cls, N, H, W, Cin, K, R, S, stride, pad):
        P = (H + 2 * pad - R) // stride + 1
        Q = (W + 2 * pad - S) // stride + 1
        return cls(N, H, W, Cin, K, R, S, stride, pad, P, Q)


class ConvEpilogue(C.Structure):
    _fields_ = [("bias", C.c_void_p), ("addend", C.c_void_p), ("addend_bits", C.c_void_p)]


_vp, _i, _i64, _f, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t
_PD = C.POINTER(ConvDesc)
_PE = C.POINTER(ConvEpilogue)

# name -> (restype, argtypes); restype None means "int status"
_SIGNATURES = {
    "srt_last_error": (C.c_char_p, []),
    "srt_version": (C.c_char_p, []),
    "srt_conv_fprop": (None, [_PD, _i, _i, _vp, _vp, _vp, _PE, _vp]),
    "srt_conv_fprop_bn_stats": (None, [_PD, _i, _i, _vp, _vp, _vp, _PE, _vp, _sz, C.POINTER(C.c_int), _vp]),
    "srt_conv_fprop_bn_stats_bytes": (_sz, [_PD]),
    "srt_conv_fprop_bn_stats_supported": (_i, [_PD, _i, _i]),
    "srt_bn_finalize": (None, [_vp, _i, _i, _i64, _vp, _vp, _f, _f, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "srt_conv_dgrad": (None, [_PD, _i, _i, _vp, _vp, _vp, _PE, _vp]),
    "srt_conv_wgrad": (None, [_PD, _i, _i, _vp, _vp, _vp, _vp, _sz, _vp]),
    "srt_conv_wgrad_scratch_bytes": (_sz, [_PD, _i, _i]),
    "srt_conv_filter_transpose": (None, [_PD, _i, _vp, _vp, _vp]),
    "srt_bn_stats": (None, [_i, _vp, _i64, _i, _vp, _vp, _f, _f, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "srt_bn_scratch_bytes": (_sz, [_i64, _i]),
    "srt_bn_stats_static": (None, [_i, _vp, _i64, _i, _vp, _vp, _f, _f, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "srt_bn_apply": (None, [_i, _vp, _vp, _vp, _i64, _i, _vp, _vp, _i, _vp]),
    "srt_bn_apply_bits": (None, [_i, _vp, _vp, _vp, _i64, _i, _vp, _vp, _vp, _vp]),
    "srt_bn_backward_bits": (None, [_i, _vp, _vp, _vp, _i64, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _vp]),
    "srt_bn_backward": (None, [_i, _vp, _vp, _vp, _i64, _i, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "srt_bn_fused_fits": (_i, [_i, _i64, _i, _i]),
    "srt_bn_forward_fused": (None, [_i, _vp, _vp, _vp, _i64, _i, _vp, _vp, _f, _f, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp]),
    "srt_bn_backward_fused": (None, [_i, _vp, _vp, _vp, _i64, _i, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp]),
    "srt_maxpool3x3s2_fwd": (None, [_i, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "srt_maxpool3x3s2_bwd": (None, [_i, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "srt_avgpool_fwd": (None, [_i, _vp, _vp, _i, _i, _i, _vp]),
    "srt_avgpool_bwd": (None, [_i, _vp, _vp, _i, _i, _i, _vp]),
    "srt_softmax_ce": (None, [_i, _vp, _vp, _i, _i, _f, _vp, _vp, _vp]),
    "srt_sum_f32": (None, [_vp, _i, _vp, _i, _vp]),
    "srt_colsum": (None, [_i, _vp, _i64, _i, _vp, _vp]),
    "srt_sgd_momentum": (None, [_vp, _vp, _vp, _vp, _i64, _f, _f, _f, _i, _vp]),
    "srt_adamw": (None, [_vp, _vp, _vp, _vp, _vp, _i64, _f, _f, _f, _f, _f, _i, _vp]),
    "srt_grad_accumulate": (None, [_vp, _vp, _i64, _vp]),
    "srt_nchw_to_nhwc": (None, [_i, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "srt_cast_f32_to_bf16": (None, [_vp, _vp, _i64, _vp]),
    "srt_cast_bf16_to_f32": (None, [_vp, _vp, _i64, _vp]),
    "srt_set_sm_mask": (None, [C.POINTER(C.c_uint64)]),
    "srt_get_sm_mask": (None, [C.POINTER(C.c_uint64)]),
    "srt_tc_status": (None, [C.POINTER(C.c_int)]),
    "srt_conv_plan_override": (None, [_i, _i, _i]),
    "srt_conv_wgrad_pairs": (_i, [_i]),
    "srt_bn_static_prepare": (None, []),
}

_lib = None


def declared_symbols() -> list[str]:
    return sorted(_SIGNATURES)


def register(sigs: dict) -> None:
    """Other modules of the package add the signatures of their entry points here."""
    _SIGNATURES.update(sigs)
    global _lib
    if _lib is not None:
        _bind(_lib, sigs)


def _bind(lib, sigs) -> None:
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)
        fn.restype = C.c_int if res is None else res
        fn.argtypes = args


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise SrtError(
                f"{LIB_PATH} is missing: build it with `python -m sirius_b200._build` "
                "(there is no CPU or PyTorch fallback)")
        l = C.CDLL(str(LIB_PATH))
        _bind(l, _SIGNATURES)
        _lib = l
    return _lib


def check(status: int, what: str = "") -> None:
    if status != 0:
        msg = lib().srt_last_error().decode(errors="replace")
        raise SrtError(f"{what or 'sirius_b200 call'} failed with status {status}: {msg}")


def call(name: str, *args) -> None:
    check(getattr(lib(), name)(*args), name)
