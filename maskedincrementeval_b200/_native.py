"""ctypes binding of libmie.so (the C ABI declared in ``include/mie.h``).

There is no fallback: if the shared library is missing or a symbol is absent the import of this
module raises, and every operator of the package fails with it.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmie.so")

OK, EINVAL, EALIGN, EUNSUPPORTED, ECUDA, ETOOBIG = 0, -1, -2, -3, -4, -5
ACT_NONE, ACT_RELU, ACT_SIGMOID, ACT_TANH = 0, 1, 2, 3
UP_BILINEAR, UP_NEAREST = 0, 1
ERR_BAD_TILE, ERR_WAIT_EXPIRED = 1, 2
OPT_TC_THRESHOLDED, OPT_TC_SPIN_LIMIT, OPT_TC_WITHHOLD_LOADS, OPT_LAUNCH_COUNT, OPT_TC_KSPLIT, OPT_TC_OWN_KERNELS = 1, 2, 3, 4, 5, 6
TAIL_MAX_TILES = 2048     # MIE_TAIL_MAX_TILES

_vp, _i, _i64, _f = C.c_void_p, C.c_int, C.c_int64, C.c_float


class TailJob(C.Structure):
    """``mie_tail_job`` of include/mie.h, field for field: a tile dilation carried by the kernel that produces its input."""
    _fields_ = [
        ("in_bits", _vp), ("N", _i), ("Hin", _i), ("Win", _i), ("Hout", _i), ("Wout", _i), ("k", _i), ("stride", _i),
        ("pad", _i), ("union_bits", _vp), ("out_bits", _vp), ("list", _vp), ("stale", _vp), ("counts", _vp), ("flags", _vp),
    ]


class ConvArgs(C.Structure):
    """``mie_conv_args`` of include/mie.h, field for field."""
    _fields_ = [
        ("in_", _vp), ("in_ps", _i64), ("cin", _i), ("hin", _i), ("win", _i),
        ("wpacked", _vp), ("cin_pad", _i), ("cout", _i), ("cout_pad", _i),
        ("n", _i), ("hout", _i), ("wout", _i), ("k", _i), ("stride", _i), ("pad", _i),
        ("list", _vp), ("stale", _vp), ("counts", _vp), ("max_tiles", _i),
        ("out", _vp), ("out_ps", _i64), ("out_bits", _vp),
        ("act", _i), ("thr", _f),
        ("res", _vp), ("res_ps", _i64),
        ("emitted", _vp), ("emitted_ps", _i64),
        ("addend", _vp), ("addend_ps", _i64),
        ("wpacked_tc", _vp),
        ("bias", _vp), ("refresh", _i),
        ("tail", _vp),
        ("head", _vp),
        ("in2", _vp), ("in2_ps", _i64),
        ("accum", _vp), ("accum_ps", _i64),
        ("own_tiles", _i), ("own_scratch", _vp),
    ]


# name -> (restype, argtypes); every symbol include/mie.h declares
SIGNATURES = {
    "mie_version": (_i, []),
    "mie_status_string": (C.c_char_p, [_i]),
    "mie_last_cuda_error": (C.c_char_p, []),
    "mie_set_option": (_i, [_i, _i]),
    "mie_get_option": (_i, [_i, C.POINTER(_i)]),
    "mie_mask_from_delta": (_i, [_vp, _i64, _i, _i, _i, _i, _f, _vp, _vp]),
    "mie_mask_from_mask": (_i, [_vp, _i, _i64, _i, _i, _i, _i, _vp, _vp]),
    "mie_tiles_compact": (_i, [_vp, _i, _vp, _vp, _vp]),
    "mie_mask_expand": (_i, [_vp, _i, _i, _i, _vp, _vp]),
    "mie_tiles_dilate": (_i, [_vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "mie_tiles_dilate_static": (_i, [_vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "mie_conv_tiles": (_i, [C.POINTER(ConvArgs), _vp]),
    "mie_conv_uses_tensor_cores": (_i, [C.POINTER(ConvArgs)]),
    "mie_conv_cluster_size": (_i, [C.POINTER(ConvArgs)]),
    "mie_conv_pack_dims": (_i, [_i, _i, _i, C.POINTER(_i), C.POINTER(_i), C.POINTER(_i64)]),
    "mie_pack_conv_weights": (_i, [_vp, _i, _i, _i, _vp, _vp]),
    "mie_conv_pack_dims_tc": (_i, [_i, _i, _i, C.POINTER(_i), C.POINTER(_i), C.POINTER(_i64)]),
    "mie_pack_conv_weights_tc": (_i, [_vp, _i, _i, _i, _vp, _vp]),
    "mie_activation_increment": (_i, [_vp, _vp, _vp, _i64, _i, _vp]),
    "mie_conv_increment_workspace_bytes": (_i64, [_i, _i, _i, _i, _i, _i, _i]),
    "mie_conv_increment_ext": (_i, [_vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _i64, _vp]),
    "mie_act_incr": (_i, [_vp, _i64, _vp, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _i, _i, _i, _i, _i, _f, _i, _vp]),
    "mie_mul_incr": (_i, [_vp, _i64, _vp, _vp, _i64, _vp, _i64, _vp, _vp, _i64, _vp, _i64, _vp, _i, _i, _i, _i, _f, _i, _vp]),
    "mie_convlstm_point": (_i, [_vp, _i64, _vp, _vp, _i64, _vp, _i64, _vp, _vp, _i64, _vp, _i64, _vp, _i64, _vp,
                                _vp, _i64, _vp, _i, _i, _i, _i, _i, _f, _vp, _i64, _vp, _vp, _vp]),
    "mie_upsample2x": (_i, [_vp, _i64, _vp, _vp, _i64, _vp, _vp, _i64, _vp, _i, _i, _i, _i, _i, _vp, _vp]),
    "mie_upsample": (_i, [_vp, _i64, _vp, _vp, _i64, _vp, _vp, _i64, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp]),
    "mie_add": (_i, [_vp, _i64, _vp, _vp, _i64, _vp, _vp, _i64, _vp, _i, _i, _i, _i, _vp, _vp]),
    "mie_cat2": (_i, [_vp, _i64, _vp, _i, _vp, _i64, _vp, _i, _vp, _i64, _vp, _i, _i, _i, _vp, _vp]),
    "mie_accumulate": (_i, [_vp, _i64, _vp, _i64, _vp, _i, _i, _i, _i, _vp]),
    "mie_delta_mask": (_i, [_vp, _i64, _vp, _i64, _vp, _i64, _vp, _i, _i, _i, _i, _f, _vp, _i64, _vp, _vp, _vp]),
    "mie_events_to_voxel": (_i, [_vp, _i, _i, _i, _i, _vp, _i64, _i, _i, _i, _i, _vp]),
    "mie_events_to_count_image": (_i, [_vp, _i, _i, _i, _vp, _i64, _i, _i, _i, _i, _vp]),
    "mie_maxpool_incr": (_i, [_vp, _i64, _vp, _vp, _i64, _vp, _i64, _vp, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "mie_reflect_border": (_i, [_vp, _i64, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "mie_split_tf32": (_i, [_vp, _i64, _vp, _i, _vp, _i64, _vp, _i, _i, _i, _vp, _vp]),
    "mie_kfenced": (_i, [_vp, _i64, _vp, _i64, _f, _vp, _i64, _vp, _i, _i, _i, _i, _vp]),
}


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python maskedincrementeval_b200/build.py` "
            "(nvcc, sm_100a).  This package has no fallback path.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export it
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


class MieError(RuntimeError):
    pass


def launch_count() -> int:
    """Kernels the library has enqueued since the last reset: counted inside the library, per launch (an entry
    point that enqueues two kernels counts two)."""
    return get_option(OPT_LAUNCH_COUNT)


def reset_launch_count() -> None:
    set_option(OPT_LAUNCH_COUNT, 0)


def check(status: int, what: str = "") -> None:
    """Map a libmie status to the exception class the reference raises for the same condition:
    unsupported kernel size / stride -> NotImplementedError (ext/pointops/pointops_functional.py:41),
    everything else -> RuntimeError (TORCH_CHECK, include/checks.h:6-8)."""
    if status == OK:
        return
    msg = lib.mie_status_string(status).decode()
    if status == ECUDA:
        msg += ": " + lib.mie_last_cuda_error().decode()
    if status == EUNSUPPORTED:
        raise NotImplementedError(f"libmie {what}: {msg}")
    raise MieError(f"libmie {what}: {msg}")


def set_option(option: int, value: int) -> None:
    check(lib.mie_set_option(option, int(value)), "set_option")


def get_option(option: int) -> int:
    v = C.c_int()
    check(lib.mie_get_option(option, C.byref(v)), "get_option")
    return v.value


def describe_error_word(word: int) -> str:
    """Text for the MIE_ERR_* bits a convolution kernel left in counts[3]."""
    parts = []
    if word & ERR_BAD_TILE:
        parts.append("a tile-list entry was outside the field (skipped)")
    if word & ERR_WAIT_EXPIRED:
        parts.append("a bounded barrier wait ran out in a tensor-core kernel (that launch's output is invalid)")
    if word & ~(ERR_BAD_TILE | ERR_WAIT_EXPIRED):
        parts.append(f"unknown bits {word:#x}")
    return "; ".join(parts)


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream_ptr(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")  # CHECK_CUDA, include/checks.h:6
    if t.dtype != torch.float32:
        raise RuntimeError(f"{name} must be float32")
