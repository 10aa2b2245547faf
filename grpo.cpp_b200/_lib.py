"""Loads ``libgrpo_b200.so`` and declares the C ABI of ``include/grpo_b200.h`` to ctypes."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libgrpo_b200.so")

OK, E_INVALID, E_NONFINITE, E_CUDA, E_WORKSPACE = 0, 1, 2, 3, 4

_f = C.POINTER(C.c_float)
_i = C.POINTER(C.c_int32)
_vp = C.c_void_p
_sz = C.c_size_t
_i64 = C.c_int64
_int = C.c_int
_flt = C.c_float


class Result(C.Structure):
    """Mirror of ``grpo_b200_result_t`` (five doubles)."""
    _fields_ = [("loss", C.c_double), ("pg_loss", C.c_double), ("kl", C.c_double),
                ("bad_grads", C.c_double), ("bad_inputs", C.c_double)]


# name -> (restype, argtypes); one entry per function declared in include/grpo_b200.h
SIGNATURES = {
    "grpo_b200_last_error": (C.c_char_p, []),
    "grpo_b200_build_info": (C.c_char_p, []),
    "grpo_b200_count_lengths": (_int, [_vp, _i64, _i64, _int, _i64, _vp, _vp]),
    "grpo_b200_weights_from_lengths": (_int, [_vp, _i64, _int, _flt, _vp, _vp, _vp]),
    "grpo_b200_count_lengths_f64": (_int, [_vp, _i64, _i64, _int, _i64, _vp, _vp]),
    "grpo_b200_weights_from_lengths_f64": (_int, [_vp, _i64, _int, _flt, _vp, _vp, _vp]),
    "grpo_b200_group_advantages": (_int, [_vp, _int, _int, _int, _flt, _vp, _vp, _vp]),
    "grpo_b200_loss_workspace_bytes": (_sz, [_i64]),
    "grpo_b200_loss": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _int, _flt, _flt, _vp, _vp, _vp, _sz, _vp]),
    "grpo_b200_loss_noalloc": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _int, _flt, _flt, _vp, _vp, _vp]),
    "grpo_b200_logits_workspace_bytes": (_sz, [_i64]),
    "grpo_b200_logits": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _int, _int, _int, _flt, _flt,
                                _int, _int, _vp, _vp, _vp, _vp, _sz, _vp]),
    "grpo_b200_row_order_bytes": (_sz, [_i64]),
    "grpo_b200_row_order": (_int, [_vp, _i64, _vp, _vp]),
    "grpo_b200_exchange_bytes": (_sz, [_i64]),
    "grpo_b200_exchange_create": (_int, [_i64, C.POINTER(_vp)]),
    "grpo_b200_exchange_export": (_int, [_vp, C.c_char_p]),
    "grpo_b200_exchange_open": (_int, [C.c_char_p, C.POINTER(_vp)]),
    "grpo_b200_exchange_close": (_int, [_vp]),
    "grpo_b200_exchange_destroy": (_int, [_vp]),
    "grpo_b200_logits_sharded": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _int, _int, _int, _flt,
                                        _flt, _int, _int, _vp, _vp, _vp, _vp, _sz, C.POINTER(_vp), _int, _int, _i64,
                                        _vp, _int, _flt, _vp, _vp, _vp, _vp]),
    "grpo_b200_lengths_sharded": (_int, [_vp, _i64, _i64, _int, _i64, C.POINTER(_vp), _int, _int, _int, _flt, _vp, _vp,
                                         _vp, _vp, _vp, _sz, _vp]),
    "grpo_b200_exchange_set_timeout_cycles": (_int, [_i64]),
    "grpo_b200_synthetic_logits": (_int, [_vp, _i64, _i64, _int, _int, _flt, C.c_uint64, _flt, _vp]),
    "grpo_b200_sample_rows": (_int, [_vp, _i64, _int, _int, _vp, _int, _vp, _vp, _vp, _vp, _vp, _vp]),
    "grpo_b200_logits_set_variant": (_int, [_int]),
    "grpo_b200_logits_variant_name": (C.c_char_p, [_int]),
    "grpo_b200_logits_plan": (C.c_char_p, [_vp, _vp, _int, _int, _i64, _int]),
    "grpo_b200_loss_host": (_int, [_f, _sz, _f, _sz, _f, _sz, _f, _sz, _i, _sz, _int, _int, _int, _flt, _flt, _int,
                                   _flt, _int, _f, _f, C.POINTER(_int)]),
    "grpo_b200_logits_host": (_int, [_f, _sz, _f, _sz, _f, _sz, _i, _sz, _f, _sz, _i, _sz, _int, _int, _int, _int,
                                     _flt, _flt, _int, _flt, _int, _f, _f, C.POINTER(_int)]),
    "grpo_b200_logits_device_inplace_host": (_int, [_vp, _f, _sz, _f, _sz, _i, _sz, _f, _sz, _i, _sz, _int, _int,
                                                    _int, _int, _int, _flt, _flt, _int, _flt, _int, _f,
                                                    C.POINTER(_int)]),
    "grpo_b200_benchmark_loss_host": (_int, [_f, _sz, _f, _sz, _f, _sz, _f, _sz, _i, _sz, _int, _int, _int, _flt,
                                             _flt, _int, _flt, _int, _int, _f, _f]),
    "grpo_b200_benchmark_logits_host": (_int, [_f, _sz, _f, _sz, _f, _sz, _i, _sz, _f, _sz, _i, _sz, _int, _int,
                                               _int, _int, _flt, _flt, _int, _flt, _int, _int, _f, _f]),
    "grpo_b200_shard_create": (_int, [_int, _int, _i64, _int, _int, _int, _i64, _i64, C.POINTER(_vp)]),
    "grpo_b200_shard_export": (_int, [_vp, C.c_char_p]),
    "grpo_b200_shard_connect_ipc": (_int, [_vp, C.c_char_p]),
    "grpo_b200_shard_connect_local": (_int, [_vp, C.POINTER(_vp)]),
    "grpo_b200_shard_destroy": (_int, [_vp]),
    "grpo_b200_logits_sharded_host": (_int, [_vp, _vp, _f, _sz, _f, _sz, _i, _sz, _f, _sz, _i, _sz, _flt, _flt, _int,
                                             _flt, _int, _f, C.POINTER(_int)]),
    "grpo_b200_gradsync_slice": (None, [_i64, _int, _int, C.POINTER(_i64), C.POINTER(_i64)]),
    "grpo_b200_gradsync_create": (_int, [_int, _int, _vp, _i64, C.POINTER(_vp)]),
    "grpo_b200_gradsync_export": (_int, [_vp, C.c_char_p]),
    "grpo_b200_gradsync_connect_ipc": (_int, [_vp, C.c_char_p]),
    "grpo_b200_gradsync_connect_local": (_int, [_vp, C.POINTER(_vp)]),
    "grpo_b200_gradsync_set_timeout_cycles": (_int, [_i64]),
    "grpo_b200_allreduce_scale": (_int, [_vp, _flt, _vp]),
    "grpo_b200_gradsync_status": (_int, [_vp, C.POINTER(_int)]),
    "grpo_b200_gradsync_destroy": (_int, [_vp]),
    "grpo_b200_lmhead_workspace_bytes": (_sz, [_i64, _int]),
    "grpo_b200_lmhead_loss": (_int, [_vp, _vp, _i64, _int, _int, _int, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _int, _flt,
                                     _flt, _vp, _vp, _vp, _vp, _sz, _vp]),
    "grpo_b200_release_cache": (_int, []),
}

_lib = None


def build(verbose: bool = False) -> str:
    """Compile the CUDA library for sm_100a in-tree (``make`` in ``csrc/``); returns its path."""
    cmd = ["make", "-C", os.path.join(_PKG, "csrc"), "-j8"] + ([] if verbose else ["-s"])
    subprocess.run(cmd, check=True)
    return LIB_PATH


def lib() -> C.CDLL:
    """The loaded library.  Raises if it has not been built: there is nothing to fall back to."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                "or `make -C grpo.cpp_b200/csrc`. This package has no CPU or eager fallback.")
        handle = C.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def last_error() -> str:
    return lib().grpo_b200_last_error().decode()


def check(status: int) -> None:
    """Raise ``RuntimeError`` with the library's message (the reference's exception text)."""
    if status != OK:
        raise RuntimeError(last_error())
