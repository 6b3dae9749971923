"""ctypes binding of libsmla_b200.so.  There is no CPU fallback: if the library is missing
the import of any op raises."""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p

from .build import LIB_PATH

IMPL_AUTO, IMPL_SCALAR, IMPL_TC = 0, 1, 2
LAYOUT_V32, LAYOUT_MODEL1 = 0, 1

_lib = None

_SIGS = {
    "smla_last_error": (c_char_p, []),
    "smla_version": (c_int, []),
    "smla_device_status": (c_int, [c_void_p, c_void_p, c_void_p]),
    "smla_status_string": (c_char_p, [c_int]),
    "smla_num_sms": (c_int, []),
    "smla_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "smla_sched_meta": (c_int, [c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "smla_decode_splitkv": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_int64, c_int,
                                    c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "smla_decode_partial": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_int64, c_int,
                                    c_void_p, c_int, c_void_p, c_void_p]),
    "smla_decode_partial_sliced": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64,
                                           c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_int64, c_int,
                                           c_void_p, c_int, c_void_p, c_void_p]),
    "smla_cp_unslice": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_void_p]),
    "smla_combine_parts": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "smla_combine_parts_strided": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64,
                                           c_void_p, c_void_p]),
    "smla_noalloc_scratch_need": (c_size_t, [c_int, c_int, c_int]),
    "smla_decode_splitkv_noalloc": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                            c_float, c_int, c_int64, c_int, c_void_p, c_void_p, c_int, c_void_p,
                                            c_void_p]),
    "smla_combine": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "smla_decode_uniform": (c_int, [c_void_p] * 7 + [c_int, c_int, c_int, c_float, c_int, c_int64, c_int, c_void_p, c_int,
                                                 c_void_p, c_void_p]),
    "smla_prefill": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                             c_float, c_int, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "smla_decode_splitkv_ext": (c_int, [c_void_p] * 11 + [c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int64,
                                                          c_int, c_int64, c_int] + [c_void_p] * 3 + [c_int, c_void_p, c_void_p]),
    "smla_prefill_ext": (c_int, [c_void_p] * 8 + [c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int64, c_int,
                                                  c_int64] + [c_void_p] * 3 + [c_int, c_void_p, c_void_p]),
    "smla_pack_kv": (c_int, [c_void_p, c_void_p, c_int64, c_void_p]),
    "smla_mqa_logits": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_int, c_int, c_int, c_int64, c_int, c_void_p, c_void_p]),
    "smla_topk": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int, c_void_p]),
    "smla_cp_partition_indices": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "smla_cp_local_window": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "smla_cp_candidates": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "smla_cp_interleave_candidates": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "smla_cp_pick_positions": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
}

EXPORTS = tuple(_SIGS)


def load():
    """Load the shared library (once) and declare the prototypes of include/smla.h."""
    global _lib
    if _lib is not None:
        return _lib
    path = os.environ.get("SMLA_LIBRARY", LIB_PATH)   # an alternative build of the same library
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python -m sparse_mla_sm120_b200.build` "
            "(needs nvcc); this library has no CPU fallback")
    lib = ctypes.CDLL(path)
    for name, (res, args) in _SIGS.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class SmlaError(RuntimeError):
    pass


def check(rc: int) -> None:
    """0 -> ok; negative -> ValueError (argument error); positive -> RuntimeError (CUDA error)."""
    if rc == 0:
        return
    msg = load().smla_last_error().decode()
    if rc < 0:
        raise ValueError(f"smla error {rc}: {msg}")
    raise SmlaError(f"CUDA error {rc}: {msg}")
