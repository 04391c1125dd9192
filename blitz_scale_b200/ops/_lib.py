"""Loader for the in-tree kernel library (``_lib/libblitz_kernels.so``).

The kernels are exported with C linkage and called through ctypes with raw
device pointers and the current CUDA stream, so a launch costs a few
microseconds of host time and is captured by CUDA graphs like any other launch
on the stream.  There is no fallback: if the library is missing the import of
any op raises, so a GPU box can never silently run a PyTorch path.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent.parent / "_lib" / "libblitz_kernels.so"
_lib = None


class KernelLibraryMissing(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            if os.environ.get("BLITZ_AUTO_BUILD", "0") == "1":
                from .. import build as _b
                _b.build_kernels()
            else:
                raise KernelLibraryMissing(
                    f"{_LIB_PATH} not found: run `python -m blitz_scale_b200.build` (needs nvcc) first")
        _lib = ctypes.CDLL(str(_LIB_PATH))
        _declare(_lib)
    return _lib


def available() -> bool:
    return _LIB_PATH.exists()


c_i = ctypes.c_int
c_i64 = ctypes.c_int64
c_u64 = ctypes.c_uint64
c_f = ctypes.c_float
c_p = ctypes.c_void_p


def _declare(L: ctypes.CDLL) -> None:
    def sig(name, args, res=c_i):
        if hasattr(L, name):
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = res

    sig("blitz_gemm", [c_p, c_i64, c_p, c_i64, c_p, c_i64, c_p, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_p, c_i64,
                       c_p, c_i, c_p, c_p])
    sig("blitz_gemm_workspace_bytes", [c_i], c_i64)
    sig("blitz_gemm_decode", [c_p, c_i64, c_p, c_i64, c_p, c_i64, c_p, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_p, c_p])
    sig("blitz_gemm_decode_supported", [c_i, c_i, c_i, c_i, c_i], c_i)
    sig("blitz_gemm_pair", [c_p, c_i64, c_p, c_i64, c_p, c_i64, c_p, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_p,
                            c_i64, c_p, c_i, c_p, c_p])
    sig("blitz_gemm_pair_supported", [c_i, c_i, c_i, c_i, c_i], c_i)
    sig("blitz_gemm_pair_workspace_bytes", [c_i], c_i64)
    sig("blitz_set_pdl", [c_i], None)
    sig("blitz_get_pdl", [], c_i)
    sig("blitz_gemm_tile_n", [c_i, c_i, c_i, c_i], c_i)
    sig("blitz_gemm_tp", [c_p, c_i64, c_p, c_i64, c_p, c_i64, c_p, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_p, c_i64,
                          c_p, c_i, c_p, c_p, c_p])
    pp_ = ctypes.POINTER(c_p)
    sig("blitz_rs_reduce_norm", [c_p, c_p, ctypes.c_uint32, c_p, c_p, pp_, pp_, c_i, c_i, c_i, c_i, c_i, c_i, c_f, c_u64,
                                 c_p, c_i, c_p])
    sig("blitz_flags_zero", [c_p, c_i, c_p])
    sig("blitz_allreduce_oneshot", [c_p, pp_, pp_, c_p, c_i, c_i, c_i64, c_u64, c_p, c_i, c_p])
    sig("blitz_allreduce_fused", [c_p, pp_, pp_, c_p, c_i, c_i, c_i64, c_u64, c_p, c_i, c_p])
    sig("blitz_ar_add_norm_mm", [c_p, c_p, c_p, c_p, c_p, pp_, c_i, c_i, c_i, c_i, c_f, c_u64, c_p, c_i, c_p])
    sig("blitz_peer_allgather", [c_p, pp_, pp_, c_i, c_i, c_i64, c_u64, c_p, c_p])
    sig("blitz_embedding", [c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_p, c_i, c_p])
    sig("blitz_rms_norm", [c_p, c_p, c_p, c_i, c_i, c_f, c_i, c_p])
    sig("blitz_add_rms_norm", [c_p, c_p, c_p, c_p, c_i, c_i, c_f, c_i, c_p])
    sig("blitz_silu_mul", [c_p, c_p, c_i, c_i, c_i64, c_i, c_p])
    sig("blitz_add_residual", [c_p, c_p, c_i64, c_i, c_p])
    sig("blitz_gather_last", [c_p, c_p, c_p, c_i, c_i, c_i, c_p])
    sig("blitz_argmax", [c_p, c_i, c_i, c_i64, c_p, c_p, c_i, c_i, c_p])
    sig("blitz_sample", [c_p, c_i, c_i, c_i64, c_p, c_p, c_p, c_p, c_u64, c_p, c_i, c_p])
    sig("blitz_rope_kv_store", [c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_i, c_f, c_p, c_i, c_p])
    sig("blitz_attn_decode_workspace_bytes", [c_i, c_i, c_i, c_i], c_i64)
    sig("blitz_attn_decode", [c_p, c_i64, c_p, c_p, c_p, c_p, c_p, c_i64, c_p, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_f,
                              c_p, c_i, c_p])
    sig("blitz_attn_prefill_paged", [c_p, c_p, c_p, c_i64, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_f, c_i, c_p,
                                     c_i, c_p])
    # comm kernels
    pp = ctypes.POINTER(c_p)
    pi64 = ctypes.POINTER(c_i64)
    sig("blitz_peer_copy_units", [c_p, pp, pp, c_i, c_p, pi64, pi64, c_i, c_i, c_i, c_i, c_p, c_i, c_p])
    sig("blitz_kv_push", [c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i64, c_i64, c_i64, c_i, c_i, c_p, c_p, c_i, c_p, c_p,
                          c_p])
    sig("blitz_flag_wait", [c_p, ctypes.c_uint32, c_u64, c_p, c_p])
    sig("blitz_flag_wait_eq", [c_p, ctypes.c_uint32, c_u64, c_p, c_p])
    sig("blitz_flag_set", [c_p, ctypes.c_uint32, c_i, c_p])
