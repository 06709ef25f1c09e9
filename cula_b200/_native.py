"""ctypes binding of libcula_kda.so (C ABI declared in include/cula_kda.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libcula_kda.so")

_vp, _ip, _fp, _i, _f = ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_float

# name -> (restype, argtypes); must list every symbol include/cula_kda.h declares
SIGNATURES = {
    "cula_kda_tile_pack_bytes": (_i, []),
    "cula_kda_fwd_intra_smem_bytes": (_i, []),
    "cula_kda_fwd_scan_smem_bytes": (_i, []),
    "cula_kda_fwd_intra": (_i, [_vp, _vp, _vp, _vp, _i, _vp, _i, _fp, _fp, _ip, _ip, _i, _i, _i,
                                _f, _i, _i, _f, _vp, _fp, _fp, _ip, _vp]),
    "cula_kda_fwd_scan": (_i, [_vp, _fp, _vp, _fp, _vp, _vp, _fp, _ip, _ip, _ip, _i, _i, _i, _ip, _vp]),
    "cula_kda_cp_transition": (_i, [_vp, _fp, _fp, _ip, _ip, _i, _i, _i, _ip, _vp]),
    "cula_kda_cp_fold": (_i, [_fp, _fp, _fp, _fp, _i, _i, ctypes.c_longlong, _vp]),
    "cula_kda_decode": (_i, [_vp, _vp, _vp, _vp, _i, _vp, _i, _fp, _fp, _fp, _ip, _vp, _i, _i, _i, _i, _i, _f, _i, _f, _f, _i, _ip, _vp]),
    "cula_kda_num_chunks": (_i, [_ip, _i]),
    "cula_kda_build_chunk_tables": (_i, [_ip, _i, _ip, _ip, _ip]),
    "cula_kda_bwd_scratch_floats": (_i, []),
    "cula_kda_bwd_grad_scale": (_i, [_vp, ctypes.c_longlong, _fp, ctypes.c_longlong, _vp, _fp, _vp]),
    "cula_kda_bwd_scan": (_i, [_vp, _vp, _fp, _fp, _vp, _fp, _fp, _ip, _ip, _ip, _i, _i, _i, _ip, _vp]),
    "cula_kda_bwd_dense": (_i, [_fp, _fp, _vp, _vp, _vp, _vp, _vp, _i, _fp, _fp, _vp, _fp, _ip, _ip, _i, _i, _i, _ip, _vp]),
    "cula_kda_bwd_gated": (_i, [_vp, _vp, _vp, _i, _vp, _i, _fp, _fp, _fp, _fp, _fp, _fp, _vp, _vp, _vp, _vp, _fp, _fp,
                                _ip, _ip, _i, _i, _i, _f, _i, _i, _f, _vp]),
    "cula_kda_noalloc_max_tiles": (_i, []),
    "cula_kda_fwd_noalloc": (_i, [_vp, _vp, _vp, _vp, _i, _vp, _i, _fp, _fp, _fp, _vp, _fp, _ip, _ip, _ip,
                                  _i, _i, _i, _i, _f, _i, _i, _f, _ip, _vp]),
    "cula_kda_gate_fwd": (_i, [_vp, _i, _fp, _fp, _vp, _i, ctypes.c_longlong, _i, _i, _i, _f, _vp]),
    "cula_kda_gate_bwd": (_i, [_vp, _i, _fp, _fp, _vp, _i, _vp, _fp, _fp, ctypes.c_longlong, _i, _i, _i, _f, _vp]),
    "cula_kda_beta_sigmoid_fwd": (_i, [_vp, _i, _fp, ctypes.c_longlong, _vp]),
    "cula_kda_beta_sigmoid_bwd": (_i, [_vp, _i, _fp, _vp, ctypes.c_longlong, _vp]),
    "cula_kda_short_conv_fwd": (_i, [_vp, _fp, _fp, _fp, _vp, _fp, _ip, _ip, _i, _i, _i, _i, _i, _vp]),
    "cula_kda_short_conv_bwd": (_i, [_vp, _fp, _fp, _fp, _vp, _vp, _fp, _fp, _ip, _ip, _i, _i, _i, _i, _i, _vp]),
    "cula_kda_rms_norm_gated_fwd": (_i, [_vp, _vp, _fp, _vp, _fp, ctypes.c_longlong, _i, _i, _f, _vp]),
    "cula_kda_rms_norm_gated_bwd": (_i, [_vp, _vp, _fp, _fp, _vp, _vp, _vp, _fp, ctypes.c_longlong, _i, _i, _vp]),
    "cula_kda_selftest_bounded_wait": (_i, [_ip, _i, _vp]),
    "cula_kda_strerror": (ctypes.c_char_p, [_i]),
}

_lib = None


def lib():
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m cula_b200.build` (needs nvcc). "
                "There is no CPU or PyTorch fallback for chunk_kda.")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(code: int, what: str):
    if code != 0:
        msg = lib().cula_kda_strerror(code).decode()
        raise RuntimeError(f"{what} failed with code {code}: {msg}")
