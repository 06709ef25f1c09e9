"""Build and call the plain-C oracle (oracle/naive_kda.c) -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Only tests/, the smoke check and the benchmark's CPU-baseline leg may import this module.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "naive_kda.c")
LIB = os.path.join(HERE, "libnaive_kda.so")


def build(force=False):
    """gcc -O3 -fopenmp the C restatement into oracle/libnaive_kda.so (skipped when up to date)."""
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    cmd = ["gcc", "-O3", "-march=x86-64-v3", "-fopenmp", "-shared", "-fPIC", SRC, "-o", LIB, "-lm"]
    subprocess.run(cmd, check=True)
    return LIB


_lib = None


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB):
            build()
        _lib = ctypes.CDLL(LIB)
        fp = ctypes.POINTER(ctypes.c_float)
        ip = ctypes.POINTER(ctypes.c_int)
        _lib.naive_kda_fwd.restype = ctypes.c_int
        _lib.naive_kda_fwd.argtypes = [fp] * 8 + [fp, fp, ip] + [ctypes.c_int] * 4 + [ctypes.c_float] + \
                                      [ctypes.c_int, ctypes.c_int, ctypes.c_float]
        _lib.naive_kda_num_threads.restype = ctypes.c_int
        _lib.naive_kda_set_num_threads.argtypes = [ctypes.c_int]
        _lib.naive_kda_set_num_threads.restype = None
    return _lib


def num_threads():
    return int(load().naive_kda_num_threads())


def use_all_cores():
    """Run on every core this process may use, whatever OMP_NUM_THREADS says (torch.distributed.run exports
    OMP_NUM_THREADS=1 to its workers). Returns the thread count now in effect."""
    load().naive_kda_set_num_threads(len(os.sched_getaffinity(0)))
    return num_threads()


def _f32(x):
    if x is None:
        return None
    return np.ascontiguousarray(np.asarray(x, dtype=np.float32))


def _ptr(a, ty=ctypes.c_float):
    return None if a is None else a.ctypes.data_as(ctypes.POINTER(ty))


def naive_kda_fwd(q, k, v, g, beta, A_log=None, dt_bias=None, h0=None, cu_seqlens=None, scale=None,
                  use_l2norm=False, gate_mode=0, lower_bound=-5.0, want_final_state=True):
    """numpy in / numpy out. q,k,g [B,T,H,K]; v [B,T,H,V]; beta [B,T,H]; h0 [N,H,K,V].

    gate_mode: 0 = g is the log decay, 1 = softplus gate, 2 = lower-bound sigmoid gate.
    With ``cu_seqlens`` the batch must be 1 and tokens are packed.
    """
    lib = load()
    q, k, v, g, beta = map(_f32, (q, k, v, g, beta))
    B, T, H, K = q.shape
    V = v.shape[-1]
    if cu_seqlens is None:
        cu = np.arange(B + 1, dtype=np.int32) * T
    else:
        assert B == 1
        cu = np.ascontiguousarray(np.asarray(cu_seqlens, dtype=np.int32))
    N = len(cu) - 1
    A_log, dt_bias, h0 = _f32(A_log), _f32(dt_bias), _f32(h0)
    o = np.zeros((B, T, H, V), dtype=np.float32)
    ht = np.zeros((N, H, K, V), dtype=np.float32) if want_final_state else None
    if scale is None:
        scale = K ** -0.5
    rc = lib.naive_kda_fwd(_ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(beta), _ptr(A_log), _ptr(dt_bias),
                           _ptr(h0), _ptr(o), _ptr(ht), _ptr(cu, ctypes.c_int), N, H, K, V,
                           float(scale), int(use_l2norm), int(gate_mode), float(lower_bound))
    if rc != 0:
        raise RuntimeError(f"naive_kda_fwd returned {rc}")
    return o, ht
