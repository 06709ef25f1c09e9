"""Single-token KDA decode against a pool of fp32 states: ``kda_decode`` and
``fused_sigmoid_gating_delta_rule_update`` with the reference's signatures
(cula/ops/kda_decode.py:1794-2096). One launch of ``kda_decode_kernel`` through the C ABI; the state pool is updated
in place. There is no fallback: without the CUDA library the call raises."""
from __future__ import annotations

import torch

from .. import _native
from ..utils import assert_blackwell
from .chunk import _ptr, _status_word


def _canonical_layout(state_layout):
    lay = "vk" if state_layout is None else str(state_layout).lower()
    if lay not in ("vk", "kv"):
        raise ValueError(f"state_layout must be 'vk' or 'kv', got {state_layout!r}")
    return lay


@torch.no_grad()
def kda_decode(A_log, dt_bias, q, k, v, a, b, initial_state_source, initial_state_indices, cu_seqlens=None, scale=None,
               use_qk_l2norm_in_kernel=True, softplus_beta=1.0, softplus_threshold=20.0, out=None, state_layout="vk"):
    """Dense decode: q/k ``(N, 1, H, 128)``, v ``(N, 1, HV, V)``, a ``(N, 1, HV, 128)``, b ``(N, 1, HV)``.
    Varlen decode: the same with the first two axes swapped (``(1, N, ...)``; a / b may drop the leading 1).
    ``initial_state_source``: ``(pool, HV, V, K)`` for ``state_layout="vk"`` (default) or ``(pool, HV, K, V)`` for
    ``"kv"``, fp32, updated in place; None means zero states that are not kept. ``initial_state_indices``: int32
    ``[N]`` pool slots (negative = skip the sequence) or None for slot = sequence. ``cu_seqlens`` is accepted for
    signature compatibility: with one token per sequence it carries no information. Returns ``o`` shaped like ``v``
    in q's dtype (cula/ops/kda_decode.py:1845-2096)."""
    B_q, T_q, H, K = q.shape
    HV, V = v.shape[2], v.shape[3]
    N = initial_state_indices.shape[0] if initial_state_indices is not None else (T_q if B_q == 1 and T_q > 1 else B_q)
    assert K == 128, f"the decode kernel requires K=128, got {K}"
    assert V % 32 == 0, f"the decode kernel requires V % 32 == 0, got V={V}"
    assert q.dtype == k.dtype == v.dtype == torch.bfloat16, "q, k, v must be in bfloat16."
    assert HV % H == 0, "the number of value heads must be a multiple of the number of q/k heads"
    assert B_q * T_q == N, "decode takes exactly one token per sequence"
    if scale is None:
        scale = K ** -0.5
    else:
        assert scale > 0, f"scale must be positive, got {scale}"
    lay = _canonical_layout(state_layout)
    assert_blackwell(q.device)
    dev = q.device
    is_varlen = B_q == 1 and T_q == N and N > 1
    state = initial_state_source
    if state is None:
        state = torch.zeros((N, HV, V, K) if lay == "vk" else (N, HV, K, V), dtype=torch.float32, device=dev)
    want = (HV, V, K) if lay == "vk" else (HV, K, V)
    if state.dim() != 4 or tuple(state.shape[1:]) != want:
        raise ValueError(f"State layout mismatch for state_layout='{lay}': got {tuple(state.shape)}, expected (..., {want})")
    assert state.dtype == torch.float32 and state.is_contiguous(), "the state pool must be contiguous float32"
    pool = state.shape[0]
    idx = initial_state_indices
    if idx is None:
        if pool < N:
            raise ValueError(f"the state pool holds {pool} states for {N} sequences and no indices were given")
    else:
        idx = idx.to(device=dev, dtype=torch.int32).contiguous()
        assert idx.numel() == N
    q, k, v = (x.contiguous() for x in (q, k, v))
    a = a.contiguous()
    b = b.contiguous()
    assert a.numel() == N * HV * K and b.numel() == N * HV, "a must be (N, HV, K) and b (N, HV) up to singleton axes"
    assert a.dtype in (torch.bfloat16, torch.float32) and b.dtype in (torch.bfloat16, torch.float32)
    A_log = A_log.reshape(-1).float().contiguous()
    assert A_log.numel() == HV
    if dt_bias is not None:
        dt_bias = dt_bias.reshape(-1).float().contiguous()
        assert dt_bias.numel() == HV * K
    shape = (1, N, HV, V) if is_varlen else (N, 1, HV, V)
    if out is None:
        out = torch.empty(shape, dtype=q.dtype, device=dev)
    else:
        if tuple(out.shape) != shape or out.dtype != q.dtype:
            raise ValueError(f"out must have shape {shape} and dtype {q.dtype}")
        if not out.is_contiguous():
            raise ValueError("out must be contiguous")
    lib = _native.lib()
    with torch.cuda.device(dev):
        _native.check(lib.cula_kda_decode(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(), int(a.dtype == torch.float32), b.data_ptr(),
            int(b.dtype == torch.float32), A_log.data_ptr(), _ptr(dt_bias), state.data_ptr(), _ptr(idx), out.data_ptr(),
            N, H, HV, V, pool, float(scale), int(use_qk_l2norm_in_kernel), float(softplus_beta), float(softplus_threshold),
            int(lay == "kv"), _status_word(dev).data_ptr(), torch.cuda.current_stream(dev).cuda_stream), "cula_kda_decode")
    return out


def fused_sigmoid_gating_delta_rule_update(A_log, a, dt_bias, softplus_beta, softplus_threshold, q, k, v, b,
                                           initial_state_source, initial_state_indices, scale=None,
                                           use_qk_l2norm_in_kernel=False, cu_seqlens=None, is_kda=False, out=None,
                                           state_layout="vk"):
    """Argument order of the reference's public decode entry (cula/ops/kda_decode.py:1794-1842)."""
    if not is_kda:
        raise NotImplementedError("cuLA fused decode currently supports only is_kda=True mode")
    return kda_decode(A_log=A_log, dt_bias=dt_bias, q=q, k=k, v=v, a=a, b=b, initial_state_source=initial_state_source,
                      initial_state_indices=initial_state_indices, cu_seqlens=cu_seqlens, scale=scale,
                      use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel, softplus_beta=softplus_beta,
                      softplus_threshold=softplus_threshold, out=out, state_layout=state_layout)
