"""``chunk_gated_delta_rule``: the scalar-gate ("GDN") variant of the chunkwise pipeline.

The gated delta rule is Kimi Delta Attention with ONE decay per (token, head) instead of one per key channel:
``S <- exp(g_t) S``, then the same delta-rule correction and read-out. It runs through the same sm_100a kernels as
``chunk_kda``: the chunk-parallel stage and the gate-dependent backward stage read ``g`` as ``[B, T, H]`` (one value
per row, broadcast over the 128 channels in registers) and the backward stage reduces the gate gradient over the
channels before it writes it, so neither ``g`` nor ``dg`` is ever expanded in HBM. Everything else (state scan, output,
dense backward stage, packed batches, initial / final states) is shared.

Call surface of flash-linear-attention's ``chunk_gated_delta_rule`` (fla/ops/gated_delta_rule/chunk.py), which the
reference lists as its modular GDN path (README.md:190; the dormant scalar-gate switch of its state scan is
cula/ops/chunk_delta_h.py:223). Restrictions of this build: K = V = 128, as many value heads as key heads.
"""
from __future__ import annotations

import torch

from ..kda.chunk import ChunkKDAFunction, _poll_status
from ..utils import assert_blackwell


@torch.compiler.disable
def chunk_gated_delta_rule(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
                           use_qk_l2norm_in_kernel=False, cu_seqlens=None, cu_seqlens_cpu=None,
                           use_gate_in_kernel=False, disable_recompute=False, **kwargs):
    r"""Chunkwise gated delta rule forward (+ autograd backward).

    Args:
        q, k, v: ``[B, T, H, 128]`` bf16.
        g: ``[B, T, H]`` fp32 or bf16: the natural-log decay of each (token, head), ``<= 0``; with
            ``use_gate_in_kernel=True`` the raw gate input, activated in-kernel as
            ``-exp(A_log[h]) * softplus(g + dt_bias[h])`` (``A_log`` ``[H]``, optional ``dt_bias`` ``[H]`` as keyword
            arguments).
        beta: ``[B, T, H]`` bf16 or fp32.
        scale: defaults to ``128 ** -0.5``.
        initial_state: ``[N, H, 128, 128]`` fp32 or None; output_final_state: also return the final state.
        use_qk_l2norm_in_kernel: L2-normalise q and k rows in-kernel.
        cu_seqlens: int32 ``[N+1]`` for a packed batch (then B must be 1).

    Returns ``(o, final_state)``. Gradients flow to q, k, v, g, beta, A_log, dt_bias and initial_state.
    """
    if cu_seqlens is not None:
        if q.shape[0] != 1:
            raise ValueError(
                f"The batch size is expected to be 1 rather than {q.shape[0]} when using `cu_seqlens`."
                f"Please flatten variable-length inputs before processing.")
        if initial_state is not None and initial_state.shape[0] != len(cu_seqlens) - 1:
            raise ValueError(
                f"The number of initial states is expected to be equal to the number of input sequences, "
                f"i.e., {len(cu_seqlens) - 1} rather than {initial_state.shape[0]}.")
    assert q.dtype == k.dtype == v.dtype == torch.bfloat16, "q, k, v must be in bfloat16."
    assert q.shape == k.shape and q.shape[-1] == v.shape[-1] == 128, "only head dim 128 is supported for keys and values"
    assert v.shape[:3] == q.shape[:3], "grouped value heads (HV > H) are not supported"
    assert g.shape == q.shape[:3] and beta.shape == q.shape[:3], "g and beta must be of shape (batch size, seq len, heads)"
    assert g.dtype in (torch.float32, torch.bfloat16) and beta.dtype in (torch.float32, torch.bfloat16)
    if initial_state is not None:
        assert initial_state.dtype == torch.float32, "initial_state must be in float32."
    A_log = dt_bias_h = dt_bias = None
    H = q.shape[2]
    if use_gate_in_kernel:
        assert "A_log" in kwargs, "A_log must be provided when use_gate_in_kernel=True."
        A_log, dt_bias_h = kwargs["A_log"], kwargs.get("dt_bias")
        if dt_bias_h is not None:      # one bias per head: the kernels take one per (head, channel)
            dt_bias = dt_bias_h.float().reshape(H, 1).expand(H, 128).reshape(H * 128)
    assert_blackwell(q.device)
    _poll_status(q.device)
    if scale is None:
        scale = k.shape[-1] ** -0.5
    keep = bool(disable_recompute) and torch.is_grad_enabled() and any(
        t is not None and t.requires_grad for t in (q, k, v, g, beta, A_log, dt_bias_h, initial_state))
    # a 3-D g tells the shared autograd function (and the kernels) that the gate is per (token, head)
    return ChunkKDAFunction.apply(q, k, v, g, beta, A_log, dt_bias, scale, initial_state, output_final_state,
                                  use_qk_l2norm_in_kernel, use_gate_in_kernel, cu_seqlens, cu_seqlens_cpu, False, None,
                                  disable_recompute, False, keep)
