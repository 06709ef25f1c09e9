"""CPU oracle for the scalar-gate variant (gated delta rule) -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Only tests/ may import this module. It restates, token by token in fp32, flash-linear-attention's
``naive_recurrent_gated_delta_rule`` (third-party dependency of the reference, installed copy 0.5.1, file
``fla/ops/gated_delta_rule/naive.py:12-66``): per (sequence, head), state S in R^{K x V}::

    S  <- exp(g_t) S                       (one decay per token and head)
    S  <- S + k_t (beta_t (v_t - S^T k_t))^T
    o_t = S^T (scale q_t)

and the gate activation used when the gate is computed in-kernel, ``g = -exp(A_log[h]) softplus(x + dt_bias[h])``
(the docstring of ``fla/ops/gated_delta_rule/chunk.py``: ``use_gate_in_kernel``).

Parity pin: ``tests/golden/gdn_*.npz`` were produced by running the third-party function itself
(``tests/golden/make_golden.py``); ``tests/test_oracle.py`` checks this restatement against them.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def gdn_gate(g, A_log, dt_bias=None):
    """``-exp(A_log[h]) * softplus(g + dt_bias[h])`` for ``g`` [..., H]."""
    x = g.float()
    if dt_bias is not None:
        x = x + dt_bias.float()
    return -A_log.float().exp() * F.softplus(x)


def naive_recurrent_gdn(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
                        dtype=torch.float32):
    """q, k [B,T,H,K]; v [B,T,H,V]; g, beta [B,T,H] (g: natural-log decay). Returns (o [B,T,H,V], S or None)."""
    B, T, H, K = q.shape
    V = v.shape[-1]
    if scale is None:
        scale = K ** -0.5
    q, k, v, g, beta = (x.to(dtype) for x in (q, k, v, g, beta))
    S = torch.zeros(B, H, K, V, dtype=dtype, device=q.device)
    if initial_state is not None:
        S = S + initial_state.to(dtype)
    outs = []
    for t in range(T):
        S = S * g[:, t].exp()[..., None, None]
        resid = (v[:, t] - torch.einsum("bhk,bhkv->bhv", k[:, t], S)) * beta[:, t].unsqueeze(-1)
        S = S + torch.einsum("bhk,bhv->bhkv", k[:, t], resid)
        outs.append(torch.einsum("bhk,bhkv->bhv", q[:, t] * scale, S))
    return torch.stack(outs, dim=1), (S if output_final_state else None)


def chunk_gdn_oracle(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
                     use_qk_l2norm_in_kernel=False, cu_seqlens=None, use_gate_in_kernel=False, A_log=None, dt_bias=None,
                     dtype=torch.float32):
    """Keyword surface of ``chunk_gated_delta_rule``, evaluated with the token recurrence (autograd gives gradients)."""
    if use_qk_l2norm_in_kernel:
        q, k = F.normalize(q.float(), p=2, dim=-1), F.normalize(k.float(), p=2, dim=-1)
    if use_gate_in_kernel:
        g = gdn_gate(g, A_log, dt_bias)
    if cu_seqlens is None:
        return naive_recurrent_gdn(q, k, v, g, beta, scale, initial_state, output_final_state, dtype)
    bounds = [int(x) for x in cu_seqlens]
    outs, finals = [], []
    for n in range(len(bounds) - 1):
        s, e = bounds[n], bounds[n + 1]
        h0 = None if initial_state is None else initial_state[n:n + 1]
        o_n, s_n = naive_recurrent_gdn(q[:, s:e], k[:, s:e], v[:, s:e], g[:, s:e], beta[:, s:e], scale, h0, True, dtype)
        outs.append(o_n)
        finals.append(s_n)
    return torch.cat(outs, dim=1), (torch.cat(finals, dim=0) if output_final_state else None)
