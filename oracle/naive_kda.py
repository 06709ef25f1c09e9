"""CPU oracle for the chunk_kda hot path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Only tests/, the smoke check and the benchmark's CPU-baseline leg may import this module.

It restates, as a plain fp32 (or fp64) token-by-token recurrence, what the reference checks
its kernels against:

* the Kimi-Delta-Attention recurrence -- semantics of flash-linear-attention's
  ``naive_recurrent_kda`` (third-party dependency of the reference, un-vendored submodule
  ``third_party/flash-linear-attention``; the installed copy is 0.5.1, file
  ``fla/ops/kda/naive.py:12-66``), which the reference's own tests call at
  ``tests/test_kda.py:106-114`` and ``tests/test_kda.py:259-267``;
* the two gate activations -- ``fla/ops/kda/gate.py:26-54`` (softplus form) and
  ``fla/ops/kda/gate.py:57-69`` (lower-bound / "safe" sigmoid form);
* the L2 normalisation the reference test applies with ``F.normalize`` (``tests/test_kda.py:107-108``).

Parity pin: ``tests/golden/*.npz`` were produced by running the third-party naive functions
themselves (script ``tests/golden/make_golden.py``); ``tests/test_oracle.py`` checks this
restatement against those stored outputs and gradients.

Published algorithm, per (sequence, head), state S in R^{K x V}::

    S  <- diag(exp(a_t)) S
    S  <- S + (beta_t k_t) (v_t - S^T k_t)^T
    o_t = S^T (scale q_t)
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def kda_gate(g, A_log, dt_bias=None, lower_bound=None):
    """Gate activation applied when ``use_gate_in_kernel=True``.

    ``lower_bound`` given  -> a = lower_bound * sigmoid(exp(A_log[h]) * (g + dt_bias[h, :]))
    ``lower_bound`` absent -> a = -exp(A_log[h]) * softplus(g + dt_bias[h, :])
    ``g`` is [..., H, K]; ``A_log`` has H elements; ``dt_bias`` has H*K elements.
    """
    H, K = g.shape[-2:]
    x = g.float()
    if dt_bias is not None:
        x = x + dt_bias.float().view(H, K)
    alpha = A_log.float().view(H, 1).exp()
    if lower_bound is not None:
        return lower_bound * torch.sigmoid(alpha * x)
    return -alpha * F.softplus(x)


def l2norm(x):
    """Row-wise L2 normalisation as the reference test does it (F.normalize, eps 1e-12)."""
    return F.normalize(x.float(), p=2, dim=-1)


def naive_recurrent_kda(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
                        dtype=torch.float32):
    """Token recurrence over [B, T, H, *] tensors; ``g`` is the natural-log decay (<= 0).

    Returns (o [B,T,H,V], S [B,H,K,V] or None) in ``dtype``.
    """
    B, T, H, K = q.shape
    V = v.shape[-1]
    if scale is None:
        scale = K ** -0.5
    q, k, v, g, beta = (x.to(dtype) for x in (q, k, v, g, beta))
    S = torch.zeros(B, H, K, V, dtype=dtype, device=q.device)     # runs wherever the inputs live (CPU by default)
    if initial_state is not None:
        S = S + initial_state.to(dtype)
    outs = []
    for t in range(T):
        S = S * g[:, t].exp().unsqueeze(-1)                       # decay each key channel
        resid = v[:, t] - torch.einsum("bhk,bhkv->bhv", k[:, t], S)
        S = S + torch.einsum("bhk,bhv->bhkv", beta[:, t].unsqueeze(-1) * k[:, t], resid)
        outs.append(torch.einsum("bhk,bhkv->bhv", q[:, t] * scale, S))
    o = torch.stack(outs, dim=1)
    return o, (S if output_final_state else None)


def chunk_kda_oracle(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
                     use_qk_l2norm_in_kernel=False, use_gate_in_kernel=False, cu_seqlens=None,
                     safe_gate=False, lower_bound=None, A_log=None, dt_bias=None,
                     dtype=torch.float32):
    """Same keyword surface as ``chunk_kda`` (``cula/kda/chunk.py:217-412``), evaluated with the
    token recurrence. Inputs may require grad; autograd supplies every gradient.

    With ``cu_seqlens`` (packed batch, B == 1) each sequence is run on its own with its own
    initial state, as ``tests/test_kda.py:259-267`` does.
    """
    if use_qk_l2norm_in_kernel:
        q, k = l2norm(q), l2norm(k)
    if use_gate_in_kernel:
        g = kda_gate(g, A_log, dt_bias, lower_bound if safe_gate else None)
    if cu_seqlens is None:
        return naive_recurrent_kda(q, k, v, g, beta, scale, initial_state, output_final_state, dtype)
    bounds = [int(x) for x in cu_seqlens]
    outs, finals = [], []
    for n in range(len(bounds) - 1):
        s, e = bounds[n], bounds[n + 1]
        h0 = None if initial_state is None else initial_state[n:n + 1]
        o_n, s_n = naive_recurrent_kda(q[:, s:e], k[:, s:e], v[:, s:e], g[:, s:e], beta[:, s:e],
                                       scale, h0, True, dtype)
        outs.append(o_n)
        finals.append(s_n)
    o = torch.cat(outs, dim=1)
    return o, (torch.cat(finals, dim=0) if output_final_state else None)


def err_ratio(ref, out):
    """Relative RMS error ||ref - out|| / ||ref|| -- the metric of the reference's ``assert_close``
    (``fla/utils.py:96-115``)."""
    ref, out = ref.double().flatten(), out.double().flatten()
    return float(((ref - out).square().mean().sqrt() / (ref.square().mean().sqrt() + 1e-300)))


from cula_b200.synthetic import make_inputs  # noqa: E402,F401  (re-exported for the tests)
