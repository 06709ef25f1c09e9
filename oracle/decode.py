"""Test infrastructure only: fp32 restatement of one KDA decode step (not part of the product path).

Follows the reference's own torch restatement of its decode kernel (tests/test_kda_decode.py:42-104) and the
docstring of kda_decode (cula/ops/kda_decode.py:1845-1878):

    gate  = exp(-exp(A_log) * softplus(a + dt_bias))
    v_new = sigmoid(b) * (v - S^T (gate * k_hat))
    S_new = diag(gate) S + k_hat v_new^T            (S as [K, V]; the pool stores it as [V, K] or [K, V])
    o     = S_new^T (scale * q_hat)

Pinned by tests/test_oracle_decode.py: one decode step must equal one token of the (golden-pinned) recurrence
oracle `naive_recurrent_kda` with the softplus gate and beta = sigmoid(b).
"""
import torch
import torch.nn.functional as F


def kda_decode_oracle(q, k, v, a, b, A_log, dt_bias, state, scale=None, use_l2norm=True, softplus_beta=1.0,
                      softplus_threshold=20.0, state_layout="vk", indices=None):
    """q, k: [N, H, K]; v: [N, HV, V]; a: [N, HV, K]; b: [N, HV]; A_log: [HV]; dt_bias: [HV, K] or None;
    state: [pool, HV, V, K] ("vk") or [pool, HV, K, V] ("kv"). Returns (o [N, HV, V], new_state) in fp32; sequences
    with a negative index are skipped (zero output row, state untouched)."""
    q, k, v, a, b = (x.float() for x in (q, k, v, a, b))
    N, H, K = q.shape
    HV, V = v.shape[1], v.shape[2]
    scale = K ** -0.5 if scale is None else scale
    new_state = state.float().clone()
    o = torch.zeros(N, HV, V)
    rep = HV // H
    for n in range(N):
        slot = n if indices is None else int(indices[n])
        if slot < 0:
            continue
        for hv in range(HV):
            hq = hv // rep
            x = a[n, hv] + (dt_bias[hv].float() if dt_bias is not None else 0.0)
            gate = torch.exp(-torch.exp(A_log[hv].float()) * F.softplus(x, beta=softplus_beta, threshold=softplus_threshold))
            qv, kv = q[n, hq], k[n, hq]
            if use_l2norm:
                qv, kv = F.normalize(qv, dim=0), F.normalize(kv, dim=0)
            S = new_state[slot, hv]
            S = S.t() if state_layout == "vk" else S            # -> [K, V]
            v_new = torch.sigmoid(b[n, hv]) * (v[n, hv] - S.t() @ (gate * kv))
            S = gate[:, None] * S + kv[:, None] * v_new[None, :]
            o[n, hv] = S.t() @ (qv * scale)
            new_state[slot, hv] = S.t() if state_layout == "vk" else S
    return o, new_state
