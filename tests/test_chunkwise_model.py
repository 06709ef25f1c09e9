"""The fp64 chunkwise forward/backward model (the specification of the CUDA kernels) against autograd
of the token recurrence."""
import pytest
import torch

from chunkwise_ref import chunk_forward_backward
from oracle.naive_kda import err_ratio, naive_recurrent_kda


@pytest.mark.parametrize("T,gate", [(64, -0.05), (150, -0.3), (200, -2.5)])
def test_chunk_model_matches_autograd(T, gate):
    torch.manual_seed(0)
    K = V = 32                      # the algebra does not depend on the head size
    dt = torch.float64
    q = torch.nn.functional.normalize(torch.randn(T, K, dtype=dt), dim=-1).requires_grad_(True)
    k = torch.nn.functional.normalize(torch.randn(T, K, dtype=dt), dim=-1).requires_grad_(True)
    v = torch.randn(T, V, dtype=dt).requires_grad_(True)
    a = (gate * torch.rand(T, K, dtype=dt)).requires_grad_(True)
    beta = torch.rand(T, dtype=dt).requires_grad_(True)
    h0 = torch.randn(K, V, dtype=dt).requires_grad_(True)
    do, dht = torch.randn(T, V, dtype=dt), torch.randn(K, V, dtype=dt)
    scale = K ** -0.5
    o, ht = naive_recurrent_kda(q[None, :, None], k[None, :, None], v[None, :, None], a[None, :, None],
                                beta[None, :, None], scale, h0[None, None], True, dtype=dt)
    ((o[0, :, 0] * do).sum() + (ht[0, 0] * dht).sum()).backward()
    with torch.no_grad():
        m = chunk_forward_backward(q, k, v, a, beta, scale, h0, do, dht)
    assert err_ratio(o[0, :, 0], m["o"]) < 1e-10 and err_ratio(ht[0, 0], m["ht"]) < 1e-10
    for name, ref in (("dq", q.grad), ("dk", k.grad), ("dv", v.grad), ("da", a.grad), ("dbeta", beta.grad),
                      ("dh0", h0.grad)):
        assert err_ratio(ref, m[name]) < 1e-9, name
