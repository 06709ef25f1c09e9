"""The CPU oracles (torch and plain C) against the stored outputs of the reference's own test oracle."""
import numpy as np
import pytest
import torch

from conftest import GDN_GOLDEN_CASES, GOLDEN_CASES, load_golden
from oracle import c_oracle
from oracle.naive_kda import chunk_kda_oracle, err_ratio, kda_gate


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_torch_oracle_matches_golden(name):
    case, inp, exp = load_golden(name)
    leaves = {n: inp[n].float().requires_grad_(True) for n in ("q", "k", "v", "g", "beta", "A_log", "dt_bias", "h0")
              if n in inp}
    o, ht = chunk_kda_oracle(
        leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"],
        initial_state=leaves.get("h0"), output_final_state=True,
        use_qk_l2norm_in_kernel=case["use_l2norm"], use_gate_in_kernel=case["use_gate_in_kernel"],
        cu_seqlens=case["cu_seqlens"], safe_gate=case["safe_gate"], lower_bound=case["lower_bound"],
        A_log=leaves.get("A_log"), dt_bias=leaves.get("dt_bias"))
    ((o * inp["do"].float()).sum() + (ht * inp["dht"]).sum()).backward()
    assert err_ratio(exp["o"], o.detach()) < 1e-6
    assert err_ratio(exp["ht"], ht.detach()) < 1e-6
    for n, t in leaves.items():
        assert err_ratio(exp["d" + n], t.grad) < 2e-6, n


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_c_oracle_matches_golden(name):
    case, inp, exp = load_golden(name)
    gate_mode = 0 if not case["use_gate_in_kernel"] else (2 if case["safe_gate"] else 1)
    f = lambda n: None if n not in inp else inp[n].float().numpy()
    o, ht = c_oracle.naive_kda_fwd(
        f("q"), f("k"), f("v"), f("g"), f("beta"), f("A_log"), f("dt_bias"), f("h0"),
        cu_seqlens=None if case["cu_seqlens"] is None else case["cu_seqlens"].numpy(),
        use_l2norm=case["use_l2norm"], gate_mode=gate_mode,
        lower_bound=case["lower_bound"] if case["lower_bound"] is not None else 0.0)
    assert err_ratio(exp["o"], torch.from_numpy(o)) < 2e-6
    assert err_ratio(exp["ht"], torch.from_numpy(ht)) < 2e-6
    assert np.isfinite(o).all()


def test_gate_forms():
    g = torch.linspace(-6, 6, 2 * 3 * 4).view(2, 3, 4)
    A_log = torch.tensor([0.1, -0.2, 0.3])
    bias = torch.arange(12, dtype=torch.float32) * 0.05
    a = kda_gate(g, A_log, bias, lower_bound=-5.0)
    assert (a < 0).all() and (a > -5).all()
    x = g + bias.view(3, 4)
    assert torch.allclose(a, -5.0 * torch.sigmoid(A_log.exp().view(3, 1) * x))
    b = kda_gate(g, A_log, bias, lower_bound=None)
    assert torch.allclose(b, -A_log.exp().view(3, 1) * torch.nn.functional.softplus(x))


def test_c_oracle_thread_count():
    assert c_oracle.num_threads() >= 1


@pytest.mark.parametrize("name", GDN_GOLDEN_CASES)
def test_scalar_gate_oracle_matches_golden(name):
    """The gated-delta-rule restatement against outputs and gradients of the third-party naive function."""
    from oracle.naive_gdn import chunk_gdn_oracle
    case, inp, exp = load_golden(name)
    leaves = {n: inp[n].float().requires_grad_(True) for n in ("q", "k", "v", "g", "beta", "A_log", "dt_bias", "h0") if n in inp}
    o, ht = chunk_gdn_oracle(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"], initial_state=leaves["h0"],
                             output_final_state=True, use_qk_l2norm_in_kernel=case["use_l2norm"],
                             cu_seqlens=case["cu_seqlens"], use_gate_in_kernel=case["use_gate_in_kernel"],
                             A_log=leaves.get("A_log"), dt_bias=leaves.get("dt_bias"))
    ((o * inp["do"].float()).sum() + (ht * inp["dht"]).sum()).backward()
    assert err_ratio(exp["o"], o.detach()) < 1e-6 and err_ratio(exp["ht"], ht.detach()) < 1e-6
    for n, t in leaves.items():
        assert err_ratio(exp["d" + n], t.grad) < 2e-6, n


def test_scalar_gate_is_the_per_channel_recurrence_with_equal_gates():
    """The kernels run the scalar-gate variant as KDA with one gate value for all channels: the two oracles agree."""
    from oracle.naive_gdn import naive_recurrent_gdn
    from oracle.naive_kda import naive_recurrent_kda
    gen = torch.Generator().manual_seed(0)
    B, T, H = 2, 40, 2
    q, k, v = (torch.randn(B, T, H, 128, generator=gen) for _ in range(3))
    k = torch.nn.functional.normalize(k, dim=-1)
    g = torch.nn.functional.logsigmoid(torch.randn(B, T, H, generator=gen))
    beta = torch.rand(B, T, H, generator=gen)
    h0 = torch.randn(B, H, 128, 128, generator=gen)
    o1, s1 = naive_recurrent_gdn(q, k, v, g, beta, None, h0, True)
    o2, s2 = naive_recurrent_kda(q, k, v, g[..., None].expand(B, T, H, 128), beta, None, h0, True)
    assert err_ratio(o1, o2) < 1e-6 and err_ratio(s1, s2) < 1e-6
