"""``fused_kda_gate`` and ``fused_beta_sigmoid``: the oracle's gate against the stored outputs of the third-party naive
functions (CPU), and the CUDA operators against both (GPU), forward and gradients. Tolerances: fp32 outputs 1e-5
relative RMS (approximate exponentials in-kernel), bf16 outputs 4e-3 (one bf16 rounding)."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN_DIR
from oracle.naive_kda import err_ratio, kda_gate


def _golden():
    z = np.load(os.path.join(GOLDEN_DIR, "gate_activations.npz"))
    g = torch.from_numpy(z["g"].view(np.int16).copy()).view(torch.bfloat16)
    t = lambda k: torch.from_numpy(z[k].copy())
    return z, g, t("A_log"), t("dt_bias"), t("dy"), t


@pytest.mark.parametrize("mode", ["softplus", "lower_bound"])
def test_oracle_gate_matches_third_party_naive_gate(mode):
    z, g, A_log, dt_bias, dy, t = _golden()
    leaves = [x.clone().float().requires_grad_(True) for x in (g, A_log, dt_bias)]
    y = kda_gate(leaves[0], leaves[1], leaves[2], lower_bound=-5.0 if mode == "lower_bound" else None)
    (y * dy).sum().backward()
    assert err_ratio(t(f"{mode}_y"), y.detach()) < 1e-6
    for leaf, name in zip(leaves, ("dg", "dA_log", "ddt_bias")):
        assert err_ratio(t(f"{mode}_{name}"), leaf.grad) < 2e-6, name


@pytest.mark.gpu
@pytest.mark.parametrize("g_dtype,out_dtype", [(torch.bfloat16, torch.float32), (torch.float32, torch.bfloat16)])
@pytest.mark.parametrize("mode", ["softplus", "lower_bound"])
def test_fused_kda_gate_matches_golden_and_oracle(mode, g_dtype, out_dtype):
    from cula_b200.kda import fused_kda_gate
    z, g, A_log, dt_bias, dy, t = _golden()
    lb = -5.0 if mode == "lower_bound" else None
    dev = [g.to(g_dtype).cuda().requires_grad_(True), A_log.cuda().requires_grad_(True), dt_bias.cuda().requires_grad_(True)]
    y = fused_kda_gate(dev[0], dev[1], dev[2], lower_bound=lb, output_dtype=out_dtype)
    assert y.dtype == out_dtype and y.shape == g.shape
    (y.float() * dy.cuda()).sum().backward()
    torch.cuda.synchronize()
    tol = 1e-5 if out_dtype == torch.float32 else 4e-3
    assert err_ratio(t(f"{mode}_y"), y.detach().float().cpu()) < tol
    assert dev[0].grad.dtype == g_dtype
    # a bf16 output hands the upstream gradient over in bf16, a bf16 gate receives its gradient in bf16
    gtol = 4e-3 if torch.bfloat16 in (g_dtype, out_dtype) else 1e-5
    assert err_ratio(t(f"{mode}_dg"), dev[0].grad.float().cpu()) < gtol
    assert err_ratio(t(f"{mode}_dA_log"), dev[1].grad.cpu()) < (2e-2 if out_dtype == torch.bfloat16 else 1e-4)   # sums of signed terms: bf16 upstream gradients do not cancel exactly
    assert err_ratio(t(f"{mode}_ddt_bias"), dev[2].grad.cpu()) < (2e-2 if out_dtype == torch.bfloat16 else 1e-4)   # sums of signed terms: bf16 upstream gradients do not cancel exactly


@pytest.mark.gpu
def test_fused_kda_gate_wide_shape_without_bias():
    """[B, T, H, K] with H = 32 (several heads per block, many token slabs), no dt_bias."""
    from cula_b200.kda import fused_kda_gate
    gen = torch.Generator().manual_seed(5)
    g = torch.randn(2, 300, 32, 128, generator=gen).to(torch.bfloat16)
    A_log = 0.3 * torch.randn(32, generator=gen)
    dy = torch.randn(2, 300, 32, 128, generator=gen)
    ref_in = [g.float().requires_grad_(True), A_log.clone().requires_grad_(True)]
    (kda_gate(ref_in[0], ref_in[1], None, lower_bound=-5.0) * dy).sum().backward()
    dev = [g.cuda().requires_grad_(True), A_log.cuda().requires_grad_(True)]
    y = fused_kda_gate(dev[0], dev[1], None, lower_bound=-5.0)
    (y * dy.cuda()).sum().backward()
    torch.cuda.synchronize()
    assert err_ratio(kda_gate(g, A_log, None, lower_bound=-5.0), y.detach().cpu()) < 1e-5
    assert err_ratio(ref_in[0].grad, dev[0].grad.float().cpu()) < 4e-3
    assert err_ratio(ref_in[1].grad, dev[1].grad.cpu()) < 1e-4


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_fused_beta_sigmoid(dtype):
    from cula_b200.kda import fused_beta_sigmoid
    gen = torch.Generator().manual_seed(6)
    x = (3.0 * torch.randn(3, 1001, 7, generator=gen)).to(dtype)
    dy = torch.randn(3, 1001, 7, generator=gen)
    ref = x.detach().float().clone().requires_grad_(True)
    (torch.sigmoid(ref) * dy).sum().backward()
    dev = x.detach().clone().cuda().requires_grad_(True)
    y = fused_beta_sigmoid(dev)
    assert y.dtype == torch.float32
    (y * dy.cuda()).sum().backward()
    torch.cuda.synchronize()
    assert err_ratio(torch.sigmoid(x.float()), y.detach().cpu()) < 1e-6
    assert dev.grad.dtype == dtype
    assert err_ratio(ref.grad, dev.grad.float().cpu()) < (4e-3 if dtype == torch.bfloat16 else 1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("beta_dtype", [torch.bfloat16, torch.float32])
def test_beta_sigmoid_inside_chunk_kda(beta_dtype):
    """Raw beta logits into chunk_kda (sigmoid in-kernel, gradient w.r.t. the logits out) equal the two-step path
    fused_beta_sigmoid -> chunk_kda, and the oracle with torch.sigmoid."""
    from cula_b200.kda import chunk_kda
    from cula_b200.synthetic import make_inputs
    from oracle.naive_kda import chunk_kda_oracle
    B, T, H = 2, 150, 2
    inp = make_inputs(B, T, H, seed=8, gate_offset=-7.0, h0_std=0.5)
    gen = torch.Generator().manual_seed(9)
    logits = (1.5 * torch.randn(B, T, H, generator=gen)).to(beta_dtype)
    do = torch.randn(B, T, H, 128, generator=gen).to(torch.bfloat16)
    kw = dict(use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, safe_gate=True, lower_bound=-5.0)
    ref_in = {n: inp[n].float().requires_grad_(True) for n in ("q", "k", "v", "g")}
    ref_b = logits.detach().float().clone().requires_grad_(True)
    o_ref, _ = chunk_kda_oracle(ref_in["q"], ref_in["k"], ref_in["v"], ref_in["g"], torch.sigmoid(ref_b),
                                initial_state=inp["initial_state"], A_log=inp["A_log"], dt_bias=inp["dt_bias"], **kw)
    (o_ref * do.float()).sum().backward()
    d = {n: inp[n].cuda() for n in ("q", "k", "v", "g", "A_log", "dt_bias", "initial_state")}
    dev_b = logits.detach().clone().cuda().requires_grad_(True)
    o, _ = chunk_kda(d["q"], d["k"], d["v"], d["g"], dev_b, initial_state=d["initial_state"], A_log=d["A_log"],
                     dt_bias=d["dt_bias"], use_beta_sigmoid_in_kernel=True, **kw)
    o.backward(do.cuda())
    torch.cuda.synchronize()
    assert err_ratio(o_ref.detach(), o.detach().float().cpu()) <= 5e-3
    assert dev_b.grad.dtype == beta_dtype and err_ratio(ref_b.grad, dev_b.grad.float().cpu()) <= 2e-2
