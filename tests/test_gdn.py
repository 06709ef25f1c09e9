"""GPU parity of the scalar-gate variant, ``chunk_gated_delta_rule`` (one decay per token and head), forward and all
gradients: against the golden vectors produced by the third-party naive function, and against this repository's
oracle on seeded inputs (fixed length, packed, in-kernel gate, fp32 and bf16 gates). Tolerances as for chunk_kda:
o rel-RMS <= 5e-3, final state <= 2e-3, gradients 8e-3 (2e-2 for the gate and beta), the reference suite's bounds
(tests/test_kda.py:145-155)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from conftest import GDN_GOLDEN_CASES, load_golden
from oracle.naive_gdn import chunk_gdn_oracle
from oracle.naive_kda import err_ratio

pytestmark = pytest.mark.gpu
TOL = {"default": 8e-3, "g": 2e-2, "beta": 2e-2, "A_log": 2e-2}


def _run(leaves_cpu, flags, do, dht, cu=None, **kw):
    from cula_b200.gdn import chunk_gated_delta_rule
    from cula_b200.kda import check_status
    dev = {n: t.detach().cuda().requires_grad_(True) for n, t in leaves_cpu.items()}
    extra = {n: dev[n] for n in ("A_log", "dt_bias") if n in dev}
    o, ht = chunk_gated_delta_rule(dev["q"], dev["k"], dev["v"], dev["g"], dev["beta"], initial_state=dev.get("h0"),
                                   output_final_state=True, cu_seqlens=None if cu is None else cu.cuda(), **flags, **extra, **kw)
    ((o.float() * do.cuda().float()).sum() + (ht * dht.cuda()).sum()).backward()
    torch.cuda.synchronize()
    check_status()
    got = {n: t.grad.float().cpu() for n, t in dev.items()}
    for n, t in dev.items():
        assert t.grad.shape == t.shape and t.grad.dtype == t.dtype, n
    return o.detach().float().cpu(), ht.detach().cpu(), got


def _check(o, ht, got, o_ref, ht_ref, ref, tag):
    bad = []
    if not err_ratio(o_ref, o) <= 5e-3:
        bad.append(f"o {err_ratio(o_ref, o):.2e}")
    if not err_ratio(ht_ref, ht) <= 2e-3:
        bad.append(f"ht {err_ratio(ht_ref, ht):.2e}")
    for n, r in ref.items():
        e = err_ratio(r, got[n])
        if not (e <= TOL.get(n, TOL["default"]) and torch.isfinite(got[n]).all()):
            bad.append(f"d{n} {e:.2e}")
    assert not bad, f"{tag}: " + "; ".join(bad)


@pytest.mark.parametrize("name", GDN_GOLDEN_CASES)
def test_scalar_gate_matches_golden(name):
    case, inp, exp = load_golden(name)
    names = [n for n in ("q", "k", "v", "g", "beta", "A_log", "dt_bias", "h0") if n in inp]
    flags = dict(use_qk_l2norm_in_kernel=case["use_l2norm"], use_gate_in_kernel=case["use_gate_in_kernel"])
    o, ht, got = _run({n: inp[n] for n in names}, flags, inp["do"], inp["dht"], cu=case["cu_seqlens"])
    _check(o, ht, got, exp["o"], exp["ht"], {n: exp["d" + n] for n in names}, name)


@pytest.mark.parametrize("B,T,H,g_dtype,gate_in,l2,recompute", [
    (2, 300, 3, torch.float32, False, True, True),
    (1, 63, 1, torch.bfloat16, False, False, False),
    (2, 1000, 4, torch.bfloat16, True, True, True),
    (1, 1, 2, torch.float32, False, True, True),
])
def test_scalar_gate_against_oracle(B, T, H, g_dtype, gate_in, l2, recompute):
    gen = torch.Generator().manual_seed(17)
    rn = lambda *s: torch.randn(*s, generator=gen)
    q, k, v = (rn(B, T, H, 128).to(torch.bfloat16) for _ in range(3))
    if not l2:
        q, k = (F.normalize(x.float(), dim=-1).to(torch.bfloat16) for x in (q, k))
    leaves = dict(q=q, k=k, v=v, beta=torch.sigmoid(rn(B, T, H)).to(torch.bfloat16), h0=0.5 * rn(B, H, 128, 128))
    if gate_in:
        leaves.update(g=(-3.0 + rn(B, T, H)).to(g_dtype), A_log=0.3 * rn(H), dt_bias=0.2 * rn(H))
    else:
        leaves["g"] = (F.logsigmoid(rn(B, T, H)) / 8.0).to(g_dtype)
    do, dht = rn(B, T, H, 128).to(torch.bfloat16), 0.3 * rn(B, H, 128, 128)
    flags = dict(use_qk_l2norm_in_kernel=l2, use_gate_in_kernel=gate_in)
    ref_in = {n: t.detach().float().requires_grad_(True) for n, t in leaves.items()}
    o_ref, ht_ref = chunk_gdn_oracle(ref_in["q"], ref_in["k"], ref_in["v"], ref_in["g"], ref_in["beta"], initial_state=ref_in["h0"],
                                     output_final_state=True, A_log=ref_in.get("A_log"), dt_bias=ref_in.get("dt_bias"), **flags)
    ((o_ref * do.float()).sum() + (ht_ref * dht).sum()).backward()
    o, ht, got = _run(leaves, flags, do, dht, disable_recompute=not recompute)
    _check(o, ht, got, o_ref.detach(), ht_ref.detach(), {n: t.grad for n, t in ref_in.items()}, f"B{B}T{T}H{H}")


def test_scalar_gate_equals_chunk_kda_with_broadcast_gate():
    """Same kernels, same arithmetic: the scalar-gate call must reproduce chunk_kda fed the gate expanded over the
    channels, bit for bit in the forward outputs."""
    from cula_b200.gdn import chunk_gated_delta_rule
    from cula_b200.kda import chunk_kda
    gen = torch.Generator().manual_seed(3)
    B, T, H = 2, 200, 2
    q, k, v = (torch.randn(B, T, H, 128, generator=gen).to(torch.bfloat16).cuda() for _ in range(3))
    g = (F.logsigmoid(torch.randn(B, T, H, generator=gen)) / 8.0).cuda()
    beta = torch.sigmoid(torch.randn(B, T, H, generator=gen)).to(torch.bfloat16).cuda()
    o1, s1 = chunk_gated_delta_rule(q, k, v, g, beta, output_final_state=True, use_qk_l2norm_in_kernel=True)
    o2, s2 = chunk_kda(q, k, v, g[..., None].expand(B, T, H, 128).contiguous(), beta, output_final_state=True,
                       use_qk_l2norm_in_kernel=True)
    torch.cuda.synchronize()
    assert torch.equal(o1, o2) and torch.equal(s1, s2)


def test_argument_errors():
    from cula_b200.gdn import chunk_gated_delta_rule
    q = torch.zeros(2, 8, 1, 128, dtype=torch.bfloat16)
    g = torch.zeros(2, 8, 1)
    with pytest.raises(ValueError, match="batch size is expected to be 1"):
        chunk_gated_delta_rule(q, q, q, g, g, cu_seqlens=torch.tensor([0, 8], dtype=torch.int32))
    with pytest.raises(AssertionError):
        chunk_gated_delta_rule(q, q, q, torch.zeros(2, 8, 1, 128), g)
    with pytest.raises(AssertionError, match="A_log"):
        chunk_gated_delta_rule(q, q, q, g, g, use_gate_in_kernel=True)
