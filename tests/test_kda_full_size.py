"""Parity at the sizes the headline configurations name. The plain-C oracle is fast enough to check the forward
outputs directly at B=2, T=2048, H=32 and on the 64-sequence / 65,536-token packed batch; larger shapes and the
backward pass are checked through size-independent properties: splitting a sequence and carrying the state
(forward) or the state gradient (backward) across the cut must reproduce the unsplit result, and the gradients
are exactly linear in the upstream gradient (the internal gradient scale is a power of two)."""
import numpy as np
import pytest
import torch

from oracle import c_oracle
from oracle.naive_kda import err_ratio, make_inputs

pytestmark = pytest.mark.gpu
KW = dict(use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, safe_gate=True, lower_bound=-5.0)


def _fwd(d, **extra):
    from cula_b200.kda import chunk_kda
    return chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], A_log=d["A_log"], dt_bias=d["dt_bias"], **KW, **extra)


def _oracle(inp, cu=None, h0=None):
    f = lambda x: None if x is None else x.float().numpy()
    o, ht = c_oracle.naive_kda_fwd(f(inp["q"]), f(inp["k"]), f(inp["v"]), f(inp["g"]), f(inp["beta"]), f(inp["A_log"]),
                                   f(inp["dt_bias"]), f(h0), cu_seqlens=None if cu is None else cu.numpy(),
                                   use_l2norm=True, gate_mode=2, lower_bound=-5.0)
    return torch.from_numpy(o), torch.from_numpy(ht)


@pytest.mark.parametrize("gate_offset", [0.0, -8.0])
def test_headline_forward_B2_T2048_H32_against_oracle(gate_offset):
    from cula_b200.kda import check_status
    inp = make_inputs(2, 2048, 32, seed=0, gate_offset=gate_offset)
    d = {k: v.cuda() for k, v in inp.items() if v is not None}
    o, ht = _fwd(d, output_final_state=True)
    torch.cuda.synchronize()
    check_status()
    o_ref, ht_ref = _oracle(inp)
    o = o.float().cpu()
    assert err_ratio(o_ref, o) <= 5e-3 and float((o_ref - o).abs().max()) <= 2e-2
    assert err_ratio(ht_ref, ht.cpu()) <= (1e-3 if gate_offset == 0.0 else 2e-3)


def test_packed_64_sequences_65536_tokens_against_oracle():
    """The varlen headline shape (64 sequences, lognormal lengths, 65,536 tokens) at H=8."""
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location("bench", os.path.join(os.path.dirname(os.path.dirname(__file__)), "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    lens = bench.varlen_lengths(64, 65536, seed=0)
    assert sum(lens) == 65536 and min(lens) >= 63 and max(lens) <= 8192
    H = 8
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)
    inp = make_inputs(1, 65536, H, seed=4, gate_offset=-7.0)
    d = {k: v.cuda() for k, v in inp.items() if v is not None}
    o, ht = _fwd(d, output_final_state=True, cu_seqlens=cu.cuda())
    torch.cuda.synchronize()
    o_ref, ht_ref = _oracle(inp, cu=cu)
    o = o.float().cpu()
    assert err_ratio(o_ref, o) <= 5e-3 and float((o_ref - o).abs().max()) <= 2e-2
    assert err_ratio(ht_ref, ht.cpu()) <= 2e-3


def test_forward_split_with_carried_state_B4_T8192_H32():
    """o(full) == o(first half) ++ o(second half started from the first half's final state)."""
    B, T, H = 4, 8192, 32
    inp = make_inputs(B, T, H, seed=1, gate_offset=-8.0, h0_std=0.1)
    d = {k: v.cuda() for k, v in inp.items()}
    o, ht = _fwd(d, output_final_state=True, initial_state=d["initial_state"])
    half = lambda t, sl: {k: (v[:, sl].contiguous() if k in ("q", "k", "v", "g", "beta") else v) for k, v in t.items()}
    o1, h1 = _fwd(half(d, slice(0, T // 2)), output_final_state=True, initial_state=d["initial_state"])
    o2, h2 = _fwd(half(d, slice(T // 2, T)), output_final_state=True, initial_state=h1)
    torch.cuda.synchronize()
    assert torch.equal(o[:, :T // 2], o1)                  # same kernels on the same chunks: bit-identical
    assert torch.equal(o[:, T // 2:], o2) and torch.equal(ht, h2)
    assert torch.isfinite(o.float()).all() and float(o.float().abs().max()) > 0


def test_backward_split_and_linearity_B2_T2048_H8():
    """Gradients of the whole sequence == gradients of the two halves chained through dh0 -> dht, and they are
    exactly linear in the upstream gradient."""
    from cula_b200.kda import chunk_kda
    B, T, H = 2, 2048, 8
    inp = make_inputs(B, T, H, seed=2, gate_offset=-8.0, h0_std=0.5)
    gen = torch.Generator().manual_seed(3)
    do = torch.randn(B, T, H, 128, generator=gen).to(torch.bfloat16).cuda()
    names = ("q", "k", "v", "g", "beta")

    def run(sl, h0, dout, dht):
        leaves = {n: inp[n][:, sl].cuda().requires_grad_(True) for n in names}
        h0 = h0.detach().clone().requires_grad_(True)
        o, ht = chunk_kda(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"], A_log=inp["A_log"].cuda(),
                          dt_bias=inp["dt_bias"].cuda(), initial_state=h0, output_final_state=True, **KW)
        loss = (o.float() * dout.float()).sum()
        if dht is not None:
            loss = loss + (ht * dht).sum()
        loss.backward()
        return {n: leaves[n].grad for n in names}, h0.grad, ht.detach()

    full, dh0_full, _ = run(slice(0, T), inp["initial_state"].cuda(), do, None)
    _, _, h_mid = run(slice(0, T // 2), inp["initial_state"].cuda(), do[:, :T // 2], None)
    g2, dh_mid, _ = run(slice(T // 2, T), h_mid, do[:, T // 2:], None)
    g1, dh0_split, _ = run(slice(0, T // 2), inp["initial_state"].cuda(), do[:, :T // 2], dh_mid)
    for n in names:
        both = torch.cat([g1[n], g2[n]], dim=1).float()
        assert err_ratio(full[n].float().cpu(), both.cpu()) <= 4e-3, n      # bf16 outputs, different gradient scales
    assert err_ratio(dh0_full.cpu(), dh0_split.cpu()) <= 1e-3
    twice, dh0_twice, _ = run(slice(0, T), inp["initial_state"].cuda(), (do.float() * 2).to(torch.bfloat16), None)
    for n in names:
        assert torch.equal(twice[n].float(), 2 * full[n].float()), n
    assert torch.equal(dh0_twice, 2 * dh0_full)
