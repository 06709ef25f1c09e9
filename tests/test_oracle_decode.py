"""Pins the decode oracle (oracle/decode.py) to the golden-pinned recurrence oracle: decode steps applied one after
the other must equal the token recurrence over the same tokens (softplus gate, beta = sigmoid(b), L2-normalised q/k,
grouped value heads), for both state layouts and with skipped sequences."""
import torch

from oracle.decode import kda_decode_oracle
from oracle.naive_kda import err_ratio, kda_gate, l2norm, naive_recurrent_kda


def _inputs(N, T, H, HV, seed):
    gen = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=gen)
    return dict(q=r(N, T, H, 128), k=r(N, T, H, 128), v=r(N, T, HV, 128), a=0.5 * r(N, T, HV, 128), b=r(N, T, HV),
                A_log=-2 * torch.rand(HV, generator=gen), dt_bias=0.1 * r(HV, 128), S0=0.1 * r(N, HV, 128, 128))


def test_decode_steps_equal_the_recurrence():
    N, T, H, HV = 2, 3, 2, 4
    d = _inputs(N, T, H, HV, 0)
    rep = HV // H
    qx, kx = d["q"].repeat_interleave(rep, dim=2), d["k"].repeat_interleave(rep, dim=2)       # one q/k head per value head
    g = kda_gate(d["a"], d["A_log"], d["dt_bias"].reshape(-1), None)                            # softplus form
    o_ref, S_ref = naive_recurrent_kda(l2norm(qx), l2norm(kx), d["v"], g, torch.sigmoid(d["b"]),
                                       initial_state=d["S0"], output_final_state=True)         # S as [N, HV, K, V]
    for layout in ("kv", "vk"):
        state = d["S0"].clone() if layout == "kv" else d["S0"].transpose(-1, -2).contiguous()
        outs = []
        for t in range(T):
            o, state = kda_decode_oracle(d["q"][:, t], d["k"][:, t], d["v"][:, t], d["a"][:, t], d["b"][:, t], d["A_log"],
                                         d["dt_bias"], state, state_layout=layout)
            outs.append(o)
        o = torch.stack(outs, dim=1)
        S = state if layout == "kv" else state.transpose(-1, -2)
        assert err_ratio(o_ref, o) < 1e-5 and err_ratio(S_ref, S) < 1e-5, layout


def test_decode_oracle_indices_and_skips():
    N, H, HV = 3, 1, 2
    d = _inputs(N, 1, H, HV, 1)
    pool = torch.randn(5, HV, 128, 128, generator=torch.Generator().manual_seed(2)) * 0.1
    idx = torch.tensor([4, -1, 0], dtype=torch.int32)
    o, new = kda_decode_oracle(d["q"][:, 0], d["k"][:, 0], d["v"][:, 0], d["a"][:, 0], d["b"][:, 0], d["A_log"], d["dt_bias"],
                               pool, indices=idx)
    assert torch.equal(new[1:4], pool[1:4]) and not torch.equal(new[4], pool[4]) and not torch.equal(new[0], pool[0])
    assert float(o[1].abs().max()) == 0.0
    o_single, _ = kda_decode_oracle(d["q"][2:, 0], d["k"][2:, 0], d["v"][2:, 0], d["a"][2:, 0], d["b"][2:, 0], d["A_log"],
                                    d["dt_bias"], pool[0:1])
    assert err_ratio(o_single[0], o[2]) < 1e-6
