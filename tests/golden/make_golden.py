"""Generate the golden vectors in this folder by running the reference's own test oracle.

The reference checks ``chunk_kda`` against flash-linear-attention's ``naive_recurrent_kda``,
``naive_kda_gate`` and ``naive_kda_lowerbound_gate`` (``tests/test_kda.py:22-23,106-114``). Those
functions are pure torch and import on a CPU-only machine that has ``fla`` installed. This script
calls THEM (not this repository's oracle) on small seeded inputs, takes gradients through torch
autograd with the reference test's loss ``(o*do).sum() + (ht*dht).sum()`` (``tests/test_kda.py:115``)
and stores inputs, outputs and gradients as ``.npz``.

    python tests/golden/make_golden.py          # needs `fla`; rewrites tests/golden/*.npz

bf16 tensors are stored as their raw uint16 bit patterns (numpy has no bfloat16).
"""
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))

# name, B, T, H, use_l2norm, use_gate_in_kernel, safe_gate, gate_offset, h0_std, seq lens (varlen) or None
CASES = [
    ("strong_gate_T130", 1, 130, 2, True, True, True, 0.0, 0.0, None),
    ("weak_gate_T200_h0", 1, 200, 2, True, True, True, -8.0, 0.5, None),
    ("softplus_gate_T96", 2, 96, 1, True, True, False, -4.0, 0.5, None),
    ("pre_gated_T63", 1, 63, 1, False, False, True, 0.0, 1.0, None),
    ("varlen_15_70_64_37", 1, 186, 1, True, True, True, -6.0, 0.5, [15, 70, 64, 37]),
    # the distributions of the reference's own grid (tests/test_kda.py:77-98): q, k, v ~ U(0,1) (all-positive,
    # highly correlated keys), log-sigmoid gates of which half are exactly 0 (no decay), h0 ~ N(0,1)
    ("uniform_qkv_masked_gate_T150", 1, 150, 2, False, False, True, "uniform", 1.0, None),
]


# Scalar-gate variant (gated delta rule): name, B, T, H, use_l2norm, use_gate_in_kernel, h0_std, seq lens or None.
# Oracle: fla.ops.gated_delta_rule.naive.naive_recurrent_gated_delta_rule and fla.ops.gated_delta_rule.gate.naive_gdn_gate.
GDN_CASES = [
    ("gdn_pre_gated_T150_h0", 1, 150, 2, True, False, 0.5, None),
    ("gdn_gate_in_kernel_varlen_40_100_65", 1, 205, 2, False, True, 0.5, [40, 100, 65]),
]


def bits(x):
    return x.view(torch.int16).numpy().view(np.uint16) if x.dtype == torch.bfloat16 else x.numpy()


def main():
    from fla.ops.kda.gate import naive_kda_gate, naive_kda_lowerbound_gate
    from fla.ops.kda.naive import naive_recurrent_kda

    K = V = 128
    for ci, (name, B, T, H, l2, gate_in, safe, goff, h0_std, lens) in enumerate(CASES):
        gen = torch.Generator().manual_seed(1000 + ci)
        rn = lambda *s: torch.randn(*s, generator=gen, dtype=torch.float32)
        uniform = goff == "uniform"
        if uniform:
            q, k, v = (torch.rand(B, T, H, K, generator=gen).to(torch.bfloat16) for _ in range(3))
        else:
            q, k, v = (rn(B, T, H, K).to(torch.bfloat16) for _ in range(3))
        if not l2:  # the caller normalises beforehand, as tests/test_kda.py:117-118 does
            q, k = (F.normalize(x.float(), p=2, dim=-1).to(torch.bfloat16) for x in (q, k))
        if gate_in:
            g = (goff + 0.1 * rn(B, T, H, K)).to(torch.bfloat16)
            A_log = 0.3 * rn(H)
            dt_bias = 0.2 * rn(H * K)
        else:  # gate already in log space, fp32, clamped to the safe range as tests/test_kda.py:88-91
            g = (F.logsigmoid(rn(B, T, H, K)) / 1.0).clamp(-5, 0)
            if uniform:
                g = g * (torch.rand(B, T, H, K, generator=gen) > 0.5)
            A_log = dt_bias = None
        beta = torch.sigmoid(rn(B, T, H)).to(torch.bfloat16)
        N = B if lens is None else len(lens)
        h0 = h0_std * rn(N, H, K, V) if h0_std > 0 else None
        do = rn(B, T, H, V).to(torch.bfloat16)
        dht = 0.3 * rn(N, H, K, V)
        lower_bound = -5.0 if (safe and gate_in) else None

        leaves = dict(q=q, k=k, v=v, g=g, beta=beta)
        if gate_in:
            leaves.update(A_log=A_log, dt_bias=dt_bias)
        if h0 is not None:
            leaves.update(h0=h0)
        req = {n: t.clone().float().requires_grad_(True) for n, t in leaves.items()}

        qn = F.normalize(req["q"], p=2, dim=-1) if l2 else req["q"]
        kn = F.normalize(req["k"], p=2, dim=-1) if l2 else req["k"]
        if gate_in:
            gate_fn = naive_kda_lowerbound_gate if safe else naive_kda_gate
            kw = dict(lower_bound=lower_bound) if safe else {}
            a = gate_fn(req["g"], req["A_log"], req["dt_bias"], **kw)
        else:
            a = req["g"]
        bounds = [0, T] if lens is None else np.concatenate([[0], np.cumsum(lens)]).tolist()
        if lens is None:
            o, ht = naive_recurrent_kda(qn, kn, req["v"], a, req["beta"],
                                        initial_state=req.get("h0"), output_final_state=True)
        else:
            os_, hs_ = [], []
            for n in range(N):
                s, e = bounds[n], bounds[n + 1]
                o_n, h_n = naive_recurrent_kda(qn[:, s:e], kn[:, s:e], req["v"][:, s:e], a[:, s:e],
                                               req["beta"][:, s:e],
                                               initial_state=None if h0 is None else req["h0"][n:n + 1],
                                               output_final_state=True)
                os_.append(o_n)
                hs_.append(h_n)
            o, ht = torch.cat(os_, 1), torch.cat(hs_, 0)
        ((o * do.float()).sum() + (ht * dht).sum()).backward()

        out = dict(B=B, T=T, H=H, use_l2norm=l2, use_gate_in_kernel=gate_in, safe_gate=safe,
                   lower_bound=np.float32(lower_bound if lower_bound is not None else np.nan),
                   cu_seqlens=np.asarray(bounds if lens is not None else [], dtype=np.int32),
                   do=bits(do), dht=dht.numpy(), o=o.detach().numpy(), ht=ht.detach().numpy())
        for n, t in leaves.items():
            out["in_" + n] = bits(t)
            out["in_" + n + "_is_bf16"] = t.dtype == torch.bfloat16
            out["d" + n] = req[n].grad.numpy()
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **out)
        print(f"{name}: wrote {os.path.getsize(path) / 1024:.0f} KiB", file=sys.stderr)


def main_gdn():
    from fla.ops.gated_delta_rule.gate import naive_gdn_gate
    from fla.ops.gated_delta_rule.naive import naive_recurrent_gated_delta_rule

    K = V = 128
    for ci, (name, B, T, H, l2, gate_in, h0_std, lens) in enumerate(GDN_CASES):
        gen = torch.Generator().manual_seed(2000 + ci)
        rn = lambda *s: torch.randn(*s, generator=gen, dtype=torch.float32)
        q, k, v = (rn(B, T, H, K).to(torch.bfloat16) for _ in range(3))
        if not l2:
            q, k = (F.normalize(x.float(), p=2, dim=-1).to(torch.bfloat16) for x in (q, k))
        if gate_in:
            g = (-2.0 + rn(B, T, H)).to(torch.bfloat16)
            A_log, dt_bias = 0.3 * rn(H), 0.2 * rn(H)
        else:
            g = F.logsigmoid(rn(B, T, H)) / 4.0            # fp32 log decay
            A_log = dt_bias = None
        beta = torch.sigmoid(rn(B, T, H)).to(torch.bfloat16)
        N = B if lens is None else len(lens)
        h0 = h0_std * rn(N, H, K, V)
        do = rn(B, T, H, V).to(torch.bfloat16)
        dht = 0.3 * rn(N, H, K, V)
        leaves = dict(q=q, k=k, v=v, g=g, beta=beta, h0=h0)
        if gate_in:
            leaves.update(A_log=A_log, dt_bias=dt_bias)
        req = {n: t.clone().float().requires_grad_(True) for n, t in leaves.items()}
        qn = F.normalize(req["q"], p=2, dim=-1) if l2 else req["q"]
        kn = F.normalize(req["k"], p=2, dim=-1) if l2 else req["k"]
        a = naive_gdn_gate(req["g"], req["A_log"], req["dt_bias"]) if gate_in else req["g"]
        bounds = [0, T] if lens is None else np.concatenate([[0], np.cumsum(lens)]).tolist()
        os_, hs_ = [], []
        for n in range(len(bounds) - 1):
            s, e = bounds[n], bounds[n + 1]
            h_in = req["h0"] if lens is None else req["h0"][n:n + 1]
            o_n, h_n = naive_recurrent_gated_delta_rule(qn[:, s:e], kn[:, s:e], req["v"][:, s:e], req["beta"][:, s:e], a[:, s:e],
                                                        initial_state=h_in, output_final_state=True)
            os_.append(o_n)
            hs_.append(h_n)
        o, ht = torch.cat(os_, 1), torch.cat(hs_, 0)
        ((o * do.float()).sum() + (ht * dht).sum()).backward()
        out = dict(B=B, T=T, H=H, use_l2norm=l2, use_gate_in_kernel=gate_in, safe_gate=False, lower_bound=np.float32(np.nan),
                   cu_seqlens=np.asarray(bounds if lens is not None else [], dtype=np.int32),
                   do=bits(do), dht=dht.numpy(), o=o.detach().numpy(), ht=ht.detach().numpy())
        for n, t in leaves.items():
            out["in_" + n] = bits(t)
            out["in_" + n + "_is_bf16"] = t.dtype == torch.bfloat16
            out["d" + n] = req[n].grad.numpy()
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **out)
        print(f"{name}: wrote {os.path.getsize(path) / 1024:.0f} KiB", file=sys.stderr)


def main_gate():
    """Stand-alone gate activations: outputs and gradients of the third-party naive_kda_gate /
    naive_kda_lowerbound_gate (fla/ops/kda/gate.py:26-69) on a small seeded tensor."""
    from fla.ops.kda.gate import naive_kda_gate, naive_kda_lowerbound_gate
    gen = torch.Generator().manual_seed(3000)
    M, H, K = 37, 3, 128
    g = (2.0 * torch.randn(M, H, K, generator=gen)).to(torch.bfloat16)
    A_log, dt_bias = 0.5 * torch.randn(H, generator=gen), 0.5 * torch.randn(H * K, generator=gen)
    dy = torch.randn(M, H, K, generator=gen)
    out = dict(g=bits(g), A_log=A_log.numpy(), dt_bias=dt_bias.numpy(), dy=dy.numpy())
    for tag, fn, kw in (("softplus", naive_kda_gate, {}), ("lower_bound", naive_kda_lowerbound_gate, dict(lower_bound=-5.0))):
        leaves = [t.clone().float().requires_grad_(True) for t in (g, A_log, dt_bias)]
        y = fn(leaves[0], leaves[1], leaves[2], **kw)
        (y * dy).sum().backward()
        out.update({f"{tag}_y": y.detach().numpy(), f"{tag}_dg": leaves[0].grad.numpy(), f"{tag}_dA_log": leaves[1].grad.numpy(),
                    f"{tag}_ddt_bias": leaves[2].grad.numpy()})
    path = os.path.join(HERE, "gate_activations.npz")
    np.savez_compressed(path, **out)
    print(f"gate_activations: wrote {os.path.getsize(path) / 1024:.0f} KiB", file=sys.stderr)


if __name__ == "__main__":
    main()
    main_gdn()
    main_gate()
