"""Seeded synthetic inputs for chunk_kda (benchmarks and tests); no dataset is involved."""
import torch


def make_inputs(B, T, H, K=128, V=128, seed=0, gate_offset=0.0, h0_std=0.0, g_dtype=torch.bfloat16,
                beta_dtype=torch.bfloat16):
    """Seeded synthetic inputs with the distributions the headline configurations name:
    q,k,v ~ N(0,1) bf16; g = gate_offset + 0.1*N(0,1); beta = sigmoid(N(0,1));
    A_log = 0.01*N(0,1) [H]; dt_bias = 0 [H*K]; initial_state = h0_std*N(0,1) fp32 (None if 0).

    ``gate_offset=-8`` gives weak gates (decay ~ -0.002 per token with lower_bound=-5) so that the
    carried state actually matters; 0 gives the nominal strong gates (~ -2.5 per token).
    """
    gen = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=gen, dtype=torch.float32)
    q = rn(B, T, H, K).to(torch.bfloat16)
    k = rn(B, T, H, K).to(torch.bfloat16)
    v = rn(B, T, H, V).to(torch.bfloat16)
    g = (gate_offset + 0.1 * rn(B, T, H, K)).to(g_dtype)
    beta = torch.sigmoid(rn(B, T, H)).to(beta_dtype)
    A_log = 0.01 * rn(H)
    dt_bias = torch.zeros(H * K)
    h0 = h0_std * rn(B, H, K, V) if h0_std > 0 else None
    return dict(q=q, k=k, v=v, g=g, beta=beta, A_log=A_log, dt_bias=dt_bias, initial_state=h0)


def make_inputs_on_device(B, T, H, device, K=128, V=128, seed=0, gate_offset=0.0, h0_std=0.0):
    """The same distributions as :func:`make_inputs`, drawn on ``device`` with its own seeded generator (a long
    sequence takes minutes to draw on the host). The same seed gives the same numbers on every GPU of one model."""
    gen = torch.Generator(device=device).manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=gen, dtype=torch.float32, device=device)
    q = rn(B, T, H, K).to(torch.bfloat16)
    k = rn(B, T, H, K).to(torch.bfloat16)
    v = rn(B, T, H, V).to(torch.bfloat16)
    g = (gate_offset + 0.1 * rn(B, T, H, K)).to(torch.bfloat16)
    beta = torch.sigmoid(rn(B, T, H)).to(torch.bfloat16)
    A_log = 0.01 * rn(H)
    dt_bias = torch.zeros(H * K, device=device)
    h0 = h0_std * rn(B, H, K, V) if h0_std > 0 else None
    return dict(q=q, k=k, v=v, g=g, beta=beta, A_log=A_log, dt_bias=dt_bias, initial_state=h0)
