"""CPU oracle for the layer operators around chunk_kda -- TEST INFRASTRUCTURE, NOT PRODUCT CODE (only tests/ import it).

* ``short_conv_ref``: the causal depthwise convolution of flash-linear-attention's ``ShortConvolution``, which is a
  ``torch.nn.Conv1d(groups=D, padding=W - 1)`` truncated to the first T outputs (fla/modules/convolution.py: the class
  derives from nn.Conv1d and its torch path is exactly that), then SiLU; the cache holds the last W inputs, newest last.
* ``rms_norm_gated_ref``: ``x * rsqrt(mean(x^2) + eps) * w * act(g)`` as computed by the kernel
  ``layer_norm_gated_fwd_kernel`` with ``IS_RMS_NORM`` (fla/modules/fused_norm_gate.py:35-105).

Parity pin: the convolution is pinned to torch's own ``F.conv1d``; the third-party Triton kernels cannot run on a CPU, so
the gated norm is a restatement of the published formula only ("parity unpinned" beyond that formula)."""
import torch
import torch.nn.functional as F


def short_conv_ref(x, weight, bias=None, initial_state=None, activation="silu", cu_seqlens=None):
    """x [B, T, D] (float), weight [D, W]; returns (y, final_state [N, D, W])."""
    B, T, D = x.shape
    W = weight.shape[-1]
    bounds = [(b, 0, T) for b in range(B)] if cu_seqlens is None else \
        [(0, int(cu_seqlens[n]), int(cu_seqlens[n + 1])) for n in range(len(cu_seqlens) - 1)]
    y = torch.zeros_like(x)
    finals = []
    for n, (b, s, e) in enumerate(bounds):
        seg = x[b, s:e]                                                     # [L, D]
        past = torch.zeros(W, D, dtype=x.dtype) if initial_state is None else initial_state[n].to(x.dtype).t()   # [W, D]
        full = torch.cat([past, seg], dim=0)                                # [W + L, D]
        out = F.conv1d(full.t().unsqueeze(0), weight.to(x.dtype).unsqueeze(1), bias if bias is None else bias.to(x.dtype),
                       groups=D)[0].t()                                     # [L + 1, D]: window ending at token i - 1
        pre = out[1:]
        y[b, s:e] = F.silu(pre) if activation in ("silu", "swish") else pre
        finals.append(full[-W:].t())
    return y, torch.stack(finals)


def rms_norm_gated_ref(x, g, weight, activation="sigmoid", eps=1e-6):
    n = x * torch.rsqrt(x.square().mean(-1, keepdim=True) + eps)
    act = torch.sigmoid(g) if activation == "sigmoid" else g * torch.sigmoid(g)
    return n * weight * act
