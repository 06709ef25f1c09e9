"""The two layer operators on either side of ``chunk_kda`` in a Kimi-Linear block (fla/layers/kda.py:147-165, 191, 306):

* ``short_conv`` -- the short causal depthwise convolution (+ SiLU) applied to the q / k / v projections; call surface of
  flash-linear-attention's ``causal_conv1d`` (fla/modules/convolution.py) for the arguments a KDA layer uses;
* ``rms_norm_gated`` -- the gated RMS norm applied to the attention output, ``rmsnorm(x) * weight * act(g)``; call
  surface of ``rms_norm_gated`` (fla/modules/fused_norm_gate.py:846-869) without residual / bias.

Both are differentiable (one streaming sm_100a kernel each way). No Triton, no fallback."""
from __future__ import annotations

import torch

from .. import _native
from ..utils import CHUNK, assert_blackwell, get_varlen_tables


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def _f32(t):
    return None if t is None else t.float().contiguous()


def _ptr(t):
    return None if t is None else t.data_ptr()


class ShortConvFunction(torch.autograd.Function):
    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda")
    def forward(ctx, x, weight, bias, initial_state, output_final_state, activation, cu_seqlens, cu_seqlens_cpu):
        B, T, D = x.shape
        W = weight.shape[-1]
        x = x.contiguous()
        w32, b32, c32 = _f32(weight), _f32(bias), _f32(initial_state)
        if cu_seqlens is not None:
            tab = get_varlen_tables(cu_seqlens, cu_seqlens_cpu)
            n_seqs, num_chunks = tab.n_seqs, tab.num_chunks
            cu_p, ci_p = tab.cu_seqlens.data_ptr(), tab.chunk_indices.data_ptr()
            y = torch.zeros_like(x)                      # rows past cu_seqlens[-1] stay zero
        else:
            n_seqs, num_chunks = B, B * ((T + CHUNK - 1) // CHUNK)
            cu_p = ci_p = None
            y = torch.empty_like(x)
        final = torch.zeros(n_seqs, D, W, dtype=torch.float32, device=x.device) if output_final_state else None
        with torch.cuda.device(x.device):
            _native.check(_native.lib().cula_kda_short_conv_fwd(
                x.data_ptr(), w32.data_ptr(), _ptr(b32), _ptr(c32), y.data_ptr(), _ptr(final), cu_p, ci_p, num_chunks, T, D, W,
                int(activation in ("silu", "swish")), _stream(x)), "cula_kda_short_conv_fwd")
        ctx.save_for_backward(x, weight, bias, initial_state, cu_seqlens)
        ctx.cu_seqlens_cpu, ctx.activation, ctx.num_chunks = cu_seqlens_cpu, activation, num_chunks
        if final is None:
            return y, None
        ctx.mark_non_differentiable(final)
        return y, final

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, dy, _dfinal):
        x, weight, bias, initial_state, cu_seqlens = ctx.saved_tensors
        B, T, D = x.shape
        W = weight.shape[-1]
        dy = dy.contiguous().to(torch.bfloat16)
        w32, b32, c32 = _f32(weight), _f32(bias), _f32(initial_state)
        cu_p = ci_p = None
        dx = torch.empty_like(x)
        if cu_seqlens is not None:
            tab = get_varlen_tables(cu_seqlens, ctx.cu_seqlens_cpu)
            cu_p, ci_p = tab.cu_seqlens.data_ptr(), tab.chunk_indices.data_ptr()
            dx = torch.zeros_like(x)
        dw = torch.zeros(D, W, dtype=torch.float32, device=x.device)
        db = None if bias is None else torch.zeros(D, dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            _native.check(_native.lib().cula_kda_short_conv_bwd(
                x.data_ptr(), w32.data_ptr(), _ptr(b32), _ptr(c32), dy.data_ptr(), dx.data_ptr(), dw.data_ptr(), _ptr(db), cu_p, ci_p,
                ctx.num_chunks, T, D, W, int(ctx.activation in ("silu", "swish")), _stream(x)), "cula_kda_short_conv_bwd")
        return (dx, dw.to(weight.dtype).view_as(weight), None if db is None else db.to(bias.dtype), None, None, None, None, None)


@torch.compiler.disable
def short_conv(x, weight, bias=None, initial_state=None, output_final_state=False, activation="silu", cu_seqlens=None,
               cu_seqlens_cpu=None):
    """Causal depthwise convolution over time, then SiLU (``activation`` ``"silu"``/``"swish"``) or nothing (``None``).

    x: ``[B, T, D]`` bf16 (``B == 1`` with ``cu_seqlens``); weight: ``[D, W]``, ``W <= 4`` (a ``[D, 1, W]`` conv1d weight
    is accepted), tap ``W - 1`` multiplies the current token; bias: ``[D]`` or None; initial_state: ``[N, D, W]`` -- the
    last ``W`` inputs of a previous call, newest last -- or None; with ``output_final_state`` the same record for this
    call is returned. Returns ``(y, final_state)``. Gradients flow to x, weight and bias."""
    assert x.dim() == 3 and x.dtype == torch.bfloat16, "x must be [B, T, D] in bfloat16."
    if weight.dim() == 3:
        weight = weight.squeeze(1)
    D, W = weight.shape
    assert x.shape[-1] == D and D % 8 == 0 and 1 <= W <= 4, "weight must be [D, W] with W <= 4 and D a multiple of 8."
    assert activation in (None, "silu", "swish"), "activation must be None, 'silu' or 'swish'."
    if cu_seqlens is not None and x.shape[0] != 1:
        raise ValueError(f"The batch size is expected to be 1 rather than {x.shape[0]} when using `cu_seqlens`.")
    n_seqs = x.shape[0] if cu_seqlens is None else len(cu_seqlens) - 1
    if initial_state is not None:
        assert tuple(initial_state.shape) == (n_seqs, D, W), "initial_state must be [N, D, W]."
    assert_blackwell(x.device)
    return ShortConvFunction.apply(x, weight, bias, initial_state, output_final_state, activation, cu_seqlens, cu_seqlens_cpu)


class RMSNormGatedFunction(torch.autograd.Function):
    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda")
    def forward(ctx, x, g, weight, activation, eps):
        D = x.shape[-1]
        x2, g2 = x.contiguous().view(-1, D), g.contiguous().view(-1, D)
        w32 = _f32(weight)
        y = torch.empty_like(x2)
        rstd = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            _native.check(_native.lib().cula_kda_rms_norm_gated_fwd(
                x2.data_ptr(), g2.data_ptr(), w32.data_ptr(), y.data_ptr(), rstd.data_ptr(), x2.shape[0], D,
                int(activation in ("swish", "silu")), float(eps), _stream(x)), "cula_kda_rms_norm_gated_fwd")
        ctx.save_for_backward(x2, g2, weight, rstd)
        ctx.activation, ctx.shape = activation, x.shape
        return y.view(x.shape)

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, dy):
        x2, g2, weight, rstd = ctx.saved_tensors
        D = x2.shape[-1]
        dy2 = dy.contiguous().view(-1, D).to(torch.bfloat16)
        w32 = _f32(weight)
        dx, dg = torch.empty_like(x2), torch.empty_like(g2)
        dw = torch.zeros(D, dtype=torch.float32, device=x2.device)
        with torch.cuda.device(x2.device):
            _native.check(_native.lib().cula_kda_rms_norm_gated_bwd(
                x2.data_ptr(), g2.data_ptr(), w32.data_ptr(), rstd.data_ptr(), dy2.data_ptr(), dx.data_ptr(), dg.data_ptr(),
                dw.data_ptr(), x2.shape[0], D, int(ctx.activation in ("swish", "silu")), _stream(x2)), "cula_kda_rms_norm_gated_bwd")
        return dx.view(ctx.shape), dg.view(ctx.shape), dw.to(weight.dtype), None, None


@torch.compiler.disable
def rms_norm_gated(x, g, weight, activation="sigmoid", eps=1e-6):
    """``x * rsqrt(mean(x^2, -1) + eps) * weight * act(g)`` with ``act`` = ``"sigmoid"`` (what the KDA layer uses) or
    ``"swish"``/``"silu"`` (``g * sigmoid(g)``). x, g: ``[..., D]`` bf16, D in {128, 256, 512, 1024}; weight ``[D]``.
    Gradients flow to x, g and weight."""
    assert x.shape == g.shape and x.dtype == g.dtype == torch.bfloat16, "x and g must be bfloat16 tensors of one shape."
    assert x.shape[-1] in (128, 256, 512, 1024) and weight.numel() == x.shape[-1], "the normalised dim must be 128/256/512/1024."
    assert activation in ("sigmoid", "swish", "silu"), "activation must be 'sigmoid', 'swish' or 'silu'."
    assert_blackwell(x.device)
    return RMSNormGatedFunction.apply(x, g, weight, activation, eps)
