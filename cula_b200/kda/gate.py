"""``fused_kda_gate`` and ``fused_beta_sigmoid``: the layer-side activations that sit next to ``chunk_kda`` in a
Kimi-Linear block, for callers that do not let ``chunk_kda`` activate the gate itself (``use_gate_in_kernel=False``).
Same call surface and autograd behaviour as flash-linear-attention's functions of the same names
(fla/ops/kda/gate.py:321-345 and :431), which callers of the reference use around ``cula.kda.chunk_kda``.
One streaming sm_100a kernel each way; no Triton, no fallback."""
from __future__ import annotations

import torch

from .. import _native
from ..utils import assert_blackwell


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


class KDAGateFunction(torch.autograd.Function):
    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda")
    def forward(ctx, g, A_log, dt_bias, lower_bound, output_dtype):
        assert g.dtype in (torch.bfloat16, torch.float32), "g must be in bfloat16 or float32."
        assert output_dtype in (torch.bfloat16, torch.float32), "output_dtype must be bfloat16 or float32."
        H, K = g.shape[-2:]
        assert A_log.numel() == H and (dt_bias is None or dt_bias.numel() == H * K)
        assert_blackwell(g.device)
        g = g.contiguous()
        a32 = A_log.float().contiguous()
        b32 = None if dt_bias is None else dt_bias.float().contiguous()
        y = torch.empty(g.shape, dtype=output_dtype, device=g.device)
        with torch.cuda.device(g.device):
            _native.check(_native.lib().cula_kda_gate_fwd(
                g.data_ptr(), int(g.dtype == torch.float32), a32.data_ptr(), None if b32 is None else b32.data_ptr(),
                y.data_ptr(), int(output_dtype == torch.float32), g.numel() // (H * K), H, K,
                int(lower_bound is not None), float(lower_bound if lower_bound is not None else 0.0), _stream(g)),
                "cula_kda_gate_fwd")
        ctx.save_for_backward(g, A_log, dt_bias)
        ctx.lower_bound = lower_bound
        return y

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, dy):
        g, A_log, dt_bias = ctx.saved_tensors
        H, K = g.shape[-2:]
        lower_bound = ctx.lower_bound
        dy = dy.contiguous()
        if dy.dtype not in (torch.bfloat16, torch.float32):
            dy = dy.float()
        a32 = A_log.float().contiguous()
        b32 = None if dt_bias is None else dt_bias.float().contiguous()
        dg = torch.empty_like(g)
        dA = torch.zeros(H, dtype=torch.float32, device=g.device)
        dbias = None if dt_bias is None else torch.zeros(H * K, dtype=torch.float32, device=g.device)
        with torch.cuda.device(g.device):
            _native.check(_native.lib().cula_kda_gate_bwd(
                g.data_ptr(), int(g.dtype == torch.float32), a32.data_ptr(), None if b32 is None else b32.data_ptr(),
                dy.data_ptr(), int(dy.dtype == torch.float32), dg.data_ptr(), dA.data_ptr(),
                None if dbias is None else dbias.data_ptr(), g.numel() // (H * K), H, K, int(lower_bound is not None),
                float(lower_bound if lower_bound is not None else 0.0), _stream(g)), "cula_kda_gate_bwd")
        dA = dA.to(A_log.dtype).view_as(A_log)
        if dbias is not None:
            dbias = dbias.to(dt_bias.dtype).view_as(dt_bias)
        return dg, dA, dbias, None, None


@torch.compiler.disable
def fused_kda_gate(g, A_log, dt_bias=None, lower_bound=None, output_dtype=torch.float32):
    """``-exp(A_log)[:, None] * softplus(g + dt_bias)`` for ``g`` ``[..., H, K]``, or, with ``lower_bound``,
    ``lower_bound * sigmoid(exp(A_log)[:, None] * (g + dt_bias))``. Differentiable in g, A_log and dt_bias."""
    return KDAGateFunction.apply(g, A_log, dt_bias, lower_bound, output_dtype)


class BetaSigmoidFunction(torch.autograd.Function):
    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda")
    def forward(ctx, x):
        assert x.dtype in (torch.bfloat16, torch.float32), "x must be in bfloat16 or float32."
        assert_blackwell(x.device)
        x = x.contiguous()
        y = torch.empty(x.shape, dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            _native.check(_native.lib().cula_kda_beta_sigmoid_fwd(x.data_ptr(), int(x.dtype == torch.float32), y.data_ptr(),
                                                                  x.numel(), _stream(x)), "cula_kda_beta_sigmoid_fwd")
        ctx.save_for_backward(x)
        return y

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        dy = dy.float().contiguous()
        dx = torch.empty_like(x)
        with torch.cuda.device(x.device):
            _native.check(_native.lib().cula_kda_beta_sigmoid_bwd(x.data_ptr(), int(x.dtype == torch.float32), dy.data_ptr(),
                                                                  dx.data_ptr(), x.numel(), _stream(x)),
                          "cula_kda_beta_sigmoid_bwd")
        return dx


def fused_beta_sigmoid(x):
    """``sigmoid(x)`` in fp32 with autograd (fla/ops/kda/gate.py:431)."""
    return BetaSigmoidFunction.apply(x)
