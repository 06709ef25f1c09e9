"""The short causal convolution and the gated RMS norm around chunk_kda: the oracle against torch's own conv1d with
left padding (CPU), and the CUDA operators against the oracle (GPU), forward, carried cache and gradients. bf16 in and
out: tolerances 4e-3 relative RMS for outputs and input gradients, 1e-2 for the parameter gradients (sums over all
tokens of bf16-rounded upstream gradients)."""
import pytest
import torch
import torch.nn.functional as F

from oracle.layer_ops import rms_norm_gated_ref, short_conv_ref
from oracle.naive_kda import err_ratio


def test_conv_oracle_is_left_padded_conv1d():
    gen = torch.Generator().manual_seed(0)
    x, w, b = torch.randn(2, 37, 16, generator=gen), torch.randn(16, 4, generator=gen), torch.randn(16, generator=gen)
    y, final = short_conv_ref(x, w, b, activation=None)
    ref = F.conv1d(x.transpose(1, 2), w.unsqueeze(1), b, padding=3, groups=16)[..., :37].transpose(1, 2)
    assert err_ratio(ref, y) < 1e-6
    assert torch.equal(final, x[:, -4:].transpose(1, 2))
    # continuing from the cache equals running the whole sequence at once
    y1, c1 = short_conv_ref(x[:, :20], w, b)
    y2, _ = short_conv_ref(x[:, 20:], w, b, initial_state=c1)
    y_all, _ = short_conv_ref(x, w, b)
    assert err_ratio(y_all, torch.cat([y1, y2], 1)) < 1e-6
    # packed sequences are independent
    cu = torch.tensor([0, 5, 37])
    yp, _ = short_conv_ref(x[:1], w, b, cu_seqlens=cu)
    assert err_ratio(short_conv_ref(x[:1, 5:], w, b)[0], yp[:, 5:]) < 1e-6


@pytest.mark.gpu
@pytest.mark.parametrize("W,bias,act,varlen", [(4, False, "silu", False), (4, True, "silu", True), (3, True, None, False),
                                               (2, False, "silu", True)])
def test_short_conv_matches_oracle(W, bias, act, varlen):
    from cula_b200.kda import short_conv
    gen = torch.Generator().manual_seed(1)
    B, T, D = (1, 333, 256) if varlen else (2, 200, 128)
    cu = torch.tensor([0, 1, 70, 198, 333], dtype=torch.int32) if varlen else None
    N = 4 if varlen else B
    x = torch.randn(B, T, D, generator=gen).to(torch.bfloat16)
    w, b = 0.5 * torch.randn(D, W, generator=gen), (0.1 * torch.randn(D, generator=gen) if bias else None)
    cache = torch.randn(N, D, W, generator=gen)
    dy = torch.randn(B, T, D, generator=gen).to(torch.bfloat16)
    ref_in = [x.float().requires_grad_(True), w.clone().requires_grad_(True)] + ([b.clone().requires_grad_(True)] if bias else [])
    y_ref, f_ref = short_conv_ref(ref_in[0], ref_in[1], ref_in[2] if bias else None, cache, act, cu)
    (y_ref * dy.float()).sum().backward()
    dev = [x.cuda().requires_grad_(True), w.cuda().requires_grad_(True)] + ([b.cuda().requires_grad_(True)] if bias else [])
    y, final = short_conv(dev[0], dev[1], dev[2] if bias else None, initial_state=cache.cuda(), output_final_state=True,
                          activation=act, cu_seqlens=None if cu is None else cu.cuda())
    y.backward(dy.cuda())
    torch.cuda.synchronize()
    assert err_ratio(y_ref.detach(), y.detach().float().cpu()) < 4e-3
    assert err_ratio(f_ref.detach(), final.cpu()) < 1e-6
    assert err_ratio(ref_in[0].grad, dev[0].grad.float().cpu()) < 4e-3
    assert err_ratio(ref_in[1].grad, dev[1].grad.cpu()) < 1e-2
    if bias:
        assert err_ratio(ref_in[2].grad, dev[2].grad.cpu()) < 1e-2


@pytest.mark.gpu
def test_short_conv_prefill_then_continue():
    """The final cache of one call is the initial cache of the next: two halves equal the whole sequence, bit for bit."""
    from cula_b200.kda import short_conv
    gen = torch.Generator().manual_seed(2)
    x = torch.randn(2, 300, 128, generator=gen).to(torch.bfloat16).cuda()
    w = torch.randn(128, 4, generator=gen).cuda()
    y_all, c_all = short_conv(x, w, output_final_state=True)
    y1, c1 = short_conv(x[:, :130].contiguous(), w, output_final_state=True)
    y2, c2 = short_conv(x[:, 130:].contiguous(), w, initial_state=c1, output_final_state=True)
    torch.cuda.synchronize()
    assert torch.equal(y_all, torch.cat([y1, y2], 1)) and torch.equal(c_all, c2)


@pytest.mark.gpu
@pytest.mark.parametrize("D,act", [(128, "sigmoid"), (128, "swish"), (256, "sigmoid"), (1024, "swish")])
def test_rms_norm_gated_matches_oracle(D, act):
    from cula_b200.kda import rms_norm_gated
    gen = torch.Generator().manual_seed(3)
    shape = (2, 77, 3, D)
    x, g = (torch.randn(*shape, generator=gen).to(torch.bfloat16) for _ in range(2))
    w = 1.0 + 0.1 * torch.randn(D, generator=gen)
    dy = torch.randn(*shape, generator=gen).to(torch.bfloat16)
    ref_in = [x.float().requires_grad_(True), g.float().requires_grad_(True), w.clone().requires_grad_(True)]
    y_ref = rms_norm_gated_ref(*ref_in, activation=act, eps=1e-5)
    (y_ref * dy.float()).sum().backward()
    dev = [x.cuda().requires_grad_(True), g.cuda().requires_grad_(True), w.cuda().requires_grad_(True)]
    y = rms_norm_gated(*dev, activation=act, eps=1e-5)
    y.backward(dy.cuda())
    torch.cuda.synchronize()
    assert y.dtype == torch.bfloat16 and err_ratio(y_ref.detach(), y.detach().float().cpu()) < 4e-3
    assert err_ratio(ref_in[0].grad, dev[0].grad.float().cpu()) < 4e-3
    assert err_ratio(ref_in[1].grad, dev[1].grad.float().cpu()) < 4e-3
    assert err_ratio(ref_in[2].grad, dev[2].grad.cpu()) < 1e-2
