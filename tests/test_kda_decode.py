"""GPU parity of the decode kernel against the fp32 decode oracle, on the shapes and input distributions of the
reference's own decode tests (tests/test_kda_decode.py:109-121, 228-300): bf16 q/k/v/a/b, grouped heads, state pool
in the (V, K) layout by default. Bar: the reference's allclose(atol=3e-2, rtol=2e-2) on o and on the state
(tests/test_kda_decode.py:187-193), plus relative RMS <= 5e-3 on o (its bf16 rounding floor) and <= 1e-5 on the
fp32 state."""
import pytest
import torch

from oracle.decode import kda_decode_oracle
from oracle.naive_kda import err_ratio

pytestmark = pytest.mark.gpu


def make_decode_inputs(N, H, HV, K, V, seed=42):
    gen = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=gen)
    q, k, v = (r(N, H, K).to(torch.bfloat16), r(N, H, K).to(torch.bfloat16), r(N, HV, V).to(torch.bfloat16))
    a = (0.1 * r(N, HV, K)).to(torch.bfloat16)
    b = r(N, HV).to(torch.bfloat16)
    A_log = -2 * torch.rand(HV, generator=gen)
    dt_bias = 0.1 * r(HV, K)
    state = 0.01 * r(N, HV, V, K)
    return q, k, v, a, b, A_log, dt_bias, state


def check(o_ref, s_ref, o, s):
    assert torch.allclose(o_ref, o.float().cpu(), atol=3e-2, rtol=2e-2)
    assert torch.allclose(s_ref, s.float().cpu(), atol=3e-2, rtol=2e-2)
    assert err_ratio(o_ref, o.float().cpu()) <= 5e-3 and err_ratio(s_ref, s.cpu()) <= 1e-5


@pytest.mark.parametrize("N", [1, 4, 33, 128])
@pytest.mark.parametrize("H,HV", [(8, 16), (16, 32), (4, 4)])
def test_decode_dense(N, H, HV):
    from cula_b200.kda import check_status, kda_decode
    q, k, v, a, b, A_log, dt_bias, state = make_decode_inputs(N, H, HV, 128, 128)
    o_ref, s_ref = kda_decode_oracle(q, k, v, a, b, A_log, dt_bias, state)
    pool = state.cuda()
    o = kda_decode(A_log=A_log.cuda(), dt_bias=dt_bias.cuda(), q=q.unsqueeze(1).cuda(), k=k.unsqueeze(1).cuda(),
                   v=v.unsqueeze(1).cuda(), a=a.unsqueeze(1).cuda(), b=b.unsqueeze(1).cuda(), initial_state_source=pool,
                   initial_state_indices=torch.arange(N, dtype=torch.int32).cuda(), scale=128 ** -0.5,
                   use_qk_l2norm_in_kernel=True)
    torch.cuda.synchronize()
    check_status()
    assert o.shape == (N, 1, HV, 128) and o.dtype == torch.bfloat16
    check(o_ref, s_ref, o.squeeze(1), pool)


@pytest.mark.parametrize("N", [2, 16, 64])
def test_decode_varlen_layout(N):
    from cula_b200.kda import check_status, kda_decode
    H, HV = 8, 16
    q, k, v, a, b, A_log, dt_bias, state = make_decode_inputs(N, H, HV, 128, 128, seed=1)
    o_ref, s_ref = kda_decode_oracle(q, k, v, a, b, A_log, dt_bias, state)
    pool = state.cuda()
    o = kda_decode(A_log=A_log.cuda(), dt_bias=dt_bias.cuda(), q=q.unsqueeze(0).cuda(), k=k.unsqueeze(0).cuda(),
                   v=v.unsqueeze(0).cuda(), a=a.cuda(), b=b.cuda(), initial_state_source=pool,
                   initial_state_indices=torch.arange(N, dtype=torch.int32).cuda(),
                   cu_seqlens=torch.arange(N + 1, dtype=torch.int32).cuda(), scale=128 ** -0.5, use_qk_l2norm_in_kernel=True)
    torch.cuda.synchronize()
    check_status()
    assert o.shape == (1, N, HV, 128)
    check(o_ref, s_ref, o.squeeze(0), pool)


@pytest.mark.parametrize("layout", ["vk", "kv"])
@pytest.mark.parametrize("V", [128, 256, 64])
def test_decode_layouts_value_widths_fp32_gates_and_pool_indices(layout, V):
    """(K, V) pools, V other than 128, fp32 a / b, a shuffled pool with a skipped sequence, no L2 norm."""
    from cula_b200.kda import check_status, fused_sigmoid_gating_delta_rule_update
    N, H, HV = 5, 2, 6
    q, k, v, a, b, A_log, dt_bias, _ = make_decode_inputs(N, H, HV, 128, V, seed=3)
    q, k = (0.1 * q.float()).to(torch.bfloat16), (0.1 * k.float()).to(torch.bfloat16)      # un-normalised path: keep it tame
    gen = torch.Generator().manual_seed(9)
    pool = 0.05 * torch.randn(9, HV, V, 128, generator=gen)
    idx = torch.tensor([7, 2, -1, 0, 5], dtype=torch.int32)
    a, b = a.float(), b.float()
    o_ref, s_ref = kda_decode_oracle(q, k, v, a, b, A_log, dt_bias, pool, use_l2norm=False, indices=idx, softplus_beta=2.0,
                                     softplus_threshold=10.0)
    dev_pool = (pool if layout == "vk" else pool.transpose(-1, -2)).contiguous().cuda()
    out = torch.full((N, 1, HV, V), 7.0, dtype=torch.bfloat16, device="cuda")
    o = fused_sigmoid_gating_delta_rule_update(A_log.cuda(), a.unsqueeze(1).cuda(), dt_bias.cuda(), 2.0, 10.0,
                                               q.unsqueeze(1).cuda(), k.unsqueeze(1).cuda(), v.unsqueeze(1).cuda(),
                                               b.unsqueeze(1).cuda(), dev_pool, idx.cuda(), scale=0.3,
                                               use_qk_l2norm_in_kernel=False, is_kda=True, out=out, state_layout=layout)
    torch.cuda.synchronize()
    check_status()
    assert o.data_ptr() == out.data_ptr()
    o_ref2, _ = kda_decode_oracle(q, k, v, a, b, A_log, dt_bias, pool, scale=0.3, use_l2norm=False, indices=idx,
                                  softplus_beta=2.0, softplus_threshold=10.0)
    got_pool = dev_pool.cpu() if layout == "vk" else dev_pool.cpu().transpose(-1, -2)
    check(o_ref2, s_ref, o.squeeze(1), got_pool)
    assert float(o[2].float().abs().max()) == 0.0                      # the skipped sequence has a zero output row


def test_decode_zero_state_and_steps_follow_prefill():
    """No state source = zero states; and: prefill T tokens with chunk_kda, decode one more token from its final
    state, compare with chunk_kda over T + 1 tokens (softplus gate on both sides)."""
    from cula_b200.kda import check_status, chunk_kda, kda_decode
    N, H, T = 2, 4, 130
    gen = torch.Generator().manual_seed(4)
    r = lambda *s: torch.randn(*s, generator=gen)
    q, k, v = (r(N, T + 1, H, 128).to(torch.bfloat16).cuda() for _ in range(3))
    g = (0.1 * r(N, T + 1, H, 128)).to(torch.bfloat16).cuda()
    braw = r(N, T + 1, H).to(torch.bfloat16).cuda()
    A_log, dt_bias = (-2 * torch.rand(H, generator=gen)).cuda(), (0.1 * r(H * 128)).cuda()
    kw = dict(use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, A_log=A_log, dt_bias=dt_bias, output_final_state=True)
    beta = torch.sigmoid(braw.float())
    o_full, s_full = chunk_kda(q, k, v, g, beta, **kw)
    _, s_pre = chunk_kda(q[:, :T], k[:, :T], v[:, :T], g[:, :T], beta[:, :T], **kw)          # [N, H, K, V]
    pool = s_pre.clone()
    o = kda_decode(A_log=A_log, dt_bias=dt_bias, q=q[:, T:], k=k[:, T:], v=v[:, T:], a=g[:, T:], b=braw[:, T:],
                   initial_state_source=pool, initial_state_indices=None, state_layout="kv")
    torch.cuda.synchronize()
    check_status()
    assert err_ratio(o_full[:, T:].float().cpu(), o.float().cpu()) <= 8e-3
    assert err_ratio(s_full.cpu(), pool.cpu()) <= 2e-3
    o0 = kda_decode(A_log=A_log, dt_bias=dt_bias, q=q[:, :1], k=k[:, :1], v=v[:, :1], a=g[:, :1], b=braw[:, :1],
                    initial_state_source=None, initial_state_indices=None)
    o_first, _ = chunk_kda(q[:, :1], k[:, :1], v[:, :1], g[:, :1], beta[:, :1], **kw)
    assert err_ratio(o_first.float().cpu(), o0.float().cpu()) <= 8e-3


def test_decode_argument_errors():
    from cula_b200.kda import fused_sigmoid_gating_delta_rule_update, kda_decode
    N, H, HV = 2, 2, 2
    q, k, v, a, b, A_log, dt_bias, state = (t.cuda() for t in make_decode_inputs(N, H, HV, 128, 128))
    args = dict(A_log=A_log, dt_bias=dt_bias, q=q.unsqueeze(1), k=k.unsqueeze(1), v=v.unsqueeze(1), a=a.unsqueeze(1),
                b=b.unsqueeze(1), initial_state_indices=torch.arange(N, dtype=torch.int32).cuda())
    with pytest.raises(ValueError):        # a (K, V)-shaped pool announced as "vk" (rectangular so the shapes differ)
        kda_decode(initial_state_source=torch.zeros(N, HV, 128, 64, device="cuda"), **args)
    with pytest.raises(ValueError):
        kda_decode(initial_state_source=state, state_layout="hv", **args)
    with pytest.raises(NotImplementedError):
        fused_sigmoid_gating_delta_rule_update(A_log, a.unsqueeze(1), dt_bias, 1.0, 20.0, q.unsqueeze(1), k.unsqueeze(1),
                                               v.unsqueeze(1), b.unsqueeze(1), state, None, is_kda=False)
    with pytest.raises(ValueError):        # out of the wrong shape
        kda_decode(initial_state_source=state, out=torch.empty(N, HV, 128, dtype=torch.bfloat16, device="cuda"), **args)


def test_decode_large_batch_and_bad_index_status():
    """A batch larger than the persistent grid, and a pool index past the end of the pool: reported, nothing touched."""
    from cula_b200.kda import check_status, kda_decode
    N, H, HV = 700, 2, 4
    q, k, v, a, b, A_log, dt_bias, state = make_decode_inputs(N, H, HV, 128, 128, seed=5)
    o_ref, s_ref = kda_decode_oracle(q, k, v, a, b, A_log, dt_bias, state)
    pool = state.cuda()
    args = dict(A_log=A_log.cuda(), dt_bias=dt_bias.cuda(), q=q.unsqueeze(1).cuda(), k=k.unsqueeze(1).cuda(),
                v=v.unsqueeze(1).cuda(), a=a.unsqueeze(1).cuda(), b=b.unsqueeze(1).cuda())
    o = kda_decode(initial_state_source=pool, initial_state_indices=None, **args)
    torch.cuda.synchronize()
    check_status()
    check(o_ref, s_ref, o.squeeze(1), pool)
    before = pool.clone()
    bad = torch.arange(N, dtype=torch.int32)
    bad[3] = N + 5
    kda_decode(initial_state_source=pool[:N], initial_state_indices=bad.cuda(), **args)
    with pytest.raises(RuntimeError, match="state-pool index"):
        check_status()
    assert torch.equal(pool[3], before[3])                   # the offending sequence touched nothing
    check_status()                                           # the status word was cleared by the failed check


def test_decode_is_capturable_in_a_cuda_graph():
    """The way a serving engine runs decode: one captured step replayed per token against the state pool. Three
    replayed steps must equal three eager steps on a copy of the pool, bit for bit."""
    from cula_b200.kda import check_status, kda_decode
    N, H, HV = 16, 8, 16
    q, k, v, a, b, A_log, dt_bias, state = make_decode_inputs(N, H, HV, 128, 128, seed=3)
    dev = lambda t: t.cuda()
    static = [dev(x.unsqueeze(1)) for x in (q, k, v, a, b)]
    A_d, bias_d, idx = dev(A_log), dev(dt_bias), torch.arange(N, dtype=torch.int32).cuda()
    pool_graph, pool_eager = dev(state), dev(state)

    def step(inputs, pool):
        return kda_decode(A_log=A_d, dt_bias=bias_d, q=inputs[0], k=inputs[1], v=inputs[2], a=inputs[3], b=inputs[4],
                          initial_state_source=pool, initial_state_indices=idx, scale=128 ** -0.5,
                          use_qk_l2norm_in_kernel=True)

    warm = dev(state)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step(static, warm)                                # warm-up outside the capture, on a scratch pool
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        o_static = step(static, pool_graph)
    pool_graph.copy_(dev(state))                          # the capture itself does not run the kernels, but be explicit
    for t in range(3):
        fresh = [dev(x.unsqueeze(1)) for x in make_decode_inputs(N, H, HV, 128, 128, seed=10 + t)[:5]]
        for dst, src in zip(static, fresh):
            dst.copy_(src)
        graph.replay()
        o_ref = step(fresh, pool_eager)
        torch.cuda.synchronize()
        assert torch.equal(o_static, o_ref) and torch.equal(pool_graph, pool_eager)
    check_status()
