"""GPU parity of the chunk_kda backward path (autograd through the C ABI) against autograd of the CPU oracle
and against the golden gradients. Tolerances (relative RMS): 5e-3 for dq, dk, dv, dg, dbeta, dh0 on the headline
distributions, the reference's own 8e-3 / 2e-2 bounds (tests/test_kda.py:147-155) elsewhere; max-abs <= 2e-2
relative to the largest reference entry."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from conftest import GOLDEN_CASES, load_golden
from oracle.naive_kda import chunk_kda_oracle, err_ratio, make_inputs

pytestmark = pytest.mark.gpu

GRADS = ("q", "k", "v", "g", "beta", "A_log", "dt_bias", "initial_state")


def run_both(inp, do, dht, cu_seqlens=None, l2=True, gate=True, safe=True, lower_bound=-5.0, **kw):
    from cula_b200.kda import check_status, chunk_kda
    names = [n for n in GRADS if inp.get(n) is not None and (gate or n not in ("A_log", "dt_bias"))]
    # oracle
    ref_in = {n: inp[n].detach().float().clone().requires_grad_(True) for n in names}
    o, ht = chunk_kda_oracle(ref_in["q"], ref_in["k"], ref_in["v"], ref_in["g"], ref_in["beta"],
                             initial_state=ref_in.get("initial_state"), output_final_state=True,
                             use_qk_l2norm_in_kernel=l2, use_gate_in_kernel=gate, cu_seqlens=cu_seqlens,
                             safe_gate=safe, lower_bound=lower_bound if (gate and safe) else None,
                             A_log=ref_in.get("A_log"), dt_bias=ref_in.get("dt_bias"))
    ((o * do.float()).sum() + (ht * dht).sum()).backward()
    ref = {n: t.grad for n, t in ref_in.items()}
    # CUDA path
    dev_in = {n: inp[n].detach().cuda().requires_grad_(True) for n in names}
    extra = dict(A_log=dev_in.get("A_log"), dt_bias=dev_in.get("dt_bias")) if gate else {}
    o2, ht2 = chunk_kda(dev_in["q"], dev_in["k"], dev_in["v"], dev_in["g"], dev_in["beta"],
                        initial_state=dev_in.get("initial_state"), output_final_state=True,
                        use_qk_l2norm_in_kernel=l2, use_gate_in_kernel=gate, safe_gate=safe,
                        lower_bound=lower_bound if (gate and safe) else None,
                        cu_seqlens=None if cu_seqlens is None else cu_seqlens.cuda(), **extra, **kw)
    ((o2.float() * do.cuda().float()).sum() + (ht2 * dht.cuda()).sum()).backward()
    torch.cuda.synchronize()
    check_status()
    got = {n: t.grad.float().cpu() for n, t in dev_in.items()}
    for n in names:
        assert got[n].shape == ref[n].shape and dev_in[n].grad.dtype == dev_in[n].dtype, n
    return ref, got


def assert_grads(ref, got, tol, tag=""):
    msgs = []
    for n in ref:
        e = err_ratio(ref[n], got[n])
        mx = float((ref[n] - got[n]).abs().max() / (ref[n].abs().max() + 1e-30))
        t = tol.get(n, tol["default"])
        if not (e <= t and mx <= 2e-2 and torch.isfinite(got[n]).all()):
            msgs.append(f"d{n}: rel {e:.2e} (tol {t}) maxabs/max {mx:.2e}")
    assert not msgs, f"{tag}: " + "; ".join(msgs)


HEADLINE_TOL = {"default": 5e-3}
SUITE_TOL = {"default": 8e-3, "g": 2e-2, "beta": 2e-2}


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_backward_matches_golden(name):
    from cula_b200.kda import chunk_kda
    case, inp, exp = load_golden(name)
    names = [n for n in ("q", "k", "v", "g", "beta", "A_log", "dt_bias", "h0") if n in inp]
    dev = {n: inp[n].detach().cuda().requires_grad_(True) for n in names}
    extra = dict(A_log=dev.get("A_log"), dt_bias=dev.get("dt_bias")) if case["use_gate_in_kernel"] else {}
    o, ht = chunk_kda(dev["q"], dev["k"], dev["v"], dev["g"], dev["beta"], initial_state=dev.get("h0"),
                      output_final_state=True, use_qk_l2norm_in_kernel=case["use_l2norm"],
                      use_gate_in_kernel=case["use_gate_in_kernel"], safe_gate=case["safe_gate"],
                      lower_bound=case["lower_bound"],
                      cu_seqlens=None if case["cu_seqlens"] is None else case["cu_seqlens"].cuda(), **extra)
    ((o.float() * inp["do"].cuda().float()).sum() + (ht * inp["dht"].cuda()).sum()).backward()
    torch.cuda.synchronize()
    ref = {n: exp["d" + n] for n in names}
    got = {n: dev[n].grad.float().cpu() for n in names}
    assert_grads(ref, got, SUITE_TOL, name)


def test_backward_headline_distribution():
    """B=1, T=512, H=4 with the headline input distributions, N(0,1) upstream gradient, 0.1*N(0,1) initial state."""
    inp = make_inputs(1, 512, 4, seed=0, h0_std=0.1)
    gen = torch.Generator().manual_seed(5)
    do = torch.randn(1, 512, 4, 128, generator=gen).to(torch.bfloat16)
    dht = torch.zeros(1, 4, 128, 128)
    ref, got = run_both(inp, do, dht)
    assert_grads(ref, got, HEADLINE_TOL, "headline")


@pytest.mark.parametrize("B,T,H,gate_offset,recompute", [
    (1, 63, 1, -6.0, True), (2, 500, 3, -8.0, False), (2, 300, 2, 0.0, True), (1, 1, 2, -8.0, True), (1, 65, 2, -3.0, False),
])
def test_backward_shapes(B, T, H, gate_offset, recompute):
    inp = make_inputs(B, T, H, seed=42, gate_offset=gate_offset, h0_std=1.0)
    inp["A_log"] = inp["A_log"] + 0.1
    gen = torch.Generator().manual_seed(7)
    inp["dt_bias"] = 0.1 * torch.randn(H * 128, generator=gen)
    do = torch.randn(B, T, H, 128, generator=gen).to(torch.bfloat16)
    dht = torch.randn(B, H, 128, 128, generator=gen)
    ref, got = run_both(inp, do, dht, disable_recompute=not recompute)
    assert_grads(ref, got, SUITE_TOL, f"B{B}T{T}H{H}")


@pytest.mark.parametrize("beta_dtype,g_fp32,safe", [(torch.float32, True, True), (torch.bfloat16, False, False)])
def test_backward_pre_gated_softplus_and_dtypes(beta_dtype, g_fp32, safe):
    """use_gate_in_kernel=False with an fp32 log-decay and fp32 beta; and the softplus gate (safe_gate=False)."""
    B, T, H = 2, 200, 2
    gen = torch.Generator().manual_seed(11)
    if g_fp32:
        inp = make_inputs(B, T, H, seed=5, h0_std=1.0, beta_dtype=beta_dtype)
        inp["g"] = (F.logsigmoid(torch.randn(B, T, H, 128, generator=gen)) / 4.0).clamp(-5, 0)
        inp["q"] = F.normalize(inp["q"].float(), dim=-1).to(torch.bfloat16)
        inp["k"] = F.normalize(inp["k"].float(), dim=-1).to(torch.bfloat16)
        kw = dict(l2=False, gate=False)
    else:
        inp = make_inputs(B, T, H, seed=5, gate_offset=-4.0, h0_std=1.0, beta_dtype=beta_dtype)
        inp["dt_bias"] = 0.2 * torch.randn(H * 128, generator=gen)
        kw = dict(safe=False)
    do = torch.randn(B, T, H, 128, generator=gen).to(torch.bfloat16)
    dht = torch.randn(B, H, 128, 128, generator=gen)
    ref, got = run_both(inp, do, dht, **kw)
    assert_grads(ref, got, SUITE_TOL, "dtypes")


@pytest.mark.parametrize("lens", [[15], [1, 63, 65], [100, 300, 56], [33, 128, 200, 95]])
def test_backward_varlen(lens):
    H, T = 2, sum(lens)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)
    inp = make_inputs(1, T, H, seed=9, gate_offset=-7.0)
    gen = torch.Generator().manual_seed(1)
    inp["initial_state"] = torch.randn(len(lens), H, 128, 128, generator=gen)
    do = torch.randn(1, T, H, 128, generator=gen).to(torch.bfloat16)
    dht = torch.randn(len(lens), H, 128, 128, generator=gen)
    ref, got = run_both(inp, do, dht, cu_seqlens=cu)
    assert_grads(ref, got, SUITE_TOL, f"varlen{lens}")


@pytest.mark.parametrize("seed", range(6))
def test_backward_varlen_random_sweep(seed):
    """Seeded random packed batches (1-5 sequences of 1-200 tokens, 1-3 heads): every gradient (with upstream gradients
    on the outputs and on the final states) against autograd of the oracle. Ragged last chunks of many lengths,
    sequences shorter than a chunk, a chunk-aligned and a single-token sequence occur across the six draws."""
    rng = np.random.default_rng(100 + seed)
    lens = [int(x) for x in rng.integers(1, 201, size=int(rng.integers(1, 6)))]
    if seed == 0:
        lens[0] = 64            # at least one chunk-aligned and one single-token sequence in the sweep
    if seed == 1:
        lens[-1] = 1
    H, T = int(rng.integers(1, 4)), sum(lens)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)
    inp = make_inputs(1, T, H, seed=20 + seed, gate_offset=-7.0)
    gen = torch.Generator().manual_seed(50 + seed)
    inp["initial_state"] = torch.randn(len(lens), H, 128, 128, generator=gen)
    do = torch.randn(1, T, H, 128, generator=gen).to(torch.bfloat16)
    dht = torch.randn(len(lens), H, 128, 128, generator=gen)
    ref, got = run_both(inp, do, dht, cu_seqlens=cu)
    assert_grads(ref, got, SUITE_TOL, f"varlen sweep {lens} H={H}")


def test_backward_small_upstream_gradient_and_no_state():
    """dO of order 1e-6 (mean-reduced losses): the power-of-two gradient scale keeps fp16 operands in range.
    Also covers initial_state=None / no final-state gradient."""
    from cula_b200.kda import chunk_kda
    B, T, H = 1, 256, 2
    inp = make_inputs(B, T, H, seed=3, gate_offset=-6.0)
    gen = torch.Generator().manual_seed(2)
    do = (1e-6 * torch.randn(B, T, H, 128, generator=gen)).to(torch.bfloat16)
    names = ("q", "k", "v", "g", "beta", "A_log", "dt_bias")
    ref_in = {n: inp[n].detach().float().clone().requires_grad_(True) for n in names}
    o, _ = chunk_kda_oracle(ref_in["q"], ref_in["k"], ref_in["v"], ref_in["g"], ref_in["beta"],
                            use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, safe_gate=True, lower_bound=-5.0,
                            A_log=ref_in["A_log"], dt_bias=ref_in["dt_bias"])
    (o * do.float()).sum().backward()
    dev = {n: inp[n].detach().cuda().requires_grad_(True) for n in names}
    o2, ht2 = chunk_kda(dev["q"], dev["k"], dev["v"], dev["g"], dev["beta"], use_qk_l2norm_in_kernel=True,
                        use_gate_in_kernel=True, safe_gate=True, lower_bound=-5.0, A_log=dev["A_log"], dt_bias=dev["dt_bias"])
    assert ht2 is None
    (o2.float() * do.cuda().float()).sum().backward()
    torch.cuda.synchronize()
    ref = {n: ref_in[n].grad for n in names}
    got = {n: dev[n].grad.float().cpu() for n in names}
    assert_grads(ref, got, SUITE_TOL, "tiny dO")


def test_backward_is_deterministic_except_atomics():
    """dq, dk, dv, dg, dbeta, dh0 are bit-identical across runs (dA_log / d dt_bias are atomic sums)."""
    inp = make_inputs(2, 300, 2, seed=1, gate_offset=-8.0, h0_std=1.0)
    gen = torch.Generator().manual_seed(3)
    do = torch.randn(2, 300, 2, 128, generator=gen).to(torch.bfloat16)
    dht = torch.randn(2, 2, 128, 128, generator=gen)
    runs = [run_both(inp, do, dht)[1] for _ in range(2)]
    for n in ("q", "k", "v", "g", "beta", "initial_state"):
        assert torch.equal(runs[0][n], runs[1][n]), n


def test_backward_with_more_scan_ctas_than_sms():
    """B * H * 2 > 148: the forward scans (plain and state-keeping) carry both value halves per CTA."""
    inp = make_inputs(5, 130, 16, seed=9, h0_std=0.1)
    gen = torch.Generator().manual_seed(10)
    do = torch.randn(5, 130, 16, 128, generator=gen).to(torch.bfloat16)
    dht = 0.1 * torch.randn(5, 16, 128, 128, generator=gen)
    ref, got = run_both(inp, do, dht)
    assert_grads(ref, got, HEADLINE_TOL, "wide grid")


def test_disable_recompute_keeps_the_forward_intermediates():
    """With ``disable_recompute=True`` the autograd node holds the forward intermediates and backward launches no
    forward kernel; without it backward re-runs the two forward launches. Both give the same gradients."""
    import cula_b200.kda.chunk as chunk_mod
    from cula_b200.kda import chunk_kda
    inp = make_inputs(2, 200, 2, seed=3, gate_offset=-7.0, h0_std=0.5)
    gen = torch.Generator().manual_seed(4)
    do = torch.randn(2, 200, 2, 128, generator=gen).to(torch.bfloat16).cuda()
    grads = {}
    for keep in (True, False):
        dev = {n: t.detach().cuda().requires_grad_(True) for n, t in inp.items()}
        o, _ = chunk_kda(dev["q"], dev["k"], dev["v"], dev["g"], dev["beta"], initial_state=dev["initial_state"],
                         output_final_state=True, use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, safe_gate=True,
                         lower_bound=-5.0, A_log=dev["A_log"], dt_bias=dev["dt_bias"], disable_recompute=keep)
        node = o.grad_fn
        assert (node.kept is not None) == keep
        if keep:
            assert all(node.kept[n] is not None for n in ("tiles", "akk", "mkk", "h32", "vnew"))
        before = chunk_mod.FORWARD_CALLS
        o.backward(do)
        torch.cuda.synchronize()
        assert chunk_mod.FORWARD_CALLS - before == (0 if keep else 1)
        grads[keep] = {n: t.grad.float().cpu() for n, t in dev.items()}
    for n in grads[True]:
        if n in ("A_log", "dt_bias"):           # atomic sums: equal up to the order of the additions
            assert err_ratio(grads[True][n], grads[False][n]) < 1e-5, n
        else:
            assert torch.equal(grads[True][n], grads[False][n]), n
    # nothing is kept when no input asks for a gradient or grad mode is off
    d = {n: t.cuda() for n, t in inp.items()}
    with torch.no_grad():
        o, _ = chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True,
                         safe_gate=True, lower_bound=-5.0, A_log=d["A_log"], dt_bias=d["dt_bias"], disable_recompute=True)
    assert o.grad_fn is None


@pytest.mark.parametrize("disable_recompute", [False, True])
def test_backward_long_sequence_all_gradients(disable_recompute):
    """One 8,192-token sequence (the length of the forward+backward configuration), weak gates so that the state and
    its gradient travel across all 128 chunks, non-zero initial state and final-state gradient: every gradient,
    dA_log and ddt_bias included, against autograd of the fp32 token recurrence (run on the CUDA device by torch so
    that 8,192 dependent steps finish in seconds)."""
    from cula_b200.kda import check_status, chunk_kda
    B, T, H = 1, 8192, 2
    inp = make_inputs(B, T, H, seed=21, gate_offset=-8.0, h0_std=0.1)
    gen = torch.Generator().manual_seed(22)
    inp["dt_bias"] = 0.1 * torch.randn(H * 128, generator=gen)
    do = torch.randn(B, T, H, 128, generator=gen).to(torch.bfloat16)
    dht = 0.1 * torch.randn(B, H, 128, 128, generator=gen)
    names = list(GRADS)
    ref_in = {n: inp[n].detach().float().cuda().requires_grad_(True) for n in names}
    o, ht = chunk_kda_oracle(ref_in["q"], ref_in["k"], ref_in["v"], ref_in["g"], ref_in["beta"],
                             initial_state=ref_in["initial_state"], output_final_state=True, use_qk_l2norm_in_kernel=True,
                             use_gate_in_kernel=True, safe_gate=True, lower_bound=-5.0, A_log=ref_in["A_log"],
                             dt_bias=ref_in["dt_bias"])
    ((o * do.cuda().float()).sum() + (ht * dht.cuda()).sum()).backward()
    dev_in = {n: inp[n].detach().cuda().requires_grad_(True) for n in names}
    o2, ht2 = chunk_kda(dev_in["q"], dev_in["k"], dev_in["v"], dev_in["g"], dev_in["beta"],
                        initial_state=dev_in["initial_state"], output_final_state=True, use_qk_l2norm_in_kernel=True,
                        use_gate_in_kernel=True, safe_gate=True, lower_bound=-5.0, A_log=dev_in["A_log"],
                        dt_bias=dev_in["dt_bias"], disable_recompute=disable_recompute)
    ((o2.float() * do.cuda().float()).sum() + (ht2 * dht.cuda()).sum()).backward()
    torch.cuda.synchronize()
    check_status()
    assert err_ratio(o.detach().cpu(), o2.detach().float().cpu()) <= 5e-3
    assert err_ratio(ht.detach().cpu(), ht2.detach().cpu()) <= 2e-3
    ref = {n: t.grad.cpu() for n, t in ref_in.items()}
    got = {n: t.grad.float().cpu() for n, t in dev_in.items()}
    assert_grads(ref, got, {"default": 5e-3, "A_log": 8e-3, "dt_bias": 8e-3}, "T8192")


@pytest.mark.parametrize("B,T,H", [(1, 64, 1), (2, 100, 3), (1, 64 * 160, 2)])
def test_dense_stage_against_torch_products(B, T, H):
    """cula_kda_bwd_dense alone, through the C ABI, on random inputs: every field of the scratch record and dv against
    fp64 matrix products of the same operands. The last shape has more tiles than SMs (persistent tile loop, TMA
    double buffering across tiles), the middle one a ragged last chunk. tf32 operands: 2e-3 relative RMS."""
    from cula_b200 import _native
    lib = _native.lib()
    g = torch.Generator().manual_seed(B * 1000 + T + H)
    nt = (T + 63) // 64
    tiles = B * nt * H
    h32 = torch.randn(tiles, 128, 128, generator=g)
    ds = torch.randn(tiles, 128, 128, generator=g)
    vnew = torch.randn(tiles, 64, 128, generator=g).half()
    dvn = torch.randn(tiles, 64, 128, generator=g).half()
    do = torch.randn(B, T, H, 128, generator=g).bfloat16()
    v = torch.randn(B, T, H, 128, generator=g).bfloat16()
    beta = torch.rand(B, T, H, generator=g)
    akk = torch.tril(torch.randn(tiles, 64, 64, generator=g) * 0.2)
    work = torch.tensor([4.0, 0.25, 0.0, 0.0])           # gradient scale s = 4 and 1 / s
    # tile = (b * nt + c) * H + h; padding rows of the last chunk carry zeros in the per-tile intermediates
    valid = torch.full((nt,), 64)
    valid[-1] = T - 64 * (nt - 1)
    for c in range(nt):
        for b in range(B):
            sl = slice((b * nt + c) * H, (b * nt + c + 1) * H)
            vnew[sl, int(valid[c]):] = 0
            dvn[sl, int(valid[c]):] = 0
    dev = {k: t.cuda() for k, t in dict(h32=h32, ds=ds, vnew=vnew, dvn=dvn, do=do, v=v, beta=beta, akk=akk, work=work).items()}
    dv = torch.zeros(B, T, H, 128, dtype=torch.bfloat16, device="cuda")
    nfl = lib.cula_kda_bwd_scratch_floats()
    scratch = torch.zeros(tiles, nfl, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.cula_kda_bwd_dense(dev["h32"].data_ptr(), dev["ds"].data_ptr(), dev["vnew"].data_ptr(), dev["dvn"].data_ptr(),
                                dev["do"].data_ptr(), dev["v"].data_ptr(), dev["beta"].data_ptr(), 1, dev["akk"].data_ptr(),
                                dev["work"].data_ptr(), dv.data_ptr(), scratch.data_ptr(), None, None, B * nt, T, H,
                                status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    scr = scratch.cpu().double()
    # reference, tile by tile in fp64
    pad = nt * 64 - T
    def tiled(x):       # [B, T, H, 128] -> [tiles, 64, 128], zero padding rows
        x = F.pad(x.double(), (0, 0, 0, 0, 0, pad)).view(B, nt, 64, H, 128).permute(0, 1, 3, 2, 4)
        return x.reshape(tiles, 64, 128)
    dO, V = 4.0 * tiled(do), tiled(v)
    bt = F.pad(beta.double(), (0, 0, 0, pad)).view(B, nt, 64, H).permute(0, 1, 3, 2).reshape(tiles, 64)
    S, dS, Vn, dVn, A = h32.double(), ds.double(), vnew.double(), dvn.double(), akk.double()
    lower, strict = torch.tril(torch.ones(64, 64, dtype=torch.float64)), torch.tril(torch.ones(64, 64, dtype=torch.float64), -1)
    Zu = A.transpose(1, 2) @ dVn
    ref = {
        "dqg": (0, dO @ S.transpose(1, 2)), "dw": (8192, -(dVn @ S.transpose(1, 2))), "dkg": (16384, Vn @ dS.transpose(1, 2)),
        "dps": (24576, (dO @ Vn.transpose(1, 2)) * lower), "dau": (28672, (dVn @ (bt[:, :, None] * V).transpose(1, 2)) * strict),
        "dbu": (32768, (Zu * V).sum(-1)), "dd": (32832, (S * dS).sum(-1)),
    }
    for name, (off, want) in ref.items():
        got = scr[:, off:off + want[0].numel()].reshape(want.shape)
        assert err_ratio(want, got) <= 2e-3, (name, err_ratio(want, got))
    dv_ref = 0.25 * bt[:, :, None] * Zu
    dv_got = tiled(dv.cpu())
    assert err_ratio(dv_ref, dv_got) <= 5e-3, err_ratio(dv_ref, dv_got)      # bf16 output


def test_forward_backward_is_capturable_in_a_cuda_graph():
    """A whole training step of the operator (forward with recomputation backward) captured once and replayed on new
    inputs: gradients equal the eager ones (dA_log / ddt_bias come from atomics: compared with a tolerance)."""
    from cula_b200.kda import check_status, chunk_kda
    B, T, H = 1, 192, 2
    names = ("q", "k", "v", "g", "beta", "A_log", "dt_bias", "initial_state")

    def step(x, do):
        for n in names:
            x[n].grad = None
        o, ht = chunk_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], A_log=x["A_log"], dt_bias=x["dt_bias"],
                          initial_state=x["initial_state"], output_final_state=True, use_qk_l2norm_in_kernel=True,
                          use_gate_in_kernel=True, safe_gate=True, lower_bound=-5.0)
        (o.float() * do.float()).sum().backward()
        return o

    def leaves(seed):
        return {n: t.cuda().requires_grad_(True) for n, t in make_inputs(B, T, H, seed=seed, gate_offset=-6.0, h0_std=0.5).items()}

    static, do = leaves(30), torch.randn(B, T, H, 128, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).cuda()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            step(static, do)                              # warm-up outside the capture (also creates the .grad buffers)
    torch.cuda.current_stream().wait_stream(side)
    for n in names:
        static[n].grad = None
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        o_static = step(static, do)
    grads_static = {n: static[n].grad for n in names}
    for seed in (31, 32):
        fresh = leaves(seed)
        with torch.no_grad():
            for n in names:
                static[n].copy_(fresh[n])
        graph.replay()
        o_ref = step(fresh, do)
        torch.cuda.synchronize()
        assert torch.equal(o_static, o_ref)
        for n in names:
            if n in ("A_log", "dt_bias"):
                assert err_ratio(fresh[n].grad.float().cpu(), grads_static[n].float().cpu()) <= 1e-5, n
            else:
                assert torch.equal(grads_static[n], fresh[n].grad), n
    check_status()
