"""GPU parity of the chunk_kda forward path (through the C ABI) against the CPU oracle and the golden
vectors. Tolerances: o relative RMS <= 5e-3 and max-abs <= 2e-2; final_state relative <= 1e-3
(headline configurations) -- the reference's own test asks 5e-3 for both (tests/test_kda.py:145-146)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from chunkwise_ref import chunk_quantities, decode_tiles
from conftest import GOLDEN_CASES, load_golden
from oracle import c_oracle
from oracle.naive_kda import err_ratio, kda_gate, make_inputs

pytestmark = pytest.mark.gpu

O_RMS, O_MAXABS, HT_REL = 5e-3, 2e-2, 1e-3


def _cuda(x):
    return None if x is None else x.cuda()


def run_chunk_kda(inp, cu_seqlens=None, l2=True, gate=True, safe=True, lower_bound=-5.0, **kw):
    from cula_b200.kda import check_status, chunk_kda
    extra = dict(A_log=_cuda(inp.get("A_log")), dt_bias=_cuda(inp.get("dt_bias"))) if gate else {}
    o, ht = chunk_kda(_cuda(inp["q"]), _cuda(inp["k"]), _cuda(inp["v"]), _cuda(inp["g"]), _cuda(inp["beta"]),
                      initial_state=_cuda(inp.get("initial_state")), output_final_state=True,
                      use_qk_l2norm_in_kernel=l2, use_gate_in_kernel=gate, safe_gate=safe,
                      lower_bound=lower_bound if (gate and safe) else None,
                      cu_seqlens=_cuda(cu_seqlens), **extra, **kw)
    torch.cuda.synchronize()
    check_status()
    return o, ht


def oracle_fwd(inp, cu_seqlens=None, l2=True, gate=True, safe=True, lower_bound=-5.0):
    f = lambda x: None if x is None else x.float().numpy()
    mode = 0 if not gate else (2 if safe else 1)
    o, ht = c_oracle.naive_kda_fwd(f(inp["q"]), f(inp["k"]), f(inp["v"]), f(inp["g"]), f(inp["beta"]),
                                   f(inp.get("A_log")) if gate else None, f(inp.get("dt_bias")) if gate else None,
                                   f(inp.get("initial_state")),
                                   cu_seqlens=None if cu_seqlens is None else cu_seqlens.numpy(),
                                   use_l2norm=l2, gate_mode=mode, lower_bound=lower_bound)
    return torch.from_numpy(o), torch.from_numpy(ht)


def assert_fwd_close(o, ht, o_ref, ht_ref, ht_tol=HT_REL, tag=""):
    o, ht = o.float().cpu(), ht.float().cpu()
    assert torch.isfinite(o).all() and torch.isfinite(ht).all(), tag
    e_o, e_h = err_ratio(o_ref, o), err_ratio(ht_ref, ht)
    mx = float((o_ref - o).abs().max())
    assert e_o <= O_RMS and mx <= O_MAXABS and e_h <= ht_tol, f"{tag}: o rms {e_o:.2e} maxabs {mx:.2e} ht {e_h:.2e}"
    return e_o, mx, e_h


@pytest.mark.parametrize("gate_offset", [0.0, -8.0])
def test_chunk_parallel_stage_against_fp64_model(gate_offset):
    """The chunk-parallel stage alone: decode its tile packs and compare each array with an fp64
    torch model of the chunk algebra (w, u, kg, qg, Aqk, decay, Akk)."""
    from cula_b200.kda.chunk import chunk_kda_fwd
    B, T, H = 1, 150, 2
    inp = make_inputs(B, T, H, seed=3, gate_offset=gate_offset)
    inp["A_log"] = inp["A_log"] + 0.2
    dev = {k: _cuda(v) for k, v in inp.items()}
    out = chunk_kda_fwd(dev["q"], dev["k"], dev["v"], dev["g"], dev["beta"], 128 ** -0.5, None, False, None, None,
                        True, True, True, -5.0, dev["A_log"], dev["dt_bias"], store_akk=True)
    torch.cuda.synchronize()
    nt = (T + 63) // 64
    got = {k: v.cpu() for k, v in decode_tiles(out["tiles"], nt * H).items()}
    akk = out["akk"].cpu()
    a = kda_gate(inp["g"], inp["A_log"], inp["dt_bias"], -5.0).double()
    qn = F.normalize(inp["q"].double(), dim=-1)
    kn = F.normalize(inp["k"].double(), dim=-1)
    msgs = []
    for h in range(H):
        ref = chunk_quantities(qn[0, :, h], kn[0, :, h], inp["v"][0, :, h].double(), a[0, :, h],
                               inp["beta"][0, :, h].double(), 128 ** -0.5)
        for c in range(nt):
            ti = c * H + h
            for name, tol in (("w", 1e-3), ("qg", 1e-3), ("kg", 1e-3), ("u", 1e-3), ("aqk", 1e-3)):
                e = err_ratio(ref[c][name], got[name][ti])
                if not e <= tol:
                    msgs.append(f"{name}[c={c},h={h}] rel {e:.2e} > {tol}")
            if not float((ref[c]["decay"] - got["decay"][ti]).abs().max()) <= 1e-5:   # underflows to 0 with strong gates
                msgs.append(f"decay[c={c},h={h}]")
            e = err_ratio(ref[c]["akk"], akk[ti])
            if not e <= 1e-4:
                msgs.append(f"akk[c={c},h={h}] rel {e:.2e}")
    assert not msgs, "; ".join(msgs[:12])


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_forward_matches_golden(name):
    case, inp, exp = load_golden(name)
    inp["initial_state"] = inp.pop("h0", None)
    o, ht = run_chunk_kda(inp, cu_seqlens=case["cu_seqlens"], l2=case["use_l2norm"], gate=case["use_gate_in_kernel"],
                          safe=case["safe_gate"], lower_bound=case["lower_bound"])
    assert_fwd_close(o, ht, exp["o"], exp["ht"], tag=name)


def test_headline_cpu_config():
    """B=1, T=512, H=4: the configuration the CPU baseline is quoted on."""
    inp = make_inputs(1, 512, 4, seed=0)
    o, ht = run_chunk_kda(inp)
    o_ref, ht_ref = oracle_fwd(inp)
    assert_fwd_close(o, ht, o_ref, ht_ref, tag="config1")


@pytest.mark.parametrize("B,T,H,gate_offset,h0_std", [
    (1, 63, 1, -6.0, 1.0), (2, 500, 3, -8.0, 1.0), (2, 1000, 3, 0.0, 1.0), (2, 1500, 4, -8.0, 0.5),
    (1, 1, 2, -8.0, 1.0), (1, 65, 2, -8.0, 0.0), (1, 127, 1, -4.0, 1.0), (4, 2048, 8, -8.0, 0.1),
])
def test_forward_shapes_of_the_reference_suite(B, T, H, gate_offset, h0_std):
    """Ragged lengths of tests/test_kda.py:52-59 plus tiny ones, weak and strong gates, with initial state."""
    inp = make_inputs(B, T, H, seed=42, gate_offset=gate_offset, h0_std=h0_std)
    inp["A_log"] = inp["A_log"] + 0.1
    inp["dt_bias"] = 0.1 * torch.randn(H * 128, generator=torch.Generator().manual_seed(7))
    o, ht = run_chunk_kda(inp)
    o_ref, ht_ref = oracle_fwd(inp)
    assert_fwd_close(o, ht, o_ref, ht_ref, ht_tol=2e-3, tag=f"B{B}T{T}H{H}")


@pytest.mark.parametrize("beta_dtype,g_fp32", [(torch.float32, False), (torch.bfloat16, True)])
def test_forward_pre_gated_and_dtypes(beta_dtype, g_fp32):
    """use_gate_in_kernel=False (g is the fp32 log decay, clamped to [-5, 0]) and fp32 beta."""
    B, T, H = 2, 200, 2
    inp = make_inputs(B, T, H, seed=5, h0_std=1.0, beta_dtype=beta_dtype)
    gen = torch.Generator().manual_seed(11)
    a = (F.logsigmoid(torch.randn(B, T, H, 128, generator=gen)) / 4.0).clamp(-5, 0)
    inp["g"] = a if g_fp32 else a.to(torch.bfloat16)
    inp["q"] = F.normalize(inp["q"].float(), dim=-1).to(torch.bfloat16)
    inp["k"] = F.normalize(inp["k"].float(), dim=-1).to(torch.bfloat16)
    o, ht = run_chunk_kda(inp, l2=False, gate=False)
    o_ref, ht_ref = oracle_fwd(inp, l2=False, gate=False)
    assert_fwd_close(o, ht, o_ref, ht_ref, ht_tol=2e-3, tag="pre-gated")


VARLEN = [[15], [64], [1, 63, 65], [100, 300, 56], [256, 100, 300, 400, 1], [33, 128, 200, 95]]


@pytest.mark.parametrize("lens", VARLEN)
def test_forward_varlen(lens):
    H, T = 3, sum(lens)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)
    inp = make_inputs(1, T, H, seed=9, gate_offset=-7.0)
    inp["initial_state"] = torch.randn(len(lens), H, 128, 128, generator=torch.Generator().manual_seed(1))
    o, ht = run_chunk_kda(inp, cu_seqlens=cu)
    o_ref, ht_ref = oracle_fwd(inp, cu_seqlens=cu)
    assert_fwd_close(o, ht, o_ref, ht_ref, ht_tol=2e-3, tag=f"varlen{lens}")
    # one packed sequence equals the fixed-length call bit for bit
    if len(lens) == 1:
        o2, ht2 = run_chunk_kda(inp)
        assert torch.equal(o, o2) and torch.equal(ht, ht2)


def test_varlen_padding_rows_stay_zero():
    """Tokens past cu_seqlens[-1] (serving stacks pad the packed batch) must come back as zeros."""
    H, T = 2, 200
    cu = torch.tensor([0, 70, 150], dtype=torch.int32)
    inp = make_inputs(1, T, H, seed=2, gate_offset=-6.0)
    o, _ = run_chunk_kda(inp, cu_seqlens=cu)
    assert float(o[:, 150:].abs().max()) == 0.0
    assert float(o[:, :150].abs().max()) > 0.0


def test_forward_is_deterministic_and_without_final_state():
    from cula_b200.kda import chunk_kda
    inp = make_inputs(2, 300, 4, seed=1, gate_offset=-8.0, h0_std=1.0)
    outs = [run_chunk_kda(inp) for _ in range(3)]
    for o, ht in outs[1:]:
        assert torch.equal(o, outs[0][0]) and torch.equal(ht, outs[0][1])
    o, ht = chunk_kda(inp["q"].cuda(), inp["k"].cuda(), inp["v"].cuda(), inp["g"].cuda(), inp["beta"].cuda(),
                      use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, safe_gate=True, lower_bound=-5.0,
                      A_log=inp["A_log"].cuda(), dt_bias=inp["dt_bias"].cuda(), initial_state=inp["initial_state"].cuda())
    assert ht is None and torch.equal(o, outs[0][0])


def test_return_intermediate_states():
    """h[b, c] is the state entering chunk c (bf16), as the reference returns it in inference mode."""
    from cula_b200.kda import chunk_kda
    B, T, H = 1, 192, 2
    inp = make_inputs(B, T, H, seed=4, gate_offset=-8.0, h0_std=1.0)
    with torch.inference_mode():
        o, ht, h = chunk_kda(inp["q"].cuda(), inp["k"].cuda(), inp["v"].cuda(), inp["g"].cuda(), inp["beta"].cuda(),
                             use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, safe_gate=True, lower_bound=-5.0,
                             A_log=inp["A_log"].cuda(), dt_bias=inp["dt_bias"].cuda(),
                             initial_state=inp["initial_state"].cuda(), output_final_state=True,
                             return_intermediate_states=True)
    assert h.shape == (B, 3, H, 128, 128)
    assert err_ratio(inp["initial_state"], h[:, 0].float().cpu()) < 4e-3      # bf16 rounding of h0
    short = {k: (v[:, :128] if k in ("q", "k", "v", "g", "beta") else v) for k, v in inp.items()}
    _, ht128 = oracle_fwd(short)
    assert err_ratio(ht128, h[:, 2].float().cpu()) < 5e-3


def test_host_pipelined_forward_matches_device_call():
    """chunk_kda_host (segments + carried state, copies overlapped) returns exactly what chunk_kda returns."""
    from cula_b200.kda import chunk_kda, chunk_kda_host
    B, T, H = 2, 1200, 3                      # not a multiple of the segment length
    inp = make_inputs(B, T, H, seed=6, gate_offset=-7.0, h0_std=0.5)
    host = {k: v.pin_memory() for k, v in inp.items()}
    o_h, ht_h = chunk_kda_host(host["q"], host["k"], host["v"], host["g"], host["beta"], segment_tokens=512,
                               initial_state=host["initial_state"], output_final_state=True, use_qk_l2norm_in_kernel=True,
                               use_gate_in_kernel=True, safe_gate=True, lower_bound=-5.0, A_log=host["A_log"],
                               dt_bias=host["dt_bias"])
    d = {k: v.cuda() for k, v in inp.items()}
    o_d, ht_d = chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["initial_state"],
                          output_final_state=True, use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, safe_gate=True,
                          lower_bound=-5.0, A_log=d["A_log"], dt_bias=d["dt_bias"])
    torch.cuda.synchronize()
    assert o_h.device.type == "cpu" and torch.equal(o_h, o_d.cpu()) and torch.equal(ht_h, ht_d.cpu())


def test_intermediate_states_do_not_depend_on_the_scan_variant():
    """return_intermediate_states for a batch wide enough for the eight-warp scan CTAs (B * H * 2 > 148) must equal,
    bit for bit, the states of the same sequences run in two narrower batches (four-warp CTAs)."""
    from cula_b200.kda import chunk_kda
    B, T, H = 6, 200, 16
    inp = make_inputs(B, T, H, seed=12, h0_std=0.3)
    d = {k: v.cuda() for k, v in inp.items()}
    kw = dict(use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, safe_gate=True, lower_bound=-5.0, A_log=d["A_log"],
              dt_bias=d["dt_bias"], output_final_state=True, return_intermediate_states=True)
    with torch.inference_mode():
        o, ht, h = chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["initial_state"], **kw)
        parts = [chunk_kda(d["q"][s], d["k"][s], d["v"][s], d["g"][s], d["beta"][s], initial_state=d["initial_state"][s], **kw)
                 for s in (slice(0, 3), slice(3, 6))]
    torch.cuda.synchronize()
    assert torch.equal(o, torch.cat([p[0] for p in parts])) and torch.equal(ht, torch.cat([p[1] for p in parts]))
    assert torch.equal(h, torch.cat([p[2] for p in parts]))


@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
def test_two_different_cu_seqlens_of_equal_length_back_to_back(dtype):
    """The index tables are cached per cu_seqlens tensor; a second tensor with the same number of sequences but
    other boundaries (int64 ones are converted, so the caller's tensor may be freed and its address reused) must
    get its own tables."""
    H, T = 2, 400
    inp = make_inputs(1, T, H, seed=13, gate_offset=-7.0)
    for bounds in ([0, 100, 300, 400], [0, 64, 130, 400], [0, 190, 191, 400]):
        cu = torch.tensor(bounds, dtype=dtype)
        o, ht = run_chunk_kda(inp, cu_seqlens=cu)
        o_ref, ht_ref = oracle_fwd(inp, cu_seqlens=torch.tensor(bounds, dtype=torch.int32))
        assert_fwd_close(o, ht, o_ref, ht_ref, ht_tol=2e-3, tag=f"{bounds}")
        del cu


def test_values_outside_the_fp16_range_are_reported():
    """|v| beyond the fp16 range cannot be carried by the tile pack: the kernel reports it through the status word,
    ``check_status`` raises, and so does the next ``chunk_kda`` call on the device."""
    from cula_b200.kda import check_status, chunk_kda
    inp = make_inputs(1, 128, 2, seed=14, gate_offset=-7.0)
    d = {k: v.cuda() for k, v in inp.items() if v is not None}
    kw = dict(use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, safe_gate=True, lower_bound=-5.0, A_log=d["A_log"],
              dt_bias=d["dt_bias"])
    torch.cuda.synchronize()
    check_status()
    big = d["v"].clone()
    big[0, 70, 1, 5] = 3.0e5
    chunk_kda(d["q"], d["k"], big, d["g"], d["beta"], **kw)
    with pytest.raises(RuntimeError, match="fp16 range"):
        check_status()
    check_status()                                   # cleared by the raise
    chunk_kda(d["q"], d["k"], big, d["g"], d["beta"], **kw)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="fp16 range"):
        chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], **kw)      # surfaced by the following call
    o, _ = chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], **kw)   # and the device is usable afterwards
    torch.cuda.synchronize()
    check_status()
    assert torch.isfinite(o).all()


def test_bounded_wait_gives_up_and_reports():
    """A wait on a barrier that nothing ever completes must run out after its (here: short) limit, set the
    time-out status and let the kernel return -- the same bounded wait every pipeline of the library uses."""
    import time
    from cula_b200 import _native
    lib = _native.lib()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    t0 = time.perf_counter()
    _native.check(lib.cula_kda_selftest_bounded_wait(status.data_ptr(), 2000, stream), "selftest")
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0
    assert int(status.item()) == 1
    # the context is intact: an ordinary forward still works
    inp = make_inputs(1, 64, 1, seed=1, gate_offset=-6.0)
    o, ht = run_chunk_kda(inp)
    assert torch.isfinite(o).all()


def test_strong_softplus_gate_matches_oracle():
    """safe_gate=False (softplus gate, no lower bound) with a decay of about 3 nats per token -- 48 nats inside a
    16-row block, well inside the range the per-block anchoring carries exactly."""
    inp = make_inputs(2, 200, 2, seed=15, gate_offset=3.0, h0_std=0.5)
    o, ht = run_chunk_kda(inp, safe=False)
    o_ref, ht_ref = oracle_fwd(inp, safe=False)
    assert_fwd_close(o, ht, o_ref, ht_ref, ht_tol=2e-3, tag="softplus strong")


def test_unbounded_gate_stays_finite():
    """A pre-gated decay of -9 nats per token is outside what the per-block anchoring can carry (a 16-row block
    spans 2^195, fp32 ends at 2^127; the safe gate, lower_bound >= -5, guarantees 2^116). The reference refuses such
    gates outright (cula/kda/chunk_intra.py:761); here the clamped factor tables must at least keep inf * 0 out of the
    Gram products: everything stays finite (the values are not claimed to be accurate in that regime)."""
    B, T, H = 1, 130, 2
    inp = make_inputs(B, T, H, seed=16, h0_std=0.5)
    gen = torch.Generator().manual_seed(17)
    inp["g"] = (-9.0 + 0.5 * torch.randn(B, T, H, 128, generator=gen)).float()
    inp["q"] = F.normalize(inp["q"].float(), dim=-1).to(torch.bfloat16)
    inp["k"] = F.normalize(inp["k"].float(), dim=-1).to(torch.bfloat16)
    o, ht = run_chunk_kda(inp, l2=False, gate=False)
    assert torch.isfinite(o).all() and torch.isfinite(ht).all()


def test_forward_is_capturable_in_a_cuda_graph():
    """Serving stacks replay the forward from a CUDA graph: nothing in the call may synchronise, allocate outside the
    graph's pool or read a device value on the host. Captured once, replayed on new input contents, compared bit for
    bit with the eager call (the kernels are deterministic)."""
    from cula_b200.kda import check_status, chunk_kda
    B, T, H = 2, 200, 3
    kw = dict(use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, safe_gate=True, lower_bound=-5.0,
              output_final_state=True)

    def call(x):
        return chunk_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], A_log=x["A_log"], dt_bias=x["dt_bias"],
                         initial_state=x["initial_state"], **kw)

    static = {n: t.cuda() for n, t in make_inputs(B, T, H, seed=5, gate_offset=-6.0, h0_std=0.5).items()}
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side), torch.no_grad():
        call(static)                                     # warm-up outside the capture
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.no_grad(), torch.cuda.graph(graph):
        o_static, ht_static = call(static)
    for seed in (6, 7):
        fresh = {n: t.cuda() for n, t in make_inputs(B, T, H, seed=seed, gate_offset=-6.0, h0_std=0.5).items()}
        for n in static:
            static[n].copy_(fresh[n])
        graph.replay()
        with torch.no_grad():
            o_ref, ht_ref = call(fresh)
        torch.cuda.synchronize()
        assert torch.equal(o_static, o_ref) and torch.equal(ht_static, ht_ref)
    check_status()
