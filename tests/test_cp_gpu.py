"""Context-parallel kernels on the GPU. With one device the W ranks are emulated one after the other in this
process (the gather is a stack), which exercises the transition launch, the fold kernel and the scan from a folded
state; with two or more devices a real NCCL run is launched through torch.distributed.run."""
import os
import subprocess
import sys

import pytest
import torch

from oracle import c_oracle
from oracle.naive_kda import err_ratio, make_inputs

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _oracle(inp):
    f = lambda x: None if x is None else x.float().numpy()
    o, ht = c_oracle.naive_kda_fwd(f(inp["q"]), f(inp["k"]), f(inp["v"]), f(inp["g"]), f(inp["beta"]), f(inp["A_log"]),
                                   f(inp["dt_bias"]), f(inp["initial_state"]), use_l2norm=True, gate_mode=2, lower_bound=-5.0)
    return torch.from_numpy(o), torch.from_numpy(ht)


@pytest.mark.parametrize("segments", [1, 2])
@pytest.mark.parametrize("world,T,gate_offset", [(2, 256, -8.0), (4, 1024, -8.0), (3, 64 * 5 + 17, -6.0), (4, 512, 0.0),
                                                 (8, 64 * 8 * 3 + 40, -8.0)])
def test_cp_emulated_ranks_match_oracle(world, T, gate_offset, segments):
    from cula_b200.kda import check_status
    from cula_b200.kda.cp import CudaBackend, cp_forward
    H = 4
    inp = make_inputs(1, T, H, seed=2, gate_offset=gate_offset, h0_std=0.5)
    per = (T // world) // 64 * 64
    bounds = [r * per for r in range(world)] + [T]
    backends = []
    for r in range(world):
        sl = slice(bounds[r], bounds[r + 1])
        backends.append(CudaBackend(inp["q"][:, sl].cuda(), inp["k"][:, sl].cuda(), inp["v"][:, sl].cuda(),
                                    inp["g"][:, sl].cuda(), inp["beta"][:, sl].cuda(), 128 ** -0.5, True, True, True, -5.0,
                                    inp["A_log"].cuda(), inp["dt_bias"].cuda(), segments=segments))
    trans = [b.transition() for b in backends]               # (C | M) per shard; some segments are empty here
    h0 = inp["initial_state"].cuda()
    # the emulated collective: every rank sees the same tensor; rank 0's pair carries the initial state
    X_all = torch.stack([backends[0].absorb_initial_state(trans[0], h0)] + trans[1:])

    outs, final = [], None
    for r, b in enumerate(backends):
        b.transition = lambda t=trans[r]: t           # already computed above
        # the state before the first token is handed to rank 0 ONLY
        o, ht = cp_forward(b, lambda x: X_all, r, world, h0 if r == 0 else None, True)
        outs.append(o)
        final = ht if ht is not None else final
    torch.cuda.synchronize()
    check_status()
    o = torch.cat(outs, dim=1).float().cpu()
    o_ref, ht_ref = _oracle(inp)
    assert err_ratio(o_ref, o) <= 5e-3 and float((o_ref - o).abs().max()) <= 2e-2
    assert err_ratio(ht_ref, final.cpu()) <= 2e-3


def test_cp_transition_is_the_affine_map_of_the_shard():
    """S_out = M S_in + C must reproduce the final state of a scan started from a random state."""
    from cula_b200.kda import chunk_kda
    from cula_b200.kda.cp import CudaBackend
    T, H = 320, 2
    inp = make_inputs(1, T, H, seed=4, gate_offset=-8.0, h0_std=1.0)
    d = {k: v.cuda() for k, v in inp.items()}
    b = CudaBackend(d["q"], d["k"], d["v"], d["g"], d["beta"], 128 ** -0.5, True, True, True, -5.0, d["A_log"], d["dt_bias"],
                    segments=1)
    C, M = b.transition()
    _, ht = chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], A_log=d["A_log"], dt_bias=d["dt_bias"],
                      initial_state=d["initial_state"], output_final_state=True, use_qk_l2norm_in_kernel=True,
                      use_gate_in_kernel=True, safe_gate=True, lower_bound=-5.0)
    pred = torch.matmul(M.double(), d["initial_state"][0].double()) + C.double()
    assert err_ratio(ht[0].double().cpu(), pred.cpu()) <= 2e-3
    X0 = b.absorb_initial_state(torch.stack([C, M]), d["initial_state"])       # what rank 0 would publish
    folded = b.incoming(X0[None].repeat(2, 1, 1, 1, 1), 1, None)[0]            # what rank 1 folds from it
    assert err_ratio(pred.cpu(), folded.double().cpu()) <= 1e-5


def test_cp_composed_segments_equal_the_whole_shard():
    """Composing the transitions of two segments must give the transition of the undivided shard."""
    from cula_b200.kda.cp import CudaBackend
    T, H = 64 * 7 + 30, 2
    inp = make_inputs(1, T, H, seed=5, gate_offset=-8.0)
    d = {k: (v.cuda() if v is not None else None) for k, v in inp.items()}
    mk = lambda P: CudaBackend(d["q"], d["k"], d["v"], d["g"], d["beta"], 128 ** -0.5, True, True, True, -5.0, d["A_log"],
                               d["dt_bias"], segments=P)
    X1, X2, X3 = mk(1).transition(), mk(2).transition(), mk(3).transition()
    for X in (X2, X3):
        assert err_ratio(X1[0].cpu(), X[0].cpu()) <= 2e-3 and err_ratio(X1[1].cpu(), X[1].cpu()) <= 2e-3


@pytest.mark.parametrize("world,T,segments", [(2, 256, 1), (4, 512, 2), (3, 64 * 5 + 17, 2)])
def test_cp_backward_emulated_ranks_match_oracle_autograd(world, T, segments):
    """Forward and backward of every shard with the exchanges emulated in-process; gradients against autograd of
    the fp32 oracle on the whole sequence. Weak gates, so the gradient that crosses shard boundaries matters."""
    from cula_b200.kda import check_status
    from cula_b200.kda.cp import CPBackwardState, CudaBackend, cp_forward
    from oracle.naive_kda import chunk_kda_oracle
    H = 2
    inp = make_inputs(1, T, H, seed=7, gate_offset=-8.0, h0_std=0.5)
    gen = torch.Generator().manual_seed(11)
    do = torch.randn(1, T, H, 128, generator=gen).to(torch.bfloat16)
    dht = 0.1 * torch.randn(1, H, 128, 128, generator=gen)
    names = ("q", "k", "v", "g", "beta", "A_log", "dt_bias", "initial_state")
    ref_in = {n: inp[n].detach().float().clone().requires_grad_(True) for n in names}
    o_ref, ht_ref = chunk_kda_oracle(ref_in["q"], ref_in["k"], ref_in["v"], ref_in["g"], ref_in["beta"],
                                     initial_state=ref_in["initial_state"], output_final_state=True,
                                     use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, safe_gate=True, lower_bound=-5.0,
                                     A_log=ref_in["A_log"], dt_bias=ref_in["dt_bias"])
    ((o_ref * do.float()).sum() + (ht_ref * dht).sum()).backward()

    per = (T // world) // 64 * 64
    bounds = [r * per for r in range(world)] + [T]
    flags = (True, True, True, -5.0)
    A_log, dt_bias = inp["A_log"].cuda(), inp["dt_bias"].cuda()
    shards, backends = [], []
    for r in range(world):
        sl = slice(bounds[r], bounds[r + 1])
        sh = {n: inp[n][:, sl].cuda().contiguous() for n in ("q", "k", "v", "g", "beta")}
        shards.append(sh)
        backends.append(CudaBackend(sh["q"], sh["k"], sh["v"], sh["g"], sh["beta"], 128 ** -0.5, *flags, A_log, dt_bias,
                                    segments=segments))
    trans = [b.transition() for b in backends]
    h0 = inp["initial_state"].cuda()
    X_all = torch.stack([backends[0].absorb_initial_state(trans[0], h0)] + trans[1:])
    states = []
    for r, b in enumerate(backends):
        b.transition = lambda t=trans[r]: t
        aux = {}
        cp_forward(b, lambda x: X_all, r, world, h0 if r == 0 else None, True, aux)
        sh = shards[r]
        states.append(CPBackwardState(sh["q"], sh["k"], sh["v"], sh["g"], sh["beta"], A_log, dt_bias, aux["s_in"], aux["X_all"],
                                      128 ** -0.5, flags, r, world))
    Y_all = torch.stack([st.prepare(do[:, bounds[r]:bounds[r + 1]].cuda(), dht.cuda() if r == world - 1 else None)
                         for r, st in enumerate(states)])
    grads = [st.finish(Y_all) for st in states]
    torch.cuda.synchronize()
    check_status()
    got = {n: torch.cat([g[i] for g in grads], dim=1).float().cpu() for i, n in enumerate(("q", "k", "v", "g", "beta"))}
    got["A_log"] = sum(g[5] for g in grads).float().cpu().view_as(inp["A_log"])
    got["dt_bias"] = sum(g[6] for g in grads).float().cpu().view_as(inp["dt_bias"])
    got["initial_state"] = grads[0][7].float().cpu()
    tol = {"g": 2e-2, "beta": 2e-2}
    for n in names:
        ref = ref_in[n].grad
        e = err_ratio(ref, got[n])
        assert e <= tol.get(n, 8e-3) and torch.isfinite(got[n]).all(), (n, e)


def _run_nccl_worker(world, port, tmp_path):
    script = os.path.join(ROOT, "tests", "cp_nccl_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                          "--master-addr", "127.0.0.1", "--master-port", str(port), script, str(tmp_path)],
                         capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert "CP_OK" in out.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_cp_two_gpus_nccl(tmp_path):
    _run_nccl_worker(2, 29611, tmp_path)


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs four GPUs")
def test_cp_all_gpus_nccl(tmp_path):
    """Forward, final state and every gradient over 4 (or 8) ranks: shards of 256 (128) tokens, so every rank but the
    first both receives and passes on a carried state, forward and backward."""
    _run_nccl_worker(8 if torch.cuda.device_count() >= 8 else 4, 29612, tmp_path)
