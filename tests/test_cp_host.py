"""Context-parallel orchestration on CPU: two gloo ranks run `cp_forward` with a compute backend built from the
oracle's token recurrence, and the stitched result must equal the single-process oracle. This covers the host
logic of the multi-GPU path (shard order, gather, fold order, which rank owns the final state) without a GPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cula_b200.kda.cp import cp_forward, gather_with_group
from oracle.naive_kda import chunk_kda_oracle, err_ratio, kda_gate, l2norm, make_inputs, naive_recurrent_kda


class OracleBackend:
    """transition / fold / forward of one shard evaluated with the fp32 token recurrence. ``bounds`` cuts the
    shard into segments (token offsets, [0, ..., T])."""

    def __init__(self, shard, bounds=None):
        self.q, self.k = l2norm(shard["q"]), l2norm(shard["k"])
        self.v, self.beta = shard["v"].float(), shard["beta"].float()
        self.a = kda_gate(shard["g"], shard["A_log"], shard["dt_bias"], -5.0)
        self.H = self.q.shape[2]
        self.bounds = bounds if bounds is not None else [0, self.q.shape[1]]
        self.n_segments = len(self.bounds) - 1

    def _seg(self, i):
        sl = slice(self.bounds[i], self.bounds[i + 1])
        return self.q[:, sl], self.k[:, sl], self.v[:, sl], self.a[:, sl], self.beta[:, sl]

    def transition(self, local_only=False):
        self.C_seg, self.M_seg = [], []
        C_tot, M_tot = torch.zeros(self.H, 128, 128), torch.eye(128).expand(self.H, 128, 128).clone()
        for i in range(self.n_segments):
            q, k, v, a, beta = self._seg(i)
            _, C = naive_recurrent_kda(q, k, v, a, beta, None, None, True)
            # M: the recurrence is linear in the state when v = 0; push the identity through it
            eye = torch.eye(128).expand(1, self.H, 128, 128)
            _, M = naive_recurrent_kda(q, k, torch.zeros_like(v), a, beta, None, eye, True)
            self.C_seg.append(C[0])
            self.M_seg.append(M[0])
            C_tot, M_tot = M[0] @ C_tot + C[0], M[0] @ M_tot
        return torch.stack([C_tot, M_tot])

    def absorb_initial_state(self, X, initial_state):
        return torch.stack([X[1] @ initial_state.reshape(self.H, 128, 128) + X[0], X[1]])

    def incoming(self, X_all, rank, initial_state):
        S = torch.zeros(self.H, 128, 128)
        if rank == 0 and initial_state is not None:
            S = initial_state.reshape(self.H, 128, 128).clone()
        for j in range(rank):
            S = X_all[j, 1] @ S + X_all[j, 0]
        states = [S]
        for i in range(1, self.n_segments):
            S = self.M_seg[i - 1] @ S + self.C_seg[i - 1]
            states.append(S)
        return states

    def forward(self, states, want_final):
        outs, ht = [], None
        for i, s_in in enumerate(states):
            q, k, v, a, beta = self._seg(i)
            s_in = None if s_in is None else s_in.reshape(1, self.H, 128, 128)
            o, ht = naive_recurrent_kda(q, k, v, a, beta, None, s_in, want_final)
            outs.append(o)
        return torch.cat(outs, dim=1), ht


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, T, H, out_dir, segmented):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        inp = make_inputs(1, T, H, seed=0, gate_offset=-8.0, h0_std=0.5)
        per = T // world
        lo, hi = rank * per, (T if rank == world - 1 else (rank + 1) * per)
        shard = {n: (t[:, lo:hi] if n in ("q", "k", "v", "g", "beta") else t) for n, t in inp.items()}
        n_loc = hi - lo
        bounds = [0, 64, n_loc] if segmented else None       # same segment count on every rank
        # the state before the first token is given on rank 0 ONLY: the exchange has to carry it to the others
        h0 = inp["initial_state"] if rank == 0 else None
        o, ht = cp_forward(OracleBackend(shard, bounds), gather_with_group(None), rank, world, h0, True)
        assert (ht is not None) == (rank == world - 1)
        torch.save((o, ht), os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
@pytest.mark.parametrize("segmented", [False, True])
def test_cp_forward_two_gloo_ranks(tmp_path, segmented):
    world, T, H = 2, 320, 2                      # 160 + 160 tokens; weak gates so the carried state matters
    port = _free_port()
    mp.spawn(_worker, args=(world, port, T, H, str(tmp_path), segmented), nprocs=world, join=True)
    parts = [torch.load(os.path.join(tmp_path, f"rank{r}.pt")) for r in range(world)]
    o = torch.cat([p[0] for p in parts], dim=1)
    ht = parts[-1][1]
    inp = make_inputs(1, T, H, seed=0, gate_offset=-8.0, h0_std=0.5)
    o_ref, ht_ref = chunk_kda_oracle(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], initial_state=inp["initial_state"],
                                     output_final_state=True, use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True,
                                     safe_gate=True, lower_bound=-5.0, A_log=inp["A_log"], dt_bias=inp["dt_bias"])
    assert err_ratio(o_ref, o) < 1e-5 and err_ratio(ht_ref, ht) < 1e-5
    # the carried state matters in this fixture: dropping it must be visible
    o_wrong, _ = OracleBackend({n: (t[:, 160:] if n in ("q", "k", "v", "g", "beta") else t)
                                for n, t in inp.items()}).forward([None], False)
    assert err_ratio(o_ref[:, 160:], o_wrong) > 1e-2


def test_cp_single_rank_is_plain_forward():
    inp = make_inputs(1, 70, 1, seed=1, gate_offset=-6.0, h0_std=0.5)
    o, ht = cp_forward(OracleBackend(inp), None, 0, 1, inp["initial_state"], True)
    o2, ht2 = cp_forward(OracleBackend(inp, [0, 64, 70]), None, 0, 1, inp["initial_state"], True)   # one rank, two segments
    assert err_ratio(o, o2) < 1e-6 and err_ratio(ht, ht2) < 1e-6
    o_ref, ht_ref = chunk_kda_oracle(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], initial_state=inp["initial_state"],
                                     output_final_state=True, use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True,
                                     safe_gate=True, lower_bound=-5.0, A_log=inp["A_log"], dt_bias=inp["dt_bias"])
    assert err_ratio(o_ref, o) < 1e-6 and err_ratio(ht_ref, ht) < 1e-6
