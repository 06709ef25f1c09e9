"""Worker of test_cp_two_gpus_nccl: one rank per GPU, chunk_kda_cp over NCCL, rank 0 compares with the oracle."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from cula_b200.kda.cp import chunk_kda_cp  # noqa: E402
from cula_b200.synthetic import make_inputs  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    T, H = 1024, 4
    inp = make_inputs(1, T, H, seed=2, gate_offset=-8.0, h0_std=0.5)
    gen = torch.Generator().manual_seed(3)
    do = torch.randn(1, T, H, 128, generator=gen).to(torch.bfloat16)
    dht = 0.1 * torch.randn(1, H, 128, 128, generator=gen)
    per = T // world
    sl = slice(rank * per, T if rank == world - 1 else (rank + 1) * per)
    sh = {n: (t[:, sl] if n in ("q", "k", "v", "g", "beta") else t).to(dev).requires_grad_(True) for n, t in inp.items()}
    # the state before the first token is given on rank 0 only; the exchange carries it to the other ranks
    o, ht = chunk_kda_cp(sh["q"], sh["k"], sh["v"], sh["g"], sh["beta"],
                         initial_state=sh["initial_state"] if rank == 0 else None, output_final_state=True,
                         use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, safe_gate=True, lower_bound=-5.0,
                         A_log=sh["A_log"], dt_bias=sh["dt_bias"])
    assert (ht is not None) == (rank == world - 1)
    loss = (o.float() * do[:, sl].to(dev).float()).sum()
    if ht is not None:
        loss = loss + (ht * dht.to(dev)).sum()
    loss.backward()                                            # every rank: the backward exchange is a collective
    parts = [torch.empty(1, per, H, 128, dtype=o.dtype, device=dev) for _ in range(world)]
    dist.all_gather(parts, o.detach().contiguous())
    ht_all = ht.detach().clone() if ht is not None else torch.empty(1, H, 128, 128, device=dev)
    dist.broadcast(ht_all, src=world - 1)
    grads = {}
    for n in ("q", "k", "v", "g", "beta"):
        gp = [torch.empty_like(sh[n].grad) for _ in range(world)]
        dist.all_gather(gp, sh[n].grad.contiguous())
        grads[n] = torch.cat(gp, dim=1).float().cpu()
    for n in ("A_log", "dt_bias"):                             # shard contributions: summed by the caller
        t = sh[n].grad.clone()
        dist.all_reduce(t)
        grads[n] = t.float().cpu()
    assert (sh["initial_state"].grad is not None) == (rank == 0)
    if rank == 0:
        grads["initial_state"] = sh["initial_state"].grad.float().cpu()
        from oracle import c_oracle
        from oracle.naive_kda import chunk_kda_oracle, err_ratio
        f = lambda x: x.float().numpy()
        o_ref, ht_ref = c_oracle.naive_kda_fwd(f(inp["q"]), f(inp["k"]), f(inp["v"]), f(inp["g"]), f(inp["beta"]),
                                               f(inp["A_log"]), f(inp["dt_bias"]), f(inp["initial_state"]),
                                               use_l2norm=True, gate_mode=2, lower_bound=-5.0)
        e_o = err_ratio(torch.from_numpy(o_ref), torch.cat(parts, 1).float().cpu())
        e_h = err_ratio(torch.from_numpy(ht_ref), ht_all.cpu())
        assert e_o <= 5e-3 and e_h <= 2e-3, (e_o, e_h)
        ref_in = {n: t.detach().float().clone().requires_grad_(True) for n, t in inp.items()}
        o2, ht2 = chunk_kda_oracle(ref_in["q"], ref_in["k"], ref_in["v"], ref_in["g"], ref_in["beta"],
                                   initial_state=ref_in["initial_state"], output_final_state=True,
                                   use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, safe_gate=True, lower_bound=-5.0,
                                   A_log=ref_in["A_log"], dt_bias=ref_in["dt_bias"])
        ((o2 * do.float()).sum() + (ht2 * dht).sum()).backward()
        worst = 0.0
        for n, gref in ((n, t.grad) for n, t in ref_in.items()):
            e = err_ratio(gref, grads[n].view_as(gref))
            assert e <= (2e-2 if n in ("g", "beta") else 8e-3), (n, e)
            worst = max(worst, e)
        print(f"CP_OK o {e_o:.2e} ht {e_h:.2e} grads {worst:.2e}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
