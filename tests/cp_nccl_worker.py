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
    per = T // world
    sl = slice(rank * per, T if rank == world - 1 else (rank + 1) * per)
    sh = {n: (t[:, sl] if n in ("q", "k", "v", "g", "beta") else t).to(dev) for n, t in inp.items()}
    o, ht = chunk_kda_cp(sh["q"], sh["k"], sh["v"], sh["g"], sh["beta"], initial_state=sh["initial_state"],
                         output_final_state=True, use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, safe_gate=True,
                         lower_bound=-5.0, A_log=sh["A_log"], dt_bias=sh["dt_bias"])
    parts = [torch.empty(1, per, H, 128, dtype=o.dtype, device=dev) for _ in range(world)]
    dist.all_gather(parts, o.contiguous())
    if ht is None:
        ht = torch.empty(1, H, 128, 128, device=dev)
    dist.broadcast(ht, src=world - 1)
    if rank == 0:
        from oracle import c_oracle
        from oracle.naive_kda import err_ratio
        f = lambda x: x.float().numpy()
        o_ref, ht_ref = c_oracle.naive_kda_fwd(f(inp["q"]), f(inp["k"]), f(inp["v"]), f(inp["g"]), f(inp["beta"]),
                                               f(inp["A_log"]), f(inp["dt_bias"]), f(inp["initial_state"]),
                                               use_l2norm=True, gate_mode=2, lower_bound=-5.0)
        e_o = err_ratio(torch.from_numpy(o_ref), torch.cat(parts, 1).float().cpu())
        e_h = err_ratio(torch.from_numpy(ht_ref), ht.cpu())
        assert e_o <= 5e-3 and e_h <= 2e-3, (e_o, e_h)
        print(f"CP_OK o {e_o:.2e} ht {e_h:.2e}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
