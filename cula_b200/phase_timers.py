"""Per-phase cycle counts of the chunk-parallel forward kernel and of the dense and gated backward kernels.

    python -m cula_b200.build --timers        # builds cula_b200/lib/libcula_kda_timers.so (-DKDA_PHASE_TIMERS)
    python -m cula_b200.phase_timers [B T H]  # on a B200; default 2 2048 32 (the headline forward configuration)

In the timers build thread 0 of every CTA adds the clock64() cycles between consecutive phase marks to a device
array; this script runs one forward (and one forward + backward) and prints the mean cycles per (chunk, head) tile
and phase. The counts include whatever the co-resident CTA makes the measured CTA wait for, so they add up to the
tile's latency, not to its issue slots. A profiling aid: the package itself never loads this library.
"""
from __future__ import annotations

import ctypes
import sys

import torch

from . import _native
from .build import TIMERS_LIB, build

FWD_PHASES = ["gate activation", "barrier (group totals)", "in-warp scan, tables", "operand generation, half 0",
              "MMA wait, half 0 (+ L2 hints)", "operand generation, half 1", "MMA wait, half 1",
              "Y staging + barrier", "triangular inverse", "Akk pack + W/U MMA issue", "W/U MMA wait", "W/U epilogue",
              "loads issued under the MMA wait", "Gram epilogue", "L2 norms, beta", "top of the tile (q/k loads issued)"]
DENSE_PHASES = ["half 0: operands widened into smem", "-",
                "half 0: store read-out + wait for the states (TMA)", "half 0: MMA issue", "half 0: next operands requested",
                "half 0: wait for the MMAs",
                "half 1: operands widened into smem", "-", "half 1: wait for the states (TMA)",
                "half 1: MMA issue", "half 1: next tile's operands requested", "half 1: wait for the MMAs", "dQg, dW staged, stores issued",
                "dKg, dPs, dAu staged, dv stored", "store read-out + end-of-tile barrier"]
BWD_PHASES = ["loads, gate, norms", "cumulative sum", "stage dW, X", "dA", "T1, dL", "Zw + accumulator set-up", "L2 hints",
              "Gram VJP, row side", "Gram VJP, column side", "reverse cumulative sum", "gate VJP, dg", "L2-norm VJP, stores"]


def main():
    B, T, H = (int(x) for x in sys.argv[1:4]) if len(sys.argv) >= 4 else (2, 2048, 32)
    build(timers=True)
    _native.LIB_PATH = TIMERS_LIB
    _native.lib()
    raw = ctypes.CDLL(TIMERS_LIB)
    from .kda import chunk_kda
    from .synthetic import make_inputs_on_device
    dev = torch.device("cuda", 0)
    d = make_inputs_on_device(B, T, H, dev, seed=0, h0_std=0.1)
    for v in d.values():
        v.requires_grad_(True)
    do = torch.randn(B, T, H, 128, device=dev).to(torch.bfloat16)
    kw = dict(use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, safe_gate=True, lower_bound=-5.0)
    buf = (ctypes.c_ulonglong * 16)()
    tiles = B * ((T + 63) // 64) * H
    for _ in range(3):                      # the last pass is the one that is read
        for v in d.values():
            v.grad = None
        raw.kda_fwd_intra_read_timers(buf, 1)
        with torch.no_grad():
            chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], A_log=d["A_log"], dt_bias=d["dt_bias"],
                      initial_state=d["initial_state"], output_final_state=True, **kw)
        torch.cuda.synchronize()
        raw.kda_fwd_intra_read_timers(buf, 0)
        fwd = [x / tiles for x in buf]
        o, _ = chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], A_log=d["A_log"], dt_bias=d["dt_bias"],
                         initial_state=d["initial_state"], output_final_state=True, **kw)
        torch.cuda.synchronize()
        raw.kda_bwd_gated_read_timers(buf, 1)
        raw.kda_bwd_dense_read_timers(buf, 1)
        o.backward(do)
        torch.cuda.synchronize()
        raw.kda_bwd_gated_read_timers(buf, 0)
        bwd = [x / tiles for x in buf]
        raw.kda_bwd_dense_read_timers(buf, 0)
        dense = [x / tiles for x in buf]
    for title, names, vals in (("kda_fwd_intra_kernel", FWD_PHASES, fwd), ("kda_bwd_dense_kernel", DENSE_PHASES, dense), ("kda_bwd_gated_kernel", BWD_PHASES, bwd)):
        print(f"{title}: cycles per tile, B={B} T={T} H={H} ({tiles} tiles)")
        for n, v in zip(names, vals):
            print(f"  {n:38s} {v:9.0f}")
        print(f"  {'total':38s} {sum(vals[:len(names)]):9.0f}")


if __name__ == "__main__":
    main()
