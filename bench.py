#!/usr/bin/env python
"""Benchmark of the chunk_kda forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one chunk_kda forward over one synthetic batch. At N=1 the workload is the headline
configuration (B=2, T=2048, H=32, K=V=128, bf16, in-kernel gate + L2 norm, safe gate, final state).
With N>1 (launched under torch.distributed.run, one rank per GPU) every rank runs the same-sized
shard of a batch that is N times larger (weak scaling over batch x head; the path has no
data-path collective there). Rank 0 prints ONE JSON line.

`--impl reference` times the reference's CPU implementation of the path (the fp32 naive token
recurrence, here the plain-C restatement under oracle/) on the host cores, same metric and config.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B, T, H, lens or None)
    "fwd_B2_T2048_H32": (2, 2048, 32),
    "fwd_B4_T8192_H32": (4, 8192, 32),
    "fwd_B1_T512_H4": (1, 512, 4),
}
KERNEL_SOURCES = {"kda_fwd_intra_kernel": "kda_fwd_intra.cu", "kda_fwd_scan_kernel": "kda_fwd_scan.cu"}


def ncu_traffic(workload, kernel):
    """DRAM bytes (read + write) of one launch from the ncu summary committed for this kernel and workload. The
    summary records the hash of the kernel source it was captured from; if the source has changed since, the
    figure is stale and None is reported instead. Returns (bytes or None, note)."""
    import hashlib
    import re
    path = os.path.join(ROOT, "profiles", f"{kernel}_{workload.replace('fwd_', '')}.md")
    src = os.path.join(ROOT, "cula_b200", "csrc", KERNEL_SOURCES.get(kernel, ""))
    if not (os.path.exists(path) and os.path.isfile(src)):
        return None, "no ncu summary for this kernel and workload"
    text = open(path).read()
    m_bytes = re.search(r"dram_bytes_per_launch:\s*(\d+)", text)
    m_sha = re.search(r"kernel_source_sha256:\s*([0-9a-f]{16})", text)
    if not (m_bytes and m_sha):
        return None, "the ncu summary carries no machine-readable traffic line"
    sha = hashlib.sha256(open(src, "rb").read()).hexdigest()[:16]
    if sha != m_sha.group(1):
        return None, f"stale: {os.path.basename(path)} was captured from another revision of {KERNEL_SOURCES[kernel]}"
    return int(m_bytes.group(1)), f"ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch ({os.path.basename(path)})"


# Secondary workloads (selected with --workload; not the headline line): forward+backward, the packed varlen
# forward, and the context-parallel forward of one long sequence split over the ranks (strong scaling).
EXTRA_WORKLOADS = {
    "fwdbwd_B4_T8192_H32": dict(kind="fwdbwd", B=4, T=8192, H=32),
    "fwdbwd_B2_T2048_H32": dict(kind="fwdbwd", B=2, T=2048, H=32),
    "varlen_64seq_65536_H32": dict(kind="varlen", n_seqs=64, total=65536, H=32),
    "cp_T262144_H32": dict(kind="cp", T=262144, H=32),
    "cp_T32768_H32": dict(kind="cp", T=32768, H=32),
    "decode_N256_H32": dict(kind="decode", N=256, H=32),
    "gdn_fwd_B2_T2048_H32": dict(kind="gdn", B=2, T=2048, H=32, backward=False),
    "gdn_fwdbwd_B2_T2048_H32": dict(kind="gdn", B=2, T=2048, H=32, backward=True),
    "layer_ops_B2_T2048_H32": dict(kind="layer", B=2, T=2048, H=32),
}


def varlen_lengths(n_seqs=64, total=65536, seed=0):
    """Seeded lognormal lengths (median 512, sigma 1, clipped to [63, 8192]) adjusted to sum to `total`."""
    import numpy as np
    rng = np.random.default_rng(seed)
    lens = np.clip(np.round(rng.lognormal(np.log(512.0), 1.0, n_seqs)), 63, 8192).astype(np.int64)
    diff = int(total - lens.sum())
    order = np.argsort(-lens)
    i = 0
    while diff != 0:
        j = order[i % n_seqs]
        step = max(-int(lens[j] - 63), min(int(8192 - lens[j]), diff))
        lens[j] += step
        diff -= step
        i += 1
    return lens.tolist()


FLOP_PER_TOKEN_HEAD = 180224          # dense-tile convention, forward
BYTES_PER_TOKEN_HEAD = 1282           # compulsory forward traffic: q,k,v,g bf16 + beta + o
TILE_PACK_BYTES = 74240


def layer_ops_section(dev, B, T, H, steps):
    """Layer-side operators on the headline shape (rows = B*T tokens, 128 channels per head): milliseconds per call and
    algorithmic GB/s (bytes every call must read and write once) as a fraction of the measured copy peak. L2 is flushed
    before every timed call; the median of `steps` calls is reported; every call is replayed from a CUDA graph so that the
    device time, not the Python around a 30-microsecond kernel, is what the events see."""
    from cula_b200.kda.gate import fused_kda_gate
    from cula_b200.kda.layer_ops import rms_norm_gated, short_conv
    peaks = load_peaks()
    gen = torch.Generator().manual_seed(0)
    n_el = B * T * H * 128
    g_raw = torch.randn(B, T, H, 128, generator=gen).to(torch.bfloat16).to(dev).requires_grad_(True)
    A_log = (0.1 * torch.randn(H, generator=gen)).to(dev).requires_grad_(True)
    dt_bias = (0.1 * torch.randn(H * 128, generator=gen)).to(dev).requires_grad_(True)
    x_conv = torch.randn(B, T, H * 128, generator=gen).to(torch.bfloat16).to(dev).requires_grad_(True)
    w_conv = (0.5 * torch.randn(H * 128, 4, generator=gen)).to(dev).requires_grad_(True)
    x_norm = torch.randn(B, T, H, 128, generator=gen).to(torch.bfloat16).to(dev).requires_grad_(True)
    g_norm = torch.randn(B, T, H, 128, generator=gen).to(torch.bfloat16).to(dev).requires_grad_(True)
    w_norm = torch.ones(128, device=dev, requires_grad=True)
    ops = {
        # name: (callable, forward bytes per element, forward+backward bytes per element)
        "fused_kda_gate (lower-bound form, fp32 out)": (lambda: fused_kda_gate(g_raw, A_log, dt_bias, lower_bound=-5.0), 2 + 4, 2 + 4 + 2 + 4 + 2),
        "short_conv (width 4) + SiLU": (lambda: short_conv(x_conv, w_conv)[0], 2 + 2, 2 + 2 + 2 + 2 + 2),
        "rms_norm_gated (sigmoid gate)": (lambda: rms_norm_gated(x_norm, g_norm, w_norm), 2 + 2 + 2, 6 + 2 + 2 + 2 + 2 + 2),
    }
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn):
        """Device time of fn(): captured in a CUDA graph once and replayed (these calls are tens of microseconds long,
        less than the Python around them costs on the host), L2 flushed before every replay."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                fn()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        ts = []
        for i in range(3 + steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize()
            if i >= 3:
                ts.append(e0.elapsed_time(e1))
        return sorted(ts)[len(ts) // 2]

    out = {}
    total_fwd = 0.0
    leaves = (g_raw, A_log, dt_bias, x_conv, w_conv, x_norm, g_norm, w_norm)
    for name, (fn, b_f, b_fb) in ops.items():
        with torch.no_grad():
            y = fn()
        dy = torch.randn_like(y)

        def fwd_only():
            with torch.no_grad():
                fn()

        def fwd_bwd():
            for t in leaves:
                t.grad = None
            fn().backward(dy)
        ms_f = timed(fwd_only)
        ms_fb = timed(fwd_bwd)
        total_fwd += ms_f
        out[name] = {"fwd_ms": ms_f, "fwd_GBps": n_el * b_f / ms_f / 1e6, "fwd_frac_of_copy_peak": n_el * b_f / ms_f / 1e6 / peaks["hbm_gbs"],
                     "fwd_bwd_ms": ms_fb, "fwd_bwd_GBps": n_el * b_fb / ms_fb / 1e6,
                     "fwd_bwd_frac_of_copy_peak": n_el * b_fb / ms_fb / 1e6 / peaks["hbm_gbs"]}
    return {"metric": "layer-side operators, forward tokens/s (sum of the three)", "value": B * T / (total_fwd * 1e-3), "unit": "tokens/s",
            "n_gpus": 1, "steps": steps, "warmup": 3, "ms_per_step": total_fwd, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "layer_ops_B2_T2048_H32", "B": B, "T": T, "H": H, "K": 128,
                       "l2": "256 MB flush buffer written before every timed call"},
            "peak_GBps": peaks["hbm_gbs"], "peak_source": peaks["source"], "ops": out}


def headline_config(workload):
    """The `config` object of the JSON line; both arms (ours, --impl reference) print exactly this."""
    B, T, H = WORKLOADS[workload]
    return {"workload": workload, "B_per_gpu": B, "T": T, "H": H, "K": 128, "V": 128,
            "flags": "l2norm+gate in kernel, safe_gate, lower_bound=-5, final state",
            "l2": "256 MB flush buffer written before every timed step",
            "sharding": "batch x head shards, one per rank, no collective"}


class stdout_to_stderr:
    """File-descriptor level redirect of stdout to stderr: the NCCL communicator prints its version banner with
    printf when it is created, and stdout must carry exactly ONE JSON line."""

    def __enter__(self):
        sys.stdout.flush()
        self.saved = os.dup(1)
        os.dup2(2, 1)

    def __exit__(self, *exc):
        sys.stdout.flush()
        os.dup2(self.saved, 1)
        os.close(self.saved)


def init_nccl(rank, world, dev):
    import torch.distributed as dist
    with stdout_to_stderr():
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        dist.barrier()                  # communicator creation (and its banner) happens here at the latest
        torch.cuda.synchronize()


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu, self.proc = gpu_index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_baseline(B, T, H, budget_s=10.0):
    """Time the plain-C oracle on the host cores on the same workload; tokens/s."""
    from cula_b200.synthetic import make_inputs
    from oracle import c_oracle
    c_oracle.use_all_cores()
    inp = make_inputs(B, T, H, seed=0)
    f = lambda x: x.float().numpy()
    args = [f(inp[k]) for k in ("q", "k", "v", "g", "beta")]
    extra = (f(inp["A_log"]), f(inp["dt_bias"]), None)
    run = lambda: c_oracle.naive_kda_fwd(*args, *extra, use_l2norm=True, gate_mode=2, lower_bound=-5.0)
    run()
    reps, t0 = 0, time.perf_counter()
    while True:
        run()
        reps += 1
        dt = time.perf_counter() - t0
        if dt > budget_s or reps >= 400:
            break
    return dict(value=B * T * reps / dt, unit="tokens/s", cores=c_oracle.num_threads(), kind="port",
                sample=f"{reps} full forward passes of B={B} T={T} H={H} ({dt:.1f} s) with the OpenMP C "
                       f"restatement of the fp32 naive recurrence"), dt / reps


def cpu_config1():
    """The reference's own CPU-runnable case (B=1, T=512, H=4): the C restatement and the torch restatement of the
    naive recurrence, tokens/s each, a few passes."""
    from cula_b200.synthetic import make_inputs
    from oracle import c_oracle
    from oracle.naive_kda import chunk_kda_oracle
    B, T, H = WORKLOADS["fwd_B1_T512_H4"]
    inp = make_inputs(B, T, H, seed=0)
    f = lambda x: x.float().numpy()
    a = [f(inp[k]) for k in ("q", "k", "v", "g", "beta")] + [f(inp["A_log"]), f(inp["dt_bias"]), None]
    c_run = lambda: c_oracle.naive_kda_fwd(*a, use_l2norm=True, gate_mode=2, lower_bound=-5.0)
    t_run = lambda: chunk_kda_oracle(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], output_final_state=True,
                                     use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, safe_gate=True, lower_bound=-5.0,
                                     A_log=inp["A_log"], dt_bias=inp["dt_bias"])
    out = {"workload": "fwd_B1_T512_H4", "torch_threads": torch.get_num_threads()}
    for name, run, reps in (("c_tokens_per_s", c_run, 20), ("torch_tokens_per_s", t_run, 3)):
        run()
        t0 = time.perf_counter()
        for _ in range(reps):
            run()
        out[name] = B * T * reps / (time.perf_counter() - t0)
    return out


def run_reference(args, rank, world):
    if rank != 0:
        return
    B, T, H = WORKLOADS[args.workload]
    from cula_b200.synthetic import make_inputs
    from oracle import c_oracle
    inp = make_inputs(B, T, H, seed=0)
    f = lambda x: x.float().numpy()
    a = [f(inp[k]) for k in ("q", "k", "v", "g", "beta")] + [f(inp["A_log"]), f(inp["dt_bias"]), None]
    run = lambda: c_oracle.naive_kda_fwd(*a, use_l2norm=True, gate_mode=2, lower_bound=-5.0)
    cores = c_oracle.use_all_cores()         # torch.distributed.run exports OMP_NUM_THREADS=1 to its workers
    for _ in range(args.warmup):
        run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run()
    dt = (time.perf_counter() - t0) / args.steps
    val = B * T / dt
    print(json.dumps({
        "impl": "reference", "metric": "chunk_kda forward tokens/s", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": headline_config(args.workload),
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": f"each step = one full forward of one rank's shard (B={B} T={T} H={H}) on {cores} "
                                   "host threads of rank 0 (plain-C restatement of the reference's fp32 naive "
                                   "recurrence); no L2 flush and no sharding apply to the CPU arm"},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }), flush=True)


CP_TOKENS, CP_HEADS = 262144, 32


def cp_section(rank, world, dev, flush, steps=10, T_total=CP_TOKENS, H=CP_HEADS):
    """Context-parallel forward of ONE sequence of ``T_total`` tokens cut into ``world`` contiguous shards (strong
    scaling): chunk-parallel stage, transition scan, NCCL all-gather of (C | M), folds, final scan -- the collective
    is inside the timed region, every step starts from a barrier, the time is the max over ranks. Also: the time
    of each stage (max over ranks, one instrumented step), the time of the same sequence on ONE GPU measured in
    this run on rank 0's device (`t1_ms`; at world 1 it is the run itself), and an untimed parity check on a
    weak-gate sequence of 4096 tokens per rank whose state really crosses the shard boundaries, against the
    single-pass, unsegmented forward of the whole sequence on rank 0."""
    import torch.distributed as dist
    import cula_b200.kda.cp as cp
    from cula_b200.kda import check_status, chunk_kda
    from cula_b200.synthetic import make_inputs_on_device
    kw = dict(use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, safe_gate=True, lower_bound=-5.0)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29577")
        # a single rank never communicates: gloo keeps NCCL (and the version banner it prints on stdout) out of it
        if world == 1:
            dist.init_process_group("gloo", rank=0, world_size=1)
        else:
            init_nccl(rank, world, dev)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def rank_max(values):
        t = torch.tensor(values, dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(x) for x in t.tolist()]

    def timed(fn, n, entry_barrier):
        evs = []
        for _ in range(n):
            flush.zero_()
            if entry_barrier and world > 1:
                dist.barrier()              # the ranks enter every step together
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            evs.append((e0, e1))
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in evs) / n

    per = T_total // world
    d = make_inputs_on_device(1, per, H, dev, seed=100 + rank)       # this rank's shard
    step = lambda marks=None: cp.chunk_kda_cp(d["q"], d["k"], d["v"], d["g"], d["beta"], A_log=d["A_log"],
                                              dt_bias=d["dt_bias"], output_final_state=True, stage_marks=marks, **kw)
    for _ in range(3):
        step()
    sync_all()
    ms = rank_max([timed(step, steps, True)])[0]
    marks = []
    timed(lambda: step(marks), 1, True)
    names = [n for n, _ in marks[1:]]
    stage_ms = rank_max([marks[i][1].elapsed_time(marks[i + 1][1]) for i in range(len(marks) - 1)])
    check_status(dev)
    sync_all()

    # ---- the same sequence on one GPU (rank 0's), for the strong-scaling efficiency ----
    t1 = ms
    if world > 1:
        del d
        if rank == 0:
            full = make_inputs_on_device(1, T_total, H, dev, seed=100)
            one = lambda: chunk_kda(full["q"], full["k"], full["v"], full["g"], full["beta"], A_log=full["A_log"],
                                    dt_bias=full["dt_bias"], output_final_state=True, **kw)
            for _ in range(3):
                one()
            torch.cuda.synchronize()
            t1 = timed(one, max(3, steps // 2), False)
            del full
        torch.cuda.empty_cache()
        t1 = rank_max([t1 if rank == 0 else 0.0])[0]
        sync_all()

    # ---- parity: weak gates, 4096 tokens per rank, initial state on rank 0 only ----
    Tp = 4096 * world
    full = make_inputs_on_device(1, Tp, H, dev, seed=7, gate_offset=-8.0, h0_std=0.5)   # the same numbers on every rank
    sl = slice(rank * 4096, (rank + 1) * 4096)
    sh = {n: (t[:, sl].contiguous() if n in ("q", "k", "v", "g", "beta") else t) for n, t in full.items()}
    o_cp, ht_cp = cp.chunk_kda_cp(sh["q"], sh["k"], sh["v"], sh["g"], sh["beta"], A_log=sh["A_log"], dt_bias=sh["dt_bias"],
                                  initial_state=sh["initial_state"] if rank == 0 else None, output_final_state=True, **kw)
    if world > 1:
        parts = [torch.empty_like(o_cp) for _ in range(world)]
        dist.all_gather(parts, o_cp.contiguous())
        o_all = torch.cat(parts, dim=1)
        ht_all = ht_cp if ht_cp is not None else torch.empty(1, H, 128, 128, dtype=torch.float32, device=dev)
        dist.broadcast(ht_all, src=world - 1)
    else:
        o_all, ht_all = o_cp, ht_cp
    parity = None
    if rank == 0:
        cp.MAX_AUTO_SEGMENTS = 1            # the yardstick is the plain single-pass scan of the whole sequence
        o_ref, ht_ref = chunk_kda(full["q"], full["k"], full["v"], full["g"], full["beta"], A_log=full["A_log"],
                                  dt_bias=full["dt_bias"], initial_state=full["initial_state"], output_final_state=True, **kw)
        cp.MAX_AUTO_SEGMENTS = 4
        rel = lambda a, b: float((a.double() - b.double()).norm() / b.double().norm())
        # what the carried state contributes: the forward of the last 4096 tokens alone, from a zero state
        tail = {n: full[n][:, -4096:].contiguous() for n in ("q", "k", "v", "g", "beta")}
        o_cut, _ = chunk_kda(tail["q"], tail["k"], tail["v"], tail["g"], tail["beta"], A_log=full["A_log"],
                             dt_bias=full["dt_bias"], **kw)
        parity = {"tokens": Tp, "gate_offset": -8.0,
                  "o_rel_rms": rel(o_all.float(), o_ref.float()), "ht_rel": rel(ht_all, ht_ref),
                  "o_rel_rms_if_state_dropped": rel(o_cut.float(), o_ref[:, -4096:].float()),
                  "against": "single-pass unsegmented chunk_kda of the whole sequence on rank 0"}
        torch.cuda.synchronize()
        check_status(dev)
        if not (parity["o_rel_rms"] <= 5e-3 and parity["ht_rel"] <= 2e-3):
            raise RuntimeError(f"context-parallel parity failed: {parity}")
    sync_all()
    return {"workload": f"cp_T{T_total}_H{H}", "scaling": "strong", "n_gpus": world, "steps": steps, "ms_per_step": ms,
            "tokens_per_s": T_total / (ms * 1e-3), "t1_ms": t1, "efficiency": t1 / (world * ms),
            "t1_source": "the same sequence through chunk_kda on rank 0's GPU alone, in this run "
                         "(segmented scan: the best single-GPU path)",
            "per_rank_ms": dict(zip(names, stage_ms)),
            "exchange": "one all-gather of (C|M) [2,H,128,128] fp32 per rank over NCCL, inside the timed region",
            "parity": parity}


def run_extra(args, rank, world, local_rank):
    """Secondary workloads: same timing rules as the headline (warm-up, L2 flush before every timed step, CUDA
    events, max over ranks); one JSON line from rank 0."""
    import torch.distributed as dist
    from cula_b200 import _native
    from cula_b200.kda import check_status, chunk_kda
    from cula_b200.synthetic import make_inputs

    if args.impl == "reference":
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "the CPU reference arm is timed on the headline workload only"}))
        return
    w = EXTRA_WORKLOADS[args.workload]
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1 or w["kind"] == "cp":
        if not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29577")
            init_nccl(rank, world, dev)
    _native.lib()
    kw = dict(use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, safe_gate=True, lower_bound=-5.0)
    H = w["H"]
    scaling, launches = "weak", 2
    if w["kind"] == "fwdbwd":
        B, T = w["B"], w["T"]
        inp = make_inputs(B, T, H, seed=rank, h0_std=0.1)
        d = {k: v.to(dev).requires_grad_(True) for k, v in inp.items()}
        do = torch.randn(B, T, H, 128, device=dev).to(torch.bfloat16)

        def step():
            for t in d.values():
                t.grad = None
            o, _ = chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], A_log=d["A_log"], dt_bias=d["dt_bias"],
                             initial_state=d["initial_state"], output_final_state=True, **kw)
            o.backward(do)
        tokens, metric, launches = B * T * world, "chunk_kda forward+backward tokens/s", 9
        cfg = {"B_per_gpu": B, "T": T, "sharding": "batch x head shards, one per rank, no collective"}
    elif w["kind"] == "gdn":
        # the scalar-gate variant (one decay per token and head) on the headline shape: raw gate activated in-kernel
        from cula_b200.gdn import chunk_gated_delta_rule
        B, T = w["B"], w["T"]
        inp = make_inputs(B, T, H, seed=rank, h0_std=0.1)
        gen = torch.Generator().manual_seed(100 + rank)
        d = {k: inp[k].to(dev) for k in ("q", "k", "v", "beta", "initial_state")}
        d["g"] = torch.randn(B, T, H, generator=gen).to(dev)
        d["A_log"] = (0.1 * torch.randn(H, generator=gen)).to(dev)
        d["dt_bias"] = (0.1 * torch.randn(H, generator=gen)).to(dev)
        do = torch.randn(B, T, H, 128, device=dev).to(torch.bfloat16)
        if w["backward"]:
            for t in d.values():
                t.requires_grad_(True)

        def step():
            for t in d.values():
                t.grad = None
            o, _ = chunk_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["initial_state"],
                                          output_final_state=True, use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True,
                                          A_log=d["A_log"], dt_bias=d["dt_bias"])
            if w["backward"]:
                o.backward(do)
        tokens = B * T * world
        metric = "chunk_gated_delta_rule forward+backward tokens/s" if w["backward"] else "chunk_gated_delta_rule forward tokens/s"
        launches = 9 if w["backward"] else 2
        cfg = {"B_per_gpu": B, "T": T, "gate": "one per (token, head), softplus form in-kernel",
               "sharding": "batch x head shards, one per rank, no collective"}
    elif w["kind"] == "varlen":
        lens = varlen_lengths(w["n_seqs"], w["total"], seed=rank)
        T = sum(lens)
        cu = torch.tensor([0] + list(__import__("itertools").accumulate(lens)), dtype=torch.int32, device=dev)
        inp = make_inputs(1, T, H, seed=rank)
        d = {k: v.to(dev) for k, v in inp.items() if v is not None}
        step = lambda: chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], A_log=d["A_log"], dt_bias=d["dt_bias"],
                                 cu_seqlens=cu, output_final_state=True, **kw)
        tokens, metric = T * world, "chunk_kda varlen forward tokens/s"
        cfg = {"sequences_per_gpu": len(lens), "tokens_per_gpu": T, "min_len": min(lens), "max_len": max(lens)}
    elif w["kind"] == "decode":
        # one token for each of N sequences against a pool of fp32 states ((V, K) layout), shuffled slots
        from cula_b200.kda import kda_decode
        N = w["N"]
        gen = torch.Generator().manual_seed(rank)
        r = lambda *s_: torch.randn(*s_, generator=gen)
        dq, dk, dv = (r(N, 1, H, 128).to(torch.bfloat16).to(dev) for _ in range(3))
        da, db = (0.1 * r(N, 1, H, 128)).to(torch.bfloat16).to(dev), r(N, 1, H).to(torch.bfloat16).to(dev)
        dA, dbias = (-2 * torch.rand(H, generator=gen)).to(dev), (0.1 * r(H, 128)).to(dev)
        pool = (0.01 * r(N, H, 128, 128)).to(dev)
        slots = torch.randperm(N, generator=gen).to(torch.int32).to(dev)
        step = lambda: kda_decode(A_log=dA, dt_bias=dbias, q=dq, k=dk, v=dv, a=da, b=db, initial_state_source=pool,
                                  initial_state_indices=slots)
        tokens, metric, launches = N * world, "kda_decode tokens/s", 1
        state_bytes = 2 * N * H * 128 * 128 * 4
        cfg = {"sequences_per_gpu": N, "state_layout": "vk", "state_bytes_read_plus_written": state_bytes}
    elif w["kind"] == "layer":
        # the streaming operators around the path (gate activation, short convolution + SiLU, gated RMS norm), each
        # timed alone, forward and forward+backward, against the bytes it has to move
        if rank == 0:
            print(json.dumps(layer_ops_section(dev, w["B"], w["T"], H, args.steps)), flush=True)
        return
    else:   # context parallel: ONE sequence of T tokens split over the ranks
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        res = cp_section(rank, world, dev, flush, steps=args.steps, T_total=w["T"], H=H)
        clocks = sampler.stop() if rank == 0 else None
        if rank == 0:
            print(json.dumps({"metric": "chunk_kda context-parallel forward tokens/s", "value": res["tokens_per_s"],
                              "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": 3,
                              "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                              "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                              "config": {"workload": args.workload, "H": H, "K": 128, "V": 128,
                                         "l2": "256 MB flush buffer written before every timed step"},
                              "cp": res, "clocks": clocks}), flush=True)
        if dist.is_initialized():
            dist.destroy_process_group()
        return
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.5)
    evs = []
    for _ in range(8):                            # untimed device work queued first: the host gets ahead of the device
        flush.zero_()
    for _ in range(args.steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step()
        e1.record()
        evs.append((e0, e1))
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    check_status(dev)
    ms = sum(a.elapsed_time(b) for a, b in evs) / args.steps
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    extra = {}
    if w["kind"] == "decode":
        peaks = load_peaks()
        ach = cfg["state_bytes_read_plus_written"] / (ms * 1e-3) / 1e9
        extra["roofline"] = {"kernel": "kda_decode_kernel", "bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"],
                             "unit": "GB/s", "frac": ach / peaks["hbm_gbs"], "traffic": None, "peak_source": peaks["source"]}
    if rank == 0:
        print(json.dumps({**extra,
            "metric": metric, "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": scaling,
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": dict({"workload": args.workload, "H": H, "K": 128, "V": 128,
                            "l2": "256 MB flush buffer written before every timed step"}, **cfg),
            "gpu_launches": launches * args.steps, "clocks": clocks}), flush=True)
    if dist.is_initialized():
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="fwd_B2_T2048_H32", choices=sorted(WORKLOADS) + sorted(EXTRA_WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-cp", action="store_true", help="skip the context-parallel section of the headline line")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.workload in EXTRA_WORKLOADS:
        return run_extra(args, rank, world, local_rank)
    if args.impl == "reference":
        return run_reference(args, rank, world)

    import torch.distributed as dist
    from cula_b200 import _native
    from cula_b200.kda import check_status, chunk_kda, chunk_kda_host
    from cula_b200.synthetic import make_inputs

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        init_nccl(rank, world, dev)
    _native.lib()                     # fail loudly if the CUDA library is missing
    # one rank per GPU: keep this rank's threads and its pinned host buffers (allocated below) on the GPU's own
    # NUMA node, so that the ranks' host<->device copies do not all go through one socket's memory
    from cula_b200.kda import bind_host_to_gpu
    host_cpus = bind_host_to_gpu(dev) if world > 1 else sorted(os.sched_getaffinity(0))

    B, T, H = WORKLOADS[args.workload]
    inp = make_inputs(B, T, H, seed=rank)          # every rank owns an equally sized shard (weak scaling)
    host = {k: v.pin_memory() for k, v in inp.items() if v is not None}
    d = {k: v.to(dev) for k, v in host.items()}
    kw = dict(use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, safe_gate=True, lower_bound=-5.0,
              output_final_state=True)
    fwd = lambda t: chunk_kda(t["q"], t["k"], t["v"], t["g"], t["beta"], A_log=t["A_log"], dt_bias=t["dt_bias"], **kw)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)      # > 126 MB L2

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(step_fn, steps, warmup):
        """Device time of `steps` calls: L2 is flushed (untimed) before each, each call has its own event pair."""
        for _ in range(warmup):
            step_fn()
        barrier()
        evs = []
        for _ in range(8):                 # untimed device work queued first, so that the host is ahead of the device
            flush.zero_()                  # when the first timed step is enqueued (the timed regions are device time)
        for _ in range(steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step_fn()
            e1.record()
            evs.append((e0, e1))
        barrier()
        total_ms = sum(a.elapsed_time(b) for a, b in evs)
        if world > 1:
            t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            total_ms = float(t.item())
        return total_ms / steps

    # ---- device-resident throughput ("value") ----
    # the clock sampler runs from before the warm-up to the end of the last timed loop (the timed region of the
    # headline number alone lasts only a few milliseconds, shorter than one nvidia-smi sampling period)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.5)
    ms = timed(lambda: fwd(d), args.steps, args.warmup)
    check_status(dev)
    tokens = B * T * world

    # ---- end to end through the public call with host buffers ----
    o_host = torch.empty(B, T, H, 128, dtype=torch.bfloat16).pin_memory()
    ht_host = torch.empty(B, H, 128, 128, dtype=torch.float32).pin_memory()

    def e2e_step():
        # the public host-buffer call: uploads, kernels and downloads are pipelined over 512-token segments
        chunk_kda_host(host["q"], host["k"], host["v"], host["g"], host["beta"], out=o_host, final_state_out=ht_host,
                       A_log=d["A_log"], dt_bias=d["dt_bias"], **kw)

    ms_e2e = timed(e2e_step, max(3, args.steps // 2), 3)
    h2d = sum(v.numel() * v.element_size() for v in host.values())
    d2h = o_host.numel() * 2 + ht_host.numel() * 4

    # ---- per-kernel device time for the roofline of the dominant kernel ----
    lib = _native.lib()
    stream = torch.cuda.current_stream(dev).cuda_stream
    nchunks = B * ((T + 63) // 64)
    tiles = torch.empty(nchunks * H * TILE_PACK_BYTES, dtype=torch.uint8, device=dev)
    o_buf = torch.empty(B, T, H, 128, dtype=torch.bfloat16, device=dev)
    ht_buf = torch.empty(B, H, 128, 128, dtype=torch.float32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    def k_intra():
        _native.check(lib.cula_kda_fwd_intra(d["q"].data_ptr(), d["k"].data_ptr(), d["v"].data_ptr(), d["g"].data_ptr(), 0,
                                             d["beta"].data_ptr(), 0, d["A_log"].data_ptr(), d["dt_bias"].data_ptr(),
                                             None, None, nchunks, T, H, 128 ** -0.5, 1, 2, -5.0, tiles.data_ptr(), None,
                                             None, status.data_ptr(), stream), "intra")

    def k_scan():
        _native.check(lib.cula_kda_fwd_scan(tiles.data_ptr(), None, o_buf.data_ptr(), ht_buf.data_ptr(), None, None,
                                            None, None, None, None, B, T, H, status.data_ptr(), stream), "scan")

    ms_intra = timed(k_intra, args.steps, 3)
    ms_scan = timed(k_scan, args.steps, 3)
    clocks = sampler.stop() if rank == 0 else None
    th = B * T * H
    kernels = {
        "kda_fwd_intra_kernel": dict(ms=ms_intra, bytes=th * (1282 - 256) + nchunks * H * TILE_PACK_BYTES),
        "kda_fwd_scan_kernel": dict(ms=ms_scan, bytes=nchunks * H * TILE_PACK_BYTES + th * 256 + B * H * 65536),
    }
    dom = max(kernels, key=lambda k: kernels[k]["ms"])
    peaks = load_peaks()
    achieved = kernels[dom]["bytes"] / (kernels[dom]["ms"] * 1e-3) / 1e9
    traffic, traffic_note = ncu_traffic(args.workload, dom)
    roofline = {"kernel": dom, "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": traffic, "traffic_source": traffic_note,
                "peak_source": peaks["source"],
                "algorithmic_bytes_per_launch": kernels[dom]["bytes"],
                "kernels_ms": {k: v["ms"] for k, v in kernels.items()}}

    # ---- the collective-bearing path: one 262,144-token sequence, context parallel over the ranks ----
    del tiles, o_buf, ht_buf
    cp = None if args.no_cp else cp_section(rank, world, dev, flush, steps=max(5, min(args.steps, 10)))

    if rank != 0:
        if dist.is_initialized():
            dist.destroy_process_group()
        return
    base = None
    if not args.no_cpu_baseline and world == 1:      # the CPU baseline is timed at N = 1 only
        base, _ = cpu_baseline(B, T, H)
        base["config1"] = cpu_config1()
    line = {
        "metric": "chunk_kda forward tokens/s", "value": tokens / (ms * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": headline_config(args.workload),
        "tflops": tokens * H * FLOP_PER_TOKEN_HEAD / (ms * 1e-3) / 1e12,
        "tflops_frac_of_bf16_peak": tokens / world * H * FLOP_PER_TOKEN_HEAD / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"],
        "hbm_frac_compulsory": tokens / world * H * BYTES_PER_TOKEN_HEAD / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
        "e2e": {"value": tokens / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e, "host_cores_rank0": len(host_cpus)},
        "gpu_launches": 2 * args.steps,
        "roofline": roofline,
        "cpu_baseline": base,
        "cp": cp,
        "clocks": clocks,
    }
    print(json.dumps(line), flush=True)
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
