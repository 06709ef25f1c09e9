"""``chunk_kda_host``: forward from HOST tensors, with the PCIe copies overlapped with the kernels.

KDA is a recurrence, so a sequence can be cut anywhere on a 64-token boundary and continued from the carried state
with bit-identical results (tests/test_kda_full_size.py). This entry point uses that to pipeline an inference
forward whose inputs live in (pinned) host memory: the time axis is cut into segments; while segment ``i`` runs on
the compute stream, segment ``i+1`` is uploaded on a copy stream and the output rows of segment ``i-1`` are
downloaded on a third stream. The reference has no such path (its callers hand it device tensors); it exists here
because the end-to-end cost of a forward on host data is dominated by the 134 MB of input traffic, not by the
0.2 ms of kernels.
"""
from __future__ import annotations

import torch

from ..utils import CHUNK
from .chunk import chunk_kda


@torch.no_grad()
def chunk_kda_host(q, k, v, g, beta, out=None, final_state_out=None, segment_tokens=512, device=None, scale=None,
                   initial_state=None, output_final_state=False, use_qk_l2norm_in_kernel=False,
                   use_gate_in_kernel=False, safe_gate=False, lower_bound=None, **kwargs):
    """Fixed-length batch ``[B, T, H, 128]`` on the host (pin the tensors for asynchronous copies).

    Returns ``(out, final_state)`` with ``out`` a host tensor (``out`` argument or a new pinned tensor) and
    ``final_state`` a host tensor or None. ``A_log`` / ``dt_bias`` / ``initial_state`` may be host or device
    tensors. The call returns after everything has landed in host memory.
    """
    assert q.device.type == "cpu" and q.dim() == 4, "chunk_kda_host takes host tensors [B, T, H, 128]"
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    B, T, H, _ = q.shape
    seg = max(CHUNK, (int(segment_tokens) // CHUNK) * CHUNK)
    n_seg = (T + seg - 1) // seg
    if out is None:
        out = torch.empty(v.shape, dtype=v.dtype).pin_memory()
    gate_kw = {}
    if use_gate_in_kernel:
        assert "A_log" in kwargs, "A_log must be provided when use_gate_in_kernel=True."
        gate_kw["A_log"] = kwargs["A_log"].to(dev)
        if kwargs.get("dt_bias") is not None:
            gate_kw["dt_bias"] = kwargs["dt_bias"].to(dev)
    state = None if initial_state is None else initial_state.to(dev, non_blocking=True)

    main = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    s_in.wait_stream(main)
    host_in = (q, k, v, g, beta)
    bufs = [[torch.empty((B, seg) + tuple(t.shape[2:]), dtype=t.dtype, device=dev) for t in host_in] for _ in range(2)]
    in_ready = [torch.cuda.Event() for _ in range(n_seg)]
    done = [torch.cuda.Event() for _ in range(n_seg)]
    outs = []

    def upload(i):
        s0, s1 = i * seg, min(T, (i + 1) * seg)
        with torch.cuda.stream(s_in):
            if i >= 2:
                s_in.wait_event(done[i - 2])              # the buffer set is free once its segment has been computed
            for src, dst in zip(host_in, bufs[i % 2]):
                for b in range(B):                        # one contiguous block per batch entry
                    dst[b, : s1 - s0].copy_(src[b, s0:s1], non_blocking=True)
            in_ready[i].record(s_in)

    upload(0)
    for i in range(n_seg):
        if i + 1 < n_seg:
            upload(i + 1)
        s0, s1 = i * seg, min(T, (i + 1) * seg)
        main.wait_event(in_ready[i])
        qd, kd, vd, gd, bd = (t[:, : s1 - s0] for t in bufs[i % 2])
        o_seg, state = chunk_kda(qd, kd, vd, gd, bd, scale=scale, initial_state=state, output_final_state=True,
                                 use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel, use_gate_in_kernel=use_gate_in_kernel,
                                 safe_gate=safe_gate, lower_bound=lower_bound, **gate_kw)
        done[i].record(main)
        outs.append(o_seg)                                # keep alive until the download has been enqueued
        with torch.cuda.stream(s_out):
            s_out.wait_event(done[i])
            for b in range(B):
                out[b, s0:s1].copy_(o_seg[b], non_blocking=True)
            o_seg.record_stream(s_out)
    final = None
    if output_final_state:
        final = final_state_out if final_state_out is not None else torch.empty(state.shape, dtype=state.dtype).pin_memory()
        final.copy_(state, non_blocking=True)
    main.wait_stream(s_out)
    main.synchronize()
    return out, final
