"""``chunk_kda_host``: forward from HOST tensors, with the PCIe copies overlapped with the kernels.

KDA is a recurrence, so a sequence can be cut anywhere on a 64-token boundary and continued from the carried state
with bit-identical results (tests/test_kda_full_size.py). This entry point uses that to pipeline an inference
forward whose inputs live in (pinned) host memory: every batch row's time axis is cut into segments; while segment ``i`` runs on
the compute stream, segment ``i+1`` is uploaded on a copy stream and the output rows of segment ``i-1`` are
downloaded on a third stream. The reference has no such path (its callers hand it device tensors); it exists here
because the end-to-end cost of a forward on host data is dominated by the 134 MB of input traffic, not by the
0.2 ms of kernels. (Letting the kernels read pinned host memory in place instead of staging it was measured too:
4.5 ms against 3.1 ms — SM-issued PCIe reads reach about 30 GB/s where the copy engine reaches 55.)
"""
from __future__ import annotations

import threading

import torch

from ..utils import CHUNK
from .chunk import chunk_kda


def bind_host_to_gpu(device=None):
    """Restrict this process to the CPU cores that sit next to ``device`` (same NUMA node / PCIe root) and return them.

    With one process per GPU, host buffers that are allocated and pinned AFTER this call land in the memory of that
    node (first-touch policy), so each rank's host<->device copies stay on its own socket instead of all ranks sharing
    one node's memory controllers and inter-socket links; the GPU's node is also made the preferred node of the
    process's page allocations (`_prefer_memory_near`). The core list comes from NVML (the ideal CPU affinity of the
    device), else from the device's ``local_cpulist`` in sysfs; it is intersected with the cores the process may already
    use, and nothing changes when that would leave no core. Only this process's own affinity mask is touched."""
    import os
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    allowed = os.sched_getaffinity(0)
    cpus = set()
    try:
        import pynvml
        pynvml.nvmlInit()
        props = torch.cuda.get_device_properties(dev)
        bus_id = f"{props.pci_domain_id:08x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        handle = pynvml.nvmlDeviceGetHandleByPciBusId(bus_id.encode())
        words = (max(allowed) // 64) + 1
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        cpus = {64 * w + b for w, m in enumerate(mask) for b in range(64) if (int(m) >> b) & 1}
    except Exception:
        cpus = set()
    if not cpus:
        try:
            props = torch.cuda.get_device_properties(dev)
            path = f"/sys/bus/pci/devices/{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0/local_cpulist"
            for part in open(path).read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        except Exception:
            cpus = set()
    _prefer_memory_near(dev)
    chosen = cpus & allowed
    if chosen and chosen != allowed:
        os.sched_setaffinity(0, chosen)
        return sorted(chosen)
    return sorted(allowed)


def _prefer_memory_near(dev, _probe=None, _syscall=None):
    """Make the NUMA node the GPU hangs off the PREFERRED node of this process's future page allocations
    (``set_mempolicy(MPOL_PREFERRED)``: other nodes are still used when it is full), so that host buffers pinned after
    this call sit next to the GPU even when the cores the process may run on do not. Returns the node, or None when the
    platform does not say (no ``numa_node`` in sysfs, one node only, the call refused): nothing changes then.
    ``_probe`` () -> (node of the GPU, number of nodes) and ``_syscall`` (nr, mode, mask, maxnode) -> rc replace sysfs
    and the system call in tests."""
    import ctypes
    import os
    import platform
    nr = {"x86_64": 238, "aarch64": 237}.get(platform.machine())

    def probe():
        props = torch.cuda.get_device_properties(dev)
        bdf = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        node = int(open(f"/sys/bus/pci/devices/{bdf}/numa_node").read())
        nodes = [d for d in os.listdir("/sys/devices/system/node") if d.startswith("node") and d[4:].isdigit()]
        return node, len(nodes)

    try:
        node, n_nodes = (_probe or probe)()
    except Exception:
        return None
    if nr is None or node < 0 or node >= 64 or n_nodes < 2:
        return None
    MPOL_PREFERRED = 1
    if _syscall is not None:
        rc = _syscall(nr, MPOL_PREFERRED, 1 << node, 65)
    else:
        mask = ctypes.c_ulong(1 << node)
        rc = ctypes.CDLL(None, use_errno=True).syscall(nr, MPOL_PREFERRED, ctypes.byref(mask), 65)
    return node if rc == 0 else None


_STREAMS: dict = {}     # device -> (upload stream, download stream), created once: stream creation costs ~10 us each
_BUFFERS: dict = {}     # (device, shapes, dtypes) -> the two device-side segment buffer sets


def _streams(dev):
    st = _STREAMS.get(str(dev))
    if st is None:
        st = _STREAMS[str(dev)] = (torch.cuda.Stream(dev), torch.cuda.Stream(dev))
    return st


def _segment_buffers(dev, host_in, B, seg):
    key = (str(dev), threading.get_ident(), B, seg, tuple((tuple(t.shape[2:]), t.dtype) for t in host_in))
    bufs = _BUFFERS.get(key)
    if bufs is None:
        if len(_BUFFERS) > 8:
            _BUFFERS.clear()
        bufs = _BUFFERS[key] = [[torch.empty((B, seg) + tuple(t.shape[2:]), dtype=t.dtype, device=dev) for t in host_in]
                                for _ in range(2)]
    return bufs


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
    # A segment is a run of tokens of ONE batch row, so that every tensor contributes one contiguous block per
    # segment (a copy costs ~6 us of set-up on top of its transfer); its length keeps the bytes per segment at
    # segment_tokens x B tokens.
    seg = min(max(CHUNK, (int(segment_tokens) * B // CHUNK) * CHUNK), ((T + CHUNK - 1) // CHUNK) * CHUNK)
    segments = [(b, s0, min(T, s0 + seg)) for b in range(B) for s0 in range(0, T, seg)]
    b_l, s0_l, s1_l = segments[-1]
    if s1_l - s0_l > 2 * CHUNK:                           # a short last segment: its compute and download are the exposed tail
        cut = s0_l + (((s1_l - s0_l) * 3 // 4) // CHUNK) * CHUNK
        segments[-1:] = [(b_l, s0_l, cut), (b_l, cut, s1_l)]
    n_seg = len(segments)
    if out is None:
        out = torch.empty(v.shape, dtype=v.dtype).pin_memory()
    gate_kw = {}
    if use_gate_in_kernel:
        assert "A_log" in kwargs, "A_log must be provided when use_gate_in_kernel=True."
        gate_kw["A_log"] = kwargs["A_log"].to(dev)
        if kwargs.get("dt_bias") is not None:
            gate_kw["dt_bias"] = kwargs["dt_bias"].to(dev)
    h0 = None if initial_state is None else initial_state.to(dev, non_blocking=True)

    main = torch.cuda.current_stream(dev)
    s_in, s_out = _streams(dev)
    s_in.wait_stream(main)
    s_out.wait_stream(main)
    host_in = (q, k, v, g)
    bufs = _segment_buffers(dev, host_in, 1, seg)       # reused across calls: a call ends synchronised (see below)
    in_ready = [torch.cuda.Event() for _ in range(n_seg)]
    done = [torch.cuda.Event() for _ in range(n_seg)]
    beta_dev = torch.empty(beta.shape, dtype=beta.dtype, device=dev)
    final_dev = torch.empty(B, H, 128, v.shape[-1], dtype=torch.float32, device=dev) if output_final_state else None

    def upload(i):
        b, s0, s1 = segments[i]
        with torch.cuda.stream(s_in):
            if i >= 2:
                s_in.wait_event(done[i - 2])              # the buffer set is free once its segment has been computed
            for src, dst in zip(host_in, bufs[i % 2]):
                dst[0, : s1 - s0].copy_(src[b, s0:s1], non_blocking=True)
            if i == 0:
                beta_dev.copy_(beta, non_blocking=True)   # small: the whole tensor in one copy, behind the first blocks
            in_ready[i].record(s_in)

    upload(0)
    state = None
    for i, (b, s0, s1) in enumerate(segments):
        if i + 1 < n_seg:
            upload(i + 1)
        main.wait_event(in_ready[i])
        if s0 == 0:
            state = None if h0 is None else h0[b:b + 1]
        qd, kd, vd, gd = (t[:, : s1 - s0] for t in bufs[i % 2])
        o_seg, state = chunk_kda(qd, kd, vd, gd, beta_dev[b:b + 1, s0:s1], scale=scale, initial_state=state,
                                 output_final_state=True, use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel,
                                 use_gate_in_kernel=use_gate_in_kernel, safe_gate=safe_gate, lower_bound=lower_bound,
                                 **gate_kw)
        if s1 == T and final_dev is not None:
            final_dev[b].copy_(state[0])
        done[i].record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(done[i])
            out[b, s0:s1].copy_(o_seg[0], non_blocking=True)
            o_seg.record_stream(s_out)
    final = None
    if output_final_state:
        final = final_state_out if final_state_out is not None else torch.empty(final_dev.shape, dtype=torch.float32).pin_memory()
        final.copy_(final_dev, non_blocking=True)
    main.wait_stream(s_out)
    main.wait_stream(s_in)
    main.synchronize()
    return out, final
