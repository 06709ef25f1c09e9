"""Context parallelism for one long sequence: ``chunk_kda_cp``.

Every rank holds a contiguous shard ``[1, T_local, H, 128]`` of the same sequence (``T_local`` a multiple of the
64-token chunk on every rank but the last). A shard acts on the carried state as ``S_out = M S_in + C`` per head, so

1. each rank runs the chunk-parallel stage on its shard and one launch that scans ``(C | M)`` (no output rows),
2. the ``(C, M)`` pairs are all-gathered (``[H, 128, 256]`` fp32 = 4 MiB per rank and segment at H = 32) into every
   rank's own memory with NCCL,
3. each rank folds its predecessors' transitions into its incoming state with a small kernel, and
4. runs the ordinary fused scan + output pass from that state.

A shard is further cut into ``P`` segments (two when it is long enough): step 1 yields one transition per segment, the
fold of step 3 also yields the state at every segment boundary, and step 4 then scans the ``P`` segments side by
side as if they were separate sequences with known initial states. The scan is a latency-bound chain that occupies
64 CTAs per segment, so this halves the time of step 4 at no extra work.

This replaces what the reference gets from flash-linear-attention's ``cp_context`` (cula/kda/chunk.py:348-355,
cula/kda/chunk_fwd.py:99-127; fla/ops/cp/chunk_delta_h.py:736-817). Forward only for now: calling backward on the
result raises.

The orchestration (`cp_forward`) is written against two small interfaces, a compute backend and a gather function,
so the same code runs on NCCL across GPUs, on gloo in CPU tests, and with all ranks emulated in one process.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import _native
from ..utils import CHUNK, VarlenTables, assert_blackwell
from .chunk import _gate_mode, _ptr, _status_word


_SEGMENT_TABLES: dict = {}      # (segment bounds, device) -> VarlenTables of the segments of a shard


class CudaBackend:
    """Compute steps of one rank on its GPU through the C ABI."""

    def __init__(self, q, k, v, g, beta, scale, use_qk_l2norm_in_kernel, use_gate_in_kernel, safe_gate, lower_bound,
                 A_log, dt_bias, segments=None):
        assert q.shape[0] == 1, "context parallelism expects one sequence (batch size 1)"
        self.lib = _native.lib()
        self.q, self.k, self.v, self.g, self.beta = (x.contiguous() for x in (q, k, v, g, beta))
        self.T, self.H = q.shape[1], q.shape[2]
        self.dev = q.device
        self.stream = torch.cuda.current_stream(self.dev).cuda_stream
        self.status = _status_word(self.dev).data_ptr()
        self.num_chunks = (self.T + CHUNK - 1) // CHUNK
        P = 2 if segments is None else max(1, int(segments))   # the same on every rank, whatever the shard length
        # segment boundaries on chunk boundaries, in tokens: [0, ..., T]
        self.bounds = [min(self.T, ((self.num_chunks * i) // P) * CHUNK) for i in range(P)] + [self.T]
        self.n_segments = P
        self.tables = None
        if P > 1:
            key = (tuple(self.bounds), str(self.dev))
            self.tables = _SEGMENT_TABLES.get(key)
            if self.tables is None:
                if len(_SEGMENT_TABLES) > 16:
                    _SEGMENT_TABLES.clear()
                cpu = torch.tensor(self.bounds, dtype=torch.int32)
                self.tables = _SEGMENT_TABLES[key] = VarlenTables(cpu.to(self.dev), cpu)
        self.tiles = torch.empty(self.num_chunks * self.H * self.lib.cula_kda_tile_pack_bytes(), dtype=torch.uint8,
                                 device=self.dev)
        A_log = None if A_log is None else A_log.float().contiguous()
        dt_bias = None if dt_bias is None else dt_bias.float().contiguous()
        _native.check(self.lib.cula_kda_fwd_intra(
            self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr(), self.g.data_ptr(), int(g.dtype == torch.float32),
            self.beta.data_ptr(), int(beta.dtype == torch.float32), _ptr(A_log), _ptr(dt_bias), None, None,
            self.num_chunks, self.T, self.H, float(scale), int(use_qk_l2norm_in_kernel),
            _gate_mode(use_gate_in_kernel, safe_gate, lower_bound), float(lower_bound if lower_bound is not None else 0.0),
            self.tiles.data_ptr(), None, None, self.status, self.stream), "cula_kda_fwd_intra")

    def _table_ptrs(self):
        if self.tables is None:
            return None, None, None
        return self.tables.cu_seqlens.data_ptr(), self.tables.chunk_offsets.data_ptr(), self.tables.seq_order.data_ptr()

    def transition(self):
        """(C, M), each [P, H, 128, 128]: the affine action of every segment of this shard on the state."""
        P = self.n_segments
        C = torch.empty(P, self.H, 128, 128, dtype=torch.float32, device=self.dev)
        M = torch.empty(P, self.H, 128, 128, dtype=torch.float32, device=self.dev)
        cu_p, co_p, _ = self._table_ptrs()
        _native.check(self.lib.cula_kda_cp_transition(self.tiles.data_ptr(), C.data_ptr(), M.data_ptr(), cu_p, co_p, P,
                                                      self.T, self.H, self.status, self.stream), "cula_kda_cp_transition")
        return C, M

    def fold(self, C_all, M_all, h0, start, n):
        """S = h0 (or 0); for j in [start, start + n): S = M_all[j] S + C_all[j] (chains of [*, H, 128, 128])."""
        s_in = torch.empty(self.H, 128, 128, dtype=torch.float32, device=self.dev)
        h0 = None if h0 is None else h0.reshape(self.H, 128, 128).float().contiguous()
        _native.check(self.lib.cula_kda_cp_fold(C_all[start:].data_ptr(), M_all[start:].data_ptr(), _ptr(h0),
                                                s_in.data_ptr(), int(n), self.H, self.stream), "cula_kda_cp_fold")
        return s_in

    def forward(self, states, want_final):
        """Scan + output of the P segments from their incoming states (None = zero state)."""
        P = self.n_segments
        o = torch.empty_like(self.v)
        ht = torch.empty(P, self.H, 128, 128, dtype=torch.float32, device=self.dev) if want_final else None
        h0 = None
        if any(s is not None for s in states):
            h0 = torch.stack([torch.zeros(self.H, 128, 128, dtype=torch.float32, device=self.dev) if s is None
                              else s.reshape(self.H, 128, 128).float() for s in states]).contiguous()
        cu_p, co_p, so_p = self._table_ptrs()
        _native.check(self.lib.cula_kda_fwd_scan(self.tiles.data_ptr(), _ptr(h0), o.data_ptr(), _ptr(ht), None, None, None,
                                                 cu_p, co_p, so_p, P, self.T, self.H, self.status, self.stream),
                      "cula_kda_fwd_scan")
        return o, (ht[P - 1:] if want_final else None)


def gather_with_group(group=None):
    """all-gather into this rank's own memory: [*shape] -> [world, *shape]."""
    def gather(x):
        world = dist.get_world_size(group)
        out = torch.empty((world,) + tuple(x.shape), dtype=x.dtype, device=x.device)
        if x.is_cuda:
            dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        else:       # gloo (CPU tests): list form
            dist.all_gather(list(out.unbind(0)), x.contiguous(), group=group)
        return out
    return gather


def cp_forward(backend, gather, rank, world, initial_state=None, output_final_state=False):
    """Rank-local part of the context-parallel forward. Returns (o_local, final_state or None); the final state
    is produced on the last rank only. ``backend.n_segments`` (P, the same on every rank) is the number of segments
    a shard is cut into; the gathered transitions form one chain of ``world * P`` elements."""
    last = rank == world - 1
    P = backend.n_segments
    if world == 1 and P == 1:
        return backend.forward([initial_state], output_final_state)
    C, M = backend.transition()                              # [P, H, 128, 128] each
    if world > 1:
        C_all, M_all = gather(C), gather(M)                  # [world, P, H, 128, 128]
        C_all, M_all = C_all.reshape((world * P,) + tuple(C.shape[1:])), M_all.reshape((world * P,) + tuple(M.shape[1:]))
    else:
        C_all, M_all = C, M
    s = initial_state if rank == 0 else backend.fold(C_all, M_all, initial_state, 0, rank * P)
    states = [s]
    for i in range(1, P):                                    # state at each inner segment boundary
        s = backend.fold(C_all, M_all, s, rank * P + i - 1, 1)
        states.append(s)
    return backend.forward(states, output_final_state and last)


class _NoBackward(torch.autograd.Function):
    @staticmethod
    def forward(ctx, o, *inputs):
        return o.view_as(o)

    @staticmethod
    def backward(ctx, do):
        raise NotImplementedError("chunk_kda_cp: the context-parallel backward pass is not implemented")


@torch.compiler.disable
def chunk_kda_cp(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
                 use_qk_l2norm_in_kernel=False, use_gate_in_kernel=False, safe_gate=False, lower_bound=None,
                 group=None, segments=None, **kwargs):
    """Context-parallel ``chunk_kda`` forward. Arguments as ``chunk_kda`` for this rank's shard of ONE sequence;
    ``initial_state`` ([1, H, 128, 128] fp32) is the state before the first token of the whole sequence and is
    read on rank 0 of ``group``; ``final_state`` is returned on the last rank (None elsewhere). ``segments`` (default 2) must be the
    same on every rank; a shard shorter than that many chunks simply gets empty segments."""
    assert q.shape[0] == 1, "context parallelism expects one sequence (batch size 1)"
    assert q.dtype == k.dtype == v.dtype == torch.bfloat16, "q, k, v must be in bfloat16."
    assert q.shape[-1] == k.shape[-1] == v.shape[-1] == 128, "Currently we only support head dim of 128 for KDA"
    A_log, dt_bias = None, None
    if use_gate_in_kernel:
        assert "A_log" in kwargs, "A_log must be provided when use_gate_in_kernel=True."
        A_log, dt_bias = kwargs["A_log"], kwargs.get("dt_bias")
    if safe_gate and use_gate_in_kernel:
        if lower_bound is None:
            raise ValueError("`lower_bound` must be specified when `safe_gate=True` and `use_gate_in_kernel=True`.")
        if not (-5 <= lower_bound < 0):
            raise ValueError(f"`lower_bound` must be in the safe range [-5, 0), got {lower_bound}.")
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    if rank != world - 1 and q.shape[1] % CHUNK != 0:
        raise ValueError(f"every shard but the last must hold a multiple of {CHUNK} tokens, got {q.shape[1]}")
    assert_blackwell(q.device)
    if scale is None:
        scale = k.shape[-1] ** -0.5
    with torch.cuda.device(q.device):
        backend = CudaBackend(q, k, v, g, beta, scale, use_qk_l2norm_in_kernel, use_gate_in_kernel, safe_gate,
                              lower_bound, A_log, dt_bias, segments=1 if world == 1 else segments)
        o, ht = cp_forward(backend, gather_with_group(group), rank, world, initial_state, output_final_state)
    if torch.is_grad_enabled() and any(t.requires_grad for t in (q, k, v, g, beta)):
        o = _NoBackward.apply(o, q, k, v, g, beta)
    return o, ht
