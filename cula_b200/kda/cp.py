"""Context parallelism for one long sequence: ``chunk_kda_cp``.

Every rank holds a contiguous shard ``[1, T_local, H, 128]`` of the same sequence (``T_local`` a multiple of the
64-token chunk on every rank but the last). A shard acts on the carried state as ``S_out = M S_in + C`` per head, so

1. each rank runs the chunk-parallel stage on its shard and one launch that scans ``(C | M)`` (no output rows),
2. the ``(C | M)`` pairs are all-gathered (``[2, H, 128, 128]`` fp32 = 4 MiB per rank at H = 32) into every rank's
   own memory with one NCCL collective,
3. each rank folds its predecessors' transitions into its incoming state with a small kernel, and
4. runs the ordinary fused scan + output pass from that state.

A shard is further cut into ``P`` segments (two by default): step 1 yields one transition per segment (composed
into the shard's transition before the gather), step 3 also yields the state at every segment boundary, and step 4
then scans the ``P`` segments side by side as if they were separate sequences with known initial states. The scan is a latency-bound chain that occupies
64 CTAs per segment, so this halves the time of step 4 at no extra work.

This replaces what the reference gets from flash-linear-attention's ``cp_context`` (cula/kda/chunk.py:348-355,
cula/kda/chunk_fwd.py:99-127; fla/ops/cp/chunk_delta_h.py:736-817). The backward pass runs the same exchange in the
other direction (`CPBackwardState`).

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


class KDACPContext:
    """What ``chunk_kda(..., cp_context=...)`` needs to run this rank's shard of one long sequence: the process
    group of the context-parallel ranks (None = the default group) and, optionally, the number of segments a shard
    is cut into. Stands where the reference takes flash-linear-attention's ``FLACPContext``
    (cula/kda/chunk.py:348-355)."""

    def __init__(self, group=None, segments=None):
        self.group = group
        self.segments = segments


class CudaBackend:
    """Compute steps of one rank on its GPU through the C ABI."""

    def __init__(self, q, k, v, g, beta, scale, use_qk_l2norm_in_kernel, use_gate_in_kernel, safe_gate, lower_bound,
                 A_log, dt_bias, segments=None, marks=None, tiles=None):
        assert q.shape[0] == 1, "context parallelism expects one sequence (batch size 1)"
        self.marks = marks          # optional list: receives (stage name, CUDA event recorded after the stage)
        self.mark("start")
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
        if tiles is not None:           # the chunk-parallel stage has already run (single-GPU segmented forward)
            self.tiles = tiles
            return
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
        self.mark("intra")

    def mark(self, name):
        if self.marks is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.marks.append((name, ev))

    def _table_ptrs(self):
        if self.tables is None:
            return None, None, None
        return self.tables.cu_seqlens.data_ptr(), self.tables.chunk_offsets.data_ptr(), self.tables.seq_order.data_ptr()

    def _fold(self, c_ptr, m_ptr, h0, n, out, stride=0):
        _native.check(self.lib.cula_kda_cp_fold(c_ptr, m_ptr, _ptr(h0), out.data_ptr(), int(n), self.H, int(stride),
                                                self.stream), "cula_kda_cp_fold")
        return out

    def transition(self, local_only=False):
        """X [2, H, 128, 128] = (C | M): the affine action of this whole shard on the state. The transitions of the
        P segments are kept for `incoming`; they are composed here so that only one pair travels. ``local_only``
        (a single rank): nobody consumes the shard's own transition, so only the first P - 1 segments are scanned
        and nothing is composed."""
        P = self.n_segments
        self.C_seg = torch.empty(P, self.H, 128, 128, dtype=torch.float32, device=self.dev)
        self.M_seg = torch.empty(P, self.H, 128, 128, dtype=torch.float32, device=self.dev)
        cu_p, co_p, _ = self._table_ptrs()
        _native.check(self.lib.cula_kda_cp_transition(self.tiles.data_ptr(), self.C_seg.data_ptr(), self.M_seg.data_ptr(),
                                                      cu_p, co_p, P - 1 if local_only else P, self.T, self.H,
                                                      self.status, self.stream), "cula_kda_cp_transition")
        self.mark("transition")
        if local_only:
            return None
        if P == 1:
            return torch.stack([self.C_seg[0], self.M_seg[0]])
        X = torch.empty(2, self.H, 128, 128, dtype=torch.float32, device=self.dev)
        self._fold(self.C_seg.data_ptr(), self.M_seg.data_ptr(), None, P, X[0])            # C = fold of the segments from 0
        self._fold(None, self.M_seg[1:].data_ptr(), self.M_seg[0], P - 1, X[1])            # M = M_{P-1} ... M_0
        return X

    def absorb_initial_state(self, X, initial_state):
        """Rank 0 of a multi-rank group: fold the state before the first token into the shard's C,
        ``C <- M h0 + C``, so that the gathered pairs carry it to every later rank."""
        h0 = initial_state.reshape(self.H, 128, 128).float().contiguous()
        out = torch.empty_like(X)
        out[1].copy_(X[1])
        self._fold(X[0].data_ptr(), X[1].data_ptr(), h0, 1, out[0])
        return out

    def incoming(self, X_all, rank, initial_state):
        """States entering each of the P segments of this shard: the fold of the shards before this one (X_all is
        [world, 2, H, 128, 128] in this GPU's memory; rank 0's pair already contains the initial state), then one
        more step per inner segment boundary. ``initial_state`` is read on rank 0 only."""
        s = None
        if rank == 0 and initial_state is not None:
            s = initial_state.reshape(self.H, 128, 128).float().contiguous()
        if rank > 0:
            per = self.H * 128 * 128
            s = self._fold(X_all.data_ptr(), X_all.data_ptr() + 4 * per, s, rank,
                           torch.empty(self.H, 128, 128, dtype=torch.float32, device=self.dev), stride=2 * per)
        states = [s]
        for i in range(1, self.n_segments):
            s = self._fold(self.C_seg[i - 1:].data_ptr(), self.M_seg[i - 1:].data_ptr(), s, 1,
                           torch.empty(self.H, 128, 128, dtype=torch.float32, device=self.dev))
            states.append(s)
        return states

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


_SM_COUNT: dict = {}
MAX_AUTO_SEGMENTS = 4       # upper bound of `auto_segments`; 1 switches the single-GPU segmentation off


def auto_segments(num_chunks, heads, device):
    """How many side-by-side segments the scan of ONE long sequence should be cut into on a single GPU: the scan is
    a chain of ``num_chunks`` dependent steps that occupies only ``2 * heads`` CTAs, so while SMs are idle a second
    pass pays for itself -- a transition scan per segment (cheaper: no output products), a fold, and then all
    segments scanned side by side from their now-known incoming states. Per chunk the two passes cost about
    (0.9 + 1.7) / P microseconds against 1.7 for the plain scan; below a few hundred chunks the extra launches eat
    the gain. The role of the intra-card mode of flash-linear-attention's merge kernel
    (fla/ops/cp/chunk_delta_h.py:321-357)."""
    key = str(device)
    if key not in _SM_COUNT:
        _SM_COUNT[key] = torch.cuda.get_device_properties(device).multi_processor_count
    fit = _SM_COUNT[key] // (2 * heads)          # segments whose four-warp scan CTAs all find an SM
    if num_chunks < 512 or fit < 2:
        return 1
    return max(1, min(MAX_AUTO_SEGMENTS, fit))


def segmented_forward(q, k, v, g, beta, tiles, initial_state, output_final_state, segments):
    """Scan + output of one sequence on one GPU in ``segments`` side-by-side pieces (see `auto_segments`); ``tiles``
    are the tile packs the chunk-parallel stage has already written. Returns (o, final_state or None)."""
    backend = CudaBackend(q, k, v, g, beta, None, None, None, None, None, None, None, segments=segments, tiles=tiles)
    return cp_forward(backend, None, 0, 1, initial_state, output_final_state)


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


def cp_forward(backend, gather, rank, world, initial_state=None, output_final_state=False, aux=None):
    """Rank-local part of the context-parallel forward. Returns (o_local, final_state or None); the final state
    is produced on the last rank only. ``aux`` (a dict) receives what the backward pass needs: the state entering
    this shard and the gathered transitions."""
    last = rank == world - 1
    if world == 1 and backend.n_segments == 1:
        if aux is not None:
            aux.update(s_in=initial_state, X_all=None)
        return backend.forward([initial_state], output_final_state)
    mark = getattr(backend, "mark", lambda name: None)
    if world == 1:
        backend.transition(local_only=True)                   # segments of one shard on one GPU: nothing travels
        X_all = None
    else:
        X = backend.transition()                              # [2, H, 128, 128]: (C | M) of this shard
        if rank == 0 and initial_state is not None:
            X = backend.absorb_initial_state(X, initial_state)    # later ranks never see initial_state itself
        mark("fold_local")
        X_all = gather(X)                                     # [world, 2, H, 128, 128]
    mark("gather")
    states = backend.incoming(X_all, rank, initial_state)
    mark("fold_incoming")
    if aux is not None:
        aux.update(s_in=states[0], X_all=X_all)
    out = backend.forward(states, output_final_state and last)
    mark("scan")
    return out


class CPBackwardState:
    """What one rank keeps from the forward pass for the context-parallel backward, and the two steps of it.

    The backward pass of a shard is affine in the gradient of the state leaving the shard:
    ``dS_in = M^T dS_out + C~`` with the forward ``M`` and ``C~`` the part that comes from the shard's own ``do``.
    So (1) `prepare` runs the reverse scan with ``dS_out = 0`` and returns ``Y = (C~ | dht)`` for the gather,
    (2) `finish` folds the successors' ``(M^T, C~)`` onto the last rank's ``dht`` to get this shard's true
    ``dS_out`` and runs the ordinary backward from it. Mirrors the forward exchange with the direction reversed
    (fla/ops/cp/chunk_delta_h.py:820-910 is the counterpart the reference reaches)."""

    def __init__(self, q, k, v, g, beta, A_log, dt_bias, s_in, X_all, scale, flags, rank, world):
        self.q, self.k, self.v, self.g, self.beta, self.A_log, self.dt_bias = q, k, v, g, beta, A_log, dt_bias
        self.s_in, self.X_all, self.scale, self.flags, self.rank, self.world = s_in, X_all, scale, flags, rank, world
        self.H = q.shape[2]

    def _s0(self):
        return None if self.s_in is None else self.s_in.reshape(1, self.H, 128, 128).float().contiguous()

    def prepare(self, do, dht):
        """Recompute the forward intermediates of the shard; reverse scan from dS_out = 0. Returns Y [2, H, 128, 128]."""
        from .chunk import chunk_kda_fwd
        lib = _native.lib()
        l2, gate_in, safe_gate, lower_bound = self.flags
        dev = self.q.device
        stream = torch.cuda.current_stream(dev).cuda_stream
        self.do = do.contiguous()
        self.saved = chunk_kda_fwd(self.q, self.k, self.v, self.g, self.beta, self.scale, self._s0(), False, None, None,
                                   l2, gate_in, safe_gate, lower_bound, self.A_log, self.dt_bias,
                                   store_for_backward=True, want_output=False)
        Y = torch.zeros(2, self.H, 128, 128, dtype=torch.float32, device=dev)
        if dht is not None:
            Y[1].copy_(dht.reshape(self.H, 128, 128))
        if self.world > 1 and self.rank > 0:                  # nobody needs rank 0's C~
            work = torch.zeros(4, dtype=torch.float32, device=dev)
            _native.check(lib.cula_kda_bwd_grad_scale(self.do.data_ptr(), self.do.numel(), None, 0, work[2:].data_ptr(),
                                                      work.data_ptr(), stream), "cula_kda_bwd_grad_scale")
            _native.check(lib.cula_kda_bwd_scan(self.saved["tiles"].data_ptr(), self.do.data_ptr(), None, work.data_ptr(),
                                                None, None, Y[0].data_ptr(), None, None, None, 1, self.q.shape[1], self.H,
                                                _status_word(dev).data_ptr(), stream), "cula_kda_bwd_scan")
        return Y

    def finish(self, Y_all):
        """Y_all [world, 2, H, 128, 128] in this GPU's memory. Returns (dq, dk, dv, dg, dbeta, dA_log, ddt_bias, dS_in);
        dA_log and ddt_bias are this shard's contributions (their sum over the group is the caller's, as it is for
        data-parallel replicas)."""
        from .chunk import chunk_kda_bwd
        lib = _native.lib()
        l2, gate_in, safe_gate, lower_bound = self.flags
        dev = self.q.device
        r, W, H = self.rank, self.world, self.H
        dht = Y_all[W - 1, 1]
        if r < W - 1:
            n = W - 1 - r
            Mt = self.X_all[r + 1:, 1].flip(0).transpose(-1, -2).contiguous()     # successors, nearest last
            Ct = Y_all[r + 1:, 0].flip(0).contiguous()
            out = torch.empty(H, 128, 128, dtype=torch.float32, device=dev)
            _native.check(lib.cula_kda_cp_fold(Ct.data_ptr(), Mt.data_ptr(), dht.contiguous().data_ptr(), out.data_ptr(), n, H,
                                               0, torch.cuda.current_stream(dev).cuda_stream), "cula_kda_cp_fold")
            dht = out
        s0 = self._s0()
        if s0 is None:                                        # a zero state still has a gradient slot (it is dS_in)
            s0 = torch.zeros(1, H, 128, 128, dtype=torch.float32, device=dev)
        return chunk_kda_bwd(self.q, self.k, self.v, self.g, self.beta, self.scale, s0, self.do,
                             dht.reshape(1, H, 128, 128), None, None, l2, gate_in, safe_gate, lower_bound, self.A_log,
                             self.dt_bias, saved=self.saved)


class ChunkKDACPFunction(torch.autograd.Function):
    """Autograd boundary of the context-parallel path: one shard per rank, exchanges inside forward and backward."""

    @staticmethod
    def forward(ctx, q, k, v, g, beta, A_log, dt_bias, initial_state, scale, output_final_state, flags, group, segments,
                marks=None):
        q, k, v, g, beta = (x.contiguous() for x in (q, k, v, g, beta))
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        l2, gate_in, safe_gate, lower_bound = flags
        aux = {}
        with torch.cuda.device(q.device):
            backend = CudaBackend(q, k, v, g, beta, scale, l2, gate_in, safe_gate, lower_bound, A_log, dt_bias,
                                  segments=segments, marks=marks)
            o, ht = cp_forward(backend, gather_with_group(group), rank, world, initial_state, output_final_state, aux)
        ctx.cp = CPBackwardState(q, k, v, g, beta, None if A_log is None else A_log.float().contiguous(),
                                 None if dt_bias is None else dt_bias.float().contiguous(), aux["s_in"], aux["X_all"],
                                 scale, flags, rank, world)
        ctx.group = group
        ctx.has_h0 = initial_state is not None
        ctx.param_dtypes = (None if A_log is None else (A_log.dtype, A_log.shape),
                            None if dt_bias is None else (dt_bias.dtype, dt_bias.shape))
        if ht is None:
            ht = torch.empty(0, device=q.device)              # autograd wants a tensor; the wrapper maps it back to None
            ctx.mark_non_differentiable(ht)
        return o, ht

    @staticmethod
    def backward(ctx, do, dht):
        cp = ctx.cp
        with torch.cuda.device(do.device):
            Y = cp.prepare(do, dht if (cp.rank == cp.world - 1 and dht is not None and dht.numel() > 0) else None)
            Y_all = gather_with_group(ctx.group)(Y) if cp.world > 1 else Y[None]
            dq, dk, dv, dg, dbeta, dA, dbias, dh0 = cp.finish(Y_all)
        if dA is not None and ctx.param_dtypes[0] is not None:
            dA = dA.to(ctx.param_dtypes[0][0]).view(ctx.param_dtypes[0][1])
        if dbias is not None and ctx.param_dtypes[1] is not None:
            dbias = dbias.to(ctx.param_dtypes[1][0]).view(ctx.param_dtypes[1][1])
        dh0 = dh0 if (ctx.has_h0 and cp.rank == 0) else None
        return dq, dk, dv, dg, dbeta, dA, dbias, dh0, None, None, None, None, None, None


@torch.compiler.disable
def chunk_kda_cp(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
                 use_qk_l2norm_in_kernel=False, use_gate_in_kernel=False, safe_gate=False, lower_bound=None,
                 group=None, segments=None, stage_marks=None, **kwargs):
    """Context-parallel ``chunk_kda`` forward. Arguments as ``chunk_kda`` for this rank's shard of ONE sequence;
    ``initial_state`` ([1, H, 128, 128] fp32) is the state before the first token of the whole sequence and is
    read on rank 0 of ``group``; ``final_state`` is returned on the last rank (None elsewhere). Differentiable: the
    gradients of ``A_log`` / ``dt_bias`` are this shard's contributions (sum them over the group as for data-parallel
    replicas), the gradient of ``initial_state`` appears on rank 0. ``segments`` (default 2) must be the
    same on every rank; a shard shorter than that many chunks simply gets empty segments. ``stage_marks`` (a
    list) receives ``(stage, torch.cuda.Event)`` pairs recorded after each stage of the forward, for profiling."""
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
    flags = (use_qk_l2norm_in_kernel, use_gate_in_kernel, safe_gate, lower_bound)
    o, ht = ChunkKDACPFunction.apply(q, k, v, g, beta, A_log, dt_bias, initial_state, scale, output_final_state, flags,
                                     group, segments, stage_marks)
    return o, (ht if ht.numel() > 0 else None)
