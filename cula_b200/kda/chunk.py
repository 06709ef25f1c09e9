"""``chunk_kda``: chunkwise Kimi Delta Attention on B200, same call surface as the reference's
``cula.kda.chunk_kda`` (cula/kda/chunk.py:217-412).

Host side only: argument checks, output allocation and two (forward) C-ABI launches on the current
torch stream. All arithmetic happens in the sm_100a kernels of libcula_kda.so; there is no Triton,
no FLA dispatch and no CPU fallback.
"""
from __future__ import annotations

import torch

from .. import _native
from ..utils import CHUNK, assert_blackwell, get_varlen_tables

GATE_NONE, GATE_SOFTPLUS, GATE_LOWER_BOUND = 0, 1, 2

_status_words: dict = {}
_status_mirrors: dict = {}      # device -> pinned host copy of the status word, refreshed after every chunk_kda forward
FORWARD_CALLS = 0               # how many times chunk_kda_fwd has run in this process (tests count recomputations)

STATUS_MESSAGES = {
    1: "a bounded in-kernel wait timed out",
    2: "a state-pool index lies past the end of the pool",
    3: "a forward intermediate (w, u, kg, qg or Aqk) left the fp16 range or is not finite; "
       "check the magnitude of v (|v| < 65504 is required) and of the gate",
}


def _status_word(device):
    key = str(device)
    if key not in _status_words:
        with torch.inference_mode(False):      # an inference tensor could not be cleared outside inference mode later
            _status_words[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status_words[key]


def _raise_status(code):
    raise RuntimeError(f"cula_b200 kernel status {code}: {STATUS_MESSAGES.get(code, 'unknown')}")


def check_status(device=None):
    """Synchronise and raise if any kernel on ``device`` reported a problem (a bounded wait that gave up, a bad
    state-pool index, an intermediate outside the fp16 range)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    word = _status_words.get(str(device))
    if word is None:
        return
    code = int(word.item())
    if code != 0:
        word.zero_()
        mirror = _status_mirrors.get(str(device))
        if mirror is not None:
            mirror.zero_()
        _raise_status(code)


def _poll_status(device):
    """Cheap, non-blocking check made at the start of every ``chunk_kda`` call: the status word of the previous
    calls is mirrored into pinned host memory by an asynchronous copy queued behind their kernels, so a problem a
    kernel reported surfaces (as RuntimeError) at the latest on the call after the one that has completed."""
    mirror = _status_mirrors.get(str(device))
    if mirror is not None and int(mirror[0]) != 0:
        check_status(device)


def _mirror_status(device):
    key = str(device)
    mirror = _status_mirrors.get(key)
    if mirror is None:
        with torch.inference_mode(False):
            mirror = _status_mirrors[key] = torch.zeros(1, dtype=torch.int32).pin_memory()
    mirror.copy_(_status_word(device), non_blocking=True)


def _ptr(t):
    return None if t is None else t.data_ptr()


def _g_flags(g):
    """Element type and layout bits of the gate tensor (CULA_KDA_G_FP32, CULA_KDA_G_PER_HEAD): a 3-D ``g`` is one
    gate per (token, head), the scalar-gate variant."""
    return int(g.dtype == torch.float32) | (2 if g.dim() == 3 else 0)


def _beta_flags(beta, beta_logit):
    """Element type bit and logit bit of the beta tensor (CULA_KDA_BETA_FP32, CULA_KDA_BETA_LOGIT)."""
    return int(beta.dtype == torch.float32) | (2 if beta_logit else 0)


def _gate_mode(use_gate_in_kernel, safe_gate, lower_bound):
    if not use_gate_in_kernel:
        return GATE_NONE
    # the lower-bound (sigmoid) form whenever a lower bound is given, as kda_gate_chunk_cumsum does
    # (fla/ops/kda/gate.py:509-548 keys on ``lower_bound is not None`` alone)
    return GATE_LOWER_BOUND if lower_bound is not None else GATE_SOFTPLUS


def chunk_kda_fwd(q, k, v, g, beta, scale, initial_state, output_final_state, cu_seqlens, cu_seqlens_cpu,
                  use_qk_l2norm_in_kernel, use_gate_in_kernel, safe_gate, lower_bound, A_log, dt_bias,
                  store_states=False, store_akk=False, store_for_backward=False, want_output=True, beta_logit=False):
    """Forward orchestration (the role of cula/kda/chunk_fwd.py:39-152): the chunk-parallel stage
    writes one tile pack per (chunk, head); the scan consumes them, carries the fp32 state and
    writes ``o``. Returns a dict with o, final_state and the intermediates kept for backward."""
    global FORWARD_CALLS
    FORWARD_CALLS += 1
    lib = _native.lib()
    B, T, H, K = q.shape
    dev = q.device
    stream = torch.cuda.current_stream(dev).cuda_stream
    if cu_seqlens is not None:
        tab = get_varlen_tables(cu_seqlens, cu_seqlens_cpu)
        if tab.total_tokens > T:
            raise ValueError(f"cu_seqlens[-1]={tab.total_tokens} exceeds the {T} packed tokens")
        n_seqs, num_chunks = tab.n_seqs, tab.num_chunks
        cu_p, ci_p, co_p, so_p = (tab.cu_seqlens.data_ptr(), tab.chunk_indices.data_ptr(),
                                  tab.chunk_offsets.data_ptr(), tab.seq_order.data_ptr())
        o = torch.zeros_like(v) if want_output else None   # rows past cu_seqlens[-1] stay zero (cula/kda/chunk_fwd.py:129-130)
    else:
        n_seqs, num_chunks = B, B * ((T + CHUNK - 1) // CHUNK)
        cu_p = ci_p = co_p = so_p = None
        o = torch.empty_like(v) if want_output else None
    tiles = torch.empty(num_chunks * H * lib.cula_kda_tile_pack_bytes(), dtype=torch.uint8, device=dev)
    akk = (torch.empty(num_chunks * H, CHUNK, CHUNK, dtype=torch.float32, device=dev)
           if (store_akk or store_for_backward) else None)
    mkk = torch.empty(num_chunks * H, CHUNK, CHUNK, dtype=torch.float32, device=dev) if store_for_backward else None
    gate_mode = _gate_mode(use_gate_in_kernel, safe_gate, lower_bound)
    _native.check(lib.cula_kda_fwd_intra(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), _g_flags(g),
        beta.data_ptr(), _beta_flags(beta, beta_logit), _ptr(A_log), _ptr(dt_bias),
        cu_p, ci_p, num_chunks, T, H, float(scale), int(use_qk_l2norm_in_kernel), gate_mode,
        float(lower_bound if lower_bound is not None else 0.0), tiles.data_ptr(), _ptr(akk), _ptr(mkk), _status_word(dev).data_ptr(), stream),
        "cula_kda_fwd_intra")
    if (cu_seqlens is None and B == 1 and want_output and not (store_states or store_for_backward)):
        from .cp import auto_segments, segmented_forward
        P = auto_segments(num_chunks, H, dev)
        if P > 1:      # one long sequence: few scan CTAs, many dependent steps -> scan it in P side-by-side segments
            o, final_state = segmented_forward(q, k, v, g, beta, tiles, initial_state, output_final_state, P)
            return dict(o=o, final_state=final_state, tiles=tiles, akk=akk, mkk=mkk, h=None, h32=None, vnew=None,
                        num_chunks=num_chunks)
    final_state = torch.empty(n_seqs, H, K, v.shape[-1], dtype=torch.float32, device=dev) if output_final_state else None
    h = vnew = h32 = None
    if store_states:
        h = torch.empty(num_chunks * H, K, v.shape[-1], dtype=torch.bfloat16, device=dev)
    if store_for_backward:
        h32 = torch.empty(num_chunks * H, K, v.shape[-1], dtype=torch.float32, device=dev)
    if store_states or store_for_backward:
        vnew = torch.empty(num_chunks * H, CHUNK, v.shape[-1], dtype=torch.float16, device=dev)
    _native.check(lib.cula_kda_fwd_scan(
        tiles.data_ptr(), _ptr(initial_state), _ptr(o), _ptr(final_state), _ptr(h), _ptr(vnew), _ptr(h32),
        cu_p, co_p, so_p, n_seqs, T, H, _status_word(dev).data_ptr(), stream), "cula_kda_fwd_scan")
    return dict(o=o, final_state=final_state, tiles=tiles, akk=akk, mkk=mkk, h=h, h32=h32, vnew=vnew,
                num_chunks=num_chunks)


def chunk_kda_bwd(q, k, v, g, beta, scale, initial_state, do, dht, cu_seqlens, cu_seqlens_cpu,
                  use_qk_l2norm_in_kernel, use_gate_in_kernel, safe_gate, lower_bound, A_log, dt_bias, saved=None,
                  beta_logit=False):
    """Backward orchestration (the role of cula/kda/chunk_bwd.py:432-604). ``saved`` holds the forward
    intermediates (tiles, akk, mkk, h32, vnew) when they were kept; otherwise they are recomputed here, as the
    reference does by default (cula/kda/chunk_bwd.py:459-500)."""
    lib = _native.lib()
    B, T, H, K = q.shape
    V = v.shape[-1]
    dev = q.device
    stream = torch.cuda.current_stream(dev).cuda_stream
    if saved is None:
        saved = chunk_kda_fwd(q, k, v, g, beta, scale, initial_state, False, cu_seqlens, cu_seqlens_cpu,
                              use_qk_l2norm_in_kernel, use_gate_in_kernel, safe_gate, lower_bound, A_log, dt_bias,
                              store_for_backward=True, want_output=False, beta_logit=beta_logit)
    if cu_seqlens is not None:
        tab = get_varlen_tables(cu_seqlens, cu_seqlens_cpu)
        n_seqs, num_chunks = tab.n_seqs, tab.num_chunks
        cu_p, ci_p, co_p, so_p = (tab.cu_seqlens.data_ptr(), tab.chunk_indices.data_ptr(),
                                  tab.chunk_offsets.data_ptr(), tab.seq_order.data_ptr())
        zeros = torch.zeros
    else:
        n_seqs, num_chunks = B, B * ((T + CHUNK - 1) // CHUNK)
        cu_p = ci_p = co_p = so_p = None
        zeros = torch.empty
    status = _status_word(dev).data_ptr()
    gate_mode = _gate_mode(use_gate_in_kernel, safe_gate, lower_bound)
    do = do.contiguous()
    if dht is not None:
        dht = dht.float().contiguous()
    work = torch.zeros(4, dtype=torch.float32, device=dev)          # [0:2] = {s, 1/s}, [2] = running max (as bits)
    _native.check(lib.cula_kda_bwd_grad_scale(do.data_ptr(), do.numel(), _ptr(dht), 0 if dht is None else dht.numel(),
                                              work[2:].data_ptr(), work.data_ptr(), stream), "cula_kda_bwd_grad_scale")
    dvn = torch.empty(num_chunks * H, CHUNK, V, dtype=torch.float16, device=dev)
    ds = torch.empty(num_chunks * H, K, V, dtype=torch.float32, device=dev)
    dh0 = torch.empty(n_seqs, H, K, V, dtype=torch.float32, device=dev) if initial_state is not None else None
    _native.check(lib.cula_kda_bwd_scan(saved["tiles"].data_ptr(), do.data_ptr(), _ptr(dht), work.data_ptr(),
                                        dvn.data_ptr(), ds.data_ptr(), _ptr(dh0), cu_p, co_p, so_p, n_seqs, T, H, status,
                                        stream), "cula_kda_bwd_scan")
    dv = zeros(v.shape, dtype=v.dtype, device=dev)
    scratch = torch.empty(num_chunks * H, lib.cula_kda_bwd_scratch_floats(), dtype=torch.float32, device=dev)
    _native.check(lib.cula_kda_bwd_dense(saved["h32"].data_ptr(), ds.data_ptr(), saved["vnew"].data_ptr(), dvn.data_ptr(),
                                         do.data_ptr(), v.data_ptr(), beta.data_ptr(), _beta_flags(beta, beta_logit),
                                         saved["akk"].data_ptr(), work.data_ptr(), dv.data_ptr(), scratch.data_ptr(),
                                         cu_p, ci_p, num_chunks, T, H, status, stream), "cula_kda_bwd_dense")
    dq, dk = zeros(q.shape, dtype=q.dtype, device=dev), zeros(k.shape, dtype=k.dtype, device=dev)
    dg, dbeta = zeros(g.shape, dtype=g.dtype, device=dev), zeros(beta.shape, dtype=beta.dtype, device=dev)
    dA = torch.zeros(H, dtype=torch.float32, device=dev) if use_gate_in_kernel else None
    dbias = torch.zeros(H * K, dtype=torch.float32, device=dev) if (use_gate_in_kernel and dt_bias is not None) else None
    _native.check(lib.cula_kda_bwd_gated(
        q.data_ptr(), k.data_ptr(), g.data_ptr(), _g_flags(g), beta.data_ptr(),
        _beta_flags(beta, beta_logit), _ptr(A_log), _ptr(dt_bias), saved["akk"].data_ptr(), saved["mkk"].data_ptr(),
        scratch.data_ptr(), work.data_ptr(), dq.data_ptr(), dk.data_ptr(), dg.data_ptr(), dbeta.data_ptr(), _ptr(dA),
        _ptr(dbias), cu_p, ci_p, num_chunks, T, H, float(scale), int(use_qk_l2norm_in_kernel), gate_mode,
        float(lower_bound if lower_bound is not None else 0.0), stream), "cula_kda_bwd_gated")
    return dq, dk, dv, dg, dbeta, dA, dbias, dh0


class ChunkKDAFunction(torch.autograd.Function):
    """Autograd boundary (cula/kda/chunk.py:28-214). Inputs are made contiguous and the device of ``q`` is made
    current (the reference's ``input_guard``); forward and backward carry the reference's autocast decorators
    (cula/kda/chunk.py:29-31,128-130), so backward runs under the autocast state forward ran under."""

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda")
    def forward(ctx, q, k, v, g, beta, A_log, dt_bias, scale, initial_state, output_final_state,
                use_qk_l2norm_in_kernel, use_gate_in_kernel, cu_seqlens, cu_seqlens_cpu, safe_gate, lower_bound,
                disable_recompute, return_intermediate_states, keep_intermediates, beta_logit=False):
        q, k, v, g, beta = (x.contiguous() for x in (q, k, v, g, beta))
        if A_log is not None:
            A_log = A_log.float().contiguous()
        if dt_bias is not None:
            dt_bias = dt_bias.float().contiguous()
        if initial_state is not None:
            initial_state = initial_state.contiguous()
        with torch.cuda.device(q.device):
            # keep_intermediates is decided by the caller of .apply: grad mode is always off in here
            out = chunk_kda_fwd(q, k, v, g, beta, scale, initial_state, output_final_state, cu_seqlens,
                                cu_seqlens_cpu, use_qk_l2norm_in_kernel, use_gate_in_kernel, safe_gate, lower_bound,
                                A_log, dt_bias, store_states=return_intermediate_states,
                                store_for_backward=bool(keep_intermediates), beta_logit=beta_logit)
            _mirror_status(q.device)
        if return_intermediate_states:
            assert torch.is_inference_mode_enabled(), "return_intermediate_states is only allowed in inference mode"
            assert disable_recompute is False, "return_intermediate_states must be used with disable_recompute=False"
            B, T, H, K = q.shape
            h = out["h"].view(out["num_chunks"], H, K, v.shape[-1])
            if cu_seqlens is None:
                h = h.view(B, -1, H, K, v.shape[-1])
            else:
                h = h.unsqueeze(0)
            return out["o"], out["final_state"], h
        ctx.save_for_backward(q, k, v, g, beta, A_log, dt_bias, initial_state, cu_seqlens)
        # disable_recompute keeps the forward intermediates alive for backward (cula/kda/chunk_fwd.py:144-151 drops
        # them otherwise); they are internal buffers nobody else can modify, so they ride on ctx directly
        ctx.kept = ({n: out[n] for n in ("tiles", "akk", "mkk", "h32", "vnew")}
                    if out["h32"] is not None else None)
        ctx.cu_seqlens_cpu = cu_seqlens_cpu
        ctx.scale = scale
        ctx.flags = (use_qk_l2norm_in_kernel, use_gate_in_kernel, safe_gate, lower_bound)
        ctx.beta_logit = beta_logit
        return out["o"], out["final_state"]

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, do, dht):
        q, k, v, g, beta, A_log, dt_bias, initial_state, cu_seqlens = ctx.saved_tensors
        l2, gate_in, safe_gate, lower_bound = ctx.flags
        with torch.cuda.device(q.device):
            dq, dk, dv, dg, dbeta, dA, dbias, dh0 = chunk_kda_bwd(
                q, k, v, g, beta, ctx.scale, initial_state, do, dht, cu_seqlens, ctx.cu_seqlens_cpu, l2, gate_in,
                safe_gate, lower_bound, A_log, dt_bias, saved=ctx.kept, beta_logit=ctx.beta_logit)
        if dA is not None and A_log is not None:
            dA = dA.to(A_log.dtype).view_as(A_log)
        if dbias is not None and dt_bias is not None:
            dbias = dbias.to(dt_bias.dtype).view_as(dt_bias)
        # gradients for: q, k, v, g, beta, A_log, dt_bias, scale, initial_state, then 11 non-tensor arguments
        return (dq, dk, dv, dg, dbeta, dA, dbias, None, dh0) + (None,) * 11


@torch.compiler.disable
def chunk_kda(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
              use_qk_l2norm_in_kernel=False, use_gate_in_kernel=False, cu_seqlens=None, cu_seqlens_cpu=None,
              safe_gate=False, lower_bound=None, disable_recompute=False, return_intermediate_states=False,
              cp_context=None, use_beta_sigmoid_in_kernel=False, **kwargs):
    r"""Chunkwise KDA forward (+ autograd backward).

    Args mirror ``cula.kda.chunk_kda`` (cula/kda/chunk.py:218-346):
        q, k: ``[B, T, H, 128]`` bf16.  v: ``[B, T, H, 128]`` bf16.
        g: ``[B, T, H, 128]``; the natural-log decay (fp32 or bf16) when ``use_gate_in_kernel=False``,
            else the raw gate input, activated in-kernel with ``A_log`` ``[H]`` and optional ``dt_bias``
            ``[H*128]`` passed as keyword arguments.
        beta: ``[B, T, H]`` bf16 or fp32.
        scale: defaults to ``128 ** -0.5``.
        initial_state: ``[N, H, 128, 128]`` fp32 (N sequences) or None.
        output_final_state: also return the ``[N, H, 128, 128]`` fp32 final state.
        use_qk_l2norm_in_kernel: L2-normalise q and k rows in-kernel.
        safe_gate / lower_bound: with ``use_gate_in_kernel`` selects
            ``lower_bound * sigmoid(exp(A_log) * (g + dt_bias))``; lower_bound must lie in [-5, 0).
        cu_seqlens: int32 ``[N+1]`` for a packed batch (then B must be 1); cu_seqlens_cpu: optional host copy.
        disable_recompute: keep forward intermediates for backward instead of recomputing them.
        return_intermediate_states: inference only; also return h ``[B, NT, H, 128, 128]`` bf16.
        use_beta_sigmoid_in_kernel: (extension) ``beta`` holds raw logits; ``sigmoid`` is applied in-kernel and the
            backward pass returns the gradient w.r.t. the logits, so the activated beta never round-trips HBM (the
            fusion of ``fused_beta_sigmoid`` into the call).
        cp_context: a :class:`cula_b200.kda.cp.KDACPContext` (process group of the context-parallel ranks); the call
            is then this rank's shard of ONE sequence and runs through ``chunk_kda_cp`` (the reference takes
            flash-linear-attention's ``FLACPContext`` here, cula/kda/chunk.py:348-355).

    Numeric range: the chunk-local intermediates w, u, kg, qg, Aqk travel as fp16 (the reference uses bf16), so
    ``|v|`` and ``|beta v|`` must stay below 65504; q and k are unrestricted when ``use_qk_l2norm_in_kernel`` is
    set and are expected to be unit rows otherwise. A value that leaves the range is reported through the device
    status word (``check_status``; also raised by the next ``chunk_kda`` call on the device).

    Returns ``(o, final_state)`` (``final_state`` is None unless requested).
    Raises ValueError / AssertionError on the same conditions as the reference (cula/kda/chunk.py:348-388).
    """
    if cp_context is not None:
        from .cp import chunk_kda_cp
        assert cu_seqlens is None, "context parallelism takes this rank's shard of one sequence, not a packed batch"
        assert not return_intermediate_states, "return_intermediate_states is not supported for context parallelism"
        return chunk_kda_cp(q, k, v, g, beta, scale=scale, initial_state=initial_state,
                            output_final_state=output_final_state, use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel,
                            use_gate_in_kernel=use_gate_in_kernel, safe_gate=safe_gate, lower_bound=lower_bound,
                            group=cp_context.group, segments=getattr(cp_context, "segments", None), **kwargs)
    if cu_seqlens is not None:
        if q.shape[0] != 1:
            raise ValueError(
                f"The batch size is expected to be 1 rather than {q.shape[0]} when using `cu_seqlens`."
                f"Please flatten variable-length inputs before processing.")
        if initial_state is not None and initial_state.shape[0] != len(cu_seqlens) - 1:
            raise ValueError(
                f"The number of initial states is expected to be equal to the number of input sequences, "
                f"i.e., {len(cu_seqlens) - 1} rather than {initial_state.shape[0]}.")
    if initial_state is not None:
        assert initial_state.dtype == torch.float32, "initial_state must be in float32."

    A_log, dt_bias = None, None
    if use_gate_in_kernel:
        assert "A_log" in kwargs, "A_log must be provided when use_gate_in_kernel=True."
        A_log, dt_bias = kwargs["A_log"], kwargs.get("dt_bias")

    if safe_gate and use_gate_in_kernel:
        if lower_bound is None:
            raise ValueError("`lower_bound` must be specified when `safe_gate=True` and `use_gate_in_kernel=True`.")
        if not (-5 <= lower_bound < 0):
            raise ValueError(f"`lower_bound` must be in the safe range [-5, 0), got {lower_bound}.")

    assert q.shape == k.shape == g.shape, "q, k, g must have the same shape."
    assert k.shape[-1] <= 256, "Currently we only support key headdim <=256 for KDA :-("
    assert beta.shape == q.shape[:3], "beta must be of shape (batch size, seq len, num of head)."
    assert v.shape == (*q.shape[:3], v.shape[-1]), "v must be of shape (batch size, seq len, num of head, head dim)."
    assert q.dtype == k.dtype == v.dtype == torch.bfloat16, "q, k, v must be in bfloat16."
    assert beta.dtype == torch.bfloat16 or beta.dtype == torch.float32, "beta must be in bfloat16 or float32."
    assert q.shape[-1] == k.shape[-1] == v.shape[-1] == 128, "Currently we only support head dim of 128 for KDA"
    assert g.dtype in (torch.bfloat16, torch.float32), "g must be in bfloat16 or float32."
    if initial_state is not None and cu_seqlens is None:
        assert initial_state.shape[0] == q.shape[0], "one initial state per batch entry is expected."
    assert_blackwell(q.device)
    _poll_status(q.device)

    if scale is None:
        scale = k.shape[-1] ** -0.5
    # the intermediates are worth keeping only if a backward pass can follow; grad mode has to be read here,
    # inside autograd.Function.forward it is always off
    keep = bool(disable_recompute) and torch.is_grad_enabled() and any(
        t is not None and t.requires_grad for t in (q, k, v, g, beta, A_log, dt_bias, initial_state))
    return ChunkKDAFunction.apply(q, k, v, g, beta, A_log, dt_bias, scale, initial_state, output_final_state,
                                  use_qk_l2norm_in_kernel, use_gate_in_kernel, cu_seqlens, cu_seqlens_cpu, safe_gate,
                                  lower_bound, disable_recompute, return_intermediate_states, keep,
                                  bool(use_beta_sigmoid_in_kernel))
