"""Host-side helpers for the KDA path: device guard and the varlen index tables."""
from __future__ import annotations

import torch

CHUNK = 64


def assert_blackwell(device=None):
    """Same guard as the reference's ``assert_blackwell`` (cula/utils.py:61-69): the kernels are
    compiled for sm_100a only."""
    if not torch.cuda.is_available():
        raise RuntimeError("cula_b200 needs a CUDA device (B200, sm_100a); there is no CPU fallback.")
    major, _ = torch.cuda.get_device_capability(device)
    if major != 10:
        raise RuntimeError(f"cula_b200 kernels are built for sm_100a; found compute capability {major}.x")


def prepare_chunk_indices(seqlens_cpu, chunk_size=CHUNK):
    """[NT, 2] int32 rows (sequence, chunk inside the sequence), sequence after sequence -- the table
    of fla.ops.utils.index.prepare_chunk_indices (fla/ops/utils/index.py:138-149) used at
    cula/kda/chunk.py:62-64."""
    lens = seqlens_cpu[1:] - seqlens_cpu[:-1]
    n_chunks = (lens + chunk_size - 1) // chunk_size
    seq = torch.repeat_interleave(torch.arange(len(lens), dtype=torch.int64), n_chunks)
    starts = torch.cumsum(n_chunks, 0) - n_chunks
    local = torch.arange(int(n_chunks.sum()), dtype=torch.int64) - torch.repeat_interleave(starts, n_chunks)
    return torch.stack([seq, local], dim=1).to(torch.int32)


def prepare_chunk_offsets(seqlens_cpu, chunk_size=CHUNK):
    """[N+1] int32: first global chunk of every sequence (cula/ops/chunk_delta_h.py:42-47)."""
    lens = seqlens_cpu[1:] - seqlens_cpu[:-1]
    n_chunks = (lens + chunk_size - 1) // chunk_size
    return torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(n_chunks, 0)]).to(torch.int32)


def prepare_uniform_cu_seqlens(batch, seqlen, device=None):
    """cu_seqlens of a fixed-length batch (cula/utils.py:215-218)."""
    return torch.arange(0, (batch + 1) * seqlen, seqlen, dtype=torch.int32, device=device)


class VarlenTables:
    """Device copies of the index tables of one packed batch."""

    def __init__(self, cu_seqlens, cu_seqlens_cpu=None):
        cpu = (cu_seqlens_cpu if cu_seqlens_cpu is not None else cu_seqlens.cpu()).to(torch.int64)
        if cpu.ndim != 1 or cpu.numel() < 1 or int(cpu[0]) != 0 or bool((cpu[1:] < cpu[:-1]).any()):
            raise ValueError("cu_seqlens must be a non-decreasing 1-D tensor starting at 0")
        dev = cu_seqlens.device
        self.n_seqs = cpu.numel() - 1
        self.total_tokens = int(cpu[-1])
        self.cu_seqlens = cu_seqlens.to(torch.int32).contiguous()
        idx = prepare_chunk_indices(cpu)
        self.num_chunks = idx.shape[0]
        self.chunk_indices = idx.contiguous().to(dev)
        self.chunk_offsets = prepare_chunk_offsets(cpu).to(dev)
        lens = cpu[1:] - cpu[:-1]
        # longest sequences first: their CTAs start first and the short ones fill in behind them
        self.seq_order = torch.argsort(lens, descending=True, stable=True).to(torch.int32).to(dev)
        self.seqlens_cpu = cpu


_TABLE_CACHE: list = []      # (source tensor, its version, cu_seqlens_cpu or None, tables), most recent last


def get_varlen_tables(cu_seqlens, cu_seqlens_cpu=None) -> VarlenTables:
    """Tables cached by tensor IDENTITY, as the reference caches its chunk indices (fla's ``tensor_cache``): an entry
    holds a reference to the caller's ``cu_seqlens`` tensor itself, so its address cannot be handed to another tensor
    while the entry lives, and is matched with ``is`` plus the tensor's version counter (an in-place edit
    invalidates it). Avoids a device->host sync on every call."""
    version = cu_seqlens._version
    for i in range(len(_TABLE_CACHE) - 1, -1, -1):
        src, ver, cpu, tab = _TABLE_CACHE[i]
        if src is cu_seqlens and ver == version and (cu_seqlens_cpu is None or cpu is None or cpu is cu_seqlens_cpu
                                                     or torch.equal(cpu, cu_seqlens_cpu)):
            return tab
    tab = VarlenTables(cu_seqlens, cu_seqlens_cpu)
    _TABLE_CACHE.append((cu_seqlens, version, cu_seqlens_cpu, tab))
    if len(_TABLE_CACHE) > 16:
        del _TABLE_CACHE[0]
    return tab
