"""CPU-side checks: index tables, argument validation of chunk_kda, and that the C-ABI library
loads and exports every symbol include/cula_kda.h declares (no compute calls without a GPU)."""
import ctypes
import os
import re

import pytest
import torch

from cula_b200 import _native
from cula_b200.kda import chunk_kda
from cula_b200.utils import VarlenTables, prepare_chunk_indices, prepare_chunk_offsets, prepare_uniform_cu_seqlens

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_chunk_tables():
    cu = torch.tensor([0, 15, 85, 149, 186])
    idx = prepare_chunk_indices(cu)
    assert idx.tolist() == [[0, 0], [1, 0], [1, 1], [2, 0], [3, 0]]
    assert prepare_chunk_offsets(cu).tolist() == [0, 1, 3, 4, 5]
    assert prepare_uniform_cu_seqlens(3, 100).tolist() == [0, 100, 200, 300]
    tab = VarlenTables(cu.to(torch.int32))
    assert tab.n_seqs == 4 and tab.num_chunks == 5 and tab.total_tokens == 186
    assert tab.seq_order.tolist() == [1, 2, 3, 0]


def test_chunk_tables_empty_sequence():
    cu = torch.tensor([0, 64, 64, 70])
    assert prepare_chunk_indices(cu).tolist() == [[0, 0], [2, 0]]
    assert prepare_chunk_offsets(cu).tolist() == [0, 1, 1, 2]


def test_bad_cu_seqlens():
    with pytest.raises(ValueError):
        VarlenTables(torch.tensor([0, 10, 5], dtype=torch.int32))
    with pytest.raises(ValueError):
        VarlenTables(torch.tensor([3, 10], dtype=torch.int32))


def _inputs(B=1, T=8, H=1, dtype=torch.bfloat16):
    q = torch.zeros(B, T, H, 128, dtype=dtype)
    return q, q.clone(), q.clone(), q.clone(), torch.zeros(B, T, H, dtype=dtype)


def test_argument_errors_match_reference():
    q, k, v, g, beta = _inputs(B=2)
    with pytest.raises(ValueError, match="batch size is expected to be 1"):
        chunk_kda(q, k, v, g, beta, cu_seqlens=torch.tensor([0, 8], dtype=torch.int32))
    q, k, v, g, beta = _inputs()
    with pytest.raises(ValueError, match="number of initial states"):
        chunk_kda(q, k, v, g, beta, cu_seqlens=torch.tensor([0, 4, 8], dtype=torch.int32),
                  initial_state=torch.zeros(1, 1, 128, 128))
    with pytest.raises(AssertionError, match="float32"):
        chunk_kda(q, k, v, g, beta, initial_state=torch.zeros(1, 1, 128, 128, dtype=torch.bfloat16))
    with pytest.raises(AssertionError, match="A_log"):
        chunk_kda(q, k, v, g, beta, use_gate_in_kernel=True)
    with pytest.raises(ValueError, match="lower_bound"):
        chunk_kda(q, k, v, g, beta, use_gate_in_kernel=True, safe_gate=True, A_log=torch.zeros(1))
    with pytest.raises(ValueError, match="safe range"):
        chunk_kda(q, k, v, g, beta, use_gate_in_kernel=True, safe_gate=True, lower_bound=-6.0, A_log=torch.zeros(1))
    with pytest.raises(AssertionError, match="bfloat16"):
        chunk_kda(q.float(), k.float(), v.float(), g, beta)
    with pytest.raises(AssertionError, match="beta must be of shape"):
        chunk_kda(q, k, v, g, beta[..., None])
    q64 = torch.zeros(1, 8, 1, 64, dtype=torch.bfloat16)
    with pytest.raises(AssertionError, match="head dim of 128"):
        chunk_kda(q64, q64, q64, q64, beta)


def test_no_cpu_fallback():
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    q, k, v, g, beta = _inputs()
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        chunk_kda(q, k, v, g, beta)


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "cula_kda.h")).read()
    declared = set(re.findall(r"\b(cula_kda_\w+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(_native.SIGNATURES), "binding table and header disagree"
    handle = ctypes.CDLL(_native.LIB_PATH)
    for name in declared:
        assert hasattr(handle, name), name
    assert handle.cula_kda_tile_pack_bytes() == 74240
    _native.lib().cula_kda_strerror.restype = ctypes.c_char_p
    assert b"invalid" in _native.lib().cula_kda_strerror(-1)


def test_header_is_plain_c(tmp_path):
    """include/cula_kda.h is the FFI contract: it must compile as C (no C++ or torch types) and every entry point
    must return int except the string helper."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("gcc is not available")
    src = tmp_path / "use_header.c"
    src.write_text('#include "cula_kda.h"\nint (*probe)(void) = cula_kda_tile_pack_bytes;\nint main(void) { return probe == 0; }\n')
    out = subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", "-fsyntax-only", "-I", os.path.join(ROOT, "include"), str(src)],
                         capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    header = open(os.path.join(ROOT, "include", "cula_kda.h")).read()
    for ret, name in re.findall(r"^(\w[\w\s\*]*?)\s*\b(cula_kda_\w+)\s*\(", header, flags=re.M):
        assert ret.strip() == ("const char*" if name == "cula_kda_strerror" else "int"), (ret, name)


def test_decode_argument_errors_without_gpu():
    from cula_b200.kda import fused_sigmoid_gating_delta_rule_update, kda_decode
    q = torch.zeros(2, 1, 2, 128, dtype=torch.bfloat16)
    v = torch.zeros(2, 1, 2, 128, dtype=torch.bfloat16)
    a, b = torch.zeros(2, 1, 2, 128, dtype=torch.bfloat16), torch.zeros(2, 1, 2, dtype=torch.bfloat16)
    A_log, dt_bias = torch.zeros(2), torch.zeros(2, 128)
    with pytest.raises(NotImplementedError):
        fused_sigmoid_gating_delta_rule_update(A_log, a, dt_bias, 1.0, 20.0, q, q, v, b, None, None, is_kda=False)
    with pytest.raises(ValueError):
        kda_decode(A_log, dt_bias, q, q, v, a, b, torch.zeros(2, 2, 128, 128), None, state_layout="hv")
    with pytest.raises(AssertionError):
        kda_decode(A_log, dt_bias, q.float(), q.float(), v, a, b, torch.zeros(2, 2, 128, 128), None)
    with pytest.raises(RuntimeError):           # valid arguments, but no Blackwell device: the call refuses, no fallback
        kda_decode(A_log, dt_bias, q, q, v, a, b, torch.zeros(2, 2, 128, 128), None)


def test_c_side_chunk_tables_match_the_python_ones():
    lib = _native.lib()
    cases = [[0, 15, 85, 149, 186], [0, 64, 64, 70], [0, 1], [0, 8192, 8255, 8255 + 63]]
    for cu in cases:
        cu_t = torch.tensor(cu, dtype=torch.int32)
        N = len(cu) - 1
        total = lib.cula_kda_num_chunks(cu_t.data_ptr(), N)
        idx_ref = prepare_chunk_indices(cu_t)
        assert total == idx_ref.shape[0]
        idx = torch.empty(max(total, 1), 2, dtype=torch.int32)
        off = torch.empty(N + 1, dtype=torch.int32)
        order = torch.empty(N, dtype=torch.int32)
        assert lib.cula_kda_build_chunk_tables(cu_t.data_ptr(), N, idx.data_ptr(), off.data_ptr(), order.data_ptr()) == 0
        assert idx[:total].tolist() == idx_ref.tolist()
        assert off.tolist() == prepare_chunk_offsets(cu_t).tolist()
        assert order.tolist() == VarlenTables(cu_t).seq_order.tolist()
    bad = torch.tensor([0, 10, 5], dtype=torch.int32)
    assert lib.cula_kda_num_chunks(bad.data_ptr(), 2) < 0
    assert lib.cula_kda_num_chunks(torch.tensor([3, 10], dtype=torch.int32).data_ptr(), 1) < 0


def test_varlen_tables_are_cached_by_identity_not_by_address():
    """Two different int64 cu_seqlens of equal length, one after the other, the first one freed in between: the
    allocator is free to hand the second one the same address, and the tables must still be rebuilt."""
    from cula_b200.utils import get_varlen_tables
    for dtype in (torch.int64, torch.int32):
        a = torch.tensor([0, 100, 300, 1000], dtype=dtype)
        tab_a = get_varlen_tables(a)
        assert get_varlen_tables(a) is tab_a                      # the same tensor: served from the cache
        assert tab_a.num_chunks == 2 + 4 + 11
        addr = a.data_ptr()
        del a
        for _ in range(50):                                       # provoke reuse of the freed address
            b = torch.tensor([0, 64, 128, 1000], dtype=dtype)
            tab_b = get_varlen_tables(b)
            assert tab_b is not tab_a
            assert tab_b.num_chunks == 1 + 1 + 14 and tab_b.chunk_offsets.tolist() == [0, 1, 2, 16]
            if b.data_ptr() == addr:
                break
            del b
    c = torch.tensor([0, 10, 20], dtype=torch.int32)
    tab_c = get_varlen_tables(c)
    c[1] = 15                                                     # an in-place edit bumps the version: rebuilt
    assert get_varlen_tables(c) is not tab_c


def test_cp_context_kwarg_dispatches_to_the_context_parallel_path(monkeypatch):
    """``chunk_kda(..., cp_context=ctx)`` keeps the reference's one-line call (cula/kda/chunk.py:348-355) and hands
    the shard to ``chunk_kda_cp`` with the group the context carries."""
    import cula_b200.kda.cp as cp
    seen = {}

    def fake(q, k, v, g, beta, **kw):
        seen.update(kw)
        return "o", None
    monkeypatch.setattr(cp, "chunk_kda_cp", fake)
    q, k, v, g, beta = _inputs(T=64)
    ctx = cp.KDACPContext(group="the-group", segments=3)
    out = chunk_kda(q, k, v, g, beta, use_gate_in_kernel=True, safe_gate=True, lower_bound=-5.0, A_log=torch.zeros(1),
                    cp_context=ctx)
    assert out == ("o", None)
    assert seen["group"] == "the-group" and seen["segments"] == 3 and seen["lower_bound"] == -5.0 and "A_log" in seen


def test_gate_mode_follows_lower_bound():
    from cula_b200.kda.chunk import GATE_LOWER_BOUND, GATE_NONE, GATE_SOFTPLUS, _gate_mode
    assert _gate_mode(False, True, -5.0) == GATE_NONE
    assert _gate_mode(True, True, -5.0) == GATE_LOWER_BOUND
    assert _gate_mode(True, False, -5.0) == GATE_LOWER_BOUND      # keyed on lower_bound alone, as fla's gate is
    assert _gate_mode(True, False, None) == GATE_SOFTPLUS


def test_noalloc_entry_point_rejects_bad_arguments_without_a_gpu():
    """Argument checks of cula_kda_fwd_noalloc come before any CUDA call: they can be exercised with dummy pointers."""
    lib = _native.lib()
    p = 0x1000          # "aligned" dummy address: never dereferenced, every call below is refused first
    ok = dict(q=p, k=p, v=p, g=p, beta=p, A=p, bias=p, o=p, ht=p, status=p)

    def call(num_chunks=2, N=1, T=128, H=2, gate_mode=2, cu=None, idx=None, off=None, **kw):
        a = dict(ok, **kw)
        return lib.cula_kda_fwd_noalloc(a["q"], a["k"], a["v"], a["g"], 0, a["beta"], 0, a["A"], a["bias"], None, a["o"], a["ht"],
                                        cu, idx, off, num_chunks, N, T, H, 0.0884, 1, gate_mode, -5.0, a["status"], None)
    assert call(q=None) == -1 and call(o=None) == -1 and call(status=None) == -1            # null pointers
    assert call(num_chunks=3) == -1                  # fixed length: num_chunks must be N * ceil(T / 64)
    assert call(gate_mode=5) == -1 and call(A=None) == -1
    assert call(cu=p) == -1                          # packed-batch tables come all three together or not at all
    assert call(num_chunks=200, T=64 * 200, H=2) == -3                                       # 400 tiles > 256
    assert call(q=p + 2) == -2 and call(o=p + 8) == -2                                       # 16-byte alignment
    assert call(num_chunks=0) == 0 and call(N=0) == 0                                        # nothing to do


def test_host_binding_helpers_without_topology_and_with_a_fake_one():
    """bind_host_to_gpu / _prefer_memory_near: nothing changes where the platform exposes no topology (this box: no
    GPU, no NUMA information); with a faked two-node topology the preferred-node policy is requested for the GPU's node
    with MPOL_PREFERRED and a one-bit mask, and a refused call reports None."""
    import os
    import platform
    from cula_b200.kda import host
    before = os.sched_getaffinity(0)
    assert host.bind_host_to_gpu("cuda:0") == sorted(before) and os.sched_getaffinity(0) == before
    assert host._prefer_memory_near("cuda:0") is None
    calls = []
    ok = lambda *a: calls.append(a) or 0
    assert host._prefer_memory_near("cuda:0", _probe=lambda: (0, 1), _syscall=ok) is None and not calls     # one node only
    assert host._prefer_memory_near("cuda:0", _probe=lambda: (-1, 2), _syscall=ok) is None and not calls    # node unknown
    if platform.machine() in ("x86_64", "aarch64"):
        assert host._prefer_memory_near("cuda:0", _probe=lambda: (1, 2), _syscall=ok) == 1
        assert calls == [({"x86_64": 238, "aarch64": 237}[platform.machine()], 1, 0b10, 65)]
        assert host._prefer_memory_near("cuda:0", _probe=lambda: (1, 2), _syscall=lambda *a: -1) is None
