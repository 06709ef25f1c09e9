"""cula_kda_fwd_noalloc: the forward pass for callers that cannot allocate device memory (a runtime whose pool
already owns all of it, a plugin under a foreign memory manager). Called straight through the C ABI and checked
against the ordinary entry points; collected last so that a failure here cannot hide other results."""
import pytest
import torch

from oracle.naive_kda import err_ratio, make_inputs

pytestmark = pytest.mark.gpu


def _call_noalloc(d, o, ht, status, B, T, H, h0=None):
    from cula_b200 import _native
    lib = _native.lib()
    nchunks = B * ((T + 63) // 64)
    return lib.cula_kda_fwd_noalloc(
        d["q"].data_ptr(), d["k"].data_ptr(), d["v"].data_ptr(), d["g"].data_ptr(), 0, d["beta"].data_ptr(), 0,
        d["A_log"].data_ptr(), d["dt_bias"].data_ptr(), None if h0 is None else h0.data_ptr(), o.data_ptr(),
        ht.data_ptr(), None, None, None, nchunks, B, T, H, 128 ** -0.5, 1, 2, -5.0, status.data_ptr(),
        torch.cuda.current_stream().cuda_stream)


def test_noalloc_forward_matches_regular_entry_points_twice_in_a_row():
    from cula_b200.kda import chunk_kda
    outs = []
    for call, (B, T, H, seed) in enumerate([(1, 200, 4, 0), (2, 130, 3, 1)]):      # two calls in a row, different shapes
        inp = make_inputs(B, T, H, seed=seed, gate_offset=-6.0, h0_std=0.5)
        d = {k: v.cuda() for k, v in inp.items()}
        o = torch.empty(B, T, H, 128, dtype=torch.bfloat16, device="cuda")
        ht = torch.empty(B, H, 128, 128, dtype=torch.float32, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        rc = _call_noalloc(d, o, ht, status, B, T, H, h0=d["initial_state"])
        assert rc == 0, rc
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        o_ref, ht_ref = chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], A_log=d["A_log"], dt_bias=d["dt_bias"],
                                  initial_state=d["initial_state"], output_final_state=True,
                                  use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, safe_gate=True, lower_bound=-5.0)
        torch.cuda.synchronize()
        # same kernels, same inputs: the forward tolerances of tests/test_kda_fwd.py are met with room to spare
        assert err_ratio(o_ref.float().cpu(), o.float().cpu()) <= 5e-3
        assert float((o_ref.float() - o.float()).abs().max()) <= 2e-2
        assert err_ratio(ht_ref.cpu(), ht.cpu()) <= 1e-3
        outs.append((o, ht))
    assert outs[0][0].shape != outs[1][0].shape


def test_noalloc_refuses_problems_beyond_its_capacity():
    from cula_b200 import _native
    lib = _native.lib()
    assert lib.cula_kda_noalloc_max_tiles() == 256
    B, T, H = 1, 64 * 33, 8                         # 33 chunks x 8 heads = 264 tiles > 256
    x = torch.zeros(B, T, H, 128, dtype=torch.bfloat16, device="cuda")
    beta = torch.zeros(B, T, H, dtype=torch.bfloat16, device="cuda")
    a_log, bias = torch.zeros(H, device="cuda"), torch.zeros(H * 128, device="cuda")
    o, ht = torch.empty_like(x), torch.empty(B, H, 128, 128, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.cula_kda_fwd_noalloc(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), 0, beta.data_ptr(), 0,
                                  a_log.data_ptr(), bias.data_ptr(), None, o.data_ptr(), ht.data_ptr(), None, None, None,
                                  33, B, T, H, 0.0884, 1, 2, -5.0, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == -3
    assert b"capacity" in lib.cula_kda_strerror(rc)


def test_noalloc_allocates_nothing_and_handles_a_packed_batch():
    """The property the entry point exists for: a warmed-up call changes neither the device's free memory nor
    torch's allocator state. Done on a packed (varlen) batch whose index tables come from the C-side builder."""
    import numpy as np
    from cula_b200 import _native
    from cula_b200.kda import chunk_kda
    lib = _native.lib()
    lens = [70, 1, 129, 64]
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)
    N, T, H = len(lens), int(cu[-1]), 2
    num_chunks = lib.cula_kda_num_chunks(cu.data_ptr(), N)
    idx, off, order = (torch.empty(num_chunks, 2, dtype=torch.int32), torch.empty(N + 1, dtype=torch.int32),
                       torch.empty(N, dtype=torch.int32))
    assert lib.cula_kda_build_chunk_tables(cu.data_ptr(), N, idx.data_ptr(), off.data_ptr(), order.data_ptr()) == 0
    inp = make_inputs(1, T, H, seed=3, gate_offset=-7.0)
    d = {k: v.cuda() for k, v in inp.items() if v is not None}
    h0 = torch.randn(N, H, 128, 128, generator=torch.Generator().manual_seed(4)).cuda()
    cu_d, idx_d, off_d = cu.cuda(), idx.cuda(), off.cuda()
    o = torch.zeros(1, T, H, 128, dtype=torch.bfloat16, device="cuda")
    ht = torch.empty(N, H, 128, 128, dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    def call():
        return lib.cula_kda_fwd_noalloc(
            d["q"].data_ptr(), d["k"].data_ptr(), d["v"].data_ptr(), d["g"].data_ptr(), 0, d["beta"].data_ptr(), 0,
            d["A_log"].data_ptr(), d["dt_bias"].data_ptr(), h0.data_ptr(), o.data_ptr(), ht.data_ptr(), cu_d.data_ptr(),
            idx_d.data_ptr(), off_d.data_ptr(), num_chunks, N, T, H, 128 ** -0.5, 1, 2, -5.0, status.data_ptr(), stream)

    assert call() == 0                       # warm-up: resolves the address of the built-in array on this device
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    allocated_before, reserved_before = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    for _ in range(3):
        assert call() == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert (torch.cuda.memory_allocated(), torch.cuda.memory_reserved()) == (allocated_before, reserved_before)
    assert int(status.item()) == 0
    o_ref, ht_ref = chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], A_log=d["A_log"], dt_bias=d["dt_bias"],
                              initial_state=h0, output_final_state=True, cu_seqlens=cu_d, use_qk_l2norm_in_kernel=True,
                              use_gate_in_kernel=True, safe_gate=True, lower_bound=-5.0)
    torch.cuda.synchronize()
    assert err_ratio(o_ref.float().cpu(), o.float().cpu()) <= 5e-3 and err_ratio(ht_ref.cpu(), ht.cpu()) <= 1e-3
