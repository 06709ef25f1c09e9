"""The C ABI from a host program written in plain C (tests/c_host/forward_from_c.c): compiled with gcc against
include/cula_kda.h and the CUDA runtime, run as its own process, compared with the oracle. No Python, torch or
ctypes sits between the program and the library, which is the point of the boundary."""
import os
import shutil
import subprocess

import numpy as np
import pytest
import torch

from cula_b200 import _native
from oracle import c_oracle
from oracle.naive_kda import err_ratio, make_inputs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _compile(out):
    gcc = shutil.which("gcc")
    if gcc is None or not os.path.exists(os.path.join(CUDA, "include", "cuda_runtime_api.h")):
        pytest.skip("gcc or the CUDA runtime headers are not available")
    lib_dir = os.path.dirname(_native.LIB_PATH)
    cmd = [gcc, "-std=c99", "-O1", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA, "include"),
           os.path.join(ROOT, "tests", "c_host", "forward_from_c.c"), "-o", out, "-L", lib_dir, "-lcula_kda",
           "-L", os.path.join(CUDA, "lib64"), "-lcudart", f"-Wl,-rpath,{lib_dir}", f"-Wl,-rpath,{os.path.join(CUDA, 'lib64')}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return out


def test_c_host_program_builds(tmp_path):
    """Links against the built library on any machine with gcc and the CUDA runtime (no GPU needed to link)."""
    _native.lib()
    _compile(str(tmp_path / "forward_from_c"))


@pytest.mark.gpu
def test_c_host_program_matches_oracle(tmp_path):
    _native.lib()
    exe = _compile(str(tmp_path / "forward_from_c"))
    B, T, H = 2, 200, 3                                  # ragged last chunk
    inp = make_inputs(B, T, H, seed=8, gate_offset=-6.0, h0_std=0.5)
    raw = lambda t: t.contiguous().view(torch.int16).numpy() if t.dtype == torch.bfloat16 else t.contiguous().numpy()
    for name, key in (("q", "q"), ("k", "k"), ("v", "v"), ("g", "g"), ("beta", "beta"), ("A_log", "A_log"),
                      ("dt_bias", "dt_bias"), ("h0", "initial_state")):
        raw(inp[key]).tofile(str(tmp_path / f"{name}.bin"))
    res = subprocess.run([exe, str(tmp_path), str(B), str(T), str(H)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "C_HOST_OK" in res.stdout, res.stdout + res.stderr
    o = torch.from_numpy(np.fromfile(str(tmp_path / "o.bin"), dtype=np.int16)).view(torch.bfloat16).view(B, T, H, 128)
    ht = torch.from_numpy(np.fromfile(str(tmp_path / "ht.bin"), dtype=np.float32)).view(B, H, 128, 128)
    f = lambda x: x.float().numpy()
    o_ref, ht_ref = c_oracle.naive_kda_fwd(f(inp["q"]), f(inp["k"]), f(inp["v"]), f(inp["g"]), f(inp["beta"]), f(inp["A_log"]),
                                           f(inp["dt_bias"]), f(inp["initial_state"]), use_l2norm=True, gate_mode=2,
                                           lower_bound=-5.0)
    assert err_ratio(torch.from_numpy(o_ref), o.float()) <= 5e-3
    assert float((torch.from_numpy(o_ref) - o.float()).abs().max()) <= 2e-2
    assert err_ratio(torch.from_numpy(ht_ref), ht) <= 2e-3


@pytest.mark.gpu
def test_c_host_program_packed_batch(tmp_path):
    """The same program on a packed batch: index tables from cula_kda_build_chunk_tables, per-sequence states."""
    _native.lib()
    exe = _compile(str(tmp_path / "forward_from_c"))
    lens, H = [15, 70, 64, 37, 130], 2
    T, N = sum(lens), len(lens)
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    inp = make_inputs(1, T, H, seed=9, gate_offset=-6.0)
    h0 = 0.5 * torch.randn(N, H, 128, 128, generator=torch.Generator().manual_seed(1))
    raw = lambda t: t.contiguous().view(torch.int16).numpy() if t.dtype == torch.bfloat16 else t.contiguous().numpy()
    for name, t in (("q", inp["q"]), ("k", inp["k"]), ("v", inp["v"]), ("g", inp["g"]), ("beta", inp["beta"]),
                    ("A_log", inp["A_log"]), ("dt_bias", inp["dt_bias"]), ("h0", h0), ("cu_seqlens", cu)):
        raw(t).tofile(str(tmp_path / f"{name}.bin"))
    res = subprocess.run([exe, str(tmp_path), "1", str(T), str(H)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "C_HOST_OK" in res.stdout, res.stdout + res.stderr
    o = torch.from_numpy(np.fromfile(str(tmp_path / "o.bin"), dtype=np.int16)).view(torch.bfloat16).view(1, T, H, 128)
    ht = torch.from_numpy(np.fromfile(str(tmp_path / "ht.bin"), dtype=np.float32)).view(N, H, 128, 128)
    f = lambda x: x.float().numpy()
    o_ref, ht_ref = c_oracle.naive_kda_fwd(f(inp["q"]), f(inp["k"]), f(inp["v"]), f(inp["g"]), f(inp["beta"]), f(inp["A_log"]),
                                           f(inp["dt_bias"]), f(h0), cu_seqlens=cu.numpy(), use_l2norm=True, gate_mode=2,
                                           lower_bound=-5.0)
    assert err_ratio(torch.from_numpy(o_ref), o.float()) <= 5e-3
    assert err_ratio(torch.from_numpy(ht_ref), ht) <= 2e-3
