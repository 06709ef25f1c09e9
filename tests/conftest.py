import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")
GOLDEN_CASES = ["strong_gate_T130", "weak_gate_T200_h0", "softplus_gate_T96", "pre_gated_T63",
                "varlen_15_70_64_37", "uniform_qkv_masked_gate_T150"]


GDN_GOLDEN_CASES = ["gdn_pre_gated_T150_h0", "gdn_gate_in_kernel_varlen_40_100_65"]


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    """Return (case dict of python scalars, inputs dict of torch tensors, expected dict of fp32 tensors)."""
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))

    def tensor(key):
        a = z[key]
        if key + "_is_bf16" in z and bool(z[key + "_is_bf16"]):
            return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
        return torch.from_numpy(a.copy())

    case = dict(B=int(z["B"]), T=int(z["T"]), H=int(z["H"]), use_l2norm=bool(z["use_l2norm"]),
                use_gate_in_kernel=bool(z["use_gate_in_kernel"]), safe_gate=bool(z["safe_gate"]),
                lower_bound=None if np.isnan(z["lower_bound"]) else float(z["lower_bound"]),
                cu_seqlens=(torch.from_numpy(z["cu_seqlens"].copy()) if z["cu_seqlens"].size else None))
    inputs = {k[3:]: tensor(k) for k in z.files if k.startswith("in_") and not k.endswith("_is_bf16")}
    inputs["do"] = torch.from_numpy(z["do"].view(np.int16).copy()).view(torch.bfloat16)
    inputs["dht"] = torch.from_numpy(z["dht"].copy())
    expected = {k: torch.from_numpy(z[k].copy()) for k in z.files
                if k in ("o", "ht") or (k.startswith("d") and k not in ("do", "dht"))}
    return case, inputs, expected
