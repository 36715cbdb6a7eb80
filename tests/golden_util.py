"""Loader for the golden vectors in ``tests/golden`` (outputs of the reference's own
pure-PyTorch implementation, see ``tests/golden/make_golden.py``)."""

import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CASES = ["fixed_d64", "varlen_gva_d128", "hardgate_d128"]


def _bf16(bits):
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)


def load_case(name):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    x = {n: _bf16(z[n + "_bf16"]) for n in ("q", "k", "v", "beta", "do")}
    for n in ("g", "h0", "dht"):
        x[n] = torch.from_numpy(z[n])
    cu = z["cu_seqlens"]
    x["cu_seqlens"] = torch.from_numpy(cu.copy()) if cu.size else None
    x["scale"] = float(z["scale"])
    ref = {n[4:]: torch.from_numpy(z[n]) for n in z.files if n.startswith("ref_")}
    return x, ref
