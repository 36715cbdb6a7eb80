"""Import the reference's own ``tests/ref_gdr.py`` from ``oracle/_ref/`` (see
``oracle/build_ref.py``).  TEST INFRASTRUCTURE ONLY.

``ref_gdr.py`` does ``from flash_qla.utils import ...``.  Importing the reference *package*
needs TileLang and a GPU, and this repository ships a drop-in package of the same name, so the
five helpers are served from the two copied helper files through a stand-in module that exists
only while ``ref_gdr.py`` is being imported.  The reference's memo decorator insists on a CUDA
runtime; the undecorated functions are plain torch and are what is exposed.
"""

from __future__ import annotations

import importlib.util
import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")


def available() -> bool:
    return all(os.path.exists(os.path.join(REF_DIR, f)) for f in ("ref_gdr.py", "pack.py", "index.py"))


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


_cached = None


def load():
    """Returns the imported ``ref_gdr`` module (the reference's code), or raises if absent."""
    global _cached
    if _cached is not None:
        return _cached
    if not available():
        raise FileNotFoundError(f"{REF_DIR} is not populated: run oracle/build_ref.py")
    pack = _load(os.path.join(REF_DIR, "pack.py"), "_fqla_ref_pack")
    try:
        index = _load(os.path.join(REF_DIR, "index.py"), "_fqla_ref_index")
        offsets = getattr(index.prepare_chunk_offsets, "__wrapped__", index.prepare_chunk_offsets)
    except Exception:  # the file imports tilelang at the top; its function is four torch lines
        import torch

        def offsets(cu_seqlens, chunk_size):
            n = (torch.diff(cu_seqlens) + chunk_size - 1) // chunk_size
            out = torch.zeros_like(cu_seqlens)
            out[1:] = torch.cumsum(n, dim=0)
            return out, out[-1].item()
    stub_pkg, stub = types.ModuleType("flash_qla"), types.ModuleType("flash_qla.utils")
    for name in ("pad_and_reshape", "pack", "unpack", "fill_last_chunk_of_g"):
        setattr(stub, name, getattr(pack, name))
    stub.prepare_chunk_offsets = offsets
    stub_pkg.utils = stub
    saved = {n: sys.modules.get(n) for n in ("flash_qla", "flash_qla.utils")}
    sys.modules["flash_qla"], sys.modules["flash_qla.utils"] = stub_pkg, stub
    try:
        _cached = _load(os.path.join(REF_DIR, "ref_gdr.py"), "_fqla_ref_gdr")
    finally:
        for n, m in saved.items():
            if m is None:
                sys.modules.pop(n, None)
            else:
                sys.modules[n] = m
    return _cached
