"""Generate the golden vectors in this folder from the reference's own code.

Run once, in a container that has the reference checkout (it is not needed afterwards):

    python tests/golden/make_golden.py /path/to/reference

What runs is the reference's unmodified pure-PyTorch implementation
(``tests/ref_gdr.py``), on CPU in float64, fed through the reference's own
``flash_qla/utils/pack.py`` and ``flash_qla/utils/index.py`` helpers loaded by file path
(importing the reference *package* needs a GPU, these two files do not).  Inputs come from
``oracle.gdr_oracle.make_inputs`` and are stored with the outputs, so the tests never depend
on a random-number generator reproducing them.
"""

from __future__ import annotations

import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle.gdr_oracle import make_inputs  # noqa: E402

CASES = {
    # name: (B, T, Hq, Hv, K, V, cu_seqlens, seed, gate)
    "fixed_d64": (1, 256, 4, 4, 64, 64, None, 11, "logsigmoid"),
    "varlen_gva_d128": (1, 200, 1, 2, 128, 128, [0, 70, 200], 12, "logsigmoid"),
    "hardgate_d128": (2, 192, 2, 2, 128, 128, None, 13, "hard"),
}

INDEX_CASES = {
    "idx_a": [0, 100, 356, 512],
    "idx_b": [0, 47, 128],
    "idx_c": [0, 64, 64, 200, 1024],
    "idx_d": [0, 211, 985],
}


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def load_reference(ref_root):
    """Expose the reference's pack/index helpers as ``flash_qla.utils`` and import its oracle."""
    pack = _load(os.path.join(ref_root, "flash_qla/utils/pack.py"), "_ref_pack")
    index = _load(os.path.join(ref_root, "flash_qla/utils/index.py"), "_ref_index")
    # The reference's memo asserts a CUDA runtime; the undecorated functions are plain torch.
    chunk_offsets = index.prepare_chunk_offsets.__wrapped__
    chunk_indices_raw = index.prepare_chunk_indices.__wrapped__
    index.prepare_lens = index.prepare_lens.__wrapped__  # used inside prepare_chunk_indices
    pkg, utils = types.ModuleType("flash_qla"), types.ModuleType("flash_qla.utils")
    for name in ("pad_and_reshape", "pack", "unpack", "fill_last_chunk_of_g"):
        setattr(utils, name, getattr(pack, name))
    utils.prepare_chunk_offsets = chunk_offsets
    pkg.utils = utils
    saved = {m: sys.modules.get(m) for m in ("flash_qla", "flash_qla.utils")}
    sys.modules["flash_qla"], sys.modules["flash_qla.utils"] = pkg, utils
    try:
        ref = _load(os.path.join(ref_root, "tests/ref_gdr.py"), "_ref_gdr")
    finally:
        for m, old in saved.items():
            if old is None:
                sys.modules.pop(m, None)
            else:
                sys.modules[m] = old
    return ref, chunk_indices_raw, chunk_offsets


def bf16_bits(x):
    return x.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def main(ref_root):
    ref, chunk_indices, chunk_offsets = load_reference(ref_root)
    for name, (B, T, Hq, Hv, K, V, cu, seed, gate) in CASES.items():
        cu_t = None if cu is None else torch.tensor(cu, dtype=torch.int32)
        x = make_inputs(B, T, Hq, Hv, K, V, seed, cu_seqlens=cu_t, gate=gate)
        d = {n: (t.double() if t is not None else None) for n, t in x.items()}
        scale = K ** -0.5
        g_cum, o, A, h, ht = ref.chunk_gated_delta_rule_fwd(
            q=d["q"], k=d["k"], v=d["v"], g=d["g"].clone(), beta=d["beta"],
            cu_seqlens=cu_t, initial_state=d["h0"], scale=scale, chunk_size=64,
        )
        dq, dk, dv, db, dg, dh0 = ref.chunk_gated_delta_rule_bwd(
            d["q"], d["k"], d["v"], g_cum, d["beta"], A, scale, d["h0"], d["do"].clone(),
            d["dht"], cu_t, chunk_size=64,
        )
        out = dict(
            q_bf16=bf16_bits(x["q"]), k_bf16=bf16_bits(x["k"]), v_bf16=bf16_bits(x["v"]),
            beta_bf16=bf16_bits(x["beta"]), do_bf16=bf16_bits(x["do"]),
            g=x["g"].numpy(), h0=x["h0"].numpy(), dht=x["dht"].numpy(),
            cu_seqlens=np.array([] if cu is None else cu, dtype=np.int32),
            scale=np.float64(scale),
        )
        for n, t in dict(g_cum=g_cum, o=o, A=A, h=h, ht=ht, dq=dq, dk=dk, dv=dv, db=db,
                         dg=dg, dh0=dh0).items():
            out["ref_" + n] = t.float().numpy()
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
        print(name, {n: a.shape for n, a in out.items() if n.startswith("ref_")})
    idx = {}
    for name, cu in INDEX_CASES.items():
        cu_t = torch.tensor(cu, dtype=torch.int32)
        idx[name + "_cu"] = np.array(cu, dtype=np.int32)
        idx[name + "_indices"] = chunk_indices(cu_t, 64).numpy()
        offs, total = chunk_offsets(cu_t, 64)
        idx[name + "_offsets"] = offs.numpy()
        idx[name + "_total"] = np.int64(total)
    np.savez_compressed(os.path.join(HERE, "index_tables.npz"), **idx)
    print("index tables", sorted(idx))


if __name__ == "__main__":
    main(sys.argv[1])
