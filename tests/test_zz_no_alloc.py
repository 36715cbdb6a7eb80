"""The allocation-free forward entry point ``fqla_fwd_noalloc`` against the ordinary entry points.

Who needs it: a host that cannot allocate device memory at the point where it calls the library,
for example a serving engine whose arena already owns the device (a later ``cudaMalloc`` there
stalls every stream or fails) or a plugin that only gets raw pointers and a stream.  The entry
point keeps the forward's two intermediates in a fixed array inside the library, so this test
passes nothing but inputs and outputs, calls it twice in a row on different problems (the second
call finds the first call's leftovers in the array), and compares with ``fqla_kkt_solve`` +
``fqla_fwd_seq`` fed by caller-owned buffers.

This file sorts after the other test files on purpose, so a run that stops at the first failure
has already been through everything else.
"""

import pytest
import torch

from oracle import gdr_oracle as orc

pytestmark = pytest.mark.gpu

TOL_FWD = 5e-3  # normalised error bound of the forward outputs used throughout the GPU tests
DEV = "cuda"


def _inputs(T, Hq, Hv, seed, cu=None):
    cu_t = None if cu is None else torch.tensor(cu, dtype=torch.int32)
    x = orc.make_inputs(1, T, Hq, Hv, 128, 128, seed, cu_seqlens=cu_t, with_h0=True)
    d = {n: x[n].to(DEV) for n in ("g", "h0")}
    for n in ("q", "k", "v", "beta"):
        d[n] = x[n].bfloat16().to(DEV)
    d["cu"] = None if cu_t is None else cu_t.to(DEV)
    return d


def _existing_entry_points(d, scale):
    from flashqla_b200 import ops

    g_cum, A = ops.kkt_solve(d["k"], d["beta"], d["g"], d["cu"], raw_gate=True)
    res = ops.fwd_seq(d["q"], d["k"], d["v"], A, g_cum, d["beta"], scale, d["h0"],
                      output_final_state=True, cu_seqlens=d["cu"])
    return res["o"], res["ht"]


def _noalloc(d, scale):
    from flashqla_b200 import _lib, ops

    B, T, Hq, D = d["k"].shape
    Hv = d["v"].shape[2]
    tb = ops.SeqTables(B, T, d["cu"])  # index tables are inputs: built before the call
    o = torch.full_like(d["v"], float("nan"))  # outputs are the caller's, pre-poisoned
    ht = torch.full((tb.N, Hv, D, D), float("nan"), dtype=torch.float32, device=DEV)
    p = lambda t: None if t is None else t.data_ptr()  # noqa: E731
    st = _lib.load().fqla_fwd_noalloc(
        p(d["q"]), p(d["k"]), p(d["v"]), p(d["g"]), p(d["beta"]), 0, p(d["h0"]), p(ht), p(o),
        B, T, Hq, Hv, D, scale, p(tb.cu), p(tb.chunk_offsets), p(tb.chunk_indices), tb.is64,
        tb.N, tb.num_chunks, torch.cuda.current_stream().cuda_stream)
    return st, o, ht


def test_noalloc_forward_matches_existing_entry_points_twice_in_a_row():
    scale = 128 ** -0.5
    problems = [
        _inputs(1024, 2, 4, seed=301),                          # fixed length, GVA
        _inputs(777, 2, 2, seed=302, cu=[0, 130, 131, 640]),    # packed, ragged, rows past the end
    ]
    for i, d in enumerate(problems):
        o_ref, ht_ref = _existing_entry_points(d, scale)
        st, o, ht = _noalloc(d, scale)
        assert st == 0, f"call {i}: status {st}"
        torch.cuda.synchronize()
        assert torch.isfinite(o.float()).all() and torch.isfinite(ht).all()
        e_o, e_h = orc.rel_err(o.float(), o_ref.float()), orc.rel_err(ht, ht_ref)
        print(f"call {i}: o {e_o:.2e} ht {e_h:.2e}")
        assert e_o <= TOL_FWD and e_h <= TOL_FWD


def test_noalloc_rejects_problems_beyond_its_fixed_array():
    from flashqla_b200 import _lib

    lib = _lib.load()
    limit = lib.fqla_fwd_noalloc_max_pairs()
    assert limit == 32768
    d = _inputs(64, 1, 1, seed=303)
    d_big = dict(d)
    B, T, Hq, D = 1, limit + 64, 1, 128  # one value head: T alone exceeds the limit
    one = d["q"].data_ptr()  # never dereferenced: the size check comes before any launch
    st = lib.fqla_fwd_noalloc(one, one, one, one, one, 0, None, None, one, B, T, Hq, 1, D,
                              128 ** -0.5, None, None, None, 0, B, 0,
                              torch.cuda.current_stream().cuda_stream)
    assert st == -3
    assert b"scratch" in lib.fqla_status_string(st)
    del d_big
