"""Parity of the CUDA path with the fp32 CPU oracle at the benchmark configurations themselves
(their exact shapes, length distributions and seeds) and over the shape matrix of the
reference's own unit tests (``tests/test_gdr_unit.py:37-78`` of the reference: CORE, DEVELOP,
VARLEN, PRODUCT lists, ``state_v_first`` x ``use_h0``), plus repeat-launch determinism of the
backward and the cache-on / cache-off routes of the context-parallel backward
(``tests/test_gdr_unit.py:478-515``, ``:682-773``).

Tolerances: normalised error ||x - ref|| / ||ref|| <= 5e-3 for o, h and the final state,
<= 1e-2 for every gradient.  Every case prints the errors it measured.
"""

import pytest
import torch

import bench
from oracle import gdr_oracle as orc

pytestmark = pytest.mark.gpu

TOL_FWD = 5e-3
TOL_BWD = 1e-2
DEV = "cuda"


def _fq():
    import flashqla_b200 as fq

    return fq


def _cpu32(t):
    return None if t is None else t.detach().float().cpu()


def _bounds(x):
    if x["cu"] is None:
        B, T = x["q"].shape[:2]
        return None, [(b, 0, T) for b in range(B)]
    cu = [int(c) for c in x["cu"].tolist()]
    return cu, [(0, s, e) for s, e in zip(cu[:-1], cu[1:])]


def _oracle_by_sequence(x, want_bwd, heads=None):
    """fp32 CPU oracle, one sequence at a time (bounds the host memory of the autograd graph).
    ``heads``: optional list of value heads (needs Hq == Hv) to restrict the oracle to."""
    c = {n: _cpu32(x[n]) for n in ("q", "k", "v", "g", "beta", "h0", "do", "dht")}
    if heads is not None:
        for n in ("q", "k", "v", "g", "beta", "do"):
            c[n] = c[n][:, :, heads].contiguous()
        for n in ("h0", "dht"):
            c[n] = None if c[n] is None else c[n][:, heads].contiguous()
    _, spans = _bounds(x)
    outs = {n: [] for n in ("o", "ht", "dq", "dk", "dv", "db", "dg", "dh0")}
    for n_seq, (b, s, e) in enumerate(spans):
        sl = lambda t: t[b:b + 1, s:e].contiguous()  # noqa: E731
        h0 = None if c["h0"] is None else c["h0"][n_seq:n_seq + 1]
        if e == s:  # empty sequence: the state passes through, and so does its gradient
            Hv, D = c["v"].shape[2], c["v"].shape[3]
            outs["o"].append(c["v"][b:b + 1, s:e])
            outs["ht"].append(torch.zeros(1, Hv, D, D) if h0 is None else h0)
            if want_bwd:
                for n, src in (("dq", "q"), ("dk", "k"), ("dv", "v"), ("db", "beta"), ("dg", "g")):
                    outs[n].append(c[src][b:b + 1, s:e])
                outs["dh0"].append(c["dht"][n_seq:n_seq + 1])
            continue
        _, _, o, _, ht = orc.chunk_gdr_fwd(sl(c["q"]), sl(c["k"]), sl(c["v"]), sl(c["g"]),
                                           sl(c["beta"]), None, h0)
        outs["o"].append(o)
        outs["ht"].append(ht)
        if want_bwd:
            gr = orc.chunk_gdr_bwd(sl(c["q"]), sl(c["k"]), sl(c["v"]), sl(c["g"]), sl(c["beta"]),
                                   sl(c["do"]), c["dht"][n_seq:n_seq + 1], None, h0)
            for n, t in zip(("dq", "dk", "dv", "db", "dg", "dh0"), gr):
                outs[n].append(t)
    dim = 1 if x["cu"] is not None else 0
    ref = {"o": torch.cat(outs["o"], dim), "ht": torch.cat(outs["ht"], 0)}
    if want_bwd:
        for n in ("dq", "dk", "dv", "db", "dg"):
            ref[n] = torch.cat(outs[n], dim)
        ref["dh0"] = None if c["h0"] is None else torch.cat(outs["dh0"], 0)
    return ref


def _cuda_fwd_bwd(x, want_bwd, auto_cp=True, state_v_first=False, cache=True, output_h=False):
    fq = _fq()
    tr = (lambda t: None if t is None else t.transpose(-1, -2).contiguous()) if state_v_first \
        else (lambda t: t)
    g_cum, A, o, h, ht, cp_cache = fq.chunk_gated_delta_rule_fwd(
        x["q"], x["k"], x["v"], x["g"], x["beta"], None, tr(x["h0"]), x["cu"],
        output_final_state=True, output_h=output_h, auto_cp=auto_cp,
        state_v_first=state_v_first, enable_fwd_cp_cache=cache and want_bwd)
    res = {"o": o, "ht": tr(ht), "h": None if h is None else tr(h)}
    if want_bwd:
        gr = fq.chunk_gated_delta_rule_bwd(
            x["q"], x["k"], x["v"], g_cum, x["beta"], A, x["do"], tr(x["dht"]), None,
            tr(x["h0"]), x["cu"], state_v_first, auto_cp, cp_cache if cache else None)
        res.update(zip(("dq", "dk", "dv", "db", "dg", "dh0"), gr))
        res["dh0"] = tr(res["dh0"])
    torch.cuda.synchronize()
    return res


def _compare(res, ref, what, heads=None):
    errs = {}
    for n, tol in (("o", TOL_FWD), ("ht", TOL_FWD), ("dq", TOL_BWD), ("dk", TOL_BWD),
                   ("dv", TOL_BWD), ("db", TOL_BWD), ("dg", TOL_BWD), ("dh0", TOL_BWD)):
        if ref.get(n) is None:
            continue
        got = res[n].float()
        if heads is not None:
            got = got[:, heads] if n in ("ht", "dh0") else got[:, :, heads]
        if n not in ("ht", "dh0"):
            got = got[:, : ref[n].shape[1]]
        errs[n] = orc.rel_err(got, ref[n])
    print(what, {k: f"{v:.2e}" for k, v in errs.items()})
    for n, e in errs.items():
        assert e <= (TOL_FWD if n in ("o", "ht") else TOL_BWD), f"{what} {n}: {e:.3e}"
    return errs


def _workload(name, **over):
    w = dict(bench.WORKLOADS[name], **over)
    return w, bench.make_batch(w, torch.device(DEV, 0), 1234)


# ---- the benchmark configurations at their own shapes --------------------------------------------

def test_config1_forward_full_size_vs_oracle():
    """B=4, T=8192, Hq=Hv=16, no initial state: the default bench workload, as the bench runs it
    (the planner splits every sequence into segments)."""
    from flashqla_b200 import cp
    from flashqla_b200.ops import SeqTables

    w, x = _workload("c1_fwd")
    assert cp.plan_segments(SeqTables(4, 8192, None), 16, device=x["q"].device) is not None
    ref = _oracle_by_sequence(x, want_bwd=False)
    _compare(_cuda_fwd_bwd(x, False, auto_cp=True), ref, "c1 split")
    _compare(_cuda_fwd_bwd(x, False, auto_cp=False), ref, "c1 unsplit")


def test_config2_forward_64_packed_sequences_with_initial_states():
    w, x = _workload("c2_fwd")
    assert x["cu"].numel() == 65 and x["h0"].shape[0] == 64
    ref = _oracle_by_sequence(x, want_bwd=False)
    _compare(_cuda_fwd_bwd(x, False), ref, "c2")


def test_config3_forward_backward_gva_lognormal_lengths():
    """32768 packed tokens, log-normal document lengths, Hq=16 / Hv=32: o, final state and all
    six gradients, with the forward's cache handed to the backward and without it."""
    w, x = _workload("c3_fwdbwd")
    assert int(x["cu"][-1]) == 32768
    ref = _oracle_by_sequence(x, want_bwd=True)
    _compare(_cuda_fwd_bwd(x, True, cache=True), ref, "c3 cache")
    _compare(_cuda_fwd_bwd(x, True, cache=False), ref, "c3 no cache")


def test_config4_long_sequence_forward_two_heads_vs_oracle():
    """1 x 262144 tokens, H=8 (4096 chunks, split into segments by the planner): the oracle walks
    the whole sequence for two of the heads; o over all tokens and the final state are compared."""
    w, x = _workload("c4_fwd")
    heads = [0, 5]
    ref = _oracle_by_sequence(x, want_bwd=False, heads=heads)
    res = _cuda_fwd_bwd(x, False, auto_cp=True)
    _compare(res, ref, "c4 fwd heads 0,5", heads=heads)
    # window by window, so that a local defect cannot hide in the norm over 262144 tokens
    worst = 0.0
    for t0 in range(0, 262144, 4096):
        got = res["o"][:, t0:t0 + 4096][:, :, heads].float()
        worst = max(worst, orc.rel_err(got, ref["o"][:, t0:t0 + 4096]))
    print(f"c4 worst 4096-token window: {worst:.2e}")
    assert worst <= TOL_FWD


def test_config4_prefix_forward_backward_with_context_parallel_split():
    """Backward of the long-sequence configuration on its first 32768 tokens (8 heads), split
    into segments by the planner in both directions."""
    from flashqla_b200 import cp
    from flashqla_b200.ops import SeqTables

    w, x = _workload("c4_fwdbwd", T=32768)
    assert cp.plan_segments(SeqTables(1, 32768, None), 8, is_bwd=True,
                            device=x["q"].device) is not None
    ref = _oracle_by_sequence(x, want_bwd=True)
    ref["dh0"] = None  # the workload has no initial state
    _compare(_cuda_fwd_bwd(x, True), ref, "c4 prefix fwd+bwd")


# ---- the reference unit tests' shape matrix ---------------------------------------------------------

# (id, B, T, Hq, Hv, varlen, cu)   -- reference tests/test_gdr_unit.py:37-78
CORE = [
    ("B1-T4096-H4", 1, 4096, 4, 4, False, None),
    ("B1-T4096-H8G2", 1, 4096, 2, 8, False, None),
    ("B1-T4096-H16G4", 1, 4096, 4, 16, False, None),
    ("B3-T4096-H4-varlen", 3, 4096, 4, 4, True, None),
    ("B1-T4096-H32G16-varlen", 1, 4096, 16, 32, True, [0, 410, 841, 1135, 2126, 2512, 4096]),
    ("B1-T1000-H64G16-padding", 1, 1000, 16, 64, True, [0, 211, 985]),
]
EXTENDED = [
    ("dev-H4", 1, 32768, 4, 4, False, None),
    ("dev-H8", 1, 32768, 8, 8, False, None),
    ("dev-H16", 1, 32768, 16, 16, False, None),
    ("varlen-B11-T33", 11, 33, 4, 4, True, None),
    ("varlen-B7-T4321", 7, 4321, 4, 4, True, None),
    ("varlen-B3-T16789", 3, 16789, 4, 4, True, None),
    ("varlen-B5-T8192", 5, 8192, 4, 4, True, None),
    ("varlen-B10-T1024", 10, 1024, 4, 4, True, None),
    ("varlen-B20-T512", 20, 512, 4, 4, True, None),
    ("prod-mixed-small", 1, 128, 4, 4, True, [0, 47, 128]),
    ("prod-mixed-segs", 1, 4096, 4, 4, True, [0, 517, 883, 1010, 3767, 4096]),
    ("prod-mixed-large", 1, 16384, 4, 4, True, [0, 4096, 6893, 7665, 8192, 12288, 16384]),
    ("prod-mixed-pad", 1, 256, 4, 4, True, [0, 73, 115, 209]),
]


def _matrix_inputs(B, T, Hq, Hv, varlen, cu, use_h0, seed=42):
    """Inputs in the style of the reference's ``_make_inputs``: the per-head ``-A softplus`` gate
    with one decay-free and one extreme-decay head; random-length packing when ``varlen`` has no
    explicit boundaries (``B`` lengths drawn from [1, T))."""
    if varlen and cu is None:
        gen = torch.Generator().manual_seed(seed)
        lens = torch.randint(1, T, (B,), generator=gen).tolist()
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        B, T = 1, cu[-1]
    cu_t = None if cu is None else torch.tensor(cu, dtype=torch.int32)
    raw = orc.make_inputs(B, T, Hq, Hv, 128, 128, seed, cu_seqlens=cu_t, with_h0=use_h0,
                          gate="hard")
    x = {n: raw[n].bfloat16().to(DEV) for n in ("q", "k", "v", "do")}
    x["beta"] = raw["beta"].to(DEV)  # fp32 beta, as the reference's tests pass it
    x["g"] = raw["g"].to(DEV)
    x["h0"] = None if raw["h0"] is None else raw["h0"].to(DEV)
    x["dht"] = raw["dht"].to(DEV)
    x["cu"] = None if cu_t is None else cu_t.to(DEV)
    return x


@pytest.mark.parametrize("use_h0", [False, True], ids=["no_h0", "h0"])
@pytest.mark.parametrize("case", CORE, ids=[c[0] for c in CORE])
def test_core_matrix_forward_backward_both_state_layouts(case, use_h0):
    name, B, T, Hq, Hv, varlen, cu = case
    x = _matrix_inputs(B, T, Hq, Hv, varlen, cu, use_h0)
    ref = _oracle_by_sequence(x, want_bwd=True)
    for svf in (False, True):
        res = _cuda_fwd_bwd(x, True, state_v_first=svf)
        if not use_h0:
            assert res["dh0"] is None
        _compare(res, ref, f"{name} h0={use_h0} v_first={svf}")


@pytest.mark.parametrize("case", EXTENDED, ids=[c[0] for c in EXTENDED])
def test_extended_matrix_forward_backward(case):
    name, B, T, Hq, Hv, varlen, cu = case
    x = _matrix_inputs(B, T, Hq, Hv, varlen, cu, use_h0=True)
    ref = _oracle_by_sequence(x, want_bwd=True)
    _compare(_cuda_fwd_bwd(x, True), ref, name)


def test_per_chunk_states_output_at_core_shape():
    """``output_h=True``: the state entering every chunk (bf16), both state layouts."""
    x = _matrix_inputs(1, 4096, 2, 8, False, None, True)
    c = {n: _cpu32(x[n]) for n in ("q", "k", "v", "g", "beta", "h0")}
    _, _, _, h_ref, _ = orc.chunk_gdr_fwd(c["q"], c["k"], c["v"], c["g"], c["beta"], None, c["h0"])
    for svf in (False, True):
        h = _cuda_fwd_bwd(x, False, state_v_first=svf, output_h=True)["h"]
        e = orc.rel_err(h.float(), h_ref)
        print(f"h v_first={svf}: {e:.2e}")
        assert e <= TOL_FWD


# ---- context-parallel split: packed batches with uneven segment counts ------------------------------

CP_CASES = [
    # id, B, T, Hq, Hv, cu
    ("packed_with_empty_seq_hv1", 1, 3700, 1, 1, [0, 2100, 2100, 3700]),
    ("packed_with_empty_seq_hv2", 1, 3700, 1, 2, [0, 2100, 2100, 3700]),
    ("fixed_b2_ragged_tail", 2, 1100, 1, 2, None),
]


@pytest.mark.parametrize("case", CP_CASES, ids=[c[0] for c in CP_CASES])
def test_split_plan_packed_and_batched_cache_on_and_off(case):
    """Segment tables of a split plan with several raw sequences (first/last segment lookups,
    keep flags, an empty sequence in the middle, T not a chunk multiple): forward and backward
    with h0 and dht against the oracle, through the autograd entry (forward cache on) and through
    the direct backward call without the cache."""
    from flashqla_b200 import cp
    from flashqla_b200.ops import SeqTables

    name, B, T, Hq, Hv, cu = case
    cu_t = None if cu is None else torch.tensor(cu, dtype=torch.int32)
    raw = orc.make_inputs(B, T, Hq, Hv, 128, 128, seed=77, cu_seqlens=cu_t, with_h0=True)
    x = {n: raw[n].bfloat16().to(DEV) for n in ("q", "k", "v", "beta", "do")}
    x.update(g=raw["g"].to(DEV), h0=raw["h0"].to(DEV), dht=raw["dht"].to(DEV),
             cu=None if cu_t is None else cu_t.to(DEV))
    plan = cp.plan_segments(SeqTables(B, T, x["cu"]), Hv, device=x["q"].device)
    assert plan is not None and plan.n_seg > (B if cu is None else len(cu) - 1)
    ref = _oracle_by_sequence(x, want_bwd=True)
    # cache off: direct calls
    _compare(_cuda_fwd_bwd(x, True, cache=False), ref, f"{name} cache off")
    # cache on: the autograd entry point
    fq = _fq()
    leaves = {n: x[n].clone().requires_grad_(True) for n in ("q", "k", "v", "g", "beta", "h0")}
    o, ht = fq.chunk_gated_delta_rule(leaves["q"], leaves["k"], leaves["v"], leaves["g"],
                                      leaves["beta"], initial_state=leaves["h0"],
                                      output_final_state=True, cu_seqlens=x["cu"])
    (o.float() * x["do"].float()).sum().add((ht * x["dht"]).sum()).backward()
    res = dict(o=o, ht=ht, dq=leaves["q"].grad, dk=leaves["k"].grad, dv=leaves["v"].grad,
               db=leaves["beta"].grad, dg=leaves["g"].grad, dh0=leaves["h0"].grad)
    _compare(res, ref, f"{name} cache on (autograd)")


# ---- determinism --------------------------------------------------------------------------------------

DETERMINISM = [
    ("fixed-H8G2", 1, 4096, 2, 8, False, None),
    ("varlen-H4", 3, 4096, 4, 4, True, None),
    ("batch32-H4G2", 32, 1024, 2, 4, False, None),
]


@pytest.mark.parametrize("case", DETERMINISM, ids=[c[0] for c in DETERMINISM])
def test_forward_and_backward_repeat_bit_identically(case):
    """Reductions are accumulated in registers in a fixed order and nothing uses atomics on
    data, so repeated launches must agree bit for bit (the reference's determinism tests only
    demand agreement within tolerance over 1000 launches)."""
    name, B, T, Hq, Hv, varlen, cu = case
    x = _matrix_inputs(B, T, Hq, Hv, varlen, cu, use_h0=True)
    first = _cuda_fwd_bwd(x, True)
    for i in range(20):
        again = _cuda_fwd_bwd(x, True, cache=(i % 2 == 0))
        for n in ("o", "ht", "dq", "dk", "dv", "db", "dg", "dh0"):
            assert torch.equal(first[n], again[n]), f"{name}: {n} differs on repeat {i}"
