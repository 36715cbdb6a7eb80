"""Kernel-level checks through the C ABI: the two implementations of each K = V = 128 kernel
(tcgen05 and mma.sync) against each other, the operand-tile hand-off against the row-major one,
and the small context-parallel kernels against host restatements."""

import os
import subprocess
import sys

import pytest
import torch

from oracle import gdr_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _inputs(T, Hq, Hv, seed, cu=None):
    cu_t = None if cu is None else torch.tensor(cu, dtype=torch.int32)
    x = orc.make_inputs(1, T, Hq, Hv, 128, 128, seed=seed, cu_seqlens=cu_t, with_h0=True)
    d = {n: t.to(DEV) for n, t in x.items()}
    for n in ("q", "k", "v", "beta", "do"):
        d[n] = d[n].bfloat16()
    d["cu_seqlens"] = None if cu_t is None else cu_t.to(DEV)
    return d


def _prep(d):
    from flashqla_b200 import ops

    cu = d.get("cu_seqlens")
    tables = ops.SeqTables(1, d["k"].shape[1], cu)
    g_cum = ops.chunk_local_cumsum(d["g"], 64, cu)
    A = ops.kkt_solve(d["k"], d["beta"], g_cum, cu)
    return tables, g_cum, A


@pytest.mark.parametrize("cu", [None, [0, 130, 130, 777, 1000]], ids=["fixed", "varlen"])
def test_operand_tiles_equal_row_major_outputs(cu):
    """h, v_new, dh, du written as operand tiles (TMA stores) hold exactly the values of the
    row-major outputs, transposed per chunk."""
    from flashqla_b200 import ops

    T = 1000 if cu is not None else 1024
    d = _inputs(T, 2, 4, seed=31, cu=cu)
    tables, g_cum, A = _prep(d)
    scale = 128 ** -0.5
    kw = dict(output_o=False, output_h=True, output_vnew=True, tables=tables)
    row = ops.fwd_seq(None, d["k"], d["v"], A, g_cum, d["beta"], scale, d["h0"], **kw)
    til = ops.fwd_seq(None, d["k"], d["v"], A, g_cum, d["beta"], scale, d["h0"], operand_tiles=True, **kw)
    assert torch.equal(til["h"].transpose(-1, -2), row["h"])
    brow = ops.bwd_dh(d["q"], d["k"], A, g_cum, d["beta"], d["do"], scale, d["dht"], tables=tables)
    btil = ops.bwd_dh(d["q"], d["k"], A, g_cum, d["beta"], d["do"], scale, d["dht"], tables=tables,
                      operand_tiles=True)
    assert torch.equal(btil["dh"].transpose(-1, -2), brow["dh"])
    assert torch.equal(btil["dh0"], brow["dh0"])
    # per chunk: tile[c, h, v, t] == row-major[token bos + 64 c' + t, h, v]; columns past the
    # sequence end are zero
    bounds = cu if cu is not None else [0, T]
    c = 0
    for bos, eos in zip(bounds[:-1], bounds[1:]):
        for t0 in range(bos, eos, 64):
            n = min(64, eos - t0)
            for name, tl, rw in (("vnew", til["vnew"], row["vnew"]), ("du", btil["du"], brow["du"])):
                got = tl[c].transpose(-1, -2)  # [Hv, 64, V]
                want = rw[0, t0:t0 + n].transpose(0, 1)
                assert torch.equal(got[:, :n], want), (name, c)
                assert not got[:, n:].any(), (name, c)
            c += 1
    assert c == tables.num_chunks
    # the chunk-parallel kernel gives the same gradients from either layout
    a = ops.bwd_main(d["q"], d["k"], d["v"], row["vnew"], A, g_cum, d["beta"], d["do"], brow["du"],
                     row["h"], brow["dh"], scale, tables=tables)
    b = ops.bwd_main(d["q"], d["k"], d["v"], til["vnew"], A, g_cum, d["beta"], d["do"], btil["du"],
                     til["h"], btil["dh"], scale, tables=tables, operand_tiles=True)
    total = tables.total
    for x, y, name in zip(a, b, ("dq", "dk", "dv", "db", "dg")):
        assert orc.rel_err(y[:, :total].float(), x[:, :total].float()) < 1e-5, name


_CHILD = r"""
import sys, torch
sys.path.insert(0, {root!r})
from oracle import gdr_oracle as orc
import flashqla_b200 as fq
cu = torch.tensor([0, 130, 130, 777, 1000], dtype=torch.int32)
x = orc.make_inputs(1, 1000, 2, 4, 128, 128, seed=77, cu_seqlens=cu, with_h0=True)
d = {{n: t.cuda() for n, t in x.items()}}
for n in ("q", "k", "v", "beta", "do"):
    d[n] = d[n].bfloat16()
cu = cu.cuda()
g_cum, A, o, h, ht, _ = fq.chunk_gated_delta_rule_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], None,
                                                      d["h0"], cu, output_h=True)
grads = fq.chunk_gated_delta_rule_bwd(d["q"], d["k"], d["v"], g_cum, d["beta"], A, d["do"], d["dht"],
                                      None, d["h0"], cu)
torch.save([t.cpu() for t in (o, h, ht, *grads)], sys.argv[1])
"""


def test_tcgen05_kernels_match_mma_sync_kernels(tmp_path):
    """The whole forward + backward with the tcgen05 kernels against the same run with every
    K = V = 128 kernel forced to its mma.sync implementation (separate process: the switch is
    read once per process)."""
    outs = []
    for force in (False, True):
        env = dict(os.environ)
        env.pop("FQLA_FORCE_MMA_SYNC", None)
        if force:
            env["FQLA_FORCE_MMA_SYNC"] = "1"
        path = str(tmp_path / f"out_{int(force)}.pt")
        subprocess.run([sys.executable, "-c", _CHILD.format(root=ROOT), path], check=True, env=env,
                       timeout=600)
        outs.append(torch.load(path))
    names = ("o", "h", "ht", "dq", "dk", "dv", "db", "dg", "dh0")
    for name, a, b in zip(names, *outs):
        tol = 5e-3 if name in ("o", "h", "ht") else 1e-2
        assert orc.rel_err(a.float(), b.float()) < tol, name


def test_warmup_scan_against_host_loop():
    from flashqla_b200 import ops

    torch.manual_seed(5)
    T, Hv = 64 * 37 + 11, 6
    # per-token log gates chosen so that some (segment, head) pairs cross the threshold early,
    # some late, some never
    g = -torch.rand(1, T, Hv) * torch.tensor([0.5, 0.05, 0.005, 0.0005, 0.2, 0.0])
    seg = [0, 64 * 5, 64 * 5, 64 * 20, 64 * 36, T]
    seg_cu = torch.tensor(seg, dtype=torch.int32)
    g_cum = orc.chunk_local_cumsum(g, seg_cu)
    keep = torch.tensor([1, 1, 0, 1, 1], dtype=torch.int32)
    for from_start in (False, True):
        warm, fb = ops.warmup_scan(g_cum.to(DEV), seg_cu.to(DEV), -10.0, from_start, keep.to(DEV))
        warm, fb = warm.cpu(), fb.cpu()
        for s, (b, e) in enumerate(zip(seg[:-1], seg[1:])):
            n_chunks = (e - b + 63) // 64
            ends = [min(e, b + 64 * (c + 1)) - 1 for c in range(n_chunks)]
            order = ends if from_start else ends[::-1]
            for h in range(Hv):
                if keep[s] == 0:
                    assert warm[s, h] == 0 and fb[s, h] == 0
                    continue
                acc, n, reached = 0.0, 0, False
                for r in order:
                    acc += float(g_cum[0, r, h])
                    n += 1
                    if acc < -10.0:
                        reached = True
                        break
                # summation order differs (warp prefix sum): allow the crossing chunk to move by
                # one only when the running sum is within rounding of the threshold
                assert abs(int(warm[s, h]) - n) <= (1 if abs(acc + 10.0) < 1e-3 else 0), (s, h)
                if int(warm[s, h]) == n:
                    assert int(fb[s, h]) == (0 if reached else 1)


def test_merge_states_against_host_chain():
    from flashqla_b200 import ops

    torch.manual_seed(6)
    n_seg, Hv, D = 7, 3, 128
    seg_begin = torch.tensor([0, 3, 3, 7], dtype=torch.int32)  # raw sequences of 3, 0 and 4 segments
    local = torch.randn(n_seg, Hv, D, D)
    M = torch.randn(n_seg, Hv, D, D) * 0.05
    use = (torch.rand(n_seg, Hv) > 0.4).int()
    raw = torch.randn(3, Hv, D, D)
    for reverse in (False, True):
        out = ops.merge_states(local.to(DEV), M.to(DEV), use.to(DEV), raw.to(DEV), seg_begin.to(DEV),
                               reverse=reverse).cpu()
        for r in range(3):
            s0, s1 = int(seg_begin[r]), int(seg_begin[r + 1])
            idx = list(range(s0, s1))[::-1] if reverse else list(range(s0, s1))
            cur = raw[r].clone()
            for j, i in enumerate(idx):
                assert orc.rel_err(out[i], cur) < 1e-5, (reverse, r, i)
                m = M[i].transpose(-1, -2) if reverse else M[i]
                cur = local[i] + use[i].view(Hv, 1, 1) * (m @ cur)
        # the same inputs as views into the records of one buffer (what an all-gather leaves),
        # flags stored as the numbers 0.0 / 1.0 and read as bits: the same result, bit for bit
        n = Hv * D * D
        rows = torch.full((n_seg, 3 * n + Hv), float("nan"), device=DEV)
        rows[:, :n] = local.to(DEV).reshape(n_seg, n)
        rows[:, n:2 * n] = M.to(DEV).reshape(n_seg, n)
        rows[:, 3 * n:] = use.to(DEV).float()
        strided = ops.merge_states(rows[:, :n].unflatten(1, (Hv, D, D)),
                                   rows[:, n:2 * n].unflatten(1, (Hv, D, D)),
                                   rows[:, 3 * n:].view(torch.int32), raw.to(DEV),
                                   seg_begin.to(DEV), reverse=reverse).cpu()
        assert torch.equal(strided, out)


@pytest.mark.parametrize("cu", [None, [0, 130, 130, 777, 1000]], ids=["fixed", "varlen"])
def test_kkt_solve_with_fused_cumsum(cu):
    """kkt_solve fed with the raw gate forms the chunk-local cumsum itself: same g_cum as the
    cumsum kernel (up to the order of the fp32 additions) and the same A."""
    from flashqla_b200 import ops

    T = 1024 if cu is None else 1000
    d = _inputs(T, 2, 4, seed=41, cu=cu)
    cu_t = d["cu_seqlens"]
    g_ref = ops.chunk_local_cumsum(d["g"], 64, cu_t)
    A_ref = ops.kkt_solve(d["k"], d["beta"], g_ref, cu_t)
    g_cum, A = ops.kkt_solve(d["k"], d["beta"], d["g"], cu_t, raw_gate=True)
    assert orc.rel_err(g_cum, g_ref) < 1e-6
    assert orc.rel_err(A.float(), A_ref.float()) < 1e-3
    want = orc.chunk_local_cumsum(d["g"].cpu(), None if cu_t is None else cu_t.cpu())
    assert orc.rel_err(g_cum.cpu(), want) < 1e-6


@pytest.mark.parametrize("cu,T", [(None, 1024), ([0, 130, 130, 777, 1000], 1000), (None, 16384)],
                         ids=["fixed", "varlen", "segmented"])
def test_forward_cache_tiles_replace_the_recomputation(cu, T):
    """With the forward cache on, the forward keeps the state entering every chunk and v_new as
    operand tiles; they equal what the backward's own state-only pass produces, and the backward
    returns the same gradients with or without them."""
    import flashqla_b200 as fq
    import flash_qla.ops.gated_delta_rule.chunk as api
    from flashqla_b200 import ops

    d = _inputs(T, 2, 4, seed=47, cu=cu)
    cu_t = d["cu_seqlens"]
    g_cum, A, o, _, ht, cache = fq.chunk_gated_delta_rule_fwd(
        d["q"], d["k"], d["v"], d["g"], d["beta"], None, d["h0"], cu_t, output_final_state=True,
        enable_fwd_cp_cache=True)
    assert cache is not None and cache[1] is not None and cache[2] is not None
    if T >= 16384:
        assert cache[0] is not None  # long sequence: split into segments, initial states kept too
    _, _, o2, _, ht2, none = fq.chunk_gated_delta_rule_fwd(
        d["q"], d["k"], d["v"], d["g"], d["beta"], None, d["h0"], cu_t, output_final_state=True)
    assert none is None
    assert torch.equal(o, o2) and torch.equal(ht, ht2)
    args = (d["q"], d["k"], d["v"], g_cum, d["beta"], A, d["do"], d["dht"], None, d["h0"], cu_t)
    with_tiles = fq.chunk_gated_delta_rule_bwd(*args, cp_cache=cache)
    recomputed = fq.chunk_gated_delta_rule_bwd(*args, cp_cache=(cache[0], None, None, cache[3]))
    for x, y, name in zip(with_tiles, recomputed, ("dq", "dk", "dv", "db", "dg", "dh0")):
        assert torch.equal(x, y), name
    # the switch turns the tiles off again
    api.SAVE_STATE_TILES = False
    try:
        cache_off = fq.chunk_gated_delta_rule_fwd(
            d["q"], d["k"], d["v"], d["g"], d["beta"], None, d["h0"], cu_t,
            enable_fwd_cp_cache=True)[5]
    finally:
        api.SAVE_STATE_TILES = True
    assert cache_off is None or cache_off[1] is None


def test_bounded_wait_runs_out_and_reports_through_the_status_word():
    """The failure path every tcgen05 kernel shares: a wait whose barrier nobody arrives at gives
    up after its budget, the kernel returns by itself, the device status word reads 1 until it is
    reset, and the launches that follow are unaffected (bit-identical to the ones before)."""
    import ctypes

    from flashqla_b200 import _lib, ops

    lib = _lib.load()
    d = _inputs(256, 1, 2, seed=61)
    scale = 128 ** -0.5
    g_cum, A = ops.kkt_solve(d["k"], d["beta"], d["g"], None, raw_gate=True)
    run = lambda: ops.fwd_seq(d["q"], d["k"], d["v"], A, g_cum, d["beta"], scale, d["h0"],  # noqa: E731
                              output_final_state=True)
    before = run()
    torch.cuda.synchronize()
    status = ctypes.c_int(-1)
    assert lib.fqla_device_status(ctypes.byref(status), 0) == 0 and status.value == 0
    assert lib.fqla_selftest_wait_timeout(3, torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()  # the kernel comes back by itself after about 3 ms
    assert lib.fqla_device_status(ctypes.byref(status), 1) == 0 and status.value == 1
    assert lib.fqla_device_status(ctypes.byref(status), 0) == 0 and status.value == 0
    after = run()
    torch.cuda.synchronize()
    assert torch.equal(before["o"], after["o"]) and torch.equal(before["ht"], after["ht"])
    assert lib.fqla_selftest_wait_timeout(0, None) == -1


def test_float16_inputs_are_accepted_and_computed_in_bfloat16():
    import flashqla_b200 as fq

    d = _inputs(320, 2, 4, seed=62)
    o_bf, ht_bf = fq.chunk_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["beta"],
                                            initial_state=d["h0"], output_final_state=True)
    h = {n: d[n].to(torch.float16) for n in ("q", "k", "v")}  # bf16 values are exact in fp16 here
    o_h, ht_h = fq.chunk_gated_delta_rule(h["q"], h["k"], h["v"], d["g"], d["beta"],
                                          initial_state=d["h0"], output_final_state=True)
    assert o_h.dtype == torch.float16
    assert orc.rel_err(o_h.float(), o_bf.float()) < 2e-3 and orc.rel_err(ht_h, ht_bf) < 1e-6


@pytest.mark.parametrize("gate", ["logsigmoid", "weak"])
def test_segment_scan_matches_per_segment_scan_and_decides_lead_in(gate):
    """The one-launch scan of a split plan: same warm / fallback as the per-segment scan, and the
    lead-in decision per (sequence, head) restated on the host."""
    from flashqla_b200 import cp, ops

    cu = [0, 2100, 2100, 3700, 5000]
    cu_t = torch.tensor(cu, dtype=torch.int32)
    x = orc.make_inputs(1, cu[-1], 1, 4, 128, 128, seed=71, cu_seqlens=cu_t, gate=gate)
    g_cum = ops.chunk_local_cumsum(x["g"].to(DEV), 64, cu_t.to(DEV))
    plan = cp.plan_segments(ops.SeqTables(1, cu[-1], cu_t.to(DEV)), 4, device=torch.device(DEV, 0))
    assert plan is not None
    begin = plan.seg_begin.tolist()
    for from_start, keep in ((False, plan.keep_fwd), (True, plan.keep_bwd)):
        w_old, f_old = ops.warmup_scan(g_cum, plan.seg_tables.cu, cp.THRESHOLD, from_start, keep)
        warm, fb, lead, exact, any_fb = ops.segment_scan(g_cum, plan.seg_tables.cu,
                                                         plan.seg_begin, cp.THRESHOLD, from_start)
        torch.cuda.synchronize()
        assert torch.equal(warm, w_old) and torch.equal(fb, f_old)
        warm, fb, lead, exact, any_fb = (t.cpu() for t in (warm, fb, lead, exact, any_fb))
        if gate == "weak":
            assert int(any_fb.sum()) > 0  # the gate-free heads never reach the threshold
        for r, (s0, s1) in enumerate(zip(begin[:-1], begin[1:])):
            for hv in range(4):
                a = int(fb[s0:s1, hv].sum() > 0)
                assert int(any_fb[r, hv]) == a
                for s in range(s0, s1):
                    giver = s + 1 if from_start else s - 1
                    has = giver < s1 if from_start else giver >= s0
                    assert int(lead[s, hv]) == (int(warm[giver, hv]) if has and not a else 0)
                    assert int(exact[s, hv]) == (int(warm[s, hv]) if a else -1)
                    if has and not a:
                        assert int(lead[s, hv]) >= 1


def test_lead_in_forward_agrees_with_explicit_start_states():
    """The recurrence kernel that starts a segment a few chunks early from zero against the same
    kernel fed by the separate state-only pass and merge chain: same truncation of the past, so
    the results agree far inside the forward tolerance (the state copy is rounded at different
    points, so not bit for bit)."""
    import flashqla_b200 as fq
    from flashqla_b200 import cp

    d = _inputs(64 * 70 + 13, 2, 4, seed=72)
    run = lambda: fq.chunk_gated_delta_rule_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], None,  # noqa: E731
                                                d["h0"], None, output_final_state=True)
    assert cp.LEAD_IN
    _, _, o_lead, _, ht_lead, _ = run()
    cp.LEAD_IN = False
    try:
        _, _, o_sep, _, ht_sep, _ = run()
    finally:
        cp.LEAD_IN = True
    assert orc.rel_err(o_lead.float(), o_sep.float()) < 2e-3
    assert orc.rel_err(ht_lead, ht_sep) < 2e-3


@pytest.mark.parametrize("case", ["one_sequence", "packed_ragged"])
def test_lead_out_backward_agrees_with_explicit_end_gradients(case):
    """The reverse recurrence kernel that starts a segment a few chunks late from a zero gradient
    against the same kernel fed by the separate dh0-only pass and the transposed merge chain, and
    both against the fp32 oracle.  The ragged case ends every sequence in a partial chunk, which
    a lead-out may have to walk first."""
    import flashqla_b200 as fq
    from flashqla_b200 import cp

    if case == "one_sequence":
        d = _inputs(64 * 70 + 13, 2, 4, seed=74)
        cu = None
    else:
        d = _inputs(64 * 40 + 5 + 64 * 17 + 30 + 64 * 9 + 1, 2, 4, seed=75,
                    cu=[0, 64 * 40 + 5, 64 * 57 + 35, 64 * 66 + 36])
        cu = d["cu_seqlens"]

    def run():
        g_cum, A, _, _, _, cache = fq.chunk_gated_delta_rule_fwd(
            d["q"], d["k"], d["v"], d["g"], d["beta"], None, d["h0"], cu,
            output_final_state=True)
        return fq.chunk_gated_delta_rule_bwd(d["q"], d["k"], d["v"], g_cum, d["beta"], A, d["do"],
                                             d["dht"], None, d["h0"], cu, cp_cache=cache)

    from flashqla_b200 import ops

    tb = ops.SeqTables(1, d["k"].shape[1], cu)
    plan = cp.plan_segments(tb, 4, device=d["k"].device)
    assert plan is not None and plan.n_seg > tb.N
    assert cp.LEAD_IN
    lead = run()
    cp.LEAD_IN = False
    try:
        sep = run()
    finally:
        cp.LEAD_IN = True
    for a, b, name in zip(lead, sep, ("dq", "dk", "dv", "db", "dg", "dh0")):
        assert orc.rel_err(a.float(), b.float()) < 3e-3, name
    want = orc.chunk_gdr_bwd(d["q"].float().cpu(), d["k"].float().cpu(), d["v"].float().cpu(),
                             d["g"].cpu(), d["beta"].float().cpu(), d["do"].float().cpu(),
                             d["dht"].cpu(), None, d["h0"].cpu(),
                             None if cu is None else cu.cpu())
    for a, b, name in zip(lead, want, ("dq", "dk", "dv", "db", "dg", "dh0")):
        assert orc.rel_err(a.float().cpu(), b) < 1e-2, name


@pytest.mark.parametrize("tiles", [False, True], ids=["row_major", "operand_tiles"])
def test_lead_out_over_a_partial_last_chunk_is_exact(tiles):
    """A lead-out that covers ALL rows after the segment, the partial last chunk of the sequence
    included, from a zero end gradient is no approximation: the segment's dh, du and dh0 must be
    the bits of the unsplit walk."""
    from flashqla_b200 import ops

    T = 64 * 10 + 30
    d = _inputs(T, 2, 4, seed=76)
    _, g_cum, A = _prep(d)
    scale = 128 ** -0.5
    full = ops.bwd_dh(d["q"], d["k"], A, g_cum, d["beta"], d["do"], scale, None,
                      tables=ops.SeqTables(1, T, None), operand_tiles=tiles)
    seg_cu = torch.tensor([0, 640, T], dtype=torch.int32, device=DEV)
    lead = torch.tensor([[1] * 4, [0] * 4], dtype=torch.int32, device=DEV)
    # a non-zero gradient offered to the leading segment must be ignored
    dht = torch.ones(2, 4, 128, 128, device=DEV)
    dht[1] = 0
    part = ops.bwd_dh(d["q"], d["k"], A, g_cum, d["beta"], d["do"], scale, dht,
                      tables=ops.SeqTables(1, T, seg_cu), operand_tiles=tiles, lead_chunks=lead)
    torch.cuda.synchronize()
    assert torch.equal(part["dh"], full["dh"])
    assert torch.equal(part["dh0"][0], full["dh0"][0])
    if tiles:
        assert torch.equal(part["du"], full["du"])
    else:
        assert torch.equal(part["du"][:, :T], full["du"][:, :T])


@pytest.mark.parametrize("dtype,D", [(torch.bfloat16, 128), (torch.float16, 96),
                                     (torch.float32, 64), (torch.bfloat16, 322)])
def test_l2norm_kernels_against_torch(dtype, D):
    """The one-pass L2-normalisation kernels against the reference's expressions
    (``flash_qla/utils/math.py:9-51``) evaluated with torch ops in fp32."""
    from flashqla_b200.utils import l2norm_bwd, l2norm_fwd

    gen = torch.Generator(device=DEV).manual_seed(5)
    x = torch.randn(3, 37, 5, D, device=DEV, generator=gen).to(dtype)
    dy = torch.randn(3, 37, 5, D, device=DEV, generator=gen).to(dtype)
    y, rstd = l2norm_fwd(x)
    assert y.dtype == dtype and y.shape == x.shape
    assert rstd.dtype == torch.float32 and rstd.shape == x.shape[:-1]
    xf = x.float()
    rstd_ref = torch.rsqrt((xf * xf).sum(-1, keepdim=True) + 1e-6)
    assert orc.rel_err(rstd, rstd_ref.squeeze(-1)) < 1e-6
    # the product is rounded once to the output dtype, as in the reference
    tol = {torch.float32: 1e-6, torch.float16: 1e-3, torch.bfloat16: 6e-3}[dtype]
    assert orc.rel_err(y.float(), xf * rstd_ref) < tol
    dx = l2norm_bwd(y, rstd, dy)
    assert dx.dtype == torch.float32 and dx.shape == x.shape
    yf, dyf = y.float(), dy.float()
    dx_ref = (dyf - (dyf * yf).sum(-1, keepdim=True) * yf) * rstd.unsqueeze(-1)
    assert orc.rel_err(dx, dx_ref) < 1e-5
    # mixed dtypes: y in the input dtype, the incoming gradient in fp32
    dx32 = l2norm_bwd(y, rstd, dyf)
    assert orc.rel_err(dx32, dx_ref) < 1e-5


def test_two_launches_with_complementary_run_masks_equal_one_launch():
    """``run_mask`` / ``run_value``: a launch walks only the (sequence, head) pairs selected; two
    launches with the two values fill one set of outputs with the bits of a single launch."""
    from flashqla_b200 import ops

    d = _inputs(1500, 2, 4, seed=77, cu=[0, 70, 700, 701, 1100, 1500])
    tables, g_cum, A = _prep(d)
    scale = 128 ** -0.5
    mask = (torch.arange(5 * 4, device=DEV).reshape(5, 4) % 3 == 0).to(torch.int32)
    kw = dict(output_final_state=True, output_h=True, output_vnew=True, tables=tables,
              operand_tiles=True)
    one = ops.fwd_seq(d["q"], d["k"], d["v"], A, g_cum, d["beta"], scale, d["h0"], **kw)
    out = ops.fwd_seq_outputs(d["k"], d["v"], tables, True, True, True, True, False, True)
    for t in out.values():
        t.fill_(float("nan"))
    for value in (1, 0):
        ops.fwd_seq(d["q"], d["k"], d["v"], A, g_cum, d["beta"], scale, d["h0"], run_mask=mask,
                    run_value=value, out=out, **kw)
    for name in ("o", "ht", "h", "vnew"):
        assert torch.equal(out[name][..., :].nan_to_num(0.0), one[name].nan_to_num(0.0)), name
    bone = ops.bwd_dh(d["q"], d["k"], A, g_cum, d["beta"], d["do"], scale, d["dht"], tables=tables,
                      operand_tiles=True)
    bout = ops.bwd_dh_outputs(d["k"], d["do"], tables, operand_tiles=True)
    for value in (0, 1):
        ops.bwd_dh(d["q"], d["k"], A, g_cum, d["beta"], d["do"], scale, d["dht"], tables=tables,
                   operand_tiles=True, run_mask=mask, run_value=value, out=bout)
    for name in ("dh", "du", "dh0"):
        assert torch.equal(bout[name], bone[name]), name


def test_longest_first_block_order_does_not_change_results():
    """Packed batches hand their sequences to the sequential kernels longest first (a block-index
    -> sequence table); the outputs must be the same bits as in index order."""
    from flashqla_b200 import ops

    d = _inputs(1500, 2, 4, seed=73, cu=[0, 70, 700, 701, 1100, 1500])
    tables, g_cum, A = _prep(d)
    assert tables.order is not None and sorted(tables.order.tolist()) == [0, 1, 2, 3, 4]
    assert tables.order.tolist()[0] == 1  # the 630-token sequence goes first
    scale = 128 ** -0.5

    def run(tb):
        fw = ops.fwd_seq(d["q"], d["k"], d["v"], A, g_cum, d["beta"], scale, d["h0"],
                         output_final_state=True, tables=tb)
        bw = ops.bwd_dh(d["q"], d["k"], A, g_cum, d["beta"], d["do"], scale, d["dht"], tables=tb)
        return fw["o"], fw["ht"], bw["dh"], bw["du"], bw["dh0"]

    with_order = run(tables)
    plain = ops.SeqTables(1, 1500, d["cu_seqlens"])
    plain.order = None
    for a, b, name in zip(with_order, run(plain), ("o", "ht", "dh", "du", "dh0")):
        assert torch.equal(a, b), name
