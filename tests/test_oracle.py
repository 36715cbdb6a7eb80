"""The CPU oracle against the golden vectors produced by the reference's own code, and the
three statements of the operator against each other.  CPU only."""

import numpy as np
import pytest
import torch

from golden_util import CASES, GOLDEN_DIR, load_case
from oracle import gdr_oracle as orc

TIGHT = 2e-5  # fp64 oracle vs fp32-stored fp64 reference output


@pytest.mark.parametrize("name", CASES)
def test_chunk_fwd_matches_reference_golden(name):
    x, ref = load_case(name)
    d = {n: x[n].double() for n in ("q", "k", "v", "g", "beta", "h0")}
    g_cum, A, o, h, ht = orc.chunk_gdr_fwd(
        d["q"], d["k"], d["v"], d["g"], d["beta"], x["scale"], d["h0"], x["cu_seqlens"]
    )
    assert orc.rel_err(g_cum, ref["g_cum"]) < TIGHT
    assert orc.rel_err(A, ref["A"]) < TIGHT
    assert orc.rel_err(o, ref["o"]) < TIGHT
    assert orc.rel_err(h, ref["h"]) < TIGHT
    assert orc.rel_err(ht, ref["ht"]) < TIGHT


@pytest.mark.parametrize("name", CASES)
def test_chunk_bwd_matches_reference_golden(name):
    x, ref = load_case(name)
    d = {n: x[n].double() for n in ("q", "k", "v", "g", "beta", "h0", "do", "dht")}
    grads = orc.chunk_gdr_bwd(
        d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], d["dht"], x["scale"], d["h0"],
        x["cu_seqlens"],
    )
    for got, n in zip(grads, ("dq", "dk", "dv", "db", "dg", "dh0")):
        assert orc.rel_err(got, ref[n]) < TIGHT, n


@pytest.mark.parametrize("name", ["varlen_gva_d128", "hardgate_d128"])
def test_recurrence_matches_reference_golden(name):
    x, ref = load_case(name)
    d = {n: x[n].double() for n in ("q", "k", "v", "g", "beta", "h0")}
    o, ht = orc.recurrent_gdr(
        d["q"], d["k"], d["v"], d["g"], d["beta"], x["scale"], d["h0"], x["cu_seqlens"]
    )
    assert orc.rel_err(o, ref["o"]) < TIGHT
    assert orc.rel_err(ht, ref["ht"]) < TIGHT


def test_cumsum_reverse_and_tail():
    g = torch.arange(1, 201, dtype=torch.float64).reshape(1, 200, 1)
    cu = torch.tensor([0, 70, 200])
    f = orc.chunk_local_cumsum(g, cu)
    r = orc.chunk_local_cumsum(g, cu, reverse=True)
    assert f[0, 63, 0] == sum(range(1, 65)) and f[0, 64, 0] == 65 and f[0, 70, 0] == 71
    assert r[0, 64, 0] == sum(range(65, 71)) and r[0, 69, 0] == 70
    # prefix + suffix - self = chunk total, on every row of a chunk
    assert torch.all((f + r - g)[0, :64, 0] == f[0, 63, 0])


def test_known_answers():
    # beta = 0: nothing is written, the state only decays and o reads the decayed h0.
    x = orc.make_inputs(1, 96, 1, 1, 16, 16, seed=3, dtype=torch.float64, round_to=None)
    beta0 = torch.zeros_like(x["beta"])
    _, A, o, _, ht = orc.chunk_gdr_fwd(x["q"], x["k"], x["v"], x["g"], beta0, None, x["h0"])
    eye_rows = torch.eye(64, dtype=torch.float64)[torch.arange(96) % 64]
    assert torch.allclose(A[0, :, 0], eye_rows)
    total = x["g"].sum(1)[0, 0].exp()
    assert torch.allclose(ht[0, 0], x["h0"][0, 0] * total)
    # g = 0, beta = 1, orthonormal keys: the delta rule overwrites, so reading key t back
    # after the sequence returns v_t exactly.
    K = 16
    k = torch.eye(K, dtype=torch.float64).reshape(1, K, 1, K)
    v = torch.randn(1, K, 1, 8, dtype=torch.float64)
    z, one = torch.zeros(1, K, 1, dtype=torch.float64), torch.ones(1, K, 1, dtype=torch.float64)
    _, _, _, _, ht = orc.chunk_gdr_fwd(k, k, v, z, one, 1.0, None)
    assert torch.allclose(ht[0, 0], v[0, :, 0])


def test_index_tables_match_reference_golden():
    from flashqla_b200.utils import prepare_chunk_indices, prepare_chunk_offsets

    z = np.load(GOLDEN_DIR + "/index_tables.npz")
    for name in ("idx_a", "idx_b", "idx_c", "idx_d"):
        for dtype in (torch.int32, torch.int64):
            cu = torch.from_numpy(z[name + "_cu"]).to(dtype)
            idx = prepare_chunk_indices(cu, 64)
            offs, total = prepare_chunk_offsets(cu, 64)
            assert idx.dtype == dtype and offs.dtype == dtype
            assert np.array_equal(idx.numpy(), z[name + "_indices"])
            assert np.array_equal(offs.numpy(), z[name + "_offsets"])
            assert total == int(z[name + "_total"])
    assert prepare_chunk_indices(torch.tensor([0, 100, 356, 512]), 64).tolist() == [
        [0, 0], [0, 1], [1, 0], [1, 1], [1, 2], [1, 3], [2, 0], [2, 1], [2, 2]]


def test_reference_copy_reproduces_its_golden_vectors_when_present():
    """Where ``oracle/_ref`` holds the reference's own ``tests/ref_gdr.py`` (the file the CPU
    baseline of the benchmark times), it must reproduce the committed golden vectors, which were
    generated from that same file."""
    from oracle import ref_loader

    if not ref_loader.available():
        pytest.skip("oracle/_ref is not populated on this machine")
    ref = ref_loader.load()
    for name in CASES:
        x, want = load_case(name)
        d = {n: x[n].double() for n in ("q", "k", "v", "g", "beta", "h0", "do", "dht")}
        g, o, A, h, ht = ref.chunk_gated_delta_rule_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"],
                                                        x["cu_seqlens"], d["h0"], x["scale"])
        assert orc.rel_err(o, want["o"]) < TIGHT and orc.rel_err(ht, want["ht"]) < TIGHT
        grads = ref.chunk_gated_delta_rule_bwd(d["q"], d["k"], d["v"], g, d["beta"], A, x["scale"],
                                               d["h0"], d["do"], d["dht"], x["cu_seqlens"])
        for got, n in zip(grads, ("dq", "dk", "dv", "db", "dg", "dh0")):
            assert orc.rel_err(got, want[n]) < TIGHT, (name, n)
