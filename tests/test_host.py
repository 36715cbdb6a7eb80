"""Host-side logic that needs no GPU: the C-ABI library loads and exports everything the header
declares, the segment planner, the memo cache, argument checking, and the autograd signature."""

import ast
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from flashqla_b200 import _lib, build

    build.build_library()
    return _lib.load()


def test_library_exports_every_declared_symbol(lib):
    header = open(os.path.join(ROOT, "include", "fqla.h")).read()
    declared = set(re.findall(r"\b(fqla_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 10
    raw = ctypes.CDLL(os.path.join(ROOT, "flashqla_b200", "libfqla_sm100.so"))
    for name in declared:
        assert hasattr(raw, name), f"{name} declared in include/fqla.h but not exported"
    from flashqla_b200._lib import SIGNATURES

    assert set(SIGNATURES) | {"fqla_version", "fqla_status_string",
                              "fqla_fwd_noalloc_max_pairs"} == declared
    assert lib.fqla_version() >= 3
    assert lib.fqla_status_string(0) == b"ok"
    assert b"invalid" in lib.fqla_status_string(-1)


def test_header_argument_counts_match_binding():
    from flashqla_b200._lib import SIGNATURES

    header = open(os.path.join(ROOT, "include", "fqla.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    for name, argtypes in SIGNATURES.items():
        m = re.search(name + r"\s*\((.*?)\)\s*;", header, flags=re.S)
        assert m, name
        assert len(m.group(1).split(",")) == len(argtypes), name


def test_invalid_arguments_are_rejected_before_any_launch(lib):
    # null pointers / bad head grouping: negative status, no CUDA call needed
    assert lib.fqla_chunk_local_cumsum(None, None, 1, 64, 1, None, 0, 1, None, 1, 0, None) == -1
    assert lib.fqla_group_reduce(None, None, 1, 1, 1, 128, None) == -1
    assert lib.fqla_merge_states(None, None, None, None, None, None, None, 1, 1, 128, 0, 0, None) == -1
    assert lib.fqla_segment_scan(None, 64, 1, None, 0, None, 1, -10.0, 0, None, None, None, None,
                                 None, None) == -1


def test_product_refuses_cpu_tensors():
    import flashqla_b200 as fq
    from flashqla_b200._lib import FqlaError

    q = torch.zeros(1, 64, 1, 128, dtype=torch.bfloat16)
    g = torch.zeros(1, 64, 1)
    with pytest.raises((FqlaError, RuntimeError, AssertionError)):
        fq.chunk_gated_delta_rule_fwd(q, q, q, g, g.bfloat16())


def test_segment_planner_properties():
    from flashqla_b200.cp import split_sequences

    # already saturated: 64 sequences x 8 heads
    assert split_sequences(list(range(0, 65 * 2048, 2048)), 8, 148) is None
    # nothing longer than a segment
    assert split_sequences([0, 256], 1, 148) is None
    # 4 sequences x 16 heads = 64 streams on 148 SMs: halving each sequence gives one full wave
    seg, begin = split_sequences([0, 8192, 16384, 24576, 32768], 16, 148)
    assert len(seg) - 1 == 8 and begin == [0, 2, 4, 6, 8]
    # 148 equal streams: exactly one wave, nothing to gain
    assert split_sequences(list(range(0, 38 * 4096, 4096)), 4, 148) is None
    # a ragged batch whose longest document would be the tail of the launch: only long ones are cut
    bounds = [0, 8192] + [8192 + 512 * i for i in range(1, 41)]
    seg, begin = split_sequences(bounds, 8, 148)
    assert begin[1] - begin[0] > 1 and all(b - a == 1 for a, b in zip(begin[1:-1], begin[2:]))
    for bounds, heads in (([0, 262144], 8), ([0, 8192, 16384, 24576, 32768], 2),
                          ([0, 100, 5000, 5064, 30000], 2), ([0, 4096 + 77], 2)):
        res = split_sequences(bounds, heads, 148)
        assert res is not None
        seg, begin = res
        assert seg[0] == bounds[0] and seg[-1] == bounds[-1]
        assert all(b > a for a, b in zip(seg[:-1], seg[1:]) if True) or 0 in [
            e - s for s, e in zip(bounds[:-1], bounds[1:])]
        assert len(begin) == len(bounds)
        for r, (s, e) in enumerate(zip(bounds[:-1], bounds[1:])):
            inner = seg[begin[r]:begin[r + 1]]
            assert inner[0] == s
            assert all((x - s) % 64 == 0 for x in inner)  # cuts are chunk aligned
            assert all(x < e for x in inner)
        # every raw boundary is a segment boundary
        assert set(bounds) <= set(seg)


def test_shard_segments_for_the_overlapped_exchange():
    from flashqla_b200.cp import shard_segment_chunks

    # config 4 on 8 / 4 / 2 GPUs (Hv = 8), 16 SMs left to the exchange
    for chunks in (512, 1024, 2048):
        for short in ("first", "last"):
            lens = shard_segment_chunks(chunks, 148 - 16, 8, short)
            assert sum(lens) == chunks and len(lens) == 16 and min(lens) >= 8
            edge, rest = (lens[0], lens[1:]) if short == "first" else (lens[-1], lens[:-1])
            assert max(rest) - min(rest) <= 1 and 0.4 * max(rest) <= edge <= 0.6 * max(rest)
    # too short to overlap anything, or too many heads for three segments
    assert shard_segment_chunks(16, 148, 4, "first") is None
    assert shard_segment_chunks(512, 148, 64, "first") is None
    # no segment below the minimum even when the half would be
    assert min(shard_segment_chunks(40, 148, 4, "first")) >= 8


def test_tensor_cache_identity_and_eviction():
    from flashqla_b200.utils import tensor_cache

    calls = []

    @tensor_cache
    def f(t, n):
        calls.append(n)
        return t + n

    xs = [torch.zeros(1) for _ in range(6)]
    assert f(xs[0], 1) is f(xs[0], 1) and calls == [1]
    f(torch.zeros(1), 1)  # equal value, different identity: recomputed
    assert len(calls) == 2
    for x in xs[1:]:
        f(x, 1)
    n = len(calls)
    f(xs[0], 1)  # evicted by now (4 slots)
    assert len(calls) == n + 1
    assert len(f.cache_entries) <= 4
    # eviction goes by identity even when a pinned entry with tensors of another size comes first
    f.cache_entries[0][3] = True
    for size in (2, 3, 5, 7, 11):
        f(torch.zeros(size), 1)
    assert sum(1 for e in f.cache_entries if not e[3]) <= 4 and f.cache_entries[0][3]


def test_pack_helpers_round_trip():
    from flashqla_b200.utils import fill_last_chunk_of_g, pack, pad_and_reshape, unpack

    cu = torch.tensor([0, 5, 12, 20])
    x = torch.arange(20.0).reshape(1, 20, 1)
    u = unpack(x, cu)
    assert u.shape == (3, 8, 1) and torch.equal(pack(u, cu), x)
    p = pad_and_reshape(torch.ones(1, 70, 2), dim=1, chunk_size=64)
    assert p.shape == (1, 2, 64, 2) and p[0, 1, 6:].sum() == 0
    g = torch.arange(1.0, 129.0).reshape(1, 2, 64).clone()
    g[0, 1, 6:] = 0
    fill_last_chunk_of_g(g, 70, None)
    assert torch.all(g[0, 1, 6:] == g[0, 1, 5])


def test_backward_returns_one_gradient_per_forward_input():
    """The check of the reference's tests/test_function_signature.py:43-66 with its own lookup
    rules: the class is a top-level definition of flash_qla/ops/gated_delta_rule/chunk/__init__.py,
    ``forward`` starts with ``ctx``, ``backward`` has exactly one ``return`` and it is a tuple
    literal with one element per non-ctx input."""
    path = os.path.join(ROOT, "flash_qla", "ops", "gated_delta_rule", "chunk", "__init__.py")
    tree = ast.parse(open(path).read())
    cls = next(n for n in tree.body
               if isinstance(n, ast.ClassDef) and n.name == "ChunkGatedDeltaRuleFunction")
    fns = {n.name: n for n in cls.body if isinstance(n, ast.FunctionDef)}
    assert fns["forward"].args.args[0].arg == "ctx"
    n_inputs = len(fns["forward"].args.args) - 1
    returns = [n for n in ast.walk(fns["backward"]) if isinstance(n, ast.Return)]
    assert len(returns) == 1 and isinstance(returns[0].value, ast.Tuple)
    assert len(returns[0].value.elts) == n_inputs == 13


def test_drop_in_package_paths():
    import flash_qla
    from flash_qla.ops.gated_delta_rule import chunk_gated_delta_rule as a
    from flash_qla.ops.gated_delta_rule.chunk import ChunkGatedDeltaRuleFunction  # noqa: F401
    from flash_qla.ops.utils import chunk_local_cumsum, group_reduce_vector  # noqa: F401
    from flash_qla.utils import (fill_last_chunk_of_g, input_guard, l2norm, pack,  # noqa: F401
                                 pad_and_reshape, prepare_chunk_indices, prepare_chunk_offsets,
                                 tensor_cache, unpack)
    import flashqla_b200

    assert flash_qla.chunk_gated_delta_rule is flashqla_b200.chunk_gated_delta_rule is a


def test_kernel_chunk_table_uses_positions_of_sequences():
    """The public chunk table keeps the reference's numbering (a zero-length sequence takes no
    id); the table handed to the kernels carries the position in cu_seqlens instead, and is
    the public one when no sequence is empty."""
    import torch

    from flashqla_b200 import ops
    from flashqla_b200.utils import prepare_chunk_indices

    cu = torch.tensor([0, 100, 100, 400], dtype=torch.int32)
    assert prepare_chunk_indices(cu, 64)[:, 0].tolist() == [0, 0, 1, 1, 1, 1, 1]
    t = ops._kernel_chunk_indices(cu)
    assert t[:, 0].tolist() == [0, 0, 2, 2, 2, 2, 2]
    assert t[:, 1].tolist() == [0, 1, 0, 1, 2, 3, 4]
    assert t.dtype == cu.dtype and t.is_contiguous()
    full = torch.tensor([0, 64, 130], dtype=torch.int64)
    assert ops._kernel_chunk_indices(full) is prepare_chunk_indices(full, 64)
