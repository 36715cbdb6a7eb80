"""Intra-GPU context parallelism along T ("gate-driven auto-CP").

Long sequences are cut into chunk-aligned segments that run as independent streams.  Every
segment's start state is obtained without running the sequence serially:

1. per (segment, head) a scan of the chunk gate totals finds how many trailing chunks matter
   before the accumulated log gate falls below ``THRESHOLD`` (earlier history is attenuated by
   more than ``exp(THRESHOLD)``);
2. a state-only pass over just those chunks, from a zero state, gives the segment's local end
   state; where the threshold is never reached inside the segment, the whole segment is walked
   and its exact transition matrix ``M`` is produced as well;
3. a merge kernel chains the segments of each sequence:
   ``start[i+1] = local[i] + fallback[i] * M[i] @ start[i]``.

The backward pass mirrors this for the state gradient with ``M^T``.  This follows the scheme of
the reference's ``flash_qla/ops/gated_delta_rule/chunk/cp_context.py:47-321``; the segment
length policy is this package's own (sized for the 148 SMs of a B200, also applied to batched
fixed-length input, which the reference never splits).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import ops
from .ops import CHUNK_SIZE, SeqTables
from .utils import tensor_cache

THRESHOLD = -10.0
MIN_SEGMENT_CHUNKS = 8
VALUE_SLICES = 1  # CTAs per (segment, head) of the tcgen05 forward kernel
SEGMENT_OVERHEAD_CHUNKS = 2  # cost of a hand-off, in chunk steps of the main kernel
CTA_START_CHUNKS = 2  # cost of starting a CTA (tensor-memory allocation, first loads), same unit
# True: the tcgen05 recurrence kernels start a segment a few chunks early (forward,
# ``forward_start``) or late (reverse, ``backward_end``) from a zero state; False: every segment's
# start state comes from the separate state-only pass and the merge chain
# (``forward_segment_states``, ``backward_segment_states``), as the mma.sync kernels always do.
LEAD_IN = True


def sm_count(device) -> int:
    return torch.cuda.get_device_properties(device).multi_processor_count


@dataclass
class SegmentPlan:
    seg_tables: SeqTables          # the segments seen as a packed batch
    seg_begin: torch.Tensor        # int32 [n_raw+1]: first segment of every raw sequence
    first_seg_of_raw: torch.Tensor  # int64 [n_raw]
    last_seg_of_raw: torch.Tensor   # int64 [n_raw]
    keep_fwd: torch.Tensor         # int32 [n_seg]: 0 for the last segment of a raw sequence
    keep_bwd: torch.Tensor         # int32 [n_seg]: 0 for the first segment of a raw sequence
    n_seg: int


def _makespan(costs: list[int], copies: int, machines: int) -> int:
    """Length of the schedule the hardware produces for CTAs of the given costs (each present
    ``copies`` times, one per head) handed out longest first to ``machines`` SMs, one CTA per SM:
    every CTA goes to the SM that frees up first."""
    import heapq

    items = sorted(costs, reverse=True)
    n = len(items) * copies
    if n <= machines:
        return items[0] if items else 0
    loads = [0] * machines
    heapq.heapify(loads)
    for c in items:
        for _ in range(copies):
            heapq.heappush(loads, heapq.heappop(loads) + c)
    return max(loads)


def split_sequences(bounds: list[int], num_heads: int, n_sm: int,
                    min_chunks: int = MIN_SEGMENT_CHUNKS, slices: int = VALUE_SLICES):
    """Host-side segment planner.  ``bounds`` are the raw cumulative sequence lengths.

    The sequential kernels keep one CTA per SM and walk their chunks in order; the CTAs of a
    launch are handed out longest first, each to the SM that frees up first.  The planner
    evaluates that schedule (``_makespan``) for the unsplit batch and for every maximum segment
    length ``ceil(longest / p)`` (sequences longer than the limit are cut into equal, chunk
    aligned parts), charging ``CTA_START_CHUNKS`` per CTA and ``SEGMENT_OVERHEAD_CHUNKS`` more
    per segment that needs a start state, and keeps the cheapest.  It therefore splits a single
    long sequence to fill the GPU, splits only the few long documents of a ragged batch that
    would otherwise be the tail of the launch, and leaves a batch alone that already keeps every
    SM busy.

    Returns ``None`` when no split beats the unsplit schedule by at least 3 %, else
    ``(seg_bounds, seg_begin)``: the cumulative lengths of the segments and, per raw sequence, the
    index of its first segment.
    """
    lens = [e - s for s, e in zip(bounds[:-1], bounds[1:])]
    chunks = [(n + CHUNK_SIZE - 1) // CHUNK_SIZE for n in lens]
    longest = max(chunks) if chunks else 0
    if longest < 2 * min_chunks:
        return None
    copies = num_heads * slices

    def layout(limit):
        parts = [max(1, math.ceil(c / limit)) for c in chunks]
        per = [math.ceil(c / p) if c else 0 for c, p in zip(chunks, parts)]
        costs = []
        for c, p, pc in zip(chunks, parts, per):
            for i in range(p):
                seg = min(pc, c - i * pc)
                if seg > 0:
                    costs.append(seg + CTA_START_CHUNKS + (SEGMENT_OVERHEAD_CHUNKS if i else 0))
        return parts, per, _makespan(costs, copies, n_sm)

    _, _, unsplit = layout(longest)
    tried, cands = set(), []
    for p in range(2, longest // min_chunks + 1):
        limit = math.ceil(longest / p)
        if limit < min_chunks:
            break
        if limit in tried:
            continue
        tried.add(limit)
        parts, per, cost = layout(limit)
        cands.append((cost, parts, per))
    if not cands:
        return None
    cheapest = min(c[0] for c in cands)
    if cheapest > 0.97 * unsplit:
        return None
    # among near-ties the coarsest split: fewer CTAs, fewer hand-offs
    best = next(c for c in cands if c[0] <= 1.03 * cheapest)
    _, parts, per = best
    seg_bounds, seg_begin = [], []
    for s, np_, pc in zip(bounds[:-1], parts, per):
        seg_begin.append(len(seg_bounds))
        for i in range(np_):
            seg_bounds.append(s + i * pc * CHUNK_SIZE)  # balanced, chunk aligned
    seg_begin.append(len(seg_bounds))
    seg_bounds.append(bounds[-1])
    return seg_bounds, seg_begin


@tensor_cache
def _host_bounds(cu_seqlens: torch.Tensor) -> list[int]:
    return [int(x) for x in cu_seqlens.tolist()]


_fixed_plan_cache: dict = {}


def _build_plan(bounds, Hv, device, idx_dtype, T_rows) -> SegmentPlan | None:
    res = split_sequences(bounds, Hv, sm_count(device))
    if res is None:
        return None
    return _plan_from_bounds(res[0], res[1], device, idx_dtype, T_rows)


def _plan_from_bounds(seg_bounds, seg_begin, device, idx_dtype, T_rows) -> SegmentPlan:
    seg_cu = torch.tensor(seg_bounds, dtype=idx_dtype, device=device)
    begin = torch.tensor(seg_begin, dtype=torch.int32, device=device)
    tables = SeqTables(1, T_rows, seg_cu)
    n_seg = len(seg_bounds) - 1
    keep_fwd = [1] * n_seg
    keep_bwd = [1] * n_seg
    for first, nxt in zip(seg_begin[:-1], seg_begin[1:]):
        if nxt > first:
            keep_bwd[first] = 0
            keep_fwd[nxt - 1] = 0
    return SegmentPlan(tables, begin, begin[:-1].long(), begin[1:].long() - 1,
                       torch.tensor(keep_fwd, dtype=torch.int32, device=device),
                       torch.tensor(keep_bwd, dtype=torch.int32, device=device), n_seg)


_shard_plan_cache: dict = {}


def shard_segment_chunks(chunks: int, n_sm: int, Hv: int, short: str,
                         min_chunks: int = MIN_SEGMENT_CHUNKS) -> list[int] | None:
    """Chunks per segment of a shard of ``chunks`` chunks for ``shard_plan``: ``n`` segments with
    ``n * Hv <= n_sm``, the waiting one (first or last) about half as long as the others and no
    segment shorter than ``min_chunks``; ``None`` when fewer than three fit."""
    n = min(n_sm // Hv, chunks // min_chunks)
    if n < 3:
        return None
    short_len = max(min_chunks, int(chunks / (n - 0.5) / 2))
    base, extra = divmod(chunks - short_len, n - 1)
    lens = [base + (1 if i < extra else 0) for i in range(n - 1)]
    return [short_len] + lens if short == "first" else lens + [short_len]


def shard_plan(T: int, Hv: int, device, short: str, reserve_sms: int = 0) -> SegmentPlan | None:
    """Segment plan of ONE sequence of ``T`` tokens (a chunk multiple) whose edge segment has to
    wait for a state from elsewhere (another GPU): as many segments as fit one CTA per SM, the
    waiting one (``short`` = "first" for the forward direction, "last" for the reverse one) about
    half as long as the others, so that it can start late and still finish with them.
    ``reserve_sms`` SMs are left without a CTA: the kernels of the exchange (the collective's
    own, the summary pass, the chains) run there while the recurrence occupies the rest.
    ``None`` when fewer than three segments fit."""
    key = (T, Hv, str(device), short, reserve_sms)
    if key not in _shard_plan_cache:
        lens = shard_segment_chunks(T // CHUNK_SIZE, sm_count(device) - reserve_sms, Hv, short)
        plan = None
        if lens is not None:
            n = len(lens)
            bounds = [0]
            for c in lens:
                bounds.append(bounds[-1] + c * CHUNK_SIZE)
            plan = _plan_from_bounds(bounds, [0, n], torch.device(device), torch.int32, T)
        _shard_plan_cache[key] = plan
    return _shard_plan_cache[key]


@tensor_cache
def _plan_for_cu(cu_seqlens: torch.Tensor, Hv: int, T_rows: int):
    return _build_plan(_host_bounds(cu_seqlens), Hv, cu_seqlens.device, cu_seqlens.dtype, T_rows)


def plan_segments(tables: SeqTables, Hv: int, is_bwd: bool = False,
                  device=None) -> SegmentPlan | None:
    """Segment plan for a batch, or ``None`` when the batch runs unsplit.  Cached per
    ``cu_seqlens`` tensor (identity) or per fixed shape, so steady-state calls do no host work."""
    if tables.cu is not None:
        return _plan_for_cu(tables.cu, Hv, tables.T)
    device = device if device is not None else torch.cuda.current_device()
    key = (tables.B, tables.T, Hv, str(device))
    if key not in _fixed_plan_cache:
        bounds = [b * tables.T for b in range(tables.B + 1)]
        _fixed_plan_cache[key] = _build_plan(bounds, Hv, torch.device("cuda", device)
                                             if isinstance(device, int) else device,
                                             torch.int32, tables.B * tables.T)
    return _fixed_plan_cache[key]


def forward_segment_states(plan: SegmentPlan, k, v, A, g_cum, beta, scale, h0):
    """Start state of every segment, fp32 ``[n_seg, Hv, D, D]``."""
    seg = plan.seg_tables
    # the last segment of a sequence hands nothing on
    warm, fallback = ops.warmup_scan(g_cum, seg.cu, THRESHOLD, from_start=False,
                                     keep=plan.keep_fwd)
    res = ops.fwd_seq(None, k, v, A, g_cum, beta, scale, None, output_o=False,
                      output_final_state=True, output_m=True, warm_chunks=warm,
                      m_mask=fallback, tables=seg)
    return ops.merge_states(res["ht"], res["M"], fallback, h0, plan.seg_begin, reverse=False)


def forward_start(plan: SegmentPlan, k, v, A, g_cum, beta, scale, h0):
    """How every segment of a split plan gets its start state, for the tcgen05 recurrence kernel:
    returns ``(seg_h0, lead)``.  Where no segment of a (sequence, head) falls back, segment ``i``
    just starts ``lead[i]`` chunks early from a zero state inside the recurrence kernel itself,
    and the three launches below find nothing to do for it (the scan is the only one that costs
    more than a launch); ``seg_h0`` then only carries the sequence's own initial state.  Where
    some segment falls back (gates too weak for the past to die out inside a segment) the exact
    chain of ``forward_segment_states`` runs for that (sequence, head) and ``lead`` is 0."""
    seg = plan.seg_tables
    _, fallback, lead, exact_warm, any_fb = ops.segment_scan(g_cum, seg.cu, plan.seg_begin,
                                                             THRESHOLD, from_start=False)
    res = ops.fwd_seq(None, k, v, A, g_cum, beta, scale, None, output_o=False,
                      output_final_state=True, output_m=True, warm_chunks=exact_warm,
                      m_mask=fallback, tables=seg)
    seg_h0 = ops.merge_states(res["ht"], res["M"], fallback, h0, plan.seg_begin, reverse=False,
                              any_fallback=any_fb)
    return seg_h0, lead


def backward_segment_states(plan: SegmentPlan, q, k, v, A, g_cum, beta, do, scale, dht):
    """Gradient of the state leaving every segment, fp32 ``[n_seg, Hv, D, D]``."""
    seg = plan.seg_tables
    # the first segment of a sequence receives nothing from before it
    warm, fallback = ops.warmup_scan(g_cum, seg.cu, THRESHOLD, from_start=True,
                                     keep=plan.keep_bwd)
    local = ops.bwd_dh(q, k, A, g_cum, beta, do, scale, None, output_dh=False, output_du=False,
                       output_dh0=True, warm_chunks=warm, tables=seg)["dh0"]
    # exact transition matrices where the gradient does not die out inside the segment
    m = ops.fwd_seq(None, k, v, A, g_cum, beta, scale, None, output_o=False, output_m=True,
                    m_mask=fallback, tables=seg)["M"]
    return ops.merge_states(local, m, fallback, dht, plan.seg_begin, reverse=True)


def backward_end(plan: SegmentPlan, q, k, v, A, g_cum, beta, do, scale, dht):
    """Mirror image of ``forward_start`` for the state gradient, for the tcgen05 reverse
    recurrence kernel: returns ``(seg_dht, lead)``.  Where no segment of a (sequence, head) falls
    back, segment ``i`` starts ``lead[i]`` chunks after its end (the head of segment ``i + 1``)
    from a zero gradient inside the recurrence kernel itself and ``seg_dht`` only carries the
    gradient of the sequence's own final state; elsewhere the exact chain of
    ``backward_segment_states`` runs and ``lead`` is 0."""
    seg = plan.seg_tables
    _, fallback, lead, exact_warm, any_fb = ops.segment_scan(g_cum, seg.cu, plan.seg_begin,
                                                             THRESHOLD, from_start=True)
    local = ops.bwd_dh(q, k, A, g_cum, beta, do, scale, None, output_dh=False, output_du=False,
                       output_dh0=True, warm_chunks=exact_warm, tables=seg)["dh0"]
    m = ops.fwd_seq(None, k, v, A, g_cum, beta, scale, None, output_o=False, output_m=True,
                    m_mask=fallback, tables=seg)["M"]
    seg_dht = ops.merge_states(local, m, fallback, dht, plan.seg_begin, reverse=True,
                               any_fallback=any_fb)
    return seg_dht, lead
