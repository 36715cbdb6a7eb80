"""Multi-GPU use of the gated-delta-rule path: one process per GPU, ``torch.distributed``.

Two ways to spread the work over the GPUs of a node (the reference has neither; its "TP4/TP8"
benchmark rows only emulate the head count one tensor-parallel shard would see):

* **(batch, head) sharding** - streams are independent per (sequence, value head), so each rank
  simply runs the operator on its own slice.  No communication.  ``shard_heads`` cuts a full
  problem into the slice of one rank.
* **T sharding of one long sequence** - rank ``r`` owns the tokens ``[r*T/R, (r+1)*T/R)``.  Each
  rank first computes, from a zero state, the end state of its own tokens and (only where the
  gates do not let the past die out inside the shard) the exact transition matrix ``M`` of its
  shard; one all-gather hands every rank all boundary summaries (``[Hv,K,V]`` + ``[Hv,K,K]`` fp32
  per rank, packed with the optional edge state into one record of about 1.5 MiB at Hv = 8 and
  moved by ONE collective per direction), every rank chains them locally
  (``start[r+1] = local[r] + M[r] start[r]``) and then runs the ordinary forward on its tokens
  with its start state.  The backward pass mirrors this for the state gradient with ``M^T`` in
  the other direction.  The payload always lands in the receiving GPU's own memory (the
  all-gather output) before any kernel reads it.

The collective is issued through ``torch.distributed`` (NCCL over NVLink on GPUs, gloo in the
CPU tests of the host logic); a rank that never joins surfaces as the process group's timeout
error on the host, no kernel ever waits on another GPU.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from . import cp, ops
from .api import chunk_gated_delta_rule_bwd, run_forward
from .ops import CHUNK_SIZE

# True (K = V = 128, at least three segments per shard): the recurrence kernels of a T-sharded
# call run in two launches.  The segments that can start from a zero state by themselves run at
# once on a side stream; this rank's summary, the all-gather and the chains run beside them, and
# only the edge segment (plus any head whose gates do not let the past die out) waits for the
# exchanged state.  False: everything waits for the exchange.
OVERLAP_EXCHANGE = True
_side_streams: dict = {}


def _side_stream(device) -> torch.cuda.Stream:
    key = str(device)
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device=device)
    return _side_streams[key]


def _two_phase_plan(k, Hv: int, short: str):
    import flash_qla.ops.gated_delta_rule.chunk as chunk_mod

    if not (OVERLAP_EXCHANGE and cp.LEAD_IN and chunk_mod._tiles_ok(k.shape[-1])):
        return None
    return cp.shard_plan(k.shape[1], Hv, k.device, short)


def _wait_mask(any_fb, n_seg: int, edge: int):
    """int32 ``[n_seg, Hv]``: 1 where a (segment, head) needs the exchanged state (the edge
    segment, and every segment of a head that falls back), 0 where it starts by itself."""
    mask = any_fb.expand(n_seg, -1).contiguous()
    mask[edge] = 1
    return mask


def shard_heads(q, k, v, g, beta, rank: int, world: int, initial_state=None):
    """Slice of a full problem owned by ``rank`` under value-head sharding (the matching q/k
    heads follow their value heads; with fewer q/k heads than ranks the group's q/k head is
    replicated).  Returns contiguous tensors ``(q, k, v, g, beta, initial_state)``."""
    Hq, Hv = q.shape[2], v.shape[2]
    if Hv % world:
        raise ValueError(f"{Hv} value heads do not divide over {world} ranks")
    hv = Hv // world
    v0 = rank * hv
    G = Hv // Hq
    if hv % G == 0:
        q0, hq = v0 // G, hv // G
    elif G % hv == 0:
        q0, hq = v0 // G, 1  # the shard lies inside one q/k group
    else:
        raise ValueError("value-head shard straddles q/k groups unevenly")
    sl = lambda x, a, n: x[:, :, a:a + n].contiguous()  # noqa: E731
    h0 = None if initial_state is None else initial_state[:, v0:v0 + hv].contiguous()
    return sl(q, q0, hq), sl(k, q0, hq), sl(v, v0, hv), sl(g, v0, hv), sl(beta, v0, hv), h0


# ---- T sharding -----------------------------------------------------------------------------

_const_cache: dict = {}


def _const_i32(values: tuple, device) -> torch.Tensor:
    """Small constant index tensors, made once per (values, device): steady-state steps then do
    no host-to-device copy, and the memo caches keyed by tensor identity keep hitting."""
    key = (values, str(device))
    if key not in _const_cache:
        _const_cache[key] = torch.tensor(values, dtype=torch.int32, device=device)
    return _const_cache[key]


def chain_boundary_states(local, M, use_m, first, rank: int, reverse: bool = False,
                          merge_fn=None):
    """Start state (or, reversed, end gradient) of ``rank`` from the gathered per-rank
    summaries.  ``local``, ``M``: ``[R, Hv, D, D]`` fp32; ``use_m``: ``[R, Hv]`` int32;
    ``first``: ``[1, Hv, D, D]`` state entering rank 0 (leaving rank R-1 when reversed) or None.
    ``merge_fn`` defaults to the CUDA merge kernel; the CPU tests pass a torch stand-in."""
    merge_fn = merge_fn or ops.merge_states
    R = local.shape[0]
    seg_begin = _const_i32((0, R), local.device)
    chained = merge_fn(local, M, use_m, first, seg_begin, reverse)
    return chained[rank:rank + 1].contiguous()


def _exchange(local, M, use_m, edge_state, edge_rank: int, reverse: bool, group, merge_fn):
    """One all-gather per direction, the same on every rank whatever its local arguments.

    Every rank contributes one record ``[local | M | edge state | use_m]``; the edge state (the
    sequence's initial state for the forward direction, the gradient of its final state for the
    reverse one) is read from the record of ``edge_rank`` only, and an owner that was given none
    sends zeros, which chain exactly like "no state".  So a caller may pass the state on the
    owning rank only, on every rank, or nowhere: the collective sequence is identical in all
    three cases."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    Hv, D = local.shape[1], local.shape[2]
    n_state = Hv * D * D
    rec = torch.zeros(3 * n_state + Hv, dtype=local.dtype, device=local.device)
    rec[:n_state] = local.reshape(-1)
    rec[n_state:2 * n_state] = M.reshape(-1)
    if edge_state is not None and rank == edge_rank:
        rec[2 * n_state:3 * n_state] = edge_state.reshape(-1)
    rec[3 * n_state:] = use_m.reshape(-1).to(local.dtype)
    flat = torch.empty(world * rec.numel(), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(flat, rec, group=group)
    everything = flat.view(world, rec.numel())
    all_local = everything[:, :n_state].reshape(world, Hv, D, D)
    all_m = everything[:, n_state:2 * n_state].reshape(world, Hv, D, D)
    edge = everything[edge_rank, 2 * n_state:3 * n_state].reshape(1, Hv, D, D)
    all_use = everything[:, 3 * n_state:].to(torch.int32)
    return chain_boundary_states(all_local.contiguous(), all_m.contiguous(), all_use.contiguous(),
                                 edge.contiguous(), rank, reverse, merge_fn)


def exchange_forward(local, M, use_m, initial_state, group=None, merge_fn=None):
    """All-gather the forward summaries of every rank and return this rank's start state
    ``[1, Hv, D, D]``.  ``local``/``M``: ``[1, Hv, D, D]``; ``use_m``: ``[1, Hv]`` int32;
    ``initial_state`` is the sequence's initial state: it is taken from rank 0, other ranks may
    pass it too or pass None."""
    return _exchange(local, M, use_m, initial_state, 0, False, group, merge_fn)


def exchange_backward(local, M, use_m, dht, group=None, merge_fn=None):
    """Mirror of ``exchange_forward`` for the state gradient: returns the gradient of the state
    leaving this rank's tokens.  ``dht`` is the gradient of the sequence's final state: it is
    taken from the last rank, other ranks may pass it too or pass None."""
    return _exchange(local, M, use_m, dht, dist.get_world_size(group) - 1, True, group, merge_fn)


def _local_summary_fwd(k, v, A, g_cum, beta, scale):
    """(end state from zero, M, fallback flag) of this rank's whole shard, shapes [1,Hv,D,D]."""
    T = k.shape[1]
    seg_cu = _const_i32((0, T), k.device)
    warm, fallback = ops.warmup_scan(g_cum, seg_cu, cp.THRESHOLD, from_start=False)
    tables = ops.SeqTables(1, T, seg_cu)
    res = ops.fwd_seq(None, k, v, A, g_cum, beta, scale, None, output_o=False,
                      output_final_state=True, output_m=True, warm_chunks=warm, m_mask=fallback,
                      tables=tables)
    return res["ht"], res["M"], fallback


def fwd_tsharded(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=True,
                 group=None, for_backward=False):
    """Forward of ONE sequence whose tokens are split evenly over the ranks of ``group``
    (this rank passes its own ``[1, T/R, ...]`` slice, a multiple of 64 tokens).  Returns
    ``(g_cum, A, o, final_state, saved)``; ``final_state`` is the sequence's final state on every
    rank, ``saved`` carries what ``bwd_tsharded`` needs.  ``initial_state`` is read on rank 0 only
    (other ranks may pass None); ``output_final_state`` and ``for_backward`` must be the same on
    every rank.  With ``for_backward`` the forward keeps the per-chunk state and v_new tiles so
    that ``bwd_tsharded`` skips its recomputation pass."""
    assert q.shape[0] == 1 and q.shape[1] % CHUNK_SIZE == 0, "T shard must be a chunk multiple"
    if scale is None:
        scale = k.shape[-1] ** -0.5
    world = dist.get_world_size(group)
    g32 = g if g.dtype == torch.float32 else g.float()
    g_cum, A = ops.kkt_solve(k, beta, g32.contiguous(), None, raw_gate=True)
    h0 = None if initial_state is None else initial_state.float().contiguous()
    plan = _two_phase_plan(k, v.shape[2], "first")
    if plan is None:
        local, M, fallback = _local_summary_fwd(k, v, A, g_cum, beta, scale)
        start = exchange_forward(local, M, fallback, h0, group)
        res, cache = run_forward(q, k, v, A, g_cum, beta, scale, start,
                                 ops.SeqTables(1, q.shape[1], None), output_final_state=True,
                                 enable_fwd_cp_cache=for_backward)
        o, ht = res["o"], res["ht"]
    else:
        seg = plan.seg_tables
        # nothing here depends on another rank: the scan, the exact local passes of heads that
        # fall back (they return at once elsewhere), and the recurrence of every (segment, head)
        # that leads in by itself
        _, fallback, lead, exact_warm, any_fb = ops.segment_scan(
            g_cum, seg.cu, plan.seg_begin, cp.THRESHOLD, from_start=False)
        waits = _wait_mask(any_fb, plan.n_seg, 0)
        exact = ops.fwd_seq(None, k, v, A, g_cum, beta, scale, None, output_o=False,
                            output_final_state=True, output_m=True, warm_chunks=exact_warm,
                            m_mask=fallback, tables=seg)
        tiles = dict(output_h=True, output_vnew=True, operand_tiles=True) if for_backward else {}
        out = ops.fwd_seq_outputs(k, v, seg, output_final_state=True, **tiles)
        main, side = torch.cuda.current_stream(k.device), _side_stream(k.device)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            ops.fwd_seq(q, k, v, A, g_cum, beta, scale, None, tables=seg, lead_chunks=lead,
                        run_mask=waits, run_value=0, out=out, operand_tiles=for_backward)
        # beside it: this rank's summary, the collective, the chain over the ranks and (for heads
        # that fall back) over this rank's segments, then the (segment, head) pairs that waited
        local, M, fb_shard = _local_summary_fwd(k, v, A, g_cum, beta, scale)
        start = exchange_forward(local, M, fb_shard, h0, group)
        seg_h0 = ops.merge_states(exact["ht"], exact["M"], fallback, start, plan.seg_begin,
                                  reverse=False, any_fallback=any_fb)
        ops.fwd_seq(q, k, v, A, g_cum, beta, scale, seg_h0, tables=seg, lead_chunks=lead,
                    run_mask=waits, run_value=1, out=out, operand_tiles=for_backward)
        main.wait_stream(side)
        o, ht = out["o"], out["ht"][plan.n_seg - 1:plan.n_seg]
        cache = (None, out["h"], out["vnew"], None) if for_backward else None
    final_state = None
    if output_final_state:
        final_state = ht.clone()
        src = world - 1
        dist.broadcast(final_state, src=dist.get_global_rank(group, src) if group else src,
                       group=group)
    return g_cum, A, o, final_state, (start, M, cache)


def bwd_tsharded(q, k, v, g_cum, beta, A, do, dht=None, scale=None, saved=None, group=None):
    """Backward of a T-sharded sequence.  ``saved`` is the tuple returned by ``fwd_tsharded``.
    Returns ``(dq, dk, dv, db, dg, dh0)`` for this rank's tokens; ``dh0`` (gradient of the
    sequence's initial state) is valid on every rank.  ``dht`` is read on the last rank only."""
    if scale is None:
        scale = k.shape[-1] ** -0.5
    start, _, cache = saved
    have_tiles = cache is not None and cache[1] is not None and cache[2] is not None
    plan = _two_phase_plan(k, v.shape[2], "last") if have_tiles else None
    if plan is not None:
        return _bwd_two_phase(plan, q, k, v, g_cum, beta, A, do, dht, scale, cache, group)
    local, M, fallback = _local_summary_bwd(q, k, v, A, g_cum, beta, do, scale)
    dht32 = None if dht is None else dht.float().contiguous()
    end = exchange_backward(local, M, fallback, dht32, group)
    dq, dk, dv, db, dg, dh0 = chunk_gated_delta_rule_bwd(q, k, v, g_cum, beta, A, do, end, scale,
                                                         start, None, cp_cache=cache)
    dh0 = dh0.clone()
    dist.broadcast(dh0, src=dist.get_global_rank(group, 0) if group else 0, group=group)
    return dq, dk, dv, db, dg, dh0


def _local_summary_bwd(q, k, v, A, g_cum, beta, do, scale):
    """(gradient entering the shard from a zero end gradient, M, fallback flag) of this rank's
    whole shard, shapes [1,Hv,D,D] / [1,Hv]."""
    T = k.shape[1]
    seg_cu = _const_i32((0, T), k.device)
    tables = ops.SeqTables(1, T, seg_cu)
    warm, fallback = ops.warmup_scan(g_cum, seg_cu, cp.THRESHOLD, from_start=True)
    local = ops.bwd_dh(q, k, A, g_cum, beta, do, scale, None, output_dh=False, output_du=False,
                       output_dh0=True, warm_chunks=warm, tables=tables)["dh0"]
    # the exact transition matrix of this shard is needed wherever the gradient survives it
    M = ops.fwd_seq(None, k, v, A, g_cum, beta, scale, None, output_o=False, output_m=True,
                    m_mask=fallback, tables=tables)["M"]
    return local, M, fallback


def _bwd_two_phase(plan, q, k, v, g_cum, beta, A, do, dht, scale, cache, group):
    """Backward of a T-sharded sequence with the reverse recurrence in two launches (see
    ``OVERLAP_EXCHANGE``); the forward's state and v_new tiles are at hand."""
    import flash_qla.ops.gated_delta_rule.chunk as chunk_mod

    in_dtype, beta_dtype = q.dtype, beta.dtype
    Hq = k.shape[2]
    seg = plan.seg_tables
    last = plan.n_seg - 1
    _, fallback, lead, exact_warm, any_fb = ops.segment_scan(
        g_cum, seg.cu, plan.seg_begin, cp.THRESHOLD, from_start=True)
    waits = _wait_mask(any_fb, plan.n_seg, last)
    local_e = ops.bwd_dh(q, k, A, g_cum, beta, do, scale, None, output_dh=False, output_du=False,
                         output_dh0=True, warm_chunks=exact_warm, tables=seg)["dh0"]
    m_e = ops.fwd_seq(None, k, v, A, g_cum, beta, scale, None, output_o=False, output_m=True,
                      m_mask=fallback, tables=seg)["M"]
    out = ops.bwd_dh_outputs(k, do, seg, operand_tiles=True)
    main, side = torch.cuda.current_stream(k.device), _side_stream(k.device)
    side.wait_stream(main)
    with torch.cuda.stream(side):
        ops.bwd_dh(q, k, A, g_cum, beta, do, scale, None, tables=seg, operand_tiles=True,
                   lead_chunks=lead, run_mask=waits, run_value=0, out=out)
    local, M, fb_shard = _local_summary_bwd(q, k, v, A, g_cum, beta, do, scale)
    dht32 = None if dht is None else dht.float().contiguous()
    end = exchange_backward(local, M, fb_shard, dht32, group)
    seg_dht = ops.merge_states(local_e, m_e, fallback, end, plan.seg_begin, reverse=True,
                               any_fallback=any_fb)
    ops.bwd_dh(q, k, A, g_cum, beta, do, scale, seg_dht, tables=seg, operand_tiles=True,
               lead_chunks=lead, run_mask=waits, run_value=1, out=out)
    main.wait_stream(side)
    dq, dk, dv, db, dg = ops.bwd_main(q, k, v, cache[2], A, g_cum, beta, do, out["du"], cache[1],
                                      out["dh"], scale, tables=seg, operand_tiles=True)
    dq, dk, dv, db, dg = chunk_mod.finish_backward(dq, dk, dv, db, dg, Hq, beta_dtype, in_dtype,
                                                   None)
    dh0 = out["dh0"][0:1].clone()
    dist.broadcast(dh0, src=dist.get_global_rank(group, 0) if group else 0, group=group)
    return dq, dk, dv, db, dg, dh0
