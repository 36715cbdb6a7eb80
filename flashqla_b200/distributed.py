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
  (``start[r+1] = local[r] + M[r] start[r]``; the step after the last rank is the final state of
  the sequence, so no second collective is needed for it) and then runs the ordinary forward on
  its tokens with its start state.  The backward pass mirrors this for the state gradient with
  ``M^T`` in the other direction.  The payload always lands in the receiving GPU's own memory
  (the all-gather output) before any kernel reads it, and the chain reads it where it landed.
  A shard is itself cut into segments (one CTA per SM), and all but the edge segment start from
  a zero state a few chunks early: those run on a side stream while the summary, the collective
  and the chains are in flight, and only the edge segment waits for the exchanged state
  (``OVERLAP_EXCHANGE``).

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
# SMs the recurrence leaves free in a T-sharded call.  A recurrence CTA owns its SM (all of its
# registers), so the collective's kernel, the summary pass and the chains only run beside it on
# SMs it does not occupy; without free SMs they finish after the recurrence and nothing overlaps.
# (Config 4 forward on 4 GPUs, same box: 0.388 ms with no SM reserved, 0.334 ms with 16; capping
# the communicator's CTAs instead made the collective itself slower: 0.378 ms at 8, 0.506 at 4.)
RESERVE_SMS = 16
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
    return cp.shard_plan(k.shape[1], Hv, k.device, short, RESERVE_SMS)


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


def _record_views(rec, Hv: int, D: int):
    """The four parts of one rank's record ``[local | M | edge state | flags]`` as views."""
    n = Hv * D * D
    return (rec[:n].view(1, Hv, D, D), rec[n:2 * n].view(1, Hv, D, D),
            rec[2 * n:3 * n].view(1, Hv, D, D), rec[3 * n:].view(1, Hv))


def _new_record(Hv: int, D: int, dtype, device):
    """A zeroed record for this rank's contribution.  Callers let their kernels write ``local``
    and ``M`` straight into its views; flags are stored as numbers (0.0 / 1.0) of ``dtype``."""
    return torch.zeros(3 * Hv * D * D + Hv, dtype=dtype, device=device)


def _exchange(rec, Hv: int, D: int, edge_rank: int, reverse: bool, group, merge_fn):
    """One all-gather per direction, the same on every rank whatever its local arguments, and
    the chain over the ranks' summaries.  Returns ``[R + 1, Hv, D, D]``:

    * forward: entry ``r`` is the state entering rank ``r``'s tokens, entry ``R`` the final state
      of the whole sequence;
    * reverse: entry ``r + 1`` is the gradient of the state leaving rank ``r``'s tokens, entry 0
      the gradient of the sequence's initial state.

    The edge state (the sequence's initial state for the forward direction, the gradient of its
    final state for the reverse one) is read from the record of ``edge_rank`` only, and an owner
    that was given none sends zeros, which chain exactly like "no state".  The records are
    gathered into one buffer with a spare record at the far end of the chain (never read: it
    only gives the chain its last step), and the chain reads local, M and the flags where the
    all-gather put them."""
    world = dist.get_world_size(group)
    merge_fn = merge_fn or ops.merge_states
    size, n = rec.numel(), Hv * D * D
    flat = torch.empty((world + 1) * size, dtype=rec.dtype, device=rec.device)
    shift = 1 if reverse else 0  # the record of rank r lands in row r + shift
    dist.all_gather_into_tensor(flat[shift * size:(shift + world) * size], rec, group=group)
    rows = flat.view(world + 1, size)
    local = rows[:, :n].unflatten(1, (Hv, D, D))
    M = rows[:, n:2 * n].unflatten(1, (Hv, D, D))
    edge = rows[edge_rank + shift, 2 * n:3 * n].view(1, Hv, D, D)
    use = rows[:, 3 * n:]
    if use.is_cuda:
        use = use.view(torch.int32)  # 0.0 is all-zero bits, 1.0 is not: the kernel tests for zero
    return merge_fn(local, M, use, edge, _const_i32((0, world + 1), rec.device), reverse)


def _record_from(local, M, use_m, edge_state, is_owner: bool):
    Hv, D = local.shape[1], local.shape[2]
    rec = _new_record(Hv, D, local.dtype, local.device)
    r_local, r_m, r_edge, r_flags = _record_views(rec, Hv, D)
    r_local.copy_(local)
    r_m.copy_(M)
    r_flags.copy_(use_m)
    if edge_state is not None and is_owner:
        r_edge.copy_(edge_state)
    return rec


def exchange_forward(local, M, use_m, initial_state, group=None, merge_fn=None):
    """All-gather the forward summaries of every rank and return this rank's start state
    ``[1, Hv, D, D]``.  ``local``/``M``: ``[1, Hv, D, D]``; ``use_m``: ``[1, Hv]`` int32;
    ``initial_state`` is the sequence's initial state: it is taken from rank 0, other ranks may
    pass it too or pass None."""
    rank = dist.get_rank(group)
    rec = _record_from(local, M, use_m, initial_state, rank == 0)
    return _exchange(rec, local.shape[1], local.shape[2], 0, False, group, merge_fn)[rank:rank + 1]


def exchange_backward(local, M, use_m, dht, group=None, merge_fn=None):
    """Mirror of ``exchange_forward`` for the state gradient: returns the gradient of the state
    leaving this rank's tokens.  ``dht`` is the gradient of the sequence's final state: it is
    taken from the last rank, other ranks may pass it too or pass None."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    rec = _record_from(local, M, use_m, dht, rank == world - 1)
    return _exchange(rec, local.shape[1], local.shape[2], world - 1, True, group,
                     merge_fn)[rank + 1:rank + 2]


def _summary_record_fwd(k, v, A, g_cum, beta, scale, edge_state, is_owner: bool):
    """This rank's forward record: the end state of its whole shard from a zero state, the exact
    transition matrix M where the gates do not let the past die out inside the shard (flag), and
    the sequence's initial state if this rank owns it.  The kernels write into the record."""
    T, Hv, D = k.shape[1], v.shape[2], k.shape[-1]
    rec = _new_record(Hv, D, torch.float32, k.device)
    r_local, r_m, r_edge, r_flags = _record_views(rec, Hv, D)
    seg_cu = _const_i32((0, T), k.device)
    warm, fallback = ops.warmup_scan(g_cum, seg_cu, cp.THRESHOLD, from_start=False)
    ops.fwd_seq(None, k, v, A, g_cum, beta, scale, None, output_o=False, warm_chunks=warm,
                m_mask=fallback, tables=ops.SeqTables(1, T, seg_cu),
                out={"ht": r_local, "M": r_m})
    r_flags.copy_(fallback)
    if edge_state is not None and is_owner:
        r_edge.copy_(edge_state)
    return rec


def _summary_record_bwd(q, k, v, A, g_cum, beta, do, scale, edge_state, is_owner: bool):
    """Mirror of ``_summary_record_fwd``: the gradient entering the shard from a zero end
    gradient, M where the gradient survives the shard, and the gradient of the sequence's final
    state if this rank owns it."""
    T, Hv, D = k.shape[1], v.shape[2], k.shape[-1]
    rec = _new_record(Hv, D, torch.float32, k.device)
    r_local, r_m, r_edge, r_flags = _record_views(rec, Hv, D)
    seg_cu = _const_i32((0, T), k.device)
    tables = ops.SeqTables(1, T, seg_cu)
    warm, fallback = ops.warmup_scan(g_cum, seg_cu, cp.THRESHOLD, from_start=True)
    ops.bwd_dh(q, k, A, g_cum, beta, do, scale, None, warm_chunks=warm, tables=tables,
               out={"dh0": r_local})
    ops.fwd_seq(None, k, v, A, g_cum, beta, scale, None, output_o=False, m_mask=fallback,
                tables=tables, out={"M": r_m})
    r_flags.copy_(fallback)
    if edge_state is not None and is_owner:
        r_edge.copy_(edge_state)
    return rec


def fwd_tsharded(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=True,
                 group=None, for_backward=False):
    """Forward of ONE sequence whose tokens are split evenly over the ranks of ``group``
    (this rank passes its own ``[1, T/R, ...]`` slice, a multiple of 64 tokens).  Returns
    ``(g_cum, A, o, final_state, saved)``; ``final_state`` is the sequence's final state on every
    rank (the last step of the chain over the gathered summaries, so it costs no second
    collective), ``saved`` carries what ``bwd_tsharded`` needs.  ``initial_state`` is read on
    rank 0 only (other ranks may pass None); ``for_backward`` must be the same on every rank.
    With ``for_backward`` the forward keeps the per-chunk state and v_new tiles so that
    ``bwd_tsharded`` skips its recomputation pass."""
    assert q.shape[0] == 1 and q.shape[1] % CHUNK_SIZE == 0, "T shard must be a chunk multiple"
    if scale is None:
        scale = k.shape[-1] ** -0.5
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    Hv, D = v.shape[2], k.shape[-1]
    g32 = g if g.dtype == torch.float32 else g.float()
    g_cum, A = ops.kkt_solve(k, beta, g32.contiguous(), None, raw_gate=True)
    h0 = None if initial_state is None else initial_state.float().contiguous()
    plan = _two_phase_plan(k, Hv, "first")
    if plan is None:
        rec = _summary_record_fwd(k, v, A, g_cum, beta, scale, h0, rank == 0)
        chained = _exchange(rec, Hv, D, 0, False, group, None)
        start = chained[rank:rank + 1]
        res, cache = run_forward(q, k, v, A, g_cum, beta, scale, start,
                                 ops.SeqTables(1, q.shape[1], None), output_final_state=False,
                                 enable_fwd_cp_cache=for_backward)
        o = res["o"]
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
        out = ops.fwd_seq_outputs(k, v, seg, **tiles)
        main, side = torch.cuda.current_stream(k.device), _side_stream(k.device)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            ops.fwd_seq(q, k, v, A, g_cum, beta, scale, None, tables=seg, lead_chunks=lead,
                        run_mask=waits, run_value=0, out=out, operand_tiles=for_backward)
        # beside it: this rank's summary, the collective, the chain over the ranks and (for heads
        # that fall back) over this rank's segments, then the (segment, head) pairs that waited
        rec = _summary_record_fwd(k, v, A, g_cum, beta, scale, h0, rank == 0)
        chained = _exchange(rec, Hv, D, 0, False, group, None)
        start = chained[rank:rank + 1]
        seg_h0 = ops.merge_states(exact["ht"], exact["M"], fallback, start, plan.seg_begin,
                                  reverse=False, any_fallback=any_fb)
        ops.fwd_seq(q, k, v, A, g_cum, beta, scale, seg_h0, tables=seg, lead_chunks=lead,
                    run_mask=waits, run_value=1, out=out, operand_tiles=for_backward)
        main.wait_stream(side)
        o = out["o"]
        cache = (None, out["h"], out["vnew"], None) if for_backward else None
    final_state = chained[world:world + 1] if output_final_state else None
    return g_cum, A, o, final_state, (start, None, cache)


def bwd_tsharded(q, k, v, g_cum, beta, A, do, dht=None, scale=None, saved=None, group=None):
    """Backward of a T-sharded sequence.  ``saved`` is the tuple returned by ``fwd_tsharded``.
    Returns ``(dq, dk, dv, db, dg, dh0)`` for this rank's tokens; ``dh0`` (gradient of the
    sequence's initial state: the last step of the reverse chain) is valid on every rank.
    ``dht`` is read on the last rank only."""
    if scale is None:
        scale = k.shape[-1] ** -0.5
    start, _, cache = saved
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    Hv, D = v.shape[2], k.shape[-1]
    dht32 = None if dht is None else dht.float().contiguous()
    have_tiles = cache is not None and cache[1] is not None and cache[2] is not None
    plan = _two_phase_plan(k, Hv, "last") if have_tiles else None
    if plan is None:
        rec = _summary_record_bwd(q, k, v, A, g_cum, beta, do, scale, dht32, rank == world - 1)
        chained = _exchange(rec, Hv, D, world - 1, True, group, None)
        grads = chunk_gated_delta_rule_bwd(q, k, v, g_cum, beta, A, do,
                                           chained[rank + 1:rank + 2], scale, start, None,
                                           cp_cache=cache)
        return grads[:5] + (chained[0:1],)
    # the reverse recurrence in two launches (see OVERLAP_EXCHANGE); the forward's state and
    # v_new tiles are at hand
    import flash_qla.ops.gated_delta_rule.chunk as chunk_mod

    seg, last = plan.seg_tables, plan.n_seg - 1
    _, fallback, lead, exact_warm, any_fb = ops.segment_scan(
        g_cum, seg.cu, plan.seg_begin, cp.THRESHOLD, from_start=True)
    waits = _wait_mask(any_fb, plan.n_seg, last)
    local_e = ops.bwd_dh(q, k, A, g_cum, beta, do, scale, None, output_dh=False, output_du=False,
                         output_dh0=True, warm_chunks=exact_warm, tables=seg)["dh0"]
    m_e = ops.fwd_seq(None, k, v, A, g_cum, beta, scale, None, output_o=False, output_m=True,
                      m_mask=fallback, tables=seg)["M"]
    out = ops.bwd_dh_outputs(k, do, seg, output_dh0=False, operand_tiles=True)
    main, side = torch.cuda.current_stream(k.device), _side_stream(k.device)
    side.wait_stream(main)
    with torch.cuda.stream(side):
        ops.bwd_dh(q, k, A, g_cum, beta, do, scale, None, tables=seg, operand_tiles=True,
                   lead_chunks=lead, run_mask=waits, run_value=0, out=out)
    rec = _summary_record_bwd(q, k, v, A, g_cum, beta, do, scale, dht32, rank == world - 1)
    chained = _exchange(rec, Hv, D, world - 1, True, group, None)
    seg_dht = ops.merge_states(local_e, m_e, fallback, chained[rank + 1:rank + 2], plan.seg_begin,
                               reverse=True, any_fallback=any_fb)
    ops.bwd_dh(q, k, A, g_cum, beta, do, scale, seg_dht, tables=seg, operand_tiles=True,
               lead_chunks=lead, run_mask=waits, run_value=1, out=out)
    main.wait_stream(side)
    dq, dk, dv, db, dg = ops.bwd_main(q, k, v, cache[2], A, g_cum, beta, do, out["du"], cache[1],
                                      out["dh"], scale, tables=seg, operand_tiles=True)
    dq, dk, dv, db, dg = chunk_mod.finish_backward(dq, dk, dv, db, dg, k.shape[2], beta.dtype,
                                                   q.dtype, None)
    return dq, dk, dv, db, dg, chained[0:1]
