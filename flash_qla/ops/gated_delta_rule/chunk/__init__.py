"""Public operator API under the reference's own module path: the three functions and the
autograd class of the reference's ``flash_qla/ops/gated_delta_rule/chunk/__init__.py`` with
unchanged signatures (``chunk_gated_delta_rule_fwd`` ``:33-88``, ``chunk_gated_delta_rule_bwd``
``:91-159``, ``ChunkGatedDeltaRuleFunction`` ``:162-266``, ``chunk_gated_delta_rule``
``:269-404``), driving the sm_100a kernels of ``flashqla_b200``.  The definitions live in this
file (not behind an alias) so that source-level checks written against the reference, such as
its ``tests/test_function_signature.py``, find the class where they look for it.

Pipeline (all launches on the current CUDA stream):

* forward:  chunk-local cumsum of g -> kkt + triangular solve (A) -> [segment planning and
  state hand-off when a sequence is split for context parallelism] -> sequential recurrence
  (o, optional h, final state).
* backward: recompute h and v_new -> reverse recurrence of the state gradient (dh, du, dh0)
  -> chunk-parallel dq/dk/dv/dbeta/dg -> GVA group sum -> reverse cumsum of dg.
"""

from __future__ import annotations

import os

import torch

from flashqla_b200 import cp, ops
from flashqla_b200.ops import CHUNK_SIZE, SeqTables
from flashqla_b200.utils import input_guard, l2norm_bwd, l2norm_fwd


def _state_in(x, state_v_first):
    """User state -> kernel layout ([key dim][value dim], fp32, contiguous)."""
    if x is None:
        return None
    if state_v_first:
        x = x.transpose(-1, -2)
    return x.to(torch.float32).contiguous()


def _state_out(x, state_v_first):
    if x is None or not state_v_first:
        return x
    return x.transpose(-1, -2).contiguous()


def _as_f32(g):
    return g if g.dtype == torch.float32 else g.float()


def _beta_in(beta):
    return beta if beta.dtype in (torch.float32, torch.bfloat16) else beta.float()


def _bf16(x):
    """float16 inputs (which the reference accepts, ``chunk/__init__.py:364-367``) are computed
    in bfloat16: the tensor cores of this build are fed bf16 operands only.  Results go back to
    the caller's dtype."""
    return x if x is None or x.dtype == torch.bfloat16 else x.to(torch.bfloat16)


# With the forward cache on (the training path), the forward also keeps what the backward would
# otherwise recompute with a second pass of the recurrence: the state entering every chunk and
# v_new, as the operand tiles the chunk-parallel backward reads (768 bytes per token and value
# head).  Set to False to trade that memory for the recomputation.
SAVE_STATE_TILES = True


def _tiles_ok(D: int) -> bool:
    return D == 128 and os.environ.get("FQLA_FORCE_MMA_SYNC") is None


def _segment_starts(plan, k, v, A, g_cum, beta, scale, h0):
    """``(segment start states, lead-in chunk counts or None)`` of a split plan.  The tcgen05
    recurrence kernel (K = V = 128) leads in by itself; the mma.sync kernels take explicit start
    states for every segment."""
    if cp.LEAD_IN and _tiles_ok(k.shape[-1]):
        return cp.forward_start(plan, k, v, A, g_cum, beta, scale, h0)
    return cp.forward_segment_states(plan, k, v, A, g_cum, beta, scale, h0), None


def run_forward(q, k, v, A, g_cum, beta, scale, h0, tables, output_final_state=True,
                output_h=False, auto_cp=True, enable_fwd_cp_cache=False):
    """The part of the forward after cumsum and kkt+solve: optional split into segments with
    state hand-off, then the sequential recurrence.  Returns ``(outputs dict, cp_cache)``;
    ``cp_cache`` is ``(segment initial states or None, h tiles or None, v_new tiles or None,
    lead-in chunk counts or None)``."""
    plan = cp.plan_segments(tables, v.shape[2], is_bwd=False, device=k.device) if auto_cp else None
    keep = enable_fwd_cp_cache and SAVE_STATE_TILES and not output_h and _tiles_ok(k.shape[-1])
    extra = dict(output_h=True, output_vnew=True, operand_tiles=True) if keep else dict(output_h=output_h)
    cp_cache = None
    lead = None
    if plan is not None:
        seg_h0, lead = _segment_starts(plan, k, v, A, g_cum, beta, scale, h0)
        res = ops.fwd_seq(q, k, v, A, g_cum, beta, scale, seg_h0,
                          output_final_state=output_final_state, tables=plan.seg_tables,
                          lead_chunks=lead, **extra)
        if output_final_state:
            res["ht"] = res["ht"][plan.last_seg_of_raw]
    else:
        seg_h0 = None
        res = ops.fwd_seq(q, k, v, A, g_cum, beta, scale, h0,
                          output_final_state=output_final_state, tables=tables, **extra)
    if keep:
        cp_cache = (seg_h0, res.pop("h"), res.pop("vnew"), lead)
    elif enable_fwd_cp_cache and seg_h0 is not None:
        cp_cache = (seg_h0, None, None, lead)
    return res, cp_cache


@ops.on_tensor_device
def chunk_gated_delta_rule_fwd(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    beta: torch.Tensor,
    scale: float | None = None,
    initial_state: torch.Tensor | None = None,
    cu_seqlens: torch.LongTensor | None = None,
    output_final_state: bool = True,
    output_h: bool = False,
    auto_cp: bool = True,
    state_v_first: bool = False,
    enable_fwd_cp_cache: bool = False,
):
    """Returns ``(g_cumsum, A, o, h, final_state, cp_cache)`` like the reference
    (``chunk/__init__.py:88``).  ``A`` is the gated inverse (the reference's oracle convention),
    consumed as-is by ``chunk_gated_delta_rule_bwd``."""
    if scale is None:
        scale = k.shape[-1] ** -0.5
    in_dtype = q.dtype
    q, k, v = _bf16(q).contiguous(), _bf16(k).contiguous(), _bf16(v).contiguous()
    g = _as_f32(g).contiguous()
    beta = _beta_in(beta).contiguous()
    B, T, Hq, D = k.shape
    tables = SeqTables(B, T, cu_seqlens)
    g_cum, A = ops.kkt_solve(k, beta, g, cu_seqlens, raw_gate=True)  # cumsum fused into the kernel
    h0 = _state_in(initial_state, state_v_first)

    res, cp_cache = run_forward(q, k, v, A, g_cum, beta, scale, h0, tables, output_final_state,
                                output_h, auto_cp, enable_fwd_cp_cache)
    o = res["o"] if in_dtype == torch.bfloat16 else res["o"].to(in_dtype)
    h = res.get("h")
    if h is not None:
        h = h.view(B, -1, *h.shape[1:]) if cu_seqlens is None else h.unsqueeze(0)
        h = _state_out(h, state_v_first)
    final_state = _state_out(res.get("ht"), state_v_first)
    return g_cum, A, o, h, final_state, cp_cache


@ops.on_tensor_device
def chunk_gated_delta_rule_bwd(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    beta: torch.Tensor,
    A: torch.Tensor,
    do: torch.Tensor,
    dht: torch.Tensor | None = None,
    scale: float | None = None,
    initial_state: torch.Tensor | None = None,
    cu_seqlens: torch.LongTensor | None = None,
    state_v_first: bool = False,
    auto_cp: bool = True,
    cp_cache: tuple | None = None,
):
    """``g`` is the cumsum returned by the forward and ``A`` the forward's ``A``.  Returns
    ``(dq, dk, dv, db, dg, dh0)`` (``chunk/__init__.py:91-159``)."""
    if scale is None:
        scale = k.shape[-1] ** -0.5
    in_dtype = q.dtype
    q, k, v, do, A = (_bf16(x).contiguous() for x in (q, k, v, do, A))
    g = _as_f32(g).contiguous()
    beta_k = _beta_in(beta).contiguous()
    B, T, Hq, D = k.shape
    Hv = v.shape[2]
    tables = SeqTables(B, T, cu_seqlens)
    h0 = _state_in(initial_state, state_v_first)
    dht_k = _state_in(dht, state_v_first)

    cached = (tuple(cp_cache) if cp_cache is not None else ()) + (None, None, None, None)
    plan = cp.plan_segments(tables, Hv, is_bwd=True, device=k.device) if auto_cp else None
    lead = lead_out = None
    if plan is not None:
        if cached[0] is not None:
            seg_h0, lead = cached[0], cached[3]
        else:
            seg_h0, lead = _segment_starts(plan, k, v, A, g, beta_k, scale, h0)
        if cp.LEAD_IN and _tiles_ok(D):
            seg_dht, lead_out = cp.backward_end(plan, q, k, v, A, g, beta_k, do, scale, dht_k)
        else:
            seg_dht = cp.backward_segment_states(plan, q, k, v, A, g, beta_k, do, scale, dht_k)
        run_tables, run_h0, run_dht = plan.seg_tables, seg_h0, seg_dht
    else:
        run_tables, run_h0, run_dht = tables, h0, dht_k

    # K = V = 128: the sequential kernels hand h, v_new, dh, du to the chunk-parallel kernel as
    # ready-made operand tiles (written by TMA), not as row-major tensors
    tiles = _tiles_ok(D)
    if tiles and cached[1] is not None and cached[2] is not None:
        fw = {"h": cached[1], "vnew": cached[2]}  # kept by the forward: no recomputation
    else:
        fw = ops.fwd_seq(None, k, v, A, g, beta_k, scale, run_h0, output_o=False, output_h=True,
                         output_vnew=True, tables=run_tables, operand_tiles=tiles,
                         lead_chunks=lead if tiles else None)
    bw = ops.bwd_dh(q, k, A, g, beta_k, do, scale, run_dht, tables=run_tables,
                    operand_tiles=tiles, lead_chunks=lead_out)
    dq, dk, dv, db, dg = ops.bwd_main(q, k, v, fw["vnew"], A, g, beta_k, do, bw["du"], fw["h"],
                                      bw["dh"], scale, tables=run_tables, operand_tiles=tiles)
    dh0 = bw["dh0"]
    if plan is not None:
        dh0 = dh0[plan.first_seg_of_raw]
    if initial_state is None:
        dh0 = None
    dh0 = _state_out(dh0, state_v_first)
    dq, dk, dv, db, dg = finish_backward(dq, dk, dv, db, dg, Hq, beta.dtype, in_dtype, cu_seqlens)
    return dq, dk, dv, db, dg, dh0


def finish_backward(dq, dk, dv, db, dg, Hq, beta_dtype, in_dtype, cu_seqlens):
    """What follows the chunk-parallel backward kernel: the sum of dq, dk over the value heads
    of a group, the reverse chunk-local cumsum of dg, and the output dtypes."""
    if Hq < dq.shape[2]:
        dq = ops.group_reduce_vector(dq, Hq)
        dk = ops.group_reduce_vector(dk, Hq)
    dg = ops.chunk_local_cumsum(dg, CHUNK_SIZE, cu_seqlens, reverse=True)
    db = db.to(beta_dtype)
    if in_dtype != torch.bfloat16:
        dq, dk, dv = dq.to(in_dtype), dk.to(in_dtype), dv.to(in_dtype)
    return dq, dk, dv, db, dg


class ChunkGatedDeltaRuleFunction(torch.autograd.Function):
    @staticmethod
    @input_guard
    @torch.amp.custom_fwd(device_type="cuda")
    def forward(
        ctx,
        q: torch.Tensor,
        k: torch.Tensor,
        v: torch.Tensor,
        g: torch.Tensor,
        beta: torch.Tensor,
        scale: float | None = None,
        initial_state: torch.Tensor | None = None,
        output_final_state: bool = False,
        cu_seqlens: torch.LongTensor | None = None,
        use_qk_l2norm_in_kernel: bool = False,
        state_v_first: bool = False,
        auto_cp: bool = True,
        enable_fwd_cp_cache: bool = True,
    ):
        q_rstd, k_rstd = None, None
        if use_qk_l2norm_in_kernel:
            q, q_rstd = l2norm_fwd(q)
            k, k_rstd = l2norm_fwd(k)
        g_cum, A, o, _, final_state, cp_cache = chunk_gated_delta_rule_fwd(
            q=q, k=k, v=v, g=g, beta=beta, scale=scale, initial_state=initial_state,
            output_final_state=output_final_state, output_h=False, cu_seqlens=cu_seqlens,
            state_v_first=state_v_first, auto_cp=auto_cp,
            enable_fwd_cp_cache=enable_fwd_cp_cache,
        )
        cached = tuple(cp_cache) if cp_cache is not None else ()
        ctx.save_for_backward(q, k, q_rstd, k_rstd, v, g_cum, beta, A, initial_state, cu_seqlens,
                              *cached)
        ctx.n_cached = len(cached)
        ctx.g_dtype = g.dtype
        ctx.scale = scale
        ctx.state_v_first = state_v_first
        ctx.auto_cp = auto_cp
        ctx.use_qk_l2norm_in_kernel = use_qk_l2norm_in_kernel
        return o.to(q.dtype), final_state

    @staticmethod
    @input_guard
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, do: torch.Tensor, dht: torch.Tensor):
        saved = ctx.saved_tensors
        q, k, q_rstd, k_rstd, v, g_cum, beta, A, initial_state, cu_seqlens = saved[:10]
        cp_cache = tuple(saved[10:]) if ctx.n_cached else None
        dq, dk, dv, db, dg, dh0 = chunk_gated_delta_rule_bwd(
            q=q, k=k, v=v, g=g_cum, beta=beta, A=A, do=do, dht=dht, scale=ctx.scale,
            initial_state=initial_state, cu_seqlens=cu_seqlens,
            state_v_first=ctx.state_v_first, auto_cp=ctx.auto_cp, cp_cache=cp_cache,
        )
        if ctx.use_qk_l2norm_in_kernel:
            dq = l2norm_bwd(q, q_rstd, dq)
            dk = l2norm_bwd(k, k_rstd, dk)
        return (
            dq.to(q),
            dk.to(k),
            dv.to(v),
            dg.to(ctx.g_dtype),
            db.to(beta),
            None,
            dh0 if initial_state is not None else None,
            None,
            None,
            None,
            None,
            None,
            None,
        )


@torch.compiler.disable
def chunk_gated_delta_rule(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    beta: torch.Tensor,
    scale: float = None,
    initial_state: torch.Tensor = None,
    output_final_state: bool = False,
    use_qk_l2norm_in_kernel: bool = False,
    cu_seqlens: torch.LongTensor | None = None,
    head_first: bool = False,
    state_v_first: bool = False,
    auto_cp: bool = True,
    enable_fwd_cp_cache: bool = True,
):
    r"""Gated delta rule, chunked prefill, with autograd.

    Args follow the reference (``chunk/__init__.py:286-329``): ``q, k [B,T,H,K]``;
    ``v [B,T,HV,V]`` with ``HV`` a multiple of ``H`` (grouped value attention); ``g [B,T,HV]``
    log-space gates; ``beta [B,T,HV]``; ``initial_state [N,HV,K,V]``; ``cu_seqlens [N+1]`` for
    packed variable-length input (batch must be 1); ``state_v_first`` stores states as ``[V,K]``.
    Returns ``(o [B,T,HV,V], final_state [N,HV,K,V] or None)``.
    """
    assert q.dtype == k.dtype == v.dtype
    assert q.dtype == torch.bfloat16 or q.dtype == torch.float16, (
        "FlashQLA only supports bfloat16 and float16."
    )
    assert not head_first, "head_first=True is not supported."
    assert v.shape[2] % k.shape[2] == 0, "num_qk_heads must be divisible to num_v_heads."
    if cu_seqlens is not None:
        if q.shape[0] != 1:
            raise ValueError(
                f"The batch size is expected to be 1 rather than {q.shape[0]} when using "
                f"`cu_seqlens`. Please flatten variable-length inputs before processing."
            )
        if initial_state is not None and initial_state.shape[0] != len(cu_seqlens) - 1:
            raise ValueError(
                f"The number of initial states is expected to be equal to the number of input "
                f"sequences, i.e., {len(cu_seqlens) - 1} rather than {initial_state.shape[0]}."
            )
    if scale is None:
        scale = k.shape[-1] ** -0.5
    o, final_state = ChunkGatedDeltaRuleFunction.apply(
        q, k, v, g, beta, scale, initial_state, output_final_state, cu_seqlens,
        use_qk_l2norm_in_kernel, state_v_first, auto_cp, enable_fwd_cp_cache,
    )
    return o, final_state
