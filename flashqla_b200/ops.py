"""Tensor-level wrappers of the C-ABI kernels.

Each function checks shapes and dtypes on the host, allocates outputs with torch, and enqueues
one kernel of ``libfqla_sm100.so`` on the current CUDA stream.  Names and argument meaning follow
the reference's kernel wrappers (``chunk_local_cumsum``, ``kkt_solve``, ``fused_gdr_fwd``,
``fused_gdr_h``, ``fused_gdr_bwd``, ``group_reduce_vector``, ``get_warmup_chunks``,
``correct_initial_states``) where one exists.
"""

from __future__ import annotations

import functools

import torch

from . import _lib
from .utils import prepare_chunk_indices, prepare_chunk_offsets, tensor_cache

CHUNK_SIZE = 64


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream(t: torch.Tensor):
    return torch.cuda.current_stream(t.device).cuda_stream


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise _lib.FqlaError(
                "flashqla_b200 kernels need CUDA tensors; there is no CPU fallback"
            )


def on_tensor_device(fn):
    """Run ``fn`` with the device of its first CUDA tensor argument current.  The C entry points
    launch on the current device (kernel attributes, the SM count and the status word are per
    device), while callers may hold tensors of another one."""

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        t = next((a for a in (*args, *kwargs.values())
                  if isinstance(a, torch.Tensor) and a.is_cuda), None)
        if t is None or t.device.index == torch.cuda.current_device():
            return fn(*args, **kwargs)
        with torch.cuda.device(t.device):
            return fn(*args, **kwargs)

    return wrapper


class SeqTables:
    """Index tables of a (possibly packed) batch: device tensors plus host-side counts."""

    def __init__(self, B: int, T: int, cu_seqlens: torch.Tensor | None):
        self.B, self.T, self.cu = B, T, cu_seqlens
        if cu_seqlens is None:
            self.N = B
            self.num_chunks = B * ((T + CHUNK_SIZE - 1) // CHUNK_SIZE)
            self.chunk_indices = self.chunk_offsets = None
            self.is64 = 0
        else:
            if cu_seqlens.dtype not in (torch.int32, torch.int64):
                raise TypeError("cu_seqlens must be int32 or int64")
            if B != 1:
                raise ValueError("packed input (cu_seqlens) needs batch size 1")
            self.N = cu_seqlens.numel() - 1
            self.chunk_indices = _kernel_chunk_indices(cu_seqlens)
            self.chunk_offsets, self.num_chunks = prepare_chunk_offsets(cu_seqlens, CHUNK_SIZE)
            self.is64 = int(cu_seqlens.dtype == torch.int64)
        # block index -> sequence, longest first (None: identity)
        self.order = None if cu_seqlens is None or self.N < 2 else _longest_first(cu_seqlens)

    @property
    def total(self) -> int:
        """Rows covered by sequences (host int, cached per ``cu_seqlens`` tensor)."""
        return self.B * self.T if self.cu is None else _total_rows(self.cu)

    @property
    def args(self):
        return _ptr(self.cu), _ptr(self.chunk_offsets), self.is64, self.N


@tensor_cache
def _kernel_chunk_indices(cu_seqlens: torch.Tensor) -> torch.Tensor:
    """``[NT, 2]`` (sequence, chunk in sequence) rows for the chunk-parallel kernels.  The public
    ``prepare_chunk_indices`` keeps the reference's numbering, in which a zero-length sequence
    does not consume a sequence id; the kernels index ``cu_seqlens`` with the id, so they get
    the position of the sequence in ``cu_seqlens`` instead.  Without zero-length sequences the
    two tables are the same tensor."""
    table = prepare_chunk_indices(cu_seqlens, CHUNK_SIZE)
    lens = torch.diff(cu_seqlens)
    if bool((lens > 0).all()):
        return table
    counts = (lens + CHUNK_SIZE - 1) // CHUNK_SIZE
    seq = torch.repeat_interleave(torch.arange(lens.numel(), device=cu_seqlens.device), counts)
    fixed = table.clone()
    fixed[:, 0] = seq.to(table.dtype)
    return fixed


@tensor_cache
def _longest_first(cu_seqlens: torch.Tensor) -> torch.Tensor:
    """int32 ``[N]``: the sequences sorted by length, longest first.  The sequential kernels start
    their CTAs in block-index order; handing the long sequences out first shortens the tail of a
    ragged batch (computed on the device, cached per ``cu_seqlens`` tensor)."""
    return torch.argsort(torch.diff(cu_seqlens), descending=True, stable=True).to(torch.int32)


@tensor_cache
def _total_rows(cu_seqlens: torch.Tensor) -> int:
    return int(cu_seqlens[-1].item())


def _beta_flag(beta: torch.Tensor) -> int:
    if beta.dtype == torch.float32:
        return 1
    if beta.dtype == torch.bfloat16:
        return 0
    raise TypeError(f"beta must be bfloat16 or float32, got {beta.dtype}")


def _check_bf16(**named):
    for name, t in named.items():
        if t is not None and t.dtype != torch.bfloat16:
            raise NotImplementedError(
                f"{name}: the sm_100a kernels are built for bfloat16 (got {t.dtype})"
            )


@on_tensor_device
def chunk_local_cumsum(g, chunk_size: int = CHUNK_SIZE, cu_seqlens=None, reverse: bool = False):
    """Chunk-local prefix (or suffix) sum of ``g [B,T,H]`` fp32
    (reference: ``ops/utils/cumsum.py:137-171``)."""
    assert chunk_size == CHUNK_SIZE, "chunk size is fixed at 64"
    _require_cuda(g)
    assert g.dtype == torch.float32 and g.is_contiguous()
    B, T, H = g.shape
    tb = SeqTables(B, T, cu_seqlens)
    out = torch.empty_like(g)
    if tb.total < B * T:  # rows past the last packed sequence come out zero
        out[:, tb.total:].zero_()
    st = _lib.load().fqla_chunk_local_cumsum(
        _ptr(g), _ptr(out), B, T, H, _ptr(tb.cu), tb.is64, tb.N, _ptr(tb.chunk_indices),
        tb.num_chunks, int(reverse), _stream(g))
    _lib.check(st, "chunk_local_cumsum")
    return out


@on_tensor_device
def kkt_solve(k, b, g_cum, cu_seqlens=None, chunk_size: int = CHUNK_SIZE, raw_gate: bool = False):
    """``A = (I + strict_lower(diag(b) K K^T * decay))^-1`` per (chunk, value head), bf16
    ``[B,T,Hv,64]`` (reference: ``blackwell/kkt_solve.py:284-324``; the gate is folded in).
    With ``raw_gate`` the third argument is the raw per-token log gate, its chunk-local cumsum is
    formed in the same kernel, and ``(g_cum, A)`` is returned."""
    assert chunk_size == CHUNK_SIZE
    _require_cuda(k, b, g_cum)
    _check_bf16(k=k)
    B, T, Hq, D = k.shape
    Hv = b.shape[-1]
    tb = SeqTables(B, T, cu_seqlens)
    A = torch.empty(B, T, Hv, CHUNK_SIZE, dtype=k.dtype, device=k.device)
    g_out = None
    if raw_gate:
        assert g_cum.dtype == torch.float32 and g_cum.is_contiguous()
        g_out = torch.empty_like(g_cum)
        if tb.total < B * T:  # rows past the last packed sequence: zero, as the cumsum kernel leaves them
            g_out[:, tb.total:].zero_()
    st = _lib.load().fqla_kkt_solve(
        _ptr(k), _ptr(b), _beta_flag(b), _ptr(g_cum), _ptr(g_out), _ptr(A), B, T, Hq, Hv, D,
        _ptr(tb.cu), tb.is64, _ptr(tb.chunk_indices), tb.num_chunks, _stream(k))
    _lib.check(st, "kkt_solve")
    return (g_out, A) if raw_gate else A


def fwd_seq_outputs(k, v, tb: SeqTables, output_o=True, output_h=False, output_vnew=False,
                    output_final_state=False, output_m=False, operand_tiles=False) -> dict:
    """The output tensors of ``fwd_seq`` (allocated on the current stream), for callers that
    fill them with more than one launch (``out=``)."""
    D, Hv, dev = k.shape[-1], v.shape[2], k.device
    out = {}
    if output_o:
        out["o"] = torch.empty_like(v)
    if output_h:
        out["h"] = torch.empty(tb.num_chunks, Hv, D, D, dtype=k.dtype, device=dev)
    if output_vnew:
        out["vnew"] = (torch.empty(tb.num_chunks, Hv, D, CHUNK_SIZE, dtype=k.dtype, device=dev)
                       if operand_tiles else torch.empty_like(v))
    if output_final_state:
        out["ht"] = torch.empty(tb.N, Hv, D, D, dtype=torch.float32, device=dev)
    if output_m:
        out["M"] = torch.empty(tb.N, Hv, D, D, dtype=torch.float32, device=dev)
    return out


@on_tensor_device
def fwd_seq(q, k, v, a, g_cum, b, scale, initial_state=None, *, output_final_state=False,
            output_o=True, output_h=False, output_vnew=False, output_m=False,
            warm_chunks=None, m_mask=None, cu_seqlens=None, tables: SeqTables | None = None,
            operand_tiles: bool = False, lead_chunks=None, run_mask=None, run_value: int = 1,
            out: dict | None = None):
    """Sequential forward recurrence.  Returns a dict with the requested outputs among
    ``o, h, vnew, ht, M`` (reference: ``blackwell/fused_fwd.py:775-915`` and
    ``blackwell/prepare_h.py:669-784``).  With ``operand_tiles`` (K = V = 128 only) ``h`` comes
    out as ``[chunks, Hv, V, K]`` and ``vnew`` as ``[chunks, Hv, V, 64]``: the layouts
    ``bwd_main(..., operand_tiles=True)`` reads as tensor-core operands.  ``lead_chunks``
    (int32 ``[N, Hv]``, K = V = 128): per (segment, head) the number of chunks before the segment
    to walk first, state-only, from a zero state (see ``segment_scan``).  ``run_mask``
    (int32 ``[N, Hv]``) with ``run_value``: only the pairs whose entry equals ``run_value`` are
    walked; with ``out`` (the dict a first call returned) a second call with the other value
    fills the rest of the same tensors."""
    _require_cuda(k, v, a, g_cum, b)
    _check_bf16(q=q, k=k, v=v, a=a)
    B, T, Hq, D = k.shape
    Hv = v.shape[2]
    tb = tables or SeqTables(B, T, cu_seqlens)
    if out is None:
        assert q is not None or not output_o
        out = fwd_seq_outputs(k, v, tb, output_o, output_h, output_vnew, output_final_state,
                              output_m, operand_tiles)
    if initial_state is not None:
        assert initial_state.dtype == torch.float32 and initial_state.is_contiguous()
        assert tuple(initial_state.shape) == (tb.N, Hv, D, D), (
            f"initial_state must be [{tb.N},{Hv},{D},{D}], got {tuple(initial_state.shape)}")
    cu, offs, is64, N = tb.args
    st = _lib.load().fqla_fwd_seq(
        _ptr(q) if output_o else None, _ptr(k), _ptr(v), _ptr(a), _ptr(g_cum), _ptr(b),
        _beta_flag(b), _ptr(initial_state), _ptr(out.get("ht")), _ptr(out.get("o")),
        _ptr(out.get("h")), _ptr(out.get("vnew")), _ptr(out.get("M")), _ptr(warm_chunks),
        _ptr(m_mask), _ptr(lead_chunks), _ptr(tb.order), _ptr(run_mask), int(run_value), tb.B,
        tb.T, Hq, Hv, D, float(scale), cu, offs, is64, N, int(operand_tiles), _stream(k))
    _lib.check(st, "fwd_seq")
    return out


def bwd_dh_outputs(k, do, tb: SeqTables, output_dh=True, output_du=True, output_dh0=True,
                   operand_tiles=False) -> dict:
    """The output tensors of ``bwd_dh`` (allocated on the current stream), see ``out=``."""
    D, Hv, dev = k.shape[-1], do.shape[2], k.device
    out = {}
    if output_dh:
        out["dh"] = torch.empty(tb.num_chunks, Hv, D, D, dtype=k.dtype, device=dev)
    if output_du:
        out["du"] = (torch.empty(tb.num_chunks, Hv, D, CHUNK_SIZE, dtype=k.dtype, device=dev)
                     if operand_tiles else torch.empty_like(do))
    if output_dh0:
        out["dh0"] = torch.empty(tb.N, Hv, D, D, dtype=torch.float32, device=dev)
    return out


@on_tensor_device
def bwd_dh(q, k, a, g_cum, b, do, scale, dht=None, *, output_dh=True, output_du=True,
           output_dh0=True, warm_chunks=None, lead_chunks=None, cu_seqlens=None,
           tables: SeqTables | None = None, operand_tiles: bool = False, run_mask=None,
           run_value: int = 1, out: dict | None = None):
    """Reverse recurrence of the state gradient; returns a dict with ``dh, du, dh0``
    (reference: ``blackwell/cp_bwd.py:592-701`` and the dS chain of ``blackwell/fused_bwd.py``).
    ``operand_tiles``: ``dh`` as ``[chunks, Hv, V, K]``, ``du`` as ``[chunks, Hv, V, 64]``.
    ``lead_chunks`` (``[N, Hv]`` int32, segments of a split plan): segment ``n`` starts that many
    chunks after its end from a zero gradient instead of taking ``dht[n]``.  ``run_mask``,
    ``run_value``, ``out``: as for ``fwd_seq``."""
    _require_cuda(q, k, a, g_cum, b, do)
    _check_bf16(q=q, k=k, a=a, do=do)
    B, T, Hq, D = k.shape
    Hv = do.shape[2]
    tb = tables or SeqTables(B, T, cu_seqlens)
    if out is None:
        out = bwd_dh_outputs(k, do, tb, output_dh, output_du, output_dh0, operand_tiles)
    if dht is not None:
        assert dht.dtype == torch.float32 and dht.is_contiguous()
        assert tuple(dht.shape) == (tb.N, Hv, D, D)
    cu, offs, is64, N = tb.args
    st = _lib.load().fqla_bwd_dh(
        _ptr(q), _ptr(k), _ptr(a), _ptr(g_cum), _ptr(b), _beta_flag(b), _ptr(do), _ptr(dht),
        _ptr(out.get("dh")), _ptr(out.get("du")), _ptr(out.get("dh0")), _ptr(warm_chunks),
        _ptr(lead_chunks), _ptr(tb.order), _ptr(run_mask), int(run_value), tb.B, tb.T, Hq, Hv, D, float(scale), cu, offs, is64, N, int(operand_tiles),
        _stream(k))
    _lib.check(st, "bwd_dh")
    return out


@on_tensor_device
def bwd_main(q, k, v, vnew, a, g_cum, b, do, du, h, dh, scale, cu_seqlens=None,
             tables: SeqTables | None = None, operand_tiles: bool = False):
    """Chunk-parallel backward.  Returns ``(dq_v, dk_v, dv, db, dg)`` with dq_v/dk_v per value
    head and ``dg`` before its reverse cumsum (reference: ``blackwell/fused_bwd.py:1325-1413``)."""
    _require_cuda(q, k, v, vnew, a, g_cum, b, do, du, h, dh)
    _check_bf16(q=q, k=k, v=v, vnew=vnew, a=a, do=do, du=du, h=h, dh=dh)
    B, T, Hq, D = k.shape
    Hv = v.shape[2]
    tb = tables or SeqTables(B, T, cu_seqlens)
    dev = k.device
    dq = torch.empty(B, T, Hv, D, dtype=k.dtype, device=dev)
    dk = torch.empty(B, T, Hv, D, dtype=k.dtype, device=dev)
    dv = torch.empty(B, T, Hv, D, dtype=k.dtype, device=dev)
    db = torch.empty(B, T, Hv, dtype=torch.float32, device=dev)
    dg = torch.empty(B, T, Hv, dtype=torch.float32, device=dev)
    if tb.total < B * T:  # rows past the last packed sequence are never written by the kernel
        for t in (dq, dk, dv, db, dg):
            t[:, tb.total:].zero_()
    cu, offs, is64, _ = tb.args
    st = _lib.load().fqla_bwd_main(
        _ptr(q), _ptr(k), _ptr(v), _ptr(vnew), _ptr(a), _ptr(g_cum), _ptr(b), _beta_flag(b),
        _ptr(do), _ptr(du), _ptr(h), _ptr(dh), _ptr(dq), _ptr(dk), _ptr(dv), _ptr(db), _ptr(dg),
        tb.B, tb.T, Hq, Hv, D, float(scale), cu, offs, _ptr(tb.chunk_indices), is64, tb.num_chunks,
        int(operand_tiles), _stream(k))
    _lib.check(st, "bwd_main")
    return dq, dk, dv, db, dg


@on_tensor_device
def group_reduce_vector(x, num_groups: int):
    """``[B,T,Hv,D] -> [B,T,num_groups,D]`` summing each run of ``Hv/num_groups`` heads
    (reference: ``ops/utils/group_reduce.py:60-79``)."""
    _require_cuda(x)
    _check_bf16(x=x)
    B, T, Hv, D = x.shape
    assert Hv % num_groups == 0
    G = Hv // num_groups
    if G == 1:
        return x
    out = torch.empty(B, T, num_groups, D, dtype=x.dtype, device=x.device)
    st = _lib.load().fqla_group_reduce(_ptr(x), _ptr(out), B * T, num_groups, G, D, _stream(x))
    _lib.check(st, "group_reduce_vector")
    return out


@on_tensor_device
def warmup_scan(g_cum, seg_cu_seqlens, threshold: float = -10.0, from_start: bool = False,
                keep=None):
    """Per (segment, head) warm-up chunk count and fallback flag, both int32 ``[n_seg, Hv]``
    (reference: ``blackwell/cp_fwd.py:81-115``, ``:224-264``).  ``keep`` (int32 ``[n_seg]``)
    marks with 0 the segments that hand nothing on: they get 0 / 0."""
    _require_cuda(g_cum, seg_cu_seqlens)
    B, T, Hv = g_cum.shape
    n_seg = seg_cu_seqlens.numel() - 1
    warm = torch.empty(n_seg, Hv, dtype=torch.int32, device=g_cum.device)
    fallback = torch.empty_like(warm)
    st = _lib.load().fqla_warmup_scan(
        _ptr(g_cum), T, Hv, _ptr(seg_cu_seqlens), int(seg_cu_seqlens.dtype == torch.int64), n_seg,
        float(threshold), int(from_start), _ptr(keep), _ptr(warm), _ptr(fallback),
        _stream(g_cum))
    _lib.check(st, "warmup_scan")
    return warm, fallback


@on_tensor_device
def segment_scan(g_cum, seg_cu_seqlens, seg_begin, threshold: float = -10.0,
                 from_start: bool = False):
    """The warm-up scan of a whole split plan plus the decision how each segment gets its start
    state; returns int32 tensors ``(warm, fallback, lead, exact_warm)`` of shape ``[n_seg, Hv]``
    and ``any_fallback [n_raw, Hv]`` (``include/fqla.h``: ``fqla_segment_scan``; reference:
    ``blackwell/cp_fwd.py:81-115``, ``:224-264`` and ``chunk/cp_context.py:148-227``)."""
    _require_cuda(g_cum, seg_cu_seqlens, seg_begin)
    B, T, Hv = g_cum.shape
    n_seg, n_raw = seg_cu_seqlens.numel() - 1, seg_begin.numel() - 1
    assert seg_begin.dtype == torch.int32
    tables = torch.empty(4, n_seg, Hv, dtype=torch.int32, device=g_cum.device)
    any_fb = torch.empty(n_raw, Hv, dtype=torch.int32, device=g_cum.device)
    st = _lib.load().fqla_segment_scan(
        _ptr(g_cum), T, Hv, _ptr(seg_cu_seqlens), int(seg_cu_seqlens.dtype == torch.int64),
        _ptr(seg_begin), n_raw, float(threshold), int(from_start), _ptr(tables[0]),
        _ptr(tables[1]), _ptr(tables[2]), _ptr(tables[3]), _ptr(any_fb), _stream(g_cum))
    _lib.check(st, "segment_scan")
    return tables[0], tables[1], tables[2], tables[3], any_fb


@on_tensor_device
def merge_states(local, M, use_m, raw, seg_begin, reverse: bool = False, any_fallback=None):
    """Chain the segment states of every raw sequence; returns the per-segment start states
    (or, reversed, end gradients) fp32 ``[n_seg, Hv, D, D]``
    (reference: ``blackwell/cp_fwd.py:483-610``).  With ``any_fallback`` (from ``segment_scan``)
    sequences without a chain only get their edge entry written; the other entries of the result
    are then undefined (their segments lead in by themselves).  ``local``, ``M`` and ``use_m``
    may be views into the records of one buffer (the output of an all-gather): their entries must
    be contiguous per segment and share one stride between segments."""
    _require_cuda(local, M, seg_begin)
    n_seg, Hv, D, _ = local.shape
    n_raw = seg_begin.numel() - 1
    assert seg_begin.dtype == torch.int32
    seg_stride = 0
    if not local.is_contiguous():
        seg_stride = local.stride(0)
        assert local[0].is_contiguous() and M[0].is_contiguous() and M.stride(0) == seg_stride
        assert use_m is None or (use_m.stride(0) == seg_stride and use_m.stride(1) == 1
                                 and use_m.element_size() == 4)
    else:
        assert M.is_contiguous() and (use_m is None or use_m.is_contiguous())
    out = torch.empty(n_seg, Hv, D, D, dtype=local.dtype, device=local.device)
    st = _lib.load().fqla_merge_states(
        _ptr(local), _ptr(M), _ptr(use_m), _ptr(raw), _ptr(seg_begin), _ptr(any_fallback),
        _ptr(out), n_raw, Hv, D, int(reverse), seg_stride, _stream(local))
    _lib.check(st, "merge_states")
    return out
