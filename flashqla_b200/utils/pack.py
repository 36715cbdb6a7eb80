"""Packing helpers shared by the host code and the parity oracle.

Behavioural mirror of the reference's ``flash_qla/utils/pack.py:7-83``; every function
works on CPU and CUDA tensors alike.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


def _bounds(cu_seqlens: torch.Tensor) -> list[int]:
    assert cu_seqlens.dim() == 1
    return [int(x) for x in cu_seqlens.tolist()]


def unpack(x: torch.Tensor, cu_seqlens: torch.Tensor) -> torch.Tensor:
    """``[1, sum(len), ...]`` -> zero-padded ``[N, max(len), ...]`` (``utils/pack.py:7-22``)."""
    assert x.shape[0] == 1
    b = _bounds(cu_seqlens)
    lens = [e - s for s, e in zip(b[:-1], b[1:])]
    out = x.new_zeros((len(lens), max(lens), *x.shape[2:]))
    for i, (s, n) in enumerate(zip(b[:-1], lens)):
        out[i, :n] = x[0, s : s + n]
    return out


def pack(x: torch.Tensor, cu_seqlens: torch.Tensor) -> torch.Tensor:
    """``[N, >=max(len), ...]`` -> ``[1, sum(len), ...]`` (``utils/pack.py:25-38``)."""
    b = _bounds(cu_seqlens)
    out = x.new_empty((1, b[-1], *x.shape[2:]))
    for i, (s, e) in enumerate(zip(b[:-1], b[1:])):
        out[0, s:e] = x[i, : e - s]
    return out


def pad_and_reshape(x: torch.Tensor, dim: int, chunk_size: int = 64) -> torch.Tensor:
    """Zero-pad ``dim`` up to a chunk multiple and split it into ``[n_chunks, chunk_size]``
    (``utils/pack.py:41-52``)."""
    n = x.shape[dim]
    pad = (-n) % chunk_size
    trailing = x.dim() - 1 - dim
    padded = F.pad(x, (0, 0) * trailing + (0, pad))
    return padded.reshape(*x.shape[:dim], -1, chunk_size, *x.shape[dim + 1 :])


def fill_last_chunk_of_g(
    g: torch.Tensor,
    num_tokens: int,
    cu_seqlens: torch.Tensor | None,
    chunk_size: int = 64,
    reverse: bool = False,
) -> torch.Tensor:
    """Fix up the padded rows of the last chunk of a chunked gate tensor ``[N, n_chunks, C, ...]``.

    Forward: pad rows take the last valid cumulative gate.  Reverse (for gradients): the
    last pad row's value is folded into the last valid row.  In place, like the reference
    (``utils/pack.py:55-83``).
    """
    if cu_seqlens is None:
        spans = [(slice(None), num_tokens)]
    else:
        b = _bounds(cu_seqlens)
        spans = [(i, e - s) for i, (s, e) in enumerate(zip(b[:-1], b[1:]))]
    for sel, length in spans:
        tail = length % chunk_size
        if tail == 0:
            continue
        c = -1 if cu_seqlens is None else length // chunk_size
        if reverse:
            g[sel, c, tail - 1] += g[sel, c, -1]
        else:
            g[sel, c, tail:] = g[sel, c, tail - 1 : tail]
    return g
