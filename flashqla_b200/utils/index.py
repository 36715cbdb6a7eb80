"""Chunk index tables for packed variable-length input, and the identity-keyed memo
that keeps them off the critical path.

Mirrors the behaviour of the reference's ``flash_qla/utils/index.py:11-107``
(``tensor_cache``, ``prepare_lens``, ``prepare_chunk_indices``, ``prepare_chunk_offsets``):
the tables must come out bit-identical, in the dtype and on the device of ``cu_seqlens``.
Unlike the reference these helpers also work on CPU tensors (the parity oracle runs there).
"""

from __future__ import annotations

import functools
from typing import Any, Callable

import torch

_CACHE_SLOTS = 4


def _is_capturing() -> bool:
    return torch.cuda.is_available() and torch.cuda.is_current_stream_capturing()


def _same_arg(a, b) -> bool:
    """Tensors (and other objects) are compared by identity, plain numbers by value: two equal
    ints are not guaranteed to be the same object."""
    if isinstance(a, (int, float, bool, str)) and type(a) is type(b):
        return a == b
    return a is b


def tensor_cache(fn: Callable[..., Any]) -> Callable[..., Any]:
    """Memoise ``fn`` on the *identity* of its arguments (reference: ``utils/index.py:11-76``).

    Up to four recent results are kept, least-recently-used first out.  A result that is
    looked up while a CUDA graph is being captured becomes pinned: it is never evicted, so
    the device tensors a captured graph refers to stay alive.  A miss during capture is an
    error, because building a table needs a host round trip.
    """

    entries: list[list[Any]] = []  # [args, kwargs, result, pinned]

    def _same(args, kwargs, e_args, e_kwargs) -> bool:
        if len(args) != len(e_args) or len(kwargs) != len(e_kwargs):
            return False
        if any(not _same_arg(a, b) for a, b in zip(args, e_args)):
            return False
        return all(k in e_kwargs and _same_arg(v, e_kwargs[k]) for k, v in kwargs.items())

    @functools.wraps(fn)
    def wrapper(*args: Any, **kwargs: Any) -> Any:
        capturing = _is_capturing()
        for pos, entry in enumerate(entries):
            if _same(args, kwargs, entry[0], entry[1]):
                if capturing:
                    entry[3] = True
                elif not entry[3]:
                    entries.append(entries.pop(pos))
                return entry[2]
        if capturing:
            raise AssertionError(
                f"tensor_cache miss during CUDA graph capture: {fn.__name__}"
            )
        result = fn(*args, **kwargs)
        unpinned = [e for e in entries if not e[3]]
        if len(unpinned) >= _CACHE_SLOTS:
            # by identity: list.remove would compare the cached tensors element by element
            del entries[next(i for i, e in enumerate(entries) if e is unpinned[0])]
        entries.append([args, kwargs, result, False])
        return result

    wrapper.cache_entries = entries  # exposed for tests
    return wrapper


def cdiv(a, b):
    return (a + b - 1) // b


@tensor_cache
def prepare_lens(cu_seqlens: torch.Tensor) -> torch.Tensor:
    return torch.diff(cu_seqlens)


@tensor_cache
def prepare_chunk_indices(cu_seqlens: torch.Tensor, chunk_size: int) -> torch.Tensor:
    """``[NT, 2]`` table of (sequence id, chunk id within the sequence), one row per chunk.

    Reference: ``utils/index.py:84-95``.  Chunks are aligned to each sequence start.
    """
    counts = cdiv(prepare_lens(cu_seqlens), chunk_size).tolist()
    seq_ids, chunk_ids = [], []
    started = -1  # the reference numbers sequences by counting chunk-0 rows, so an
    for n in counts:  # empty sequence does not consume an id; keep that
        for c in range(n):
            started += c == 0
            seq_ids.append(started)
            chunk_ids.append(c)
    table = torch.tensor(list(zip(seq_ids, chunk_ids)), dtype=torch.int64).reshape(-1, 2)
    return table.to(cu_seqlens).contiguous()  # row-major: the kernels index it as [2*i + j]


@tensor_cache
def prepare_chunk_offsets(cu_seqlens: torch.Tensor, chunk_size: int):
    """``[N+1]`` exclusive prefix sum of per-sequence chunk counts, plus the total as an int.

    Reference: ``utils/index.py:98-107``.
    """
    counts = cdiv(torch.diff(cu_seqlens), chunk_size)
    offsets = torch.zeros_like(cu_seqlens)
    offsets[1:] = torch.cumsum(counts, dim=0)
    return offsets, int(offsets[-1].item())
