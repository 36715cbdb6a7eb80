"""Argument hygiene for the autograd entry points (reference: ``flash_qla/utils/contiguous.py:10-41``)."""

from __future__ import annotations

import contextlib
import functools

import torch


def input_guard(fn):
    """Make every tensor argument contiguous and run ``fn`` with the first tensor's CUDA
    device current, so that kernels launch on that device's current stream."""

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        args = tuple(a.contiguous() if isinstance(a, torch.Tensor) else a for a in args)
        kwargs = {k: (v.contiguous() if isinstance(v, torch.Tensor) else v) for k, v in kwargs.items()}
        first = next(
            (t for t in list(args) + list(kwargs.values()) if isinstance(t, torch.Tensor)), None
        )
        if first is not None and first.is_cuda:
            guard = torch.cuda.device(first.device.index)
        else:
            guard = contextlib.nullcontext()
        with guard:
            return fn(*args, **kwargs)

    return wrapper
