"""Host utilities of the gated-delta-rule path (same names as the reference's ``flash_qla.utils``)."""

from .contiguous import input_guard
from .index import cdiv, prepare_chunk_indices, prepare_chunk_offsets, prepare_lens, tensor_cache
from .math import l2norm, l2norm_bwd, l2norm_fwd
from .pack import fill_last_chunk_of_g, pack, pad_and_reshape, unpack

__all__ = [
    "pad_and_reshape",
    "pack",
    "unpack",
    "fill_last_chunk_of_g",
    "l2norm",
    "l2norm_fwd",
    "l2norm_bwd",
    "prepare_chunk_indices",
    "prepare_chunk_offsets",
    "prepare_lens",
    "tensor_cache",
    "input_guard",
    "cdiv",
]
