"""Alias of the chunk-local cumsum and GVA group-sum wrappers under the reference's path."""

from flashqla_b200.ops import chunk_local_cumsum, group_reduce_vector

__all__ = ["chunk_local_cumsum", "group_reduce_vector"]
