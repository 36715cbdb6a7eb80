"""flashqla_b200: gated-delta-rule chunked prefill (forward and backward) for NVIDIA B200.

Hand-written sm_100a CUDA kernels behind a C ABI (``include/fqla.h``,
``libfqla_sm100.so``), driven through the same Python operator API as the reference
``flash_qla`` package.
"""

__version__ = "0.1.0"

from .api import (  # noqa: E402
    ChunkGatedDeltaRuleFunction,
    chunk_gated_delta_rule,
    chunk_gated_delta_rule_bwd,
    chunk_gated_delta_rule_fwd,
)

__all__ = [
    "chunk_gated_delta_rule",
    "chunk_gated_delta_rule_fwd",
    "chunk_gated_delta_rule_bwd",
    "ChunkGatedDeltaRuleFunction",
]
