"""Alias of ``flashqla_b200.api`` under the reference's orchestrator module path."""

from flashqla_b200.api import (
    ChunkGatedDeltaRuleFunction,
    chunk_gated_delta_rule,
    chunk_gated_delta_rule_bwd,
    chunk_gated_delta_rule_fwd,
)
from flashqla_b200.ops import CHUNK_SIZE

__all__ = [
    "ChunkGatedDeltaRuleFunction",
    "chunk_gated_delta_rule",
    "chunk_gated_delta_rule_fwd",
    "chunk_gated_delta_rule_bwd",
    "CHUNK_SIZE",
]
