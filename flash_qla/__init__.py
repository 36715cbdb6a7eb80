"""Drop-in import path: ``flash_qla`` resolves to the B200-native implementation
(same public names as the reference's ``flash_qla/__init__.py:6-16``)."""

from flashqla_b200 import __version__  # noqa: F401
from flash_qla.ops.gated_delta_rule.chunk import (
    chunk_gated_delta_rule,
    chunk_gated_delta_rule_bwd,
    chunk_gated_delta_rule_fwd,
)

__all__ = [
    "chunk_gated_delta_rule_fwd",
    "chunk_gated_delta_rule_bwd",
    "chunk_gated_delta_rule",
]
