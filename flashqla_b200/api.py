"""Operator API of the package.  The definitions sit under the reference's module path,
``flash_qla/ops/gated_delta_rule/chunk/__init__.py``; this module re-exports them so that
``flashqla_b200.api`` and ``flash_qla.ops.gated_delta_rule.chunk`` are one and the same set of
objects (module-level switches such as ``SAVE_STATE_TILES`` must be set on the latter)."""

from flash_qla.ops.gated_delta_rule.chunk import (  # noqa: F401
    CHUNK_SIZE,
    ChunkGatedDeltaRuleFunction,
    chunk_gated_delta_rule,
    chunk_gated_delta_rule_bwd,
    chunk_gated_delta_rule_fwd,
    run_forward,
)
