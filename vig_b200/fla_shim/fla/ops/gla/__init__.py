"""``fla.ops.gla``: the three one-direction entry points (``fla/ops/gla/__init__.py`` of the reference)."""
from vig_b200.ops import chunk_gla, fused_chunk_gla, fused_recurrent_gla  # noqa: F401

__all__ = ["chunk_gla", "fused_chunk_gla", "fused_recurrent_gla"]
