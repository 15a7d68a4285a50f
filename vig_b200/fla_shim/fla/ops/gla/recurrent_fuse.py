"""``fla.ops.gla.recurrent_fuse``: the recurrent entry points (``fla/ops/gla/recurrent_fuse.py:631-685``)."""
from vig_b200.ops import bid_fused_recurrent_gla, fused_recurrent_gla  # noqa: F401

__all__ = ["bid_fused_recurrent_gla", "fused_recurrent_gla"]
