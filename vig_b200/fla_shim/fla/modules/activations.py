"""``fla.modules.activations``: ``swiglu`` and ``swiglu_linear`` (``fla/modules/activations.py:109-174``)."""
from vig_b200.ops import swiglu, swiglu_linear  # noqa: F401

__all__ = ["swiglu", "swiglu_linear"]
