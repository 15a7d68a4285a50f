"""``fla.modules``: ``RMSNorm`` and ``FusedRMSNormSwishGate`` (``fla/modules/rmsnorm.py:491-512``,
``fla/modules/fused_norm_gate.py:514-536``)."""
import torch
import torch.nn as nn

from vig_b200 import ops
from vig_b200.modules import RMSNorm  # noqa: F401


class FusedRMSNormSwishGate(nn.Module):
    """``RMSNorm(x) * weight * o * sigmoid(o)`` (``fused_norm_gate.py:514-536``).  ViG's model files import it but never
    build one; it is here so that the import line resolves, as the norm kernel followed by the gate."""

    def __init__(self, hidden_size, eps=1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.register_parameter("bias", None)

    def forward(self, x, o, residual=None, prenorm=False, residual_in_fp32=False):
        res = ops.add_rmsnorm(x.contiguous(), self.weight, residual=residual, eps=self.eps, prenorm=prenorm)
        y, r = res if prenorm else (res, None)
        y = y * o * torch.sigmoid(o)
        return (y, r) if prenorm else y


__all__ = ["RMSNorm", "FusedRMSNormSwishGate"]
