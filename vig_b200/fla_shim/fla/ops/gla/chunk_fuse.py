"""``fla.ops.gla.chunk_fuse``: ``FusedChunkGLAFunction``, ``pad`` and ``fused_chunk_gla``
(``fla/ops/gla/chunk_fuse.py:317-572`` of the reference)."""
import torch.nn.functional as F

from vig_b200.ops import fused_chunk_gla  # noqa: F401


def ceildiv(a, b):
    return -(a // -b)


def pad(x, chunk_size=16):
    """Zero-pad the token dimension to a multiple of ``chunk_size`` (``chunk_fuse.py:521-527``).  The CUDA kernels take
    any length, so callers need it no more; padded tokens (k = v = 0, log-gate 0) change nothing."""
    seq_len = x.shape[-2]
    padded = ceildiv(seq_len, chunk_size) * chunk_size
    if padded != seq_len:
        x = F.pad(x, (0, 0, 0, padded - seq_len))
    return x


class FusedChunkGLAFunction:
    """Only ``apply`` is offered, with the reference's positional arguments
    ``(q, k, v, g, scale, initial_state, output_final_state)`` and its ``(o, final_state)`` result
    (``chunk_fuse.py:317-408``); differentiable through ``vig_b200``'s own autograd function."""

    @staticmethod
    def apply(q, k, v, g, scale, initial_state, output_final_state):
        return fused_chunk_gla(q, k, v, g, scale=scale, initial_state=initial_state, output_final_state=output_final_state)
