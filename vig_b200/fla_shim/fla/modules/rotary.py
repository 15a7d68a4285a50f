"""``fla.modules.rotary``: ``RotaryEmbedding`` (``fla/modules/rotary.py:137-310`` of the reference), which
``classification/models/vig.py:26`` imports and uses only with ``rope_mode='1d'`` in its training branch (no shipped
configuration sets it).  Plain PyTorch: rotary position embedding (RoFormer) over the first ``dim`` channels of
``[batch, seqlen, heads, headdim]`` tensors, first-half / second-half pairing unless ``interleaved``."""
import torch


class RotaryEmbedding(torch.nn.Module):
    def __init__(self, dim, base=10000.0, interleaved=False, scale_base=None, pos_idx_in_fp32=True, device=None):
        super().__init__()
        if scale_base is not None:
            raise NotImplementedError("the XPos scaling of the reference's class is not part of ViG's path")
        self.dim, self.base, self.interleaved = dim, float(base), interleaved
        inv_freq = 1.0 / (self.base ** (torch.arange(0, dim, 2, device=device, dtype=torch.float32) / dim))
        self.register_buffer("inv_freq", inv_freq, persistent=False)

    def _rotate(self, x, cos, sin):
        rot, rest = x[..., :self.dim], x[..., self.dim:]
        if self.interleaved:
            x1, x2 = rot[..., 0::2], rot[..., 1::2]
            out = torch.stack([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1).flatten(-2)
        else:
            x1, x2 = rot[..., :self.dim // 2], rot[..., self.dim // 2:]
            out = torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1)
        return torch.cat([out.to(x.dtype), rest], dim=-1)

    def forward(self, q, k, seqlen_offset=0, max_seqlen=None):
        """``q``, ``k``: ``[batch, seqlen, heads, headdim]``; position of token ``i`` is ``i + seqlen_offset``."""
        seqlen = q.shape[1]
        t = torch.arange(seqlen, device=q.device, dtype=torch.float32) + float(seqlen_offset)
        freqs = torch.outer(t, self.inv_freq.to(q.device, torch.float32))          # [seqlen, dim/2]
        cos, sin = freqs.cos()[None, :, None, :], freqs.sin()[None, :, None, :]
        return self._rotate(q.float(), cos, sin).to(q.dtype), self._rotate(k.float(), cos, sin).to(k.dtype)
