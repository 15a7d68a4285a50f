"""``fla.models``: ``GLAConfig`` (``fla/models/gla/configuration_gla.py``) as a plain attribute bag.

The reference's class derives from ``transformers.PretrainedConfig``; ViG only builds one and reads attributes from it
(``classification/models/vig.py:750-766, 531-580``), including ones the constructor does not name (they arrive through
``**kwargs`` and become attributes, which is what ``PretrainedConfig`` does with unknown keys)."""
from typing import Optional


class GLAConfig:
    model_type = "gla"

    def __init__(self, vocab_size: int = 32000, hidden_size: int = 2048, expand_k: float = 0.5, expand_v: float = 1,
                 hidden_ratio: Optional[int] = 4, intermediate_size: Optional[int] = None, num_hidden_layers: int = 24,
                 num_heads: int = 4, attn_mode: str = "chunk", use_short_conv: bool = False, conv_size: int = 4,
                 share_conv_kernel: bool = True, clamp_min: Optional[float] = None, hidden_act: str = "swish",
                 max_position_embeddings: int = 2048, rms_norm_eps: float = 1e-6, use_gk: bool = True, use_gv: bool = False,
                 use_cache: bool = True, initializer_range: float = 0.02, fuse_norm: bool = True,
                 fuse_cross_entropy: bool = True, **kwargs):
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self.expand_k, self.expand_v = expand_k, expand_v
        self.hidden_ratio, self.intermediate_size = hidden_ratio, intermediate_size
        self.num_hidden_layers, self.num_heads = num_hidden_layers, num_heads
        self.attn_mode, self.use_short_conv, self.conv_size = attn_mode, use_short_conv, conv_size
        self.share_conv_kernel, self.clamp_min, self.hidden_act = share_conv_kernel, clamp_min, hidden_act
        self.max_position_embeddings, self.rms_norm_eps = max_position_embeddings, rms_norm_eps
        self.use_gk, self.use_gv, self.use_cache = use_gk, use_gv, use_cache
        self.initializer_range, self.fuse_norm, self.fuse_cross_entropy = initializer_range, fuse_norm, fuse_cross_entropy
        for name, value in kwargs.items():
            setattr(self, name, value)


__all__ = ["GLAConfig"]
