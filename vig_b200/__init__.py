"""B200-native bi-directional gated linear attention and ViG block kernels behind the reference's operator API."""
from .ops import (bi_gla, bi_gla_backward, bid_fused_recurrent_gla, fused_chunk_gla, chunk_gla, fused_recurrent_gla,  # noqa: F401
                  dwconv3x3, gate_inject, add_rmsnorm, layernorm_act, swiglu, swiglu_linear, linear_swiglu,
                  check_status, status_word)
from .modules import RMSNorm, GatedLinearAttention, GLAMLP, GLABlock  # noqa: F401
from .vig import ViG, build_vig  # noqa: F401
from .hier import HierViG, GLA2D, VSSBlock  # noqa: F401
