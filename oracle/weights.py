"""Seeded synthetic weights and inputs shared by the oracle, the tests and the benchmark.

ImageNet-1K and the released checkpoints are not available offline, so weights are drawn
from a NumPy ``Generator`` (a bit stream that does not depend on the torch version) with
the reference's initialisation scales: Linear N(0, 0.02) (``classification/models/vig.py:832-837``),
GLA projections and the depthwise conv xavier-uniform with gain 2^-2.5 (``vig.py:332-349``),
norm weights 1, pos-embed N(0, 0.02) truncated at 2 sigma (``vig.py:825``).  Parity never
depends on the law: the same state dict is loaded into both sides.
"""
import math
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch


@dataclass(frozen=True)
class ViGShape:
    """Model hyper-parameters (``classification/configs/vig/vig-{t,s,b}.yaml``)."""
    embed_dim: int = 192
    num_heads: int = 3
    depth: int = 12
    expand_k: float = 0.5
    expand_v: float = 1.0
    use_act_in_conv: bool = True
    use_out_act: bool = False
    num_classes: int = 1000
    pretrain_grid: int = 14
    gate_low_rank_dim: int = 16
    gate_logit_normalizer: int = 16
    clamp_min: Optional[float] = None
    eps: float = 1e-6

    @property
    def key_dim(self):
        return int(self.embed_dim * self.expand_k)

    @property
    def value_dim(self):
        return int(self.embed_dim * self.expand_v)

    @property
    def intermediate_size(self):
        i = int(self.embed_dim * 4 * 2 / 3)
        return 256 * ((i + 255) // 256)


# "ref" = the shipped YAMLs (dk=32); "dk64" = the benchmark configuration (expand_k 1.0 -> dk=dv=64).
PRESETS = {
    "vig_t": ViGShape(192, 3, 12, 0.5, 1.0, True, True),
    "vig_s": ViGShape(384, 6, 12, 0.5, 1.0, False, False),
    "vig_b": ViGShape(768, 12, 12, 0.5, 1.0, False, False),
    "vig_t_dk64": ViGShape(192, 3, 12, 1.0, 1.0, True, True),
    "vig_s_dk64": ViGShape(384, 6, 12, 1.0, 1.0, False, False),
    "vig_b_dk64": ViGShape(768, 12, 12, 1.0, 1.0, False, False),
}


def _xavier(rng, shape, fan_in, fan_out, gain=2 ** -2.5):
    a = gain * math.sqrt(6.0 / (fan_in + fan_out))
    return torch.from_numpy(rng.uniform(-a, a, size=shape).astype(np.float32))


def _normal(rng, shape, std=0.02):
    return torch.from_numpy((rng.standard_normal(size=shape) * std).astype(np.float32))


def make_state_dict(shape: ViGShape, seed: int = 0, with_stem: bool = True):
    rng = np.random.default_rng(seed)
    C, kd, vd, I, r = shape.embed_dim, shape.key_dim, shape.value_dim, shape.intermediate_size, shape.gate_low_rank_dim
    dv = vd // shape.num_heads
    sd = {}
    if with_stem:
        sd["patch_embed.proj.0.weight"] = _normal(rng, (C // 2, 3, 9, 9), 0.05)
        sd["patch_embed.proj.0.bias"] = _normal(rng, (C // 2,), 0.02)
        sd["patch_embed.proj.1.weight"] = torch.ones(C // 2)
        sd["patch_embed.proj.1.bias"] = torch.zeros(C // 2)
        sd["patch_embed.proj.3.weight"] = _normal(rng, (C, C // 2, 3, 3), 0.05)
        sd["patch_embed.proj.3.bias"] = _normal(rng, (C,), 0.02)
        sd["patch_embed.proj.4.weight"] = torch.ones(C)
        sd["patch_embed.proj.4.bias"] = torch.zeros(C)
        sd["pos_embed"] = _normal(rng, (1, shape.pretrain_grid ** 2, C), 0.02).clamp_(-0.04, 0.04)
        sd["norm.weight"] = torch.ones(C)
        sd["head.weight"] = _normal(rng, (shape.num_classes, C))
        sd["head.bias"] = torch.zeros(shape.num_classes)
    for i in range(shape.depth):
        p = f"blocks.{i}."
        sd[p + "attn_norm.weight"] = torch.ones(C)
        sd[p + "mlp_norm.weight"] = torch.ones(C)
        sd[p + "attn.in_proj.0.weight"] = _xavier(rng, (C, 1, 3, 3), 9, 9 * C)
        sd[p + "attn.qkv_proj.weight"] = _xavier(rng, (2 * kd + vd, C), C, 2 * kd + vd)
        sd[p + "attn.gk_proj.0.weight"] = _xavier(rng, (r, C), C, r)
        sd[p + "attn.gk_proj.1.weight"] = _xavier(rng, (2 * kd, r), r, 2 * kd)
        sd[p + "attn.gk_proj.1.bias"] = _normal(rng, (2 * kd,), 0.5)
        sd[p + "attn.g_proj.weight"] = _xavier(rng, (vd, C), C, vd)
        sd[p + "attn.g_proj.bias"] = _normal(rng, (vd,), 0.1)
        sd[p + "attn.g_norm.weight"] = 1.0 + _normal(rng, (dv,), 0.1)
        sd[p + "attn.l_norm.weight"] = 1.0 + _normal(rng, (dv,), 0.1)
        sd[p + "attn.o_proj.weight"] = _xavier(rng, (C, vd), vd, C)
        sd[p + "mlp.gate_proj.weight"] = _normal(rng, (2 * I, C))
        sd[p + "mlp.down_proj.weight"] = _normal(rng, (C, I))
    return sd


def make_images(batch, size, seed=0):
    rng = np.random.default_rng(seed + 7919)
    return torch.from_numpy(rng.standard_normal(size=(batch, 3, size, size)).astype(np.float32))


def make_bigla_inputs(B, H, L, dk, dv, seed=0, gate_normalizer=16.0):
    """Operator inputs of the benchmark's first configuration: q,k,v ~ N(0,1) (q unscaled, the
    operator applies dk^-0.5), log-gates = logsigmoid(N(0,1)) / 16; drawn in the order
    q, k, v, g_fwd, g_bwd from ``torch.manual_seed(seed)``."""
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, L, dk, generator=gen)
    k = torch.randn(B, H, L, dk, generator=gen)
    v = torch.randn(B, H, L, dv, generator=gen)
    g_fwd = torch.nn.functional.logsigmoid(torch.randn(B, H, L, dk, generator=gen)) / gate_normalizer
    g_bwd = torch.nn.functional.logsigmoid(torch.randn(B, H, L, dk, generator=gen)) / gate_normalizer
    return q, k, v, g_fwd, g_bwd


def seeded_like(template, seed=0):
    """Deterministic values for every entry of ``template`` (a state dict: name -> tensor), keyed by NAME, so that two
    implementations with the same parameter names get the same weights whatever their parameter order: matrices and
    convolution kernels N(0, 1/fan_in), vectors named ``*.bias`` N(0, 0.02^2), other vectors (norm weights) 1 + N(0, 0.1^2)."""
    import zlib
    out = {}
    for name, t in template.items():
        rng = np.random.default_rng([seed, zlib.crc32(name.encode())])
        shape = tuple(t.shape)
        if len(shape) >= 2:
            fan_in = int(np.prod(shape[1:]))
            v = rng.standard_normal(size=shape) / math.sqrt(fan_in)
        elif name.endswith("bias"):
            v = 0.02 * rng.standard_normal(size=shape)
        else:
            v = 1.0 + 0.1 * rng.standard_normal(size=shape)
        out[name] = torch.from_numpy(v.astype(np.float32))
    return out
