"""Hierarchical ViG (``HierViG``, ``classification/models/vig_h.py:686-923``) on the CUDA-backed operators: four stages
of ``VSSBlock`` s (``:610-683``) around ``GLA2D`` (``:338-606``), the same bidirectional gated-linear-attention operator
with 2-D glue, LayerNorm instead of RMSNorm and a GELU or gated MLP.  Inference only, like the rest of the package.

Parameter names and shapes are the reference's (its ``Linear2d`` / ``LayerNorm2d`` keep ``nn.Linear`` / ``nn.LayerNorm``
parameters, ``vig_h.py:202-217``), so a reference state dict loads unchanged for either of its layouts
(``norm_layer`` "ln" = channels last, "ln2d" = channels first).  Internally activations are always token-major
``[B, h*w, C]``: LayerNorm over channels per pixel, 1x1 "convolutions" as linear layers and the channel-first
rearranges of the reference are the same arithmetic in that layout.
"""
from collections import OrderedDict

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from .modules import GatedLinearAttention


class GLA2D(GatedLinearAttention):
    """``vig_h.py:338-606``: ViG's attention module with the summed directions halved once (``:577-578``) and no bias in
    the depthwise convolution.  ``forward(x [B, L, C], patch_resolution=(h, w)) -> [B, L, C]``."""

    def __init__(self, d_model, expand_v=1.0, expand_k=0.5, num_heads=3, gate_fn="swish", layernorm_eps=1e-5, mode="fused_chunk",
                 use_out_act=False, use_act_in_conv=True, **unused):
        super().__init__(d_model=d_model, expand_v=expand_v, expand_k=expand_k, num_heads=num_heads, gate_fn=gate_fn,
                         layernorm_eps=layernorm_eps, mode=mode, use_out_act=use_out_act, use_act_in_conv=use_act_in_conv,
                         use_bias_in_dwconv=False)
        self.out_scale = 0.5


def _conv(conv, x):
    """Convolution through the library; fp32 inputs keep fp32 arithmetic (cuDNN would otherwise pick TF32, which misses
    the 1e-4 bar of the fp32 path)."""
    if x.dtype == torch.float32:
        with torch.backends.cudnn.flags(enabled=True, allow_tf32=False):
            return conv(x)
    return conv(x)


def _layer_norm(x, norm):
    """LayerNorm over the channels of token-major activations with the library's kernel."""
    return ops.layernorm_act(x.contiguous(), norm.weight, norm.bias, norm.eps)


class Mlp(nn.Module):
    """``vig_h.py:268-287``: fc1 -> activation -> fc2, biases on."""

    def __init__(self, in_features, hidden_features, act_layer=nn.GELU):
        super().__init__()
        self.fc1, self.act, self.fc2 = nn.Linear(in_features, hidden_features), act_layer(), nn.Linear(hidden_features, in_features)

    def forward(self, x):
        return self.fc2(self.act(self.fc1(x)))


class gMlp(nn.Module):
    """``vig_h.py:290-323``: SwiGLU MLP without biases; intermediate size 2/3 * 4 * C rounded up to a multiple of 32."""

    def __init__(self, in_features, **unused):
        super().__init__()
        inter = int(in_features * 4 * 2 / 3)
        self.intermediate_size = 32 * ((inter + 31) // 32)
        self.fc1 = nn.Linear(in_features, 2 * self.intermediate_size, bias=False)
        self.fc2 = nn.Linear(self.intermediate_size, in_features, bias=False)

    def forward(self, x):
        if ops.linear_swiglu_supported(x, self.fc1.weight, preferred=True):
            return self.fc2(ops.linear_swiglu(x, self.fc1.weight))
        gate, y = self.fc1(x).chunk(2, -1)
        return self.fc2(ops.swiglu(gate, y))


class VSSBlock(nn.Module):
    """``vig_h.py:610-683`` (pre-norm form): ``x + op(norm(x))`` then ``x + mlp(norm2(x))``."""

    def __init__(self, hidden_dim, num_head, expand_k, expand_v, hidden_act, use_out_act, use_act_in_conv, eps, mlp_ratio,
                 mlp_act_layer, gmlp, attn_model):
        super().__init__()
        self.norm = nn.LayerNorm(hidden_dim)
        self.op = GLA2D(hidden_dim, expand_k=expand_k, expand_v=expand_v, num_heads=num_head, gate_fn=hidden_act,
                        layernorm_eps=eps, mode=attn_model, use_out_act=use_out_act, use_act_in_conv=use_act_in_conv)
        self.norm2 = nn.LayerNorm(hidden_dim)
        self.mlp = gMlp(hidden_dim) if gmlp else Mlp(hidden_dim, int(hidden_dim * mlp_ratio), mlp_act_layer)

    def forward(self, x, hw):
        x = x + self.op(_layer_norm(x, self.norm), patch_resolution=hw)
        return x + self.mlp(_layer_norm(x, self.norm2))


class _Conv(nn.Module):
    """A strided convolution between token-major activations: ``[B, h*w, Cin], (h, w) -> [B, h'*w', Cout], (h', w')``."""

    def __init__(self, conv):
        super().__init__()
        self.conv = conv

    def forward(self, x, hw):
        B, _, C = x.shape
        y = _conv(self.conv, x.view(B, hw[0], hw[1], C).permute(0, 3, 1, 2))
        return y.permute(0, 2, 3, 1).reshape(B, -1, y.shape[1]), (y.shape[2], y.shape[3])


class HierViG(nn.Module):
    def __init__(self, patch_size=4, in_chans=3, num_classes=1000, depths=(2, 2, 9, 2), dims=(96, 192, 384, 768),
                 num_heads=(3, 6, 12, 24), attn_models=("fused_chunk", "fused_chunk", "fused_recurrent", "fused_recurrent"),
                 expand_k=0.5, expand_v=1.0, hidden_act="swish", use_out_act=False, use_act_in_conv=True, rope_mode="none",
                 mlp_ratio=4.0, mlp_act_layer="gelu", gmlp=False, patch_norm=True, norm_layer="LN", downsample_version="v2",
                 patchembed_version="v1", rms_norm_eps=1e-6, **unused):
        super().__init__()
        if rope_mode != "none":
            raise NotImplementedError("rotary variants are not part of the shipped configurations")
        if norm_layer.lower() not in ("ln", "ln2d"):
            raise NotImplementedError("only the LayerNorm variants (channels last 'ln', channels first 'ln2d') are implemented")
        if isinstance(dims, int):
            dims = [int(dims * 2 ** i) for i in range(len(depths))]
        self.dims, self.num_classes = list(dims), num_classes
        act = dict(silu=nn.SiLU, gelu=nn.GELU, relu=nn.ReLU, sigmoid=nn.Sigmoid)[mlp_act_layer.lower()]
        ident = nn.Identity
        # same module indices inside every nn.Sequential as the reference, so that parameter names match
        if patchembed_version == "v1":
            self.patch_embed = nn.Sequential(nn.Conv2d(in_chans, dims[0], patch_size, patch_size), ident(),
                                             nn.LayerNorm(dims[0]) if patch_norm else ident())
        elif patchembed_version == "v2":
            s = patch_size // 2
            self.patch_embed = nn.Sequential(nn.Conv2d(in_chans, dims[0] // 2, s + 1, s, 1), ident(),
                                             nn.LayerNorm(dims[0] // 2) if patch_norm else ident(), ident(), nn.GELU(),
                                             nn.Conv2d(dims[0] // 2, dims[0], s + 1, s, 1), ident(),
                                             nn.LayerNorm(dims[0]) if patch_norm else ident())
        else:
            raise ValueError(f"unknown patch embedding version {patchembed_version}")
        self.layers = nn.ModuleList()
        for i, depth in enumerate(depths):
            blocks = nn.Sequential(*[VSSBlock(dims[i], num_heads[i], expand_k, expand_v, hidden_act, use_out_act, use_act_in_conv,
                                              rms_norm_eps, mlp_ratio, act, gmlp, attn_models[i]) for _ in range(depth)])
            if i + 1 < len(depths):
                if downsample_version == "v2":
                    conv = nn.Conv2d(dims[i], dims[i + 1], 2, 2)
                elif downsample_version == "v3":
                    conv = nn.Conv2d(dims[i], dims[i + 1], 3, 2, 1)
                else:
                    raise NotImplementedError("downsample versions v2 and v3 (strided convolution + norm) are implemented")
                down = nn.Sequential(ident(), conv, ident(), nn.LayerNorm(dims[i + 1]))
            else:
                down = ident()
            self.layers.append(nn.Sequential(OrderedDict(blocks=blocks, downsample=down)))
        self.classifier = nn.Sequential(OrderedDict(norm=nn.LayerNorm(dims[-1]), head=nn.Linear(dims[-1], num_classes)))

    def _embed(self, images):
        pe = self.patch_embed
        y = images.contiguous(memory_format=torch.channels_last)
        for m in pe:
            if isinstance(m, nn.Conv2d):
                y = _conv(m, y)
            elif isinstance(m, nn.LayerNorm):
                y = F.layer_norm(y.permute(0, 2, 3, 1), m.normalized_shape, m.weight, m.bias, m.eps).permute(0, 3, 1, 2)
            elif isinstance(m, nn.GELU):
                y = m(y)
        B, C, h, w = y.shape
        return y.permute(0, 2, 3, 1).reshape(B, h * w, C), (h, w)

    def forward_features(self, images, return_stages=False):
        x, hw = self._embed(images)
        stages = []
        for layer in self.layers:
            for blk in layer.blocks:
                x = blk(x, hw)
            stages.append((x, hw))
            if not isinstance(layer.downsample, nn.Identity):
                x, hw = _Conv(layer.downsample[1])(x, hw)
                x = _layer_norm(x, layer.downsample[3])
        return stages if return_stages else x

    def forward(self, images):
        status = ops.status_word(images.device)
        status.poll()
        x = self.forward_features(images)
        x = _layer_norm(x, self.classifier.norm).mean(dim=1)
        logits = self.classifier.head(x)
        status.snapshot()
        return logits
