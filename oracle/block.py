"""CPU fp32 restatement of the ViG block and model shell around the bi-GLA operator.

Functional form over a plain ``{name: tensor}`` state dict whose keys are the
reference's parameter names (``blocks.{i}.attn.qkv_proj.weight`` ...), so the same
state dict loads into the reference modules, this oracle and the CUDA-backed modules.
Every function cites the reference lines it follows.
"""
import math
import torch
import torch.nn.functional as F

from .gla import naive_bi_gla


def rms_norm(x, weight, residual=None, eps=1e-6, prenorm=False):
    """``fla/modules/rmsnorm.py:38-52`` (``rms_norm_ref``): optional residual add, then
    ``x * rsqrt(mean(x^2) + eps) * weight``; ``prenorm`` also returns the summed input."""
    if residual is not None:
        x = x + residual
    rstd = 1.0 / torch.sqrt(x.square().mean(dim=-1, keepdim=True) + eps)
    out = x * rstd * weight
    return (out, x) if prenorm else out


def swiglu(gate, y):
    """``fla/modules/activations.py:109-113``: ``x * y / (1 + exp(-x))``."""
    return gate * y / (1.0 + torch.exp(-gate))


def dwconv3x3_nlc(x, weight, bias, hw, act):
    """Depthwise 3x3, zero padding 1, on tokens laid out [B, L=h*w, C]; optional SiLU.
    ``classification/models/vig.py:291-294,428-430`` (the reference goes through NCHW)."""
    B, L, C = x.shape
    h, w = hw
    x2d = x.transpose(1, 2).reshape(B, C, h, w)
    y = F.conv2d(x2d, weight.reshape(C, 1, 3, 3), bias, padding=1, groups=C)
    if act:
        y = F.silu(y)
    return y.flatten(2).transpose(1, 2).contiguous()


def gate_inject(o_bhld, local, gate_logits, w_gnorm, w_lnorm, eps, out_act):
    """2-D gating locality injection, ``vig.py:444-457``: head-wise RMSNorm of the scan
    output and of the conv output, sigmoid blend, optional swish.  o_bhld [B,H,L,dv];
    local, gate_logits [B,L,H*dv]; returns [B,L,H*dv]."""
    B, H, L, dv = o_bhld.shape
    o = rms_norm(o_bhld.permute(0, 2, 1, 3), w_gnorm, eps=eps)
    loc = rms_norm(local.reshape(B, L, H, dv), w_lnorm, eps=eps)
    g = torch.sigmoid(gate_logits).reshape(B, L, H, dv)
    y = (o * g + loc * (1.0 - g)).reshape(B, L, H * dv)
    if out_act:
        y = y * torch.sigmoid(y)
    return y


def gla_attention_forward(sd, p, x, hw, shape, return_parts=False):
    """Eval branch of ``GatedLinearAttention.forward``, ``vig.py:427-464``."""
    B, L, C = x.shape
    H = shape.num_heads
    key_dim, value_dim = shape.key_dim, shape.value_dim
    dk, dv = key_dim // H, value_dim // H
    xs = dwconv3x3_nlc(x, sd[p + "in_proj.0.weight"], sd.get(p + "in_proj.0.bias"), hw, shape.use_act_in_conv)
    qkv = xs @ sd[p + "qkv_proj.weight"].t()
    q, k, v = torch.split(qkv, [key_dim, key_dim, value_dim], dim=2)
    gk = (xs @ sd[p + "gk_proj.0.weight"].t()) @ sd[p + "gk_proj.1.weight"].t() + sd[p + "gk_proj.1.bias"]
    gk = F.logsigmoid(gk) / shape.gate_logit_normalizer
    if shape.clamp_min is not None:
        gk = torch.clamp_min(gk, shape.clamp_min)
    g_fwd, g_bwd = gk.chunk(2, dim=2)
    to_heads = lambda t, d: t.reshape(B, L, H, d).permute(0, 2, 1, 3)
    q, k, g_fwd, g_bwd = (to_heads(t, dk) for t in (q, k, g_fwd, g_bwd))
    v = to_heads(v, dv)
    # (o_f + o_b)/2 inside the operator wrapper (recurrent_fuse.py:442), /2 again at vig.py:443
    o = naive_bi_gla(q, k, v, g_fwd, g_bwd, out_scale=0.25)
    gate_logits = xs @ sd[p + "g_proj.weight"].t() + sd[p + "g_proj.bias"]
    y = gate_inject(o, xs, gate_logits, sd[p + "g_norm.weight"], sd[p + "l_norm.weight"], shape.eps, shape.use_out_act)
    out = y @ sd[p + "o_proj.weight"].t()
    if return_parts:
        return out, dict(xs=xs, q=q, k=k, v=v, g_fwd=g_fwd, g_bwd=g_bwd, o=o, gate_logits=gate_logits, y=y)
    return out


def mlp_forward(sd, p, x):
    """``GLAMLP.forward``, ``vig.py:494-497``: down(silu(gate) * y), [gate, y] = chunk(gate_proj(x))."""
    gy = x @ sd[p + "gate_proj.weight"].t()
    gate, y = gy.chunk(2, -1)
    return swiglu(gate, y) @ sd[p + "down_proj.weight"].t()


def block_forward(sd, p, x, hw, shape):
    """``GLABlock.forward``, ``vig.py:582-618`` (eval: DropPath is identity, no LayerScale)."""
    residual = x
    h = rms_norm(x, sd[p + "attn_norm.weight"], eps=shape.eps)
    h = gla_attention_forward(sd, p + "attn.", h, hw, shape)
    h, residual = rms_norm(h, sd[p + "mlp_norm.weight"], residual=residual, eps=shape.eps, prenorm=True)
    return residual + mlp_forward(sd, p + "mlp.", h)


def _layer_norm_2d(x, w, b, eps=1e-5):
    """``LayerNorm2d``, ``vig.py:619-624``: LayerNorm over channels of an NCHW tensor."""
    return F.layer_norm(x.permute(0, 2, 3, 1), (x.shape[1],), w, b, eps).permute(0, 3, 1, 2)


def patch_embed_v2(sd, images):
    """``V2PatchEmbed``, ``vig.py:625-672``: conv k9 s8 p1 -> LN2d -> swish -> conv k3 s2 p1 -> LN2d."""
    p = "patch_embed.proj."
    x = F.conv2d(images, sd[p + "0.weight"], sd[p + "0.bias"], stride=8, padding=1)
    x = _layer_norm_2d(x, sd[p + "1.weight"], sd[p + "1.bias"])
    x = x * torch.sigmoid(x)
    x = F.conv2d(x, sd[p + "3.weight"], sd[p + "3.bias"], stride=2, padding=1)
    x = _layer_norm_2d(x, sd[p + "4.weight"], sd[p + "4.bias"])
    hw = (x.shape[2], x.shape[3])
    return x.flatten(2).transpose(1, 2), hw


def resize_pos_embed(pos_embed, src_hw, dst_hw):
    """``resize_pos_embed``, ``vig.py:915-958``: bicubic, align_corners=False, in fp32."""
    if tuple(src_hw) == tuple(dst_hw):
        return pos_embed
    _, L, C = pos_embed.shape
    w = pos_embed.reshape(1, src_hw[0], src_hw[1], C).permute(0, 3, 1, 2)
    w = F.interpolate(w.float(), size=tuple(dst_hw), align_corners=False, mode="bicubic")
    return torch.flatten(w, 2).transpose(1, 2).to(pos_embed.dtype)


def vig_forward(sd, images, shape, return_features=False):
    """``ViG.forward``, ``vig.py:843-912`` with no cls token, absolute pos-embed, avg-pool head."""
    sd = {k: v.float() for k, v in sd.items()}
    x, hw = patch_embed_v2(sd, images.float())
    src = int(round(math.sqrt(sd["pos_embed"].shape[1])))
    x = x + resize_pos_embed(sd["pos_embed"], (src, src), hw)
    for i in range(shape.depth):
        x = block_forward(sd, f"blocks.{i}.", x, hw, shape)
    x = rms_norm(x, sd["norm.weight"], eps=shape.eps)
    feat = x.mean(dim=1)
    if return_features:
        return feat
    return feat @ sd["head.weight"].t() + sd["head.bias"]
