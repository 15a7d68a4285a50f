"""ViG model shell around the CUDA-backed block: ``ViG`` of ``classification/models/vig.py:705-912`` in
the configuration every shipped YAML uses (v2 patch embed, absolute pos-embed, no cls token, average-pool
head, RMSNorm + SwiGLU blocks).  Parameter names match the reference so its checkpoints load.
The stem's first stage (convolution + LayerNorm2d + swish) is one kernel of this library for ViG-T in 16 bits; its
second convolution, wider first stages, the bicubic pos-embed resize, pooling and the classifier run as PyTorch
library calls; everything inside the blocks except the stacked input projection is this library's kernels.
"""
import math
from types import SimpleNamespace

import torch
import torch.nn as nn
import torch.nn.functional as F

from .modules import GLABlock, RMSNorm


class LayerNorm2d(nn.LayerNorm):
    def forward(self, x):
        return F.layer_norm(x.permute(0, 2, 3, 1), self.normalized_shape, self.weight, self.bias, self.eps).permute(0, 3, 1, 2)


class V2PatchEmbed(nn.Module):
    """``vig.py:625-672``: conv k(p/2+1) s(p/2) p1 -> LN2d -> swish -> conv k3 s2 p1 -> LN2d.

    Same parameters as the reference; the forward keeps activations channels-last so both LayerNorm2d stages
    run as this library's fused LayerNorm(+swish) kernel on contiguous rows, and evaluates the first
    convolution (kernel s+1, stride s, 3 input channels -- a shape cuDNN serves without tensor cores) as a
    2x2 convolution over s x s pixel blocks (space-to-depth), which is the same sum with zero weights at the
    taps the original kernel does not have.
    """

    def __init__(self, img_size=224, patch_size=16, in_chans=3, embed_dim=768, use_bias_in_patch=True):
        super().__init__()
        stride = patch_size // 2
        self.stride = stride
        self.proj = nn.Sequential(
            nn.Conv2d(in_chans, embed_dim // 2, kernel_size=stride + 1, stride=stride, padding=1, bias=use_bias_in_patch),
            LayerNorm2d(embed_dim // 2), nn.SiLU(),
            nn.Conv2d(embed_dim // 2, embed_dim, kernel_size=3, stride=2, padding=1, bias=use_bias_in_patch),
            LayerNorm2d(embed_dim))
        self.num_patches = (img_size // patch_size) ** 2
        self._w_blocks = None
        self._w_gemm = None
        self.fuse_conv1 = True          # first convolution + LayerNorm2d + swish as one kernel where there is one (ViG-T, 16-bit)

    def _block_weight(self):
        """[O, s*s*Cin, 2, 2] weight of the space-to-depth form, channels-last, cached per parameter version."""
        w = self.proj[0].weight
        key = (w.dtype, w.device, w._version)
        if self._w_blocks is None or self._w_blocks[0] != key:
            s = self.stride
            O, Cin = w.shape[0], w.shape[1]
            big = w.new_zeros(O, Cin, 2 * s, 2 * s)
            big[:, :, :s + 1, :s + 1] = w.detach()
            # (O, Cin, cy, dy, cx, dx) -> (O, dy, dx, Cin, cy, cx) -> (O, s*s*Cin, 2, 2)
            wb = big.view(O, Cin, 2, s, 2, s).permute(0, 3, 5, 1, 2, 4).reshape(O, s * s * Cin, 2, 2)
            self._w_blocks = (key, wb.contiguous(memory_format=torch.channels_last))
        return self._w_blocks[1]

    def _gemm_weight(self):
        """[O, 512] weight of the fused first stage (``ops.stem_conv_ln``) for cells folded on 8-pixel boundaries, value
        order (dy, ic, dx).  The 9 x 9 window of output pixel (oy, ox) starts at image pixel (8oy - 1, 8ox - 1): kernel rows /
        columns 1..8 fall into cell (oy, ox), kernel column 0 into the last pixel column of cell (oy, ox-1), kernel row 0 into
        the last pixel row of the cells above.  Columns: cell (oy, ox) | cell (oy, ox-1) | last 64 values of cell (oy-1, ox) |
        last 64 values of cell (oy-1, ox-1).  Cached per parameter version."""
        w = self.proj[0].weight
        key = (w.dtype, w.device, w._version)
        if self._w_gemm is None or self._w_gemm[0] != key:
            wd = w.detach()
            O = wd.shape[0]
            main = wd[:, :, 1:, 1:].permute(0, 2, 1, 3).reshape(O, 192)                  # (dy, ic, dx) <- kernel (dy+1, dx+1)
            left = wd.new_zeros(O, 8, 3, 8)
            left[:, :, :, 7] = wd[:, :, 1:, 0].permute(0, 2, 1)                          # dx = 7 <- kernel column 0
            top = wd.new_zeros(O, 64)                                                    # values 128..191 of the cell above
            top.view(O, 8, 8)[:, 5:, :] = wd[:, :, 0, 1:]                                # dy = 7: values 168 + 8 ic + dx
            corner = wd.new_zeros(O, 64)
            corner.view(O, 8, 8)[:, 5:, 7] = wd[:, :, 0, 0]
            self._w_gemm = (key, torch.cat([main, left.reshape(O, 192), top, corner], dim=1).contiguous())
        return self._w_gemm[1]

    def _conv1_ln_fused(self, x):
        """Convolution + bias + LayerNorm2d + swish in one tensor-core kernel, channels-last ``[B, h, w, C/2]``; None when
        the shape has no such kernel (then the two steps run separately)."""
        from . import ops
        conv, ln1, s = self.proj[0], self.proj[1], self.stride
        if not (self.fuse_conv1 and s == 8 and conv.weight.dtype == x.dtype and ops.stem_conv_ln_supported_for_image(x, conv.weight.shape[0])):
            return None
        cells = ops.stem_fold(x)
        return ops.stem_conv_ln(cells, self._gemm_weight(), conv.bias, ln1.weight, ln1.bias, ln1.eps, act_swish=True)

    def _conv1(self, x):
        conv = self.proj[0]
        s = self.stride
        B, Cin, H, W = x.shape
        if H % s or W % s or Cin * s * s % 8:
            return F.conv2d(x.contiguous(memory_format=torch.channels_last), conv.weight, None, conv.stride, conv.padding)
        if s * Cin == 24:
            from . import ops
            cells = ops.stem_unfold(x, s)                                  # one gather kernel: pad + fold in a single pass
        else:
            # pad one pixel before (the conv's padding) and s-1 after, then fold s x s pixels into channels
            xp = F.pad(x.permute(0, 2, 3, 1), (0, 0, 1, s - 1, 1, s - 1))                 # [B, H+s, W+s, Cin]
            cells = xp.view(B, H // s + 1, s, W // s + 1, s, Cin).permute(0, 1, 3, 2, 4, 5).reshape(B, H // s + 1, W // s + 1, s * s * Cin)
        return F.conv2d(cells.permute(0, 3, 1, 2), self._block_weight(), None)

    def forward(self, x, pos_fn=None, next_norm=None):
        """``pos_fn(hw) -> [1, h*w, C]`` (optional): the position embedding, added inside the last LayerNorm kernel.
        ``next_norm`` (optional, an ``RMSNorm``): its output on the tokens comes out of the same kernel; the call then
        returns ``(tokens, hw, next_norm(tokens))``."""
        from . import ops
        ln1, ln2, conv2 = self.proj[1], self.proj[4], self.proj[3]
        # the convolutions run without their bias; it is added inside the LayerNorm kernel that follows
        y = self._conv1_ln_fused(x)                                       # [B, h, w, C/2], or None
        if y is None:
            y = self._conv1(x)                                            # logical NCHW, channels-last memory
            y = ops.layernorm_act(y.permute(0, 2, 3, 1).contiguous(), ln1.weight, ln1.bias, ln1.eps, act_swish=True,
                                  pre_bias=self.proj[0].bias)
        y = F.conv2d(y.permute(0, 3, 1, 2), conv2.weight, None, conv2.stride, conv2.padding)
        y = y.permute(0, 2, 3, 1).contiguous()
        pos = pos_fn((y.shape[1], y.shape[2])) if pos_fn is not None else None
        B, h, w, C = y.shape
        if next_norm is not None:
            y, normed = ops.layernorm_act(y, ln2.weight, ln2.bias, ln2.eps, act_swish=False, pre_bias=conv2.bias, post_add=pos,
                                          rms_weight=next_norm.weight, rms_eps=next_norm.eps)
            return y.view(B, h * w, C), (h, w), normed.view(B, h * w, C)
        y = ops.layernorm_act(y, ln2.weight, ln2.bias, ln2.eps, act_swish=False, pre_bias=conv2.bias, post_add=pos)
        return y.view(B, h * w, C), (h, w)


def resize_pos_embed(pos_embed, src_shape, dst_shape, mode="bicubic"):
    """``vig.py:915-958`` without extra tokens: bicubic in fp32, align_corners=False."""
    if tuple(src_shape) == tuple(dst_shape):
        return pos_embed
    C = pos_embed.shape[-1]
    w = pos_embed.reshape(1, src_shape[0], src_shape[1], C).permute(0, 3, 1, 2)
    w = F.interpolate(w.float(), size=tuple(dst_shape), align_corners=False, mode=mode)
    return torch.flatten(w, 2).transpose(1, 2).to(pos_embed.dtype)


class ViG(nn.Module):
    def __init__(self, img_size=224, patch_size=16, depth=12, num_heads=3, embed_dim=192, channels=3, num_classes=1000,
                 use_out_act=False, use_act_in_conv=True, expand_k=0.5, expand_v=1, use_bias_in_patch=True,
                 use_bias_in_dwconv=False, clamp_min=None, rms_norm_eps=1e-6, **unused):
        super().__init__()
        self.fuse_norm_epilogues = True
        self.embed_dim, self.num_classes = embed_dim, num_classes
        self.config = SimpleNamespace(hidden_size=embed_dim, num_hidden_layers=depth, num_attention_heads=num_heads,
                                      expand_k=expand_k, expand_v=expand_v, rms_norm_eps=rms_norm_eps, use_out_act=use_out_act,
                                      use_act_in_conv=use_act_in_conv, use_bias_in_dwconv=use_bias_in_dwconv,
                                      clamp_min=clamp_min, attn_mode="fused_chunk", intermediate_size=None, hidden_act="swish")
        self.patch_embed = V2PatchEmbed(img_size, patch_size, channels, embed_dim, use_bias_in_patch)
        self.patch_resolution = (img_size // patch_size, img_size // patch_size)
        self.pos_embed = nn.Parameter(torch.zeros(1, self.patch_embed.num_patches, embed_dim))
        self.head = nn.Linear(embed_dim, num_classes) if num_classes > 0 else nn.Identity()
        self.blocks = nn.ModuleList([GLABlock(self.config, i) for i in range(depth)])
        self.norm = RMSNorm(embed_dim, eps=rms_norm_eps)
        self._pos_cache = {}

    def _apply(self, fn, *args, **kwargs):
        # keep the stem's conv weights in channels_last after every .to() / .cuda() / .bfloat16()
        super()._apply(fn, *args, **kwargs)
        for m in self.patch_embed.proj:
            if isinstance(m, nn.Conv2d):
                m.weight.data = m.weight.data.contiguous(memory_format=torch.channels_last)
        return self

    @classmethod
    def from_shape(cls, shape, **kw):
        """Build from an object with embed_dim / num_heads / depth / expand_k / ... attributes."""
        return cls(depth=shape.depth, num_heads=shape.num_heads, embed_dim=shape.embed_dim, num_classes=shape.num_classes,
                   use_out_act=shape.use_out_act, use_act_in_conv=shape.use_act_in_conv, expand_k=shape.expand_k,
                   expand_v=shape.expand_v, clamp_min=shape.clamp_min, rms_norm_eps=shape.eps, **kw)

    def _pos(self, hw):
        key = (tuple(hw), self.pos_embed.dtype, self.pos_embed.device, self.pos_embed._version)
        if key not in self._pos_cache:
            self._pos_cache = {key: resize_pos_embed(self.pos_embed.detach(), self.patch_resolution, hw)}
        return self._pos_cache[key]

    def forward_features(self, x):
        # ``fuse_norm_epilogues``: every residual add + RMSNorm runs as the epilogue of the projection in front of it
        # (hidden size <= 192, 16-bit tensors; measured 74 + 104 us against 112 + 141 us for cuBLAS + the norm kernel),
        # and the first block's norm comes out of the stem's last kernel.
        probe = x.new_empty(1, 1, self.embed_dim)
        if self.fuse_norm_epilogues and len(self.blocks) and all(blk.fused_epilogues_supported(probe) for blk in self.blocks):
            x, hw, h = self.patch_embed(x, pos_fn=self._pos, next_norm=self.blocks[0].attn_norm)
            residual = x
            for i, blk in enumerate(self.blocks):
                nxt = self.blocks[i + 1].attn_norm if i + 1 < len(self.blocks) else self.norm
                h, residual = blk.forward_prenormed(h, residual, nxt, patch_resolution=hw)
            return h.mean(dim=1)
        x, hw = self.patch_embed(x, pos_fn=self._pos)  # position embedding added by the stem's last kernel
        h, residual = x, None
        for blk in self.blocks:
            h, residual = blk.forward_deferred(h, residual, patch_resolution=hw)
        x = self.norm(h, residual)                      # last residual add fused into the final norm
        return x.mean(dim=1)

    def forward(self, x, **kwargs):
        """Logits.  The kernels' error word is looked at without stalling the stream: this call raises if a kernel of an
        EARLIER forward reported an error (its status copy has landed by now), and queues the copy for its own;
        ``vig_b200.check_status()`` is the blocking form."""
        from . import ops
        status = ops.status_word(x.device)
        status.poll()
        logits = self.head(self.forward_features(x))
        status.snapshot()
        return logits


_PRESETS = {
    "vig_t": dict(embed_dim=192, num_heads=3, use_out_act=True, use_act_in_conv=True),
    "vig_s": dict(embed_dim=384, num_heads=6, use_out_act=False, use_act_in_conv=False),
    "vig_b": dict(embed_dim=768, num_heads=12, use_out_act=False, use_act_in_conv=False),
}


def build_vig(name="vig_t", expand_k=0.5, **kw):
    """ViG-T / S / B of ``classification/configs/vig/vig-{t,s,b}.yaml`` (depth 12, expand_v 1)."""
    return ViG(depth=12, expand_k=expand_k, expand_v=1, **{**_PRESETS[name], **kw})
