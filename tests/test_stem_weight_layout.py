"""Host logic of the fused first stem stage (no GPU): the [O, 512] weight that ``V2PatchEmbed._gemm_weight`` lays out for
cells folded on 8-pixel boundaries reproduces the 9 x 9 / stride 8 / padding 1 convolution when the GEMM the kernel
performs is written with torch on the CPU."""
import pytest
import torch
import torch.nn.functional as F

from vig_b200.vig import V2PatchEmbed


@pytest.mark.parametrize("H,W", [(64, 40), (8, 8), (224, 224)])
def test_cell_weight_matches_convolution(H, W):
    torch.manual_seed(H + W)
    pe = V2PatchEmbed(img_size=H, patch_size=16, in_chans=3, embed_dim=192, use_bias_in_patch=True).double()
    conv = pe.proj[0]
    B = 2
    x = torch.randn(B, 3, H, W, dtype=torch.float64)
    # the fold of vig_stem_fold_fwd: cells[b, cy, cx, (dy*3 + ic)*8 + dx] = x[b, ic, 8cy + dy, 8cx + dx]
    cells = x.view(B, 3, H // 8, 8, W // 8, 8).permute(0, 2, 4, 3, 1, 5).reshape(B, H // 8, W // 8, 192)
    cp = F.pad(cells, (0, 0, 1, 0, 1, 0))                      # cells at coordinate -1 are zeros (the TMA unit's fill)
    # row of the GEMM for output pixel (oy, ox): cell (oy, ox) | cell (oy, ox-1) | last 64 of cell (oy-1, ox) | last 64 of cell (oy-1, ox-1)
    A = torch.cat([cp[:, 1:, 1:, :], cp[:, 1:, :-1, :], cp[:, :-1, 1:, 128:], cp[:, :-1, :-1, 128:]], dim=-1)
    w2 = pe._gemm_weight()
    assert tuple(w2.shape) == (96, 512)
    got = A @ w2.t() + conv.bias
    ref = F.conv2d(x, conv.weight, conv.bias, conv.stride, conv.padding).permute(0, 2, 3, 1)
    assert got.shape == ref.shape
    assert (got - ref).abs().max().item() < 1e-12


def test_cell_weight_follows_parameter_updates():
    pe = V2PatchEmbed(img_size=64, patch_size=16, in_chans=3, embed_dim=192)
    w_a = pe._gemm_weight()
    assert pe._gemm_weight() is w_a                           # cached
    with torch.no_grad():
        pe.proj[0].weight.mul_(2.0)
    assert torch.allclose(pe._gemm_weight(), 2.0 * w_a)
