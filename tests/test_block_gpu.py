"""Parity of the block's bandwidth kernels, the block and the model (CUDA, through the C ABI) with the oracle."""
import pytest
import torch

import oracle
from conftest import rel_err

pytestmark = pytest.mark.gpu
TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2, torch.float16: 2e-2}
DTYPES = [torch.float32, torch.bfloat16, torch.float16]


@pytest.fixture(autouse=True)
def _no_tf32():
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,rows", [(192, 392), (384, 77), (768, 33), (64, 1000), (1024, 5)])
def test_add_rmsnorm(dtype, N, rows):
    import vig_b200
    g = torch.Generator().manual_seed(N)
    x, r, w = torch.randn(rows, N, generator=g).to(dtype), torch.randn(rows, N, generator=g).to(dtype), (1 + 0.1 * torch.randn(N, generator=g)).to(dtype)
    y_ref = oracle.rms_norm(x.float(), w.float())
    assert rel_err(vig_b200.add_rmsnorm(x.cuda(), w.cuda()).float(), y_ref) < TOL[dtype]
    s_ref = (x.float() + r.float()).to(dtype).float()
    y2_ref = oracle.rms_norm(s_ref, w.float())
    y2, s = vig_b200.add_rmsnorm(x.cuda(), w.cuda(), residual=r.cuda(), prenorm=True)
    assert rel_err(y2.float(), y2_ref) < TOL[dtype]
    assert torch.equal(s.cpu(), s_ref.to(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hw,C,act,bias", [((14, 14), 192, True, False), ((7, 9), 384, False, True), ((1, 1), 64, True, True), ((20, 20), 768, False, False)])
def test_dwconv3x3(dtype, hw, C, act, bias):
    import vig_b200
    g = torch.Generator().manual_seed(C)
    x = torch.randn(2, hw[0] * hw[1], C, generator=g).to(dtype)
    w = (0.3 * torch.randn(C, 1, 3, 3, generator=g)).to(dtype)
    b = torch.randn(C, generator=g).to(dtype) if bias else None
    ref = oracle.dwconv3x3_nlc(x.float(), w.float(), b.float() if bias else None, hw, act)
    y = vig_b200.dwconv3x3(x.cuda(), w.reshape(C, 9).t().contiguous().cuda(), b.cuda() if bias else None, hw, act)
    assert rel_err(y.float(), ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,hw,C,act,bias", [(8, (64, 64), 192, True, False), (8, (33, 47), 384, True, True), (2, (61, 130), 768, False, False),
                                             (8, (50, 60), 200, True, True), (4, (3, 700), 512, True, False),
                                             (4096, (7, 5), 192, True, False), (64, (64, 300), 8, False, True)])
def test_dwconv3x3_tma_form(dtype, B, hw, C, act, bias):
    """Inputs of 4M elements and more run the TMA-fed kernel (tiles of 2 rows with a zero-filled border): against the
    oracle at the type's bar, and bit for bit against the sliding-window kernel, reached through the halo entry point
    with no halo rows.  Shapes: the headline one, ragged widths and heights, channel counts cut into chunks of 256 / 192
    channels, a width cut into several column blocks, images narrower than a thread's run of 8 columns, 8 channels."""
    import vig_b200
    from vig_b200 import _lib
    h, w = hw
    assert B * h * w * C >= 1 << 22
    g = torch.Generator().manual_seed(C + h)
    x = torch.randn(B, h * w, C, generator=g).to(dtype)
    wt = (0.3 * torch.randn(C, 1, 3, 3, generator=g)).to(dtype)
    b = torch.randn(C, generator=g).to(dtype) if bias else None
    taps = wt.reshape(C, 9).t().contiguous().cuda()
    xc, bc = x.cuda(), (b.cuda() if bias else None)
    y = vig_b200.dwconv3x3(xc, taps, bc, hw, act)
    vig_b200.check_status()
    ref = oracle.dwconv3x3_nlc(x.float(), wt.float(), b.float() if bias else None, hw, act)
    assert rel_err(y.float(), ref) < TOL[dtype]
    y_rows = torch.empty_like(xc)
    st = _lib.lib().vig_dwconv3x3_halo_fwd(_lib.ptr(xc), None, None, _lib.ptr(taps), _lib.ptr(bc), _lib.ptr(y_rows), B, h, w, C,
                                           int(act), _lib.dtype_code(xc), _lib.stream_ptr())
    _lib.check(st, "vig_dwconv3x3_halo_fwd")
    assert torch.equal(y, y_rows)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("out_act", [False, True])
def test_gate_inject(dtype, out_act):
    import vig_b200
    B, H, L, dv = 2, 3, 50, 64
    g = torch.Generator().manual_seed(3)
    o = torch.randn(B, H, L, dv, generator=g).to(dtype)
    wide = torch.randn(B, L, 3 * H * dv, generator=g).to(dtype)        # local / gate logits as column slices
    wg, wl = (1 + 0.1 * torch.randn(dv, generator=g)).to(dtype), (1 + 0.1 * torch.randn(dv, generator=g)).to(dtype)
    loc, gl = wide[..., :H * dv], wide[..., 2 * H * dv:]
    ref = oracle.gate_inject(o.float(), loc.float(), gl.float(), wg.float(), wl.float(), 1e-6, out_act)
    wc = wide.cuda()
    y = vig_b200.gate_inject(o.cuda(), wc[..., :H * dv], wc[..., 2 * H * dv:], wg.cuda(), wl.cuda(), 1e-6, out_act)
    assert rel_err(y.float(), ref) < TOL[dtype]
    # scan output stored token-major ([B,L,H,dv]) and passed as a permuted view
    o_tm = o.permute(0, 2, 1, 3).contiguous().cuda().permute(0, 2, 1, 3)
    y2 = vig_b200.gate_inject(o_tm, wc[..., :H * dv], wc[..., 2 * H * dv:], wg.cuda(), wl.cuda(), 1e-6, out_act)
    assert torch.equal(y, y2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,act", [(96, True), (192, False), (384, True), (768, False)])
def test_layernorm_act(dtype, N, act):
    import vig_b200
    g = torch.Generator().manual_seed(N)
    x = (3 * torch.randn(3, 5, 7, N, generator=g) + 1).to(dtype)
    w, b = (1 + 0.2 * torch.randn(N, generator=g)).to(dtype), (0.3 * torch.randn(N, generator=g)).to(dtype)
    ref = torch.nn.functional.layer_norm(x.float(), (N,), w.float(), b.float(), 1e-5)
    if act:
        ref = ref * torch.sigmoid(ref)
    y = vig_b200.layernorm_act(x.cuda(), w.cuda(), b.cuda(), 1e-5, act)
    assert rel_err(y.float(), ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_layernorm_with_trailing_add(dtype):
    """LayerNorm followed by `+ post_add[row % P]` in one kernel == the kernel plus a separate add."""
    import vig_b200
    g = torch.Generator().manual_seed(9)
    x = torch.randn(3, 35, 192, generator=g).to(dtype).cuda()
    w, b = (1 + 0.1 * torch.randn(192, generator=g)).to(dtype).cuda(), (0.1 * torch.randn(192, generator=g)).to(dtype).cuda()
    pos = torch.randn(1, 35, 192, generator=g).to(dtype).cuda()
    got = vig_b200.ops.layernorm_act(x, w, b, 1e-6, False, post_add=pos)
    ref = vig_b200.ops.layernorm_act(x, w, b, 1e-6, False) + pos
    assert torch.equal(got, ref)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,with_pos", [(192, True), (384, True), (768, False), (96, False)])
def test_layernorm_with_rmsnorm_as_second_output(dtype, N, with_pos):
    """LayerNorm (+ position add) with the following RMSNorm out of the same pass == the two kernels run one after the other."""
    import vig_b200
    g = torch.Generator().manual_seed(N)
    x = torch.randn(3, 35, N, generator=g).to(dtype).cuda()
    w, b = (1 + 0.1 * torch.randn(N, generator=g)).to(dtype).cuda(), (0.1 * torch.randn(N, generator=g)).to(dtype).cuda()
    pb = (0.2 * torch.randn(N, generator=g)).to(dtype).cuda()
    rw = (1 + 0.1 * torch.randn(N, generator=g)).to(dtype).cuda()
    pos = torch.randn(1, 35, N, generator=g).to(dtype).cuda() if with_pos else None
    y, h = vig_b200.ops.layernorm_act(x, w, b, 1e-6, False, pre_bias=pb, post_add=pos, rms_weight=rw, rms_eps=1e-6)
    y_ref = vig_b200.ops.layernorm_act(x, w, b, 1e-6, False, pre_bias=pb, post_add=pos)
    h_ref = vig_b200.ops.add_rmsnorm(y_ref, rw, eps=1e-6)
    assert torch.equal(y, y_ref)
    assert torch.equal(h, h_ref)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("B,H,W", [(2, 32, 48), (1, 8, 8), (3, 224, 224)])
def test_stem_unfold(dtype, B, H, W):
    """Pad + space-to-depth gather against the same rearrangement written with pad / view / permute."""
    import torch.nn.functional as F
    import vig_b200
    s, Cin = 8, 3
    g = torch.Generator().manual_seed(H + W)
    x = torch.randn(B, Cin, H, W, generator=g).to(dtype)
    xp = F.pad(x.permute(0, 2, 3, 1), (0, 0, 1, s - 1, 1, s - 1))
    ref = xp.view(B, H // s + 1, s, W // s + 1, s, Cin).permute(0, 1, 3, 2, 4, 5).reshape(B, H // s + 1, W // s + 1, s * s * Cin)
    got = vig_b200.ops.stem_unfold(x.cuda(), s).cpu()
    assert torch.equal(got, ref)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,W,bias,act", [(2, 1024, 1024, True, True), (3, 224, 224, True, True), (2, 320, 320, False, True),
                                            (1, 8, 8, True, False), (5, 264, 1000, True, True), (150, 224, 224, True, True)])
def test_stem_conv_layernorm_fused_gemm(dtype, B, H, W, bias, act):
    """First stem convolution + bias + LayerNorm2d + swish as one tensor-core kernel: against the fp32 convolution of the
    same 16-bit operands followed by LayerNorm (+ swish), and against the separate steps (library convolution on the
    unfolded cells, then the LayerNorm kernel) it replaces.  Output widths that fill a 128-pixel tile exactly, that split
    into 32 x 4 and 64 x 2 tiles with clipped edges, a single pixel, a ragged wide image, and more tiles than SMs."""
    import torch.nn.functional as F
    import vig_b200
    from vig_b200.vig import V2PatchEmbed
    g = torch.Generator().manual_seed(H + W + B)
    pe = V2PatchEmbed(img_size=H, patch_size=16, in_chans=3, embed_dim=192, use_bias_in_patch=bias)
    with torch.no_grad():
        for prm in pe.parameters():
            prm.copy_(torch.randn(prm.shape, generator=g) * (0.08 if prm.dim() > 1 else 0.3) + (1.0 if prm.dim() == 1 and prm.numel() == 96 else 0.0))
    pe = pe.to(dtype).cuda().eval()
    x = torch.randn(B, 3, H, W, generator=g).to(dtype).cuda()
    conv, ln1 = pe.proj[0], pe.proj[1]
    with torch.no_grad():
        cells = vig_b200.ops.stem_fold(x)
        assert torch.equal(cells, x.view(B, 3, H // 8, 8, W // 8, 8).permute(0, 2, 4, 3, 1, 5).reshape(B, H // 8, W // 8, 192))
        assert vig_b200.ops.stem_conv_ln_supported(cells, 96)
        got = vig_b200.ops.stem_conv_ln(cells, pe._gemm_weight(), conv.bias, ln1.weight, ln1.bias, ln1.eps, act_swish=act)
        # the steps it replaces
        y = pe._conv1(x)
        sep = vig_b200.ops.layernorm_act(y.permute(0, 2, 3, 1).contiguous(), ln1.weight, ln1.bias, ln1.eps, act_swish=act, pre_bias=conv.bias)
        # fp32 reference from the same 16-bit operands
        ref = F.conv2d(x.float(), conv.weight.float(), conv.bias.float() if bias else None, conv.stride, conv.padding).permute(0, 2, 3, 1)
        ref = F.layer_norm(ref, (96,), ln1.weight.float(), ln1.bias.float(), ln1.eps)
        if act:
            ref = ref * torch.sigmoid(ref)
    assert got.shape == sep.shape == ref.shape
    assert rel_err(got.float(), ref) < TOL[dtype]
    assert rel_err(got.float(), sep.float()) < TOL[dtype]
    vig_b200.check_status()


def test_patch_embed_matches_oracle():
    import vig_b200
    shape = oracle.ViGShape(192, 3, 1, 0.5, 1.0, True, True, num_classes=16)
    sd = oracle.make_state_dict(shape, seed=2)
    model = vig_b200.ViG.from_shape(shape)
    model.load_state_dict(sd)
    model = model.cuda().eval()
    for size in (224, 320):
        img = oracle.make_images(2, size, seed=size)
        ref, hw = oracle.patch_embed_v2({k: v.float() for k, v in sd.items()}, img)
        with torch.no_grad():
            tok, hw2 = model.patch_embed(img.cuda())
        assert tuple(hw) == tuple(hw2)
        assert rel_err(tok, ref) < 1e-4


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(dtype):
    import vig_b200
    g = torch.Generator().manual_seed(4)
    gy = (2 * torch.randn(3, 37, 1024, generator=g)).to(dtype)
    gate, y = gy.chunk(2, -1)
    ref = oracle.swiglu(gate.float(), y.float())
    gc = gy.cuda()
    out = vig_b200.swiglu(*gc.chunk(2, -1))
    assert rel_err(out.float(), ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,K,N,with_res", [(392, 192, 192, True), (1000, 512, 192, True), (128, 64, 64, False), (70, 384, 384, True),
                                            (5000, 1024, 384, True), (300, 192, 128, True), (260, 128, 256, True)])
def test_linear_add_rmsnorm_fused_gemm(dtype, M, K, N, with_res):
    """Projection + residual add + RMSNorm in one tcgen05 kernel against F.linear followed by vig_add_rmsnorm_fwd
    (same roundings) and against fp32 arithmetic."""
    import torch.nn.functional as F
    import vig_b200
    g = torch.Generator().manual_seed(M + K + N)
    x = torch.randn(M, K, generator=g).to(dtype).cuda()
    w = (torch.randn(N, K, generator=g) / K ** 0.5).to(dtype).cuda()
    res = torch.randn(M, N, generator=g).to(dtype).cuda() if with_res else None
    nw = (1 + 0.1 * torch.randn(N, generator=g)).to(dtype).cuda()
    assert vig_b200.ops.linear_add_rmsnorm_supported(x, w)
    h, r = vig_b200.ops.linear_add_rmsnorm(x, w, res, nw, 1e-6)
    y = F.linear(x, w)
    if with_res:
        h_ref, r_ref = vig_b200.add_rmsnorm(y, nw, residual=res, eps=1e-6, prenorm=True)
    else:
        h_ref, r_ref = vig_b200.add_rmsnorm(y, nw, eps=1e-6), y
    assert rel_err(r.float(), r_ref.float()) < 5e-3          # the two GEMMs sum in different orders before rounding
    assert rel_err(h.float(), h_ref.float()) < 5e-3
    r32 = x.float() @ w.float().t() + (res.float() if with_res else 0)
    h32 = r32 * torch.rsqrt(r32.pow(2).mean(-1, keepdim=True) + 1e-6) * nw.float()
    assert rel_err(r.float(), r32) < 2e-2 and rel_err(h.float(), h32) < 2e-2


def test_model_with_norms_fused_into_projection_epilogues_matches_default_path():
    """``ViG.fuse_norm_epilogues``: same logits as the default path (same roundings, different GEMM kernels)."""
    import vig_b200
    shape = oracle.ViGShape(192, 3, 3, 1.0, 1.0, True, True, num_classes=16)
    model = vig_b200.ViG.from_shape(shape)
    model.load_state_dict(oracle.make_state_dict(shape, seed=4))
    model = model.cuda().bfloat16().eval()
    images = oracle.make_images(2, 224, seed=5).cuda().bfloat16()
    with torch.no_grad():
        model.fuse_norm_epilogues = False
        ref = model(images)
        model.fuse_norm_epilogues = True
        got = model(images)
    assert rel_err(got.float(), ref.float()) < 2e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,K,I", [(392, 192, 512), (1000, 384, 1024), (128, 64, 64), (70, 192, 128), (5000, 192, 512),
                                   (40000, 192, 512), (38000, 64, 128), (37930, 128, 384)])   # the last three: the N = 256 form (many row tiles)
def test_linear_swiglu_fused_gemm(dtype, M, K, I):
    import vig_b200
    g = torch.Generator().manual_seed(M + K)
    x = torch.randn(2, M // 2, K, generator=g).to(dtype)
    w = (torch.randn(2 * I, K, generator=g) / K ** 0.5).to(dtype)
    gy = x.float() @ w.float().t()
    ref = oracle.swiglu(*gy.chunk(2, -1))
    assert vig_b200.ops.linear_swiglu_supported(x.cuda(), w.cuda())
    out = vig_b200.linear_swiglu(x.cuda(), w.cuda())
    assert out.shape == (2, M // 2, I)
    assert rel_err(out.float(), ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,K,N,bias", [(40000, 192, 1152, True), (38000, 64, 96, True), (37930, 128, 320, False), (262144, 192, 1152, True)])
def test_linear_bias_gemm(dtype, M, K, N, bias):
    """The stacked input projection as the library's own tensor-core GEMM: against the fp32 product at the type's bar, and
    against the vendor GEMM (same roundings: fp32 accumulate, bias added in fp32, one rounding) to a few output steps.
    Shapes: the block's N = 1152 at a ragged M, a last column block that is mostly past N, no bias, the benchmark's M."""
    import vig_b200
    from vig_b200 import ops
    g = torch.Generator().manual_seed(M + N)
    x = torch.randn(M, K, generator=g).to(dtype).cuda()
    w = (torch.randn(N, K, generator=g) / K ** 0.5).to(dtype).cuda()
    b = torch.randn(N, generator=g).to(dtype).cuda() if bias else None
    assert ops.linear_bias_supported(x, w)
    out = ops.linear_bias(x.view(2, M // 2, K), w, b)
    vig_b200.check_status()
    assert out.shape == (2, M // 2, N)
    out = out.view(M, N)
    rows = torch.cat([torch.arange(0, 4096), torch.arange(M - 4096, M)]).cuda()      # both ends (the last tile is ragged)
    ref = x[rows].float() @ w.float().t() + (b.float() if bias else 0.0)
    assert rel_err(out[rows].float().cpu(), ref.cpu()) < TOL[dtype]
    lib = torch.nn.functional.linear(x, w, b)
    assert rel_err(out.float().cpu(), lib.float().cpu()) < (1.6e-2 if dtype == torch.bfloat16 else 2e-3)


def _shape(preset):
    base = oracle.PRESETS[preset]
    return oracle.ViGShape(**{**base.__dict__, "depth": 2, "num_classes": 16})


MODEL_CASES = [("t224", "vig_t", 224, 2), ("t320", "vig_t", 320, 1), ("s224", "vig_s", 224, 1), ("tdk64", "vig_t_dk64", 224, 1)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tag,preset,size,batch", MODEL_CASES)
def test_block_and_model_match_reference_vectors(golden_block, tag, preset, size, batch, dtype):
    import vig_b200
    shape = _shape(preset)
    sd = oracle.make_state_dict(shape, seed=11)
    model = vig_b200.ViG.from_shape(shape)
    model.load_state_dict(sd, strict=True)
    model = model.to("cuda", dtype).eval()
    g = size // 16
    x = torch.randn(batch, g * g, shape.embed_dim, generator=torch.Generator().manual_seed(21))
    with torch.no_grad():
        blk = model.blocks[0]
        a = blk.attn(blk.attn_norm(x.to("cuda", dtype)), patch_resolution=(g, g))
        y = blk(x.to("cuda", dtype), patch_resolution=(g, g))[0]
        logits = model(oracle.make_images(batch, size, seed=3).to("cuda", dtype))
    tol = TOL[dtype]
    errs = (rel_err(a.float(), golden_block[f"attn_{tag}_y"]), rel_err(y.float(), golden_block[f"block_{tag}_y"]),
            rel_err(logits.float(), golden_block[f"vig_{tag}_logits"]))
    print(f"{tag} {dtype}: attn {errs[0]:.2e} block {errs[1]:.2e} logits {errs[2]:.2e} (bar {tol:.0e})")
    vig_b200.check_status()
    assert errs[0] < tol and errs[1] < tol and errs[2] < tol, errs


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_dwconv3x3_band_with_halo_rows(dtype):
    """A band of image rows with the rows above and below handed over separately (what a rank of the sequence split
    holds) gives exactly the rows the whole-image call gives."""
    import vig_b200
    B, h, w, C = 2, 12, 10, 192
    x = torch.randn(B, h * w, C, generator=torch.Generator().manual_seed(31)).to("cuda", dtype)
    taps = (0.3 * torch.randn(9, C, generator=torch.Generator().manual_seed(32))).to("cuda", dtype)
    whole = vig_b200.dwconv3x3(x, taps, None, (h, w), True)
    for r0, r1 in ((0, 5), (5, 9), (9, 12)):
        band = x[:, r0 * w:r1 * w].contiguous()
        top = x[:, (r0 - 1) * w:r0 * w].contiguous() if r0 > 0 else None
        bottom = x[:, r1 * w:(r1 + 1) * w].contiguous() if r1 < h else None
        y = vig_b200.dwconv3x3(band, taps, None, (r1 - r0, w), True, top=top, bottom=bottom)
        assert torch.equal(y, whole[:, r0 * w:r1 * w])


def test_model_forward_captures_into_a_cuda_graph_after_eager_forwards():
    """The model's forward can be captured into a CUDA graph at any point: eager forwards leave an asynchronous read of
    the status word pending, and the forward must not query it while the stream is capturing.  The replay gives the eager
    result bit for bit."""
    import vig_b200
    shape = _shape("vig_t_dk64")
    model = vig_b200.ViG.from_shape(shape)
    model.load_state_dict(oracle.make_state_dict(shape, seed=0))
    model = model.to("cuda", torch.bfloat16).eval()
    x = oracle.make_images(2, 320, seed=3).to("cuda", torch.bfloat16)
    with torch.no_grad():
        for _ in range(3):
            eager = model(x)                                   # leaves a snapshot of the status word in flight
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            captured = model(x)
        captured.zero_()
        graph.replay()
    torch.cuda.synchronize()
    vig_b200.check_status()
    assert torch.equal(captured, eager)
