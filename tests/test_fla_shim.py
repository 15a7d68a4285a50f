"""The stand-in ``fla`` package: every import line of the reference's model file resolves to ``vig_b200`` objects, and
(where the reference checkout is present) the reference's own ``classification/models/vig.py`` imports unchanged and
builds its model on top of them."""
import importlib.util
import os
import sys
import types

import pytest
import torch
import torch.nn as nn

import oracle

# the reference checkout: named by VIG_REFERENCE_ROOT, else looked for as a `reference` folder beside this repository
_REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_VIG = os.path.join(os.environ.get("VIG_REFERENCE_ROOT", os.path.join(os.path.dirname(_REPO), "reference")),
                       "classification", "models", "vig.py")


@pytest.fixture
def shim():
    from vig_b200 import fla_shim
    saved_path, saved_mods = list(sys.path), {n: m for n, m in sys.modules.items() if n == "fla" or n.startswith("fla.")}
    fla_shim.install()
    yield fla_shim
    sys.path[:] = saved_path
    for n in [n for n in sys.modules if n == "fla" or n.startswith("fla.")]:
        del sys.modules[n]
    sys.modules.update(saved_mods)


def test_every_name_the_reference_imports_resolves(shim):
    import vig_b200
    from fla.models import GLAConfig
    from fla.modules import FusedRMSNormSwishGate, RMSNorm
    from fla.ops.gla import chunk_gla, fused_chunk_gla, fused_recurrent_gla
    from fla.ops.gla.chunk_fuse import FusedChunkGLAFunction, pad
    from fla.modules.activations import swiglu, swiglu_linear
    from fla.ops.gla.recurrent_fuse import bid_fused_recurrent_gla
    import fla
    assert os.path.dirname(fla.__file__).startswith(shim.SHIM_DIR)
    assert RMSNorm is vig_b200.RMSNorm and bid_fused_recurrent_gla is vig_b200.bid_fused_recurrent_gla
    assert fused_chunk_gla is vig_b200.fused_chunk_gla and chunk_gla is vig_b200.chunk_gla
    assert fused_recurrent_gla is vig_b200.fused_recurrent_gla and swiglu is vig_b200.swiglu and swiglu_linear is vig_b200.swiglu_linear
    cfg = GLAConfig(hidden_size=192, num_attention_heads=3, use_swiglu=True, rope_mode="none")
    assert cfg.hidden_size == 192 and cfg.num_attention_heads == 3 and cfg.use_swiglu and cfg.rms_norm_eps == 1e-6
    assert pad(torch.zeros(1, 2, 17, 8)).shape == (1, 2, 32, 8) and pad(torch.zeros(1, 2, 32, 8)).shape == (1, 2, 32, 8)
    assert callable(FusedChunkGLAFunction.apply) and isinstance(FusedRMSNormSwishGate(8), nn.Module)


@pytest.mark.skipif(not os.path.exists(REF_VIG), reason="reference checkout not present")
def test_reference_model_file_imports_unchanged_and_builds(shim):
    import vig_b200
    import transformers  # noqa: F401  (the model file takes ACT2FN from it)

    def mk(name, **attrs):
        m = types.ModuleType(name); m.__dict__.update(attrs); sys.modules[name] = m
        return m

    class DropPath(nn.Identity):
        def __init__(self, p=0.0):
            super().__init__()
    # packages the model file imports but the evaluation path never calls
    added = ["timm", "timm.models", "timm.models.vision_transformer", "timm.models.registry", "timm.models.layers",
             "causal_conv1d", "causal_conv1d.causal_conv1d_interface"]
    mk("timm"); mk("timm.models")
    mk("timm.models.vision_transformer", VisionTransformer=object, _cfg=lambda **k: k, Attention=nn.Module)
    mk("timm.models.registry", register_model=lambda f: f)
    mk("timm.models.layers", trunc_normal_=lambda t, std=1.0: nn.init.trunc_normal_(t, std=std), DropPath=DropPath,
       to_2tuple=lambda x: tuple(x) if isinstance(x, (tuple, list)) else (x, x))
    mk("causal_conv1d"); mk("causal_conv1d.causal_conv1d_interface", CausalConv1dFn=object)
    sys.path.insert(0, os.path.dirname(REF_VIG))
    try:
        spec = importlib.util.spec_from_file_location("ref_vig_via_shim", REF_VIG)
        ref = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(ref)
        assert ref.bid_fused_recurrent_gla is vig_b200.bid_fused_recurrent_gla
        assert ref.RMSNorm is vig_b200.RMSNorm and ref.swiglu_linear is vig_b200.swiglu_linear
        shape = oracle.ViGShape(192, 3, 2, 0.5, 1.0, True, True, num_classes=16)
        model = ref.ViG(img_size=224, patch_size=16, stride=16, depth=shape.depth, num_heads=shape.num_heads,
                        embed_dim=shape.embed_dim, num_classes=shape.num_classes, if_cls_token=False,
                        classification_mode="avgpool", use_out_act=True, use_swiglu=True, use_act_in_conv=True,
                        expand_k=shape.expand_k, expand_v=shape.expand_v, patch_embed_version="v2", drop_path_rate=0.0)
        missing, unexpected = model.load_state_dict(oracle.make_state_dict(shape, seed=1), strict=False)
        assert not missing and not unexpected
        assert isinstance(model.blocks[0].attn_norm, vig_b200.RMSNorm)
    finally:
        for n in added:
            sys.modules.pop(n, None)
        sys.modules.pop("ref_vig_via_shim", None)


@pytest.mark.gpu
def test_reference_call_conventions_through_the_shim(shim):
    """The calls ``classification/models/vig.py`` makes, with its argument conventions, against the oracle."""
    from fla.modules import RMSNorm
    from fla.ops.gla.chunk_fuse import FusedChunkGLAFunction, pad
    from fla.ops.gla.recurrent_fuse import bid_fused_recurrent_gla
    from fla.modules.activations import swiglu_linear
    from conftest import rel_err
    B, H, L, d = 2, 3, 196, 32
    q, k, v, gf, gb = oracle.make_bigla_inputs(B, H, L, d, 64, seed=5)
    # eval branch (vig.py:431-443): strided views of packed projections, gates stacked along the batch
    packed = torch.cat([t.permute(0, 2, 1, 3).reshape(B, L, -1) for t in (q, k, v)], dim=-1).cuda()
    heads = lambda t, dd: t.unflatten(-1, (H, dd)).permute(0, 2, 1, 3)
    qd, kd, vd = heads(packed[..., :H * d], d), heads(packed[..., H * d:2 * H * d], d), heads(packed[..., 2 * H * d:], 64)
    o, _ = bid_fused_recurrent_gla(qd, kd, vd, torch.cat([gf, gb]).cuda(), None)
    assert rel_err(o, oracle.naive_bi_gla(q, k, v, gf, gb, out_scale=0.5)) < 1e-4
    # fp32_fused_chunk_gla (vig.py:190-216): pad, FusedChunkGLAFunction.apply, slice
    args = [pad(t.cuda()) for t in (q, k, v, gf)]
    o2, final = FusedChunkGLAFunction.apply(*args, -1, None, True)
    ref_o, ref_h = oracle.naive_gla(q, k, v, gf)
    assert rel_err(o2[..., :L, :], ref_o) < 1e-4 and rel_err(final, ref_h) < 1e-4
    # norms and the MLP tail
    x, r = torch.randn(4, 50, 192), torch.randn(4, 50, 192)
    norm = RMSNorm(192, eps=1e-6).cuda()
    y, res = norm(x.cuda(), r.cuda(), True)
    s = x + r
    assert rel_err(res, s) < 1e-6 and rel_err(y, oracle.rms_norm(s, norm.weight.detach().cpu(), eps=1e-6)) < 1e-4
    gate, yy, w = torch.randn(4, 50, 512), torch.randn(4, 50, 512), 0.05 * torch.randn(192, 512)
    out = swiglu_linear(gate.cuda(), yy.cuda(), w.cuda(), None)
    assert rel_err(out, torch.nn.functional.linear(gate * torch.sigmoid(gate) * yy, w)) < 1e-4
