"""Generate the golden vectors in this folder from the REFERENCE's own Python code on CPU.

Run once, in a container that has the reference checkout, as
    python tests/golden/make_golden.py /path/to/reference [ops] [blocks] [full] [hier]
(no selection = all four files: ``bigla_ref.npz``, ``block_ref.npz``, ``model_ref.npz``, ``hier_ref.npz``; ``full`` alone takes
about a quarter of an hour on 8 cores, most of it the 16384-token case).
It cannot run where the reference is absent; the committed ``.npz`` files are what the
tests read.  What is executed on the reference side:
  * ``fla/ops/gla/naive.py`` ``naive_recurrent_gla`` (the operator pin), and
  * ``classification/models/vig.py`` ``GLABlock`` / ``ViG`` built from the reference classes,
    in ``eval()`` mode, with the three GPU-only leaf ops replaced by the reference's own
    PyTorch references: ``RMSNorm.forward -> rms_norm_ref`` (``fla/modules/rmsnorm.py:38-52``),
    ``bid_fused_recurrent_gla ->`` the naive recurrence /2 (``recurrent_fuse.py:442``), and
    ``swiglu_linear -> F.linear(x*sigmoid(x)*y, W, b)`` (``fla/modules/activations.py:109-113``).
Packages the reference imports but that are not installed (timm, causal_conv1d) are stubbed
with the handful of names ``vig.py`` needs; none of them is on the eval path.
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import oracle  # noqa: E402  (only for the seeded weight / input generators)


def load_reference(ref_root):
    import transformers  # noqa: F401  must be imported before the stubs
    fla_root = os.path.join(ref_root, "flash-linear-attention", "fla")
    fla = types.ModuleType("fla"); fla.__path__ = [fla_root]; sys.modules["fla"] = fla
    for name in ("fla.models",):
        m = types.ModuleType(name); m.__path__ = []; sys.modules[name] = m
    spec = importlib.util.spec_from_file_location(
        "fla.models.gla_config", os.path.join(fla_root, "models", "gla", "configuration_gla.py"))
    cfgmod = importlib.util.module_from_spec(spec); spec.loader.exec_module(cfgmod)
    sys.modules["fla.models"].GLAConfig = cfgmod.GLAConfig
    # fla.modules: load only rmsnorm + activations (the package __init__ pulls GPU-only code)
    mods = types.ModuleType("fla.modules"); mods.__path__ = [os.path.join(fla_root, "modules")]
    sys.modules["fla.modules"] = mods
    import fla.modules.rmsnorm as rmsnorm
    mods.RMSNorm = rmsnorm.RMSNorm
    mods.FusedRMSNormSwishGate = object
    # timm / causal_conv1d stubs
    def mk(name, **attrs):
        m = types.ModuleType(name); m.__dict__.update(attrs); sys.modules[name] = m; return m
    class DropPath(nn.Identity):
        def __init__(self, p=0.): super().__init__()
    def to_2tuple(x): return tuple(x) if isinstance(x, (tuple, list)) else (x, x)
    def trunc_normal_(t, std=1.): return nn.init.trunc_normal_(t, std=std, a=-2 * std, b=2 * std)
    mk("timm"); mk("timm.models")
    mk("timm.models.vision_transformer", VisionTransformer=object, _cfg=lambda **k: k, Attention=nn.Module)
    mk("timm.models.registry", register_model=lambda f: f)
    mk("timm.models.layers", trunc_normal_=trunc_normal_, DropPath=DropPath, to_2tuple=to_2tuple)
    mk("causal_conv1d"); mk("causal_conv1d.causal_conv1d_interface", CausalConv1dFn=object)
    # the jiterator strings need CUDA at import time: provide the module with CPU restatements
    act = mk("fla.modules.activations",
             swiglu=lambda x, y: x * torch.sigmoid(x) * y,
             swiglu_linear=lambda x, y, w, b: F.linear(x * torch.sigmoid(x) * y, w, b))
    sys.path.insert(0, os.path.join(ref_root, "classification", "models"))
    spec = importlib.util.spec_from_file_location("ref_vig", os.path.join(ref_root, "classification", "models", "vig.py"))
    vig = importlib.util.module_from_spec(spec); spec.loader.exec_module(vig)
    from fla.ops.gla.naive import naive_recurrent_gla

    def rms_forward(self, x, residual=None, prenorm=False, residual_in_fp32=False):
        return rmsnorm.rms_norm_ref(x, self.weight, self.bias, residual=residual, eps=self.eps, prenorm=prenorm)
    rmsnorm.RMSNorm.forward = rms_forward

    def bid_naive(q, k, v, gk, gv=None, *a, **kw):
        B = q.shape[0]
        o_f, _ = naive_recurrent_gla(q, k, v, gk[:B])
        o_b, _ = naive_recurrent_gla(q.flip(2), k.flip(2), v.flip(2), gk[B:].flip(2))
        return (o_f + o_b.flip(2)) / 2, None
    vig.bid_fused_recurrent_gla = bid_naive
    return vig, naive_recurrent_gla


def ref_bigla(naive, q, k, v, gf, gb):
    o_f, _ = naive(q, k, v, gf)
    o_b, _ = naive(q.flip(2), k.flip(2), v.flip(2), gb.flip(2))
    return o_f + o_b.flip(2)


def build_reference_model(vig, shape, sd):
    model = vig.ViG(img_size=224, patch_size=16, stride=16, depth=shape.depth, num_heads=shape.num_heads,
                    embed_dim=shape.embed_dim, num_classes=shape.num_classes, if_cls_token=False,
                    classification_mode="avgpool", use_out_act=shape.use_out_act, use_swiglu=True,
                    use_act_in_conv=shape.use_act_in_conv, expand_k=shape.expand_k, expand_v=shape.expand_v,
                    patch_embed_version="v2", drop_path_rate=0.0)
    missing, unexpected = model.load_state_dict(sd, strict=False)
    assert not unexpected and not missing, (missing, unexpected)
    return model.eval()


# Full-depth models at the benchmark's configurations: the same seeded weights and images the benchmark uses
# (weights seed 0, 1000 classes, images seed 0), so the vectors pin the very model the throughput is quoted on.
FULL_CASES = (("t1024", "vig_t_dk64", 1024, 1), ("s224x16", "vig_s_dk64", 224, 16), ("t224x4_dk32", "vig_t", 224, 4),
              ("b2048", "vig_b_dk64", 2048, 1))


def full_models(vig):
    import time
    out = {}
    for tag, preset, size, batch in FULL_CASES:
        shape = oracle.PRESETS[preset]
        model = build_reference_model(vig, shape, oracle.make_state_dict(shape, seed=0))
        t0 = time.time()
        out[f"vig_{tag}_logits"] = model(oracle.make_images(batch, size, seed=0)).numpy().astype(np.float32)
        print(tag, f"{time.time() - t0:.1f} s", flush=True)
    np.savez_compressed(os.path.join(HERE, "model_ref.npz"), **out)


# Hierarchical model (classification/models/vig_h.py): two tiny four-stage models, one per layout of the reference
# (channels first with LayerNorm2d / gated MLP / v2 stem / v3 downsampling as in configs/vig-h/*.yaml, and channels last
# with plain LayerNorm / GELU MLP / v1 stem / v2 downsampling), weights from oracle.seeded_like (keyed by parameter name).
HIER_CASES = {
    "cf": dict(depths=[1, 1, 2, 1], dims=96, num_heads=[3, 6, 12, 24], norm_layer="ln2d", patchembed_version="v2",
               downsample_version="v3", gmlp=True, use_act_in_conv=False, use_out_act=False, num_classes=12, drop_path_rate=0.0),
    "cl": dict(depths=[1, 1, 1, 1], dims=64, num_heads=[2, 4, 8, 16], norm_layer="ln", patchembed_version="v1",
               downsample_version="v2", gmlp=False, use_act_in_conv=True, use_out_act=True, num_classes=12, drop_path_rate=0.0,
               expand_k=1.0),
}


def hier_models(ref_root, vig):
    def mk(name, **attrs):
        m = types.ModuleType(name); m.__dict__.update(attrs); sys.modules[name] = m; return m
    mk("fvcore"); mk("fvcore.nn", FlopCountAnalysis=object, flop_count_str=None, flop_count=None, parameter_count=None)
    mk("torchvision"); mk("torchvision.models", VisionTransformer=object)
    spec = importlib.util.spec_from_file_location("ref_vig_h", os.path.join(ref_root, "classification", "models", "vig_h.py"))
    vh = importlib.util.module_from_spec(spec); spec.loader.exec_module(vh)
    vh.bid_fused_recurrent_gla = vig.bid_fused_recurrent_gla          # the naive recurrence / 2, as for the plain model
    out = {}
    for tag, kw in HIER_CASES.items():
        model = vh.HierViG(**kw).eval()
        sd = oracle.seeded_like(model.state_dict(), seed=5)
        model.load_state_dict(sd, strict=True)
        images = oracle.make_images(2, 64, seed=9)
        out[f"hier_{tag}_logits"] = model(images).numpy().astype(np.float32)
        x = model.patch_embed(images)
        x = model.layers[0].blocks(x)                                 # the first stage, before its downsampling
        if kw["norm_layer"] == "ln2d":
            x = x.permute(0, 2, 3, 1)
        out[f"hier_{tag}_stage0"] = x.reshape(2, -1, x.shape[-1]).numpy().astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "hier_ref.npz"), **out)


def main(ref_root, only=()):
    vig, naive = load_reference(ref_root)
    torch.set_grad_enabled(False)
    if not only or "hier" in only:
        hier_models(ref_root, vig)
    if not only or "ops" in only:
        operator_pins(naive)
    if not only or "blocks" in only:
        block_pins(vig)
    if not only or "full" in only:
        full_models(vig)
    print("written", sorted(os.listdir(HERE)))


def operator_pins(naive):
    out = {}
    # ---- operator pins -------------------------------------------------------------------
    cases = {"cfg1": (2, 3, 196, 64, 64, 0), "dk32": (1, 3, 196, 32, 64, 1), "L1": (1, 2, 1, 64, 64, 2),
             "L17": (2, 1, 17, 32, 64, 3), "L300": (1, 2, 300, 64, 64, 4)}
    for name, (B, H, L, dk, dv, seed) in cases.items():
        q, k, v, gf, gb = oracle.make_bigla_inputs(B, H, L, dk, dv, seed)
        out[f"bigla_{name}_shape"] = np.array([B, H, L, dk, dv, seed])
        out[f"bigla_{name}_o"] = ref_bigla(naive, q, k, v, gf, gb).numpy()
    # same-gate both-direction form of the reference (naive.py:44-58, causal=False)
    q, k, v, gf, _ = oracle.make_bigla_inputs(1, 2, 64, 64, 64, 5)
    o, o_rev = naive(q, k, v, gf, causal=False)
    out["bigla_samegate_o"] = (o + o_rev).numpy()
    # one-direction with initial / final state (naive.py:30-31,43)
    h0 = torch.randn(1, 2, 64, 64, generator=torch.Generator().manual_seed(6))
    o, hT = naive(q, k, v, gf, initial_state=h0, output_final_state=True)
    out["gla_state_o"], out["gla_state_hT"] = o.numpy(), hT.numpy()
    np.savez_compressed(os.path.join(HERE, "bigla_ref.npz"), **out)


def block_pins(vig):
    # ---- block / model pins --------------------------------------------------------------
    out = {}
    for tag, preset, size, batch in (("t224", "vig_t", 224, 2), ("t320", "vig_t", 320, 1),
                                     ("s224", "vig_s", 224, 1), ("tdk64", "vig_t_dk64", 224, 1)):
        base = oracle.PRESETS[preset]
        shape = oracle.ViGShape(**{**base.__dict__, "depth": 2, "num_classes": 16})
        sd = oracle.make_state_dict(shape, seed=11)
        model = build_reference_model(vig, shape, sd)
        images = oracle.make_images(batch, size, seed=3)
        out[f"vig_{tag}_logits"] = model(images).numpy()
        # one block in isolation on a random token tensor
        g = size // 16
        x = torch.randn(batch, g * g, shape.embed_dim, generator=torch.Generator().manual_seed(21))
        blk = model.blocks[0]
        out[f"block_{tag}_y"] = blk(x, patch_resolution=(g, g), token_position=None, lower_bound=0)[0].numpy()
        blk.attn.__DEBUG__ = True
        h = blk.attn(blk.attn_norm(x), patch_resolution=(g, g), token_position=None)
        out[f"attn_{tag}_y"] = h.numpy()
        blk.attn.__DEBUG__ = False
    np.savez_compressed(os.path.join(HERE, "block_ref.npz"), **{k: v.astype(np.float32) for k, v in out.items()})


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py /path/to/reference [ops] [blocks] [full] [hier]")
    main(sys.argv[1], tuple(sys.argv[2:]))
