"""The CPU oracle against vectors produced by the reference's own code (tests/golden/make_golden.py)."""
import numpy as np
import pytest
import torch

import oracle
from conftest import rel_err

OP_CASES = ["cfg1", "dk32", "L1", "L17", "L300"]


@pytest.mark.parametrize("name", OP_CASES)
def test_bigla_oracle_matches_reference(golden_bigla, name):
    B, H, L, dk, dv, seed = (int(x) for x in golden_bigla[f"bigla_{name}_shape"])
    q, k, v, gf, gb = oracle.make_bigla_inputs(B, H, L, dk, dv, seed)
    o = oracle.naive_bi_gla(q, k, v, gf, gb)
    assert rel_err(o, golden_bigla[f"bigla_{name}_o"]) < 1e-6


@pytest.mark.parametrize("name", OP_CASES)
def test_chunked_form_matches_reference(golden_bigla, name):
    B, H, L, dk, dv, seed = (int(x) for x in golden_bigla[f"bigla_{name}_shape"])
    q, k, v, gf, gb = oracle.make_bigla_inputs(B, H, L, dk, dv, seed)
    for chunk in (16, 64, 128):
        o = oracle.chunked_bi_gla_f64(q, k, v, gf, gb, chunk=chunk)
        assert rel_err(o, golden_bigla[f"bigla_{name}_o"]) < 1e-5


def test_same_gate_and_state_pins(golden_bigla):
    q, k, v, gf, _ = oracle.make_bigla_inputs(1, 2, 64, 64, 64, 5)
    assert rel_err(oracle.naive_bi_gla(q, k, v, gf, gf), golden_bigla["bigla_samegate_o"]) < 1e-6
    h0 = torch.randn(1, 2, 64, 64, generator=torch.Generator().manual_seed(6))
    o, hT = oracle.naive_gla(q, k, v, gf, initial_state=h0)
    assert rel_err(o, golden_bigla["gla_state_o"]) < 1e-6
    assert rel_err(hT, golden_bigla["gla_state_hT"]) < 1e-6


def _shape(preset):
    base = oracle.PRESETS[preset]
    return oracle.ViGShape(**{**base.__dict__, "depth": 2, "num_classes": 16})


MODEL_CASES = [("t224", "vig_t", 224, 2), ("t320", "vig_t", 320, 1), ("s224", "vig_s", 224, 1),
               ("tdk64", "vig_t_dk64", 224, 1)]


@pytest.mark.parametrize("tag,preset,size,batch", MODEL_CASES)
def test_block_and_model_oracle_match_reference(golden_block, tag, preset, size, batch):
    shape = _shape(preset)
    sd = oracle.make_state_dict(shape, seed=11)
    g = size // 16
    x = torch.randn(batch, g * g, shape.embed_dim, generator=torch.Generator().manual_seed(21))
    h = oracle.rms_norm(x, sd["blocks.0.attn_norm.weight"], eps=shape.eps)
    a = oracle.gla_attention_forward(sd, "blocks.0.attn.", h, (g, g), shape)
    assert rel_err(a, golden_block[f"attn_{tag}_y"]) < 2e-5
    y = oracle.block_forward(sd, "blocks.0.", x, (g, g), shape)
    assert rel_err(y, golden_block[f"block_{tag}_y"]) < 2e-5
    logits = oracle.vig_forward(sd, oracle.make_images(batch, size, seed=3), shape)
    assert rel_err(logits, golden_block[f"vig_{tag}_logits"]) < 5e-5


@pytest.mark.parametrize("tag,preset,size,batch", [("t1024", "vig_t_dk64", 1024, 1), ("s224x16", "vig_s_dk64", 224, 16),
                                                   ("t224x4_dk32", "vig_t", 224, 4)])
def test_full_depth_model_oracle_matches_reference(tag, preset, size, batch):
    """12-block models with the benchmark's weights and images (seed 0) against the reference's logits.  (The 16384-token
    ViG-B vector in the same file takes the oracle a minute and is compared on the GPU only.)"""
    import os
    from conftest import GOLDEN
    ref = np.load(os.path.join(GOLDEN, "model_ref.npz"))[f"vig_{tag}_logits"]
    shape = oracle.PRESETS[preset]
    logits = oracle.vig_forward(oracle.make_state_dict(shape, seed=0), oracle.make_images(batch, size, seed=0), shape)
    assert rel_err(logits, ref) < 1e-4
