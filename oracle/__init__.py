"""CPU restatement of the reference's bi-GLA operator and ViG block (TEST INFRASTRUCTURE ONLY).

This package is the parity checker.  It is imported by the tests, by the smoke
check and by the CPU-baseline / reference legs of the benchmark, and by nothing
else: the product path (``vig_b200``) never imports it and has no CPU fallback.

Parity status: PINNED.  The reference ships no golden vectors for this path, so
the pins are outputs of the reference's own Python code (its naive recurrent GLA
and its ``classification/models/vig.py`` module graph with the three GPU-only
leaf ops replaced by the reference's own PyTorch references) run on CPU; the
generating script and the vectors live in ``tests/golden/``.
"""
from .gla import naive_gla, naive_bi_gla, chunked_bi_gla_f64      # noqa: F401
from .block import (rms_norm, swiglu, dwconv3x3_nlc, gate_inject,  # noqa: F401
                    gla_attention_forward, mlp_forward, block_forward, vig_forward,
                    patch_embed_v2, resize_pos_embed)
from .weights import ViGShape, PRESETS, make_state_dict, make_images, make_bigla_inputs, seeded_like  # noqa: F401
