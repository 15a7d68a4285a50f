"""An ``fla`` package made of ``vig_b200`` operators, so that the reference's model files import unchanged.

``classification/models/vig.py:14-27`` imports its operators by name from ``fla``::

    from fla.models import GLAConfig
    from fla.modules import FusedRMSNormSwishGate, RMSNorm
    from fla.ops.gla import chunk_gla, fused_chunk_gla, fused_recurrent_gla
    from fla.ops.gla.chunk_fuse import FusedChunkGLAFunction, pad
    from fla.modules.activations import swiglu, swiglu_linear
    from fla.ops.gla.recurrent_fuse import bid_fused_recurrent_gla

``install()`` puts the folder that holds this stand-in ``fla`` package at the front of ``sys.path`` (and drops an ``fla``
that was imported before), after which those lines resolve to the CUDA kernels of this library.
"""
import os
import sys

SHIM_DIR = os.path.dirname(os.path.abspath(__file__))


def install():
    """Make ``import fla`` resolve to the stand-in package.  Returns the folder that was added to ``sys.path``."""
    for name in [n for n in sys.modules if n == "fla" or n.startswith("fla.")]:
        del sys.modules[name]
    if SHIM_DIR in sys.path:
        sys.path.remove(SHIM_DIR)
    sys.path.insert(0, SHIM_DIR)
    return SHIM_DIR
