"""Stand-in for the ``fla`` package (flash-linear-attention) exposing exactly the names ViG's model files import,
backed by the ``vig_b200`` CUDA library.  See ``vig_b200.fla_shim``."""
