"""hyperion_b200: a single-GPU inference engine for sm_100a, built from parts.

A model folder (config.json + safetensors) is read into a typed configuration, turned into a model
of registered parts, and stepped over a paged cache by hand-written CUDA kernels.  See
:mod:`hyperion_b200.api` for the Python entry point.
"""
__version__ = "0.1.0"
