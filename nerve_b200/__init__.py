"""B200-native CUDA backend for NERVE's route-native MXFP4 sparse-expert (MoE) layer.

The product is ``libnerve_cuda_moe.so`` (hand-written CUDA for sm_100a behind the C ABI of
``include/nerve_cuda_moe.h``); this package is the thin host side: the ctypes binding, a mirror
of the reference's device object model, the expert-parallel driver and seeded synthetic inputs.
There is no CPU fallback: importing the backend without the built library raises.
"""
from .synthetic import CONFIGS, MoeConfig, make_case, small_variant  # noqa: F401

__all__ = ["CONFIGS", "MoeConfig", "make_case", "small_variant"]
