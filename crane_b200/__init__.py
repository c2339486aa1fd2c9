"""crane_b200: a single-GPU inference engine for Hunyuan Dense on B200 (sm_100a).

Config and registry, weights, parts, paged cache, step function, scheduler,
sampling and the generation API; every kernel on the product path is CUDA
written for this package.
"""
__version__ = "0.1.0"
