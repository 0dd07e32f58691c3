"""llmx_b200: a small, whole inference engine for one GPU (NVIDIA B200, sm_100a).

Everything between a request's tokens and its next token: typed configuration,
weights by name, layers put together from parts, a paged cache, one step
function, a scheduler, sampling, and hand-written CUDA kernels.
"""
__version__ = "0.1.0"
