"""r4dx_b200: a Blackwell-native (sm_100a) inference engine for Qwen-style hybrid models.

Framework layer in PyTorch (module graph, scheduler, paged-KV allocator, server); hot paths are
hand-written CUDA kernels behind a plain C ABI in ``r4dx_b200/native``.
"""
__version__ = "0.1.0"
