"""coffin_b200: a Blackwell-native (sm_100a) LLM inference engine for Qwen3.5-style hybrid models.

Layers (lower ones never import higher ones): ``_C`` (CUDA kernels) <- ``ops`` <- ``models`` <-
``engine`` / ``cache`` <- ``serving`` <- ``entrypoints``; ``oracle`` is the CPU fp32 test oracle,
``weights`` the checkpoint formats, ``parallel`` the multi-GPU layer.
"""
__version__ = "0.1.0"
