"""B200-native attention hot path of the Qwen3.5-0.8B hybrid stack (gated full attention +
Gated DeltaNet, their caches, graph-captured decode).

This package is the Python mirror of the operator interface; all compute happens in
``libb200attn.so`` (hand-written sm_100a CUDA behind the C ABI of ``include/b200attn.h``).
There is no CPU or PyTorch fallback: importing :mod:`ops` without the built library raises.
"""
from . import synth  # noqa: F401  (pure numpy, importable without the native library)

__all__ = ["synth", "ops", "build"]
