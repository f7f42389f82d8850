"""B200-native (sm_100a) implementation of Bonsai-27B's full-attention path over a
KHQ-compressed KV cache, behind the reference project's C-ABI launch signatures.

Importing this package loads nothing; the CUDA library is loaded on first use by ``lib.load()``
and there is no CPU or PyTorch fallback for any kernel.
"""
from . import calib, lib, synth  # noqa: F401

__all__ = ["calib", "lib", "synth"]
