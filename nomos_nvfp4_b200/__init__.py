"""B200-native (sm_100a) quantized-KV attention for the Nomos kernel.

``ops`` mirrors the reference's operator interface for the attention path and
calls ``libnomos_attn.so`` through its C ABI (``include/nomos_attn.h``).  The shared
object is loaded on first use; there is no CPU or PyTorch fallback.
"""
from . import ops  # noqa: F401

__all__ = ["ops"]
