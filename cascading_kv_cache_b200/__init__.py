"""B200-native cascading KV cache hot path: the cache update and the attention over the cache.

The package is a host-side mirror of the reference's ``cascade/models`` interface for this path;
all device work is done by hand-written sm_100a kernels in ``libckv_b200.so`` (C ABI in
``include/cascade_kv_b200.h``).  There is no CPU or PyTorch fallback.
"""
from .cascading_cache import CascadingKVCache, cascade_every_n, sink_cache  # noqa: F401
from .flash_attention import attention  # noqa: F401
from .cascade_attention import (  # noqa: F401
    CascadeAttention, LlamaCascadeAttention, Qwen2CascadeAttention, cascade_attention, sample_monkeypatch)

__all__ = ["CascadingKVCache", "cascade_every_n", "sink_cache", "attention", "CascadeAttention",
           "LlamaCascadeAttention", "Qwen2CascadeAttention", "cascade_attention", "sample_monkeypatch"]
