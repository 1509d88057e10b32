"""B200-native (sm_100a) decode-attention engine with the SGLang backend surface of DirectKV.

Public pieces: ``kernel`` (entry points over the C ABI), ``DirectKVBackend`` /
``DirectKVSmpV2Backend`` (attention backends), ``DirectKVTokenToKVPool`` / ``DirectKVRequestPool``
(host-pinned KV stores), ``sharding`` (head-sharded and sequence-split multi-GPU helpers).
The CUDA library is built in-tree with ``python -m directkv_b200.build``; nothing here computes on
the CPU.
"""

from .directkv_request_pool import DirectKVRequestPool  # noqa: F401
from .directkv_pool import DirectKVTokenToKVPool  # noqa: F401

__all__ = ["DirectKVRequestPool", "DirectKVTokenToKVPool", "DirectKVBackend", "DirectKVSmpV2Backend"]


def __getattr__(name):
    # The backends import the engine binding; keep the package importable for host-side tooling.
    if name == "DirectKVBackend":
        from .directkv_backend import DirectKVBackend
        return DirectKVBackend
    if name == "DirectKVSmpV2Backend":
        from .directkv_smpv2_backend import DirectKVSmpV2Backend
        return DirectKVSmpV2Backend
    raise AttributeError(name)
