"""``directkv-smpv2`` backend name of the reference (directkv/directkv_smpv2_backend.py).

In the reference the two backend files differ only in names (class, log tag, error prefix and the
``smpv2_*`` entry points they bind); here the second class derives from the first.
"""

from __future__ import annotations

from . import kernel
from .directkv_backend import DirectKVBackend


class DirectKVSmpV2Backend(DirectKVBackend):
    _NAME = "directkv-smpv2"
    _TAG = "[DirectKV-SMPv2]"

    def __init__(self, model_runner):
        super().__init__(model_runner)
        # attribute names of directkv/directkv_smpv2_backend.py:94-96
        self._smpv2_fwd = kernel.smpv2_fwd
        self._smpv2_init_tma = kernel.smpv2_init_tma
        self._smpv2_fwd_graph = kernel.smpv2_fwd_graph
