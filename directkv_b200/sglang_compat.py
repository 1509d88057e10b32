"""Third-party base classes the backends and pools derive from.

The reference subclasses SGLang's ``AttentionBackend`` and ``KVCache``
(directkv/directkv_backend.py:32-33, directkv/directkv_pool.py:39).  When SGLang is
importable those classes are used; otherwise minimal stand-ins with the same constructor and
attributes are defined here so that the package, its tests and its benchmark run without it.
"""

from __future__ import annotations

import enum
from typing import Optional

import torch

try:  # pragma: no cover - exercised only where SGLang is installed
    from sglang.srt.layers.attention.base_attn_backend import AttentionBackend  # type: ignore
    from sglang.srt.mem_cache.memory_pool import KVCache  # type: ignore
    from sglang.srt.layers.dp_attention import get_attention_tp_size  # type: ignore
    from sglang.srt.model_executor.forward_batch_info import ForwardMode  # type: ignore

    HAVE_SGLANG = True
except Exception:  # ImportError, or a broken install
    HAVE_SGLANG = False

    class AttentionBackend:  # type: ignore[no-redef]
        """Interface of sglang.srt.layers.attention.base_attn_backend.AttentionBackend."""

        def init_forward_metadata(self, forward_batch):
            raise NotImplementedError

        def init_cuda_graph_state(self, max_bs: int, max_num_tokens: int):
            raise NotImplementedError

        def init_forward_metadata_capture_cuda_graph(self, bs, num_tokens, req_pool_indices, seq_lens,
                                                     encoder_lens, forward_mode, spec_info):
            raise NotImplementedError

        def init_forward_metadata_replay_cuda_graph(self, bs, req_pool_indices, seq_lens, seq_lens_sum,
                                                    encoder_lens, forward_mode, spec_info, seq_lens_cpu=None):
            raise NotImplementedError

        def get_cuda_graph_seq_len_fill_value(self):
            raise NotImplementedError

        def forward(self, q, k, v, layer, forward_batch, save_kv_cache: bool = True, **kwargs):
            if forward_batch.forward_mode.is_idle():
                return q.new_empty(q.shape[0], layer.tp_q_head_num * layer.v_head_dim)
            if forward_batch.forward_mode.is_decode():
                return self.forward_decode(q, k, v, layer, forward_batch, save_kv_cache=save_kv_cache, **kwargs)
            return self.forward_extend(q, k, v, layer, forward_batch, save_kv_cache=save_kv_cache, **kwargs)

        def forward_decode(self, q, k, v, layer, forward_batch, save_kv_cache: bool = True):
            raise NotImplementedError

        def forward_extend(self, q, k, v, layer, forward_batch, save_kv_cache: bool = True):
            raise NotImplementedError

    class KVCache:  # type: ignore[no-redef]
        """Constructor contract of sglang.srt.mem_cache.memory_pool.KVCache (0.4.9)."""

        def __init__(self, size: int, page_size: int, dtype: torch.dtype, layer_num: int, device: str,
                     enable_memory_saver: bool, start_layer: Optional[int] = None,
                     end_layer: Optional[int] = None):
            self.size = size
            self.page_size = page_size
            self.dtype = dtype
            self.device = device
            self.store_dtype = dtype
            self.layer_num = layer_num
            self.start_layer = start_layer or 0
            self.end_layer = end_layer or layer_num - 1
            self.mem_usage = 0

    def get_attention_tp_size() -> int:  # type: ignore[no-redef]
        return 1

    class ForwardMode(enum.IntEnum):  # type: ignore[no-redef]
        EXTEND = 1
        DECODE = 2
        MIXED = 3
        IDLE = 4

        def is_extend(self):
            return self in (ForwardMode.EXTEND, ForwardMode.MIXED)

        def is_decode(self):
            return self == ForwardMode.DECODE

        def is_idle(self):
            return self == ForwardMode.IDLE


def pinned_zeros(shape, dtype: torch.dtype) -> torch.Tensor:
    """Zero-filled page-locked host tensor, placed in the memory of the socket the current CUDA device hangs off
    where the machine has more than one (directkv_b200/numa.py; a no-op elsewhere).

    Without a CUDA driver nothing can be page-locked; then a pageable tensor is returned so the
    host-side logic (indexing, free-list) can still be exercised.  The engine itself refuses
    pageable pools (the C ABI checks the pointer's memory type).
    """
    if torch.cuda.is_available():
        from .numa import local_to_gpu

        with local_to_gpu(torch.cuda.current_device()):
            return torch.zeros(shape, dtype=dtype, pin_memory=True)
    return torch.zeros(shape, dtype=dtype)
