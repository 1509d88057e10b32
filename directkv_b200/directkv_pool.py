"""Token-indexed host-pinned KV cache for the B200 engine.

Drop-in for the reference's ``DirectKVTokenToKVPool`` (directkv/directkv_pool.py:44-267): same
constructor, same ``KVCache`` methods, same errors.  Per layer the buffers are
``(size + page_size, head_num, head_dim)`` in page-locked host memory; token ``t`` of request
``r`` lives at slot ``req_to_token[r, t]`` (directkv/directkv_backend.py:846-852) and slot 0 is
the reserved padding row (directkv/directkv_pool.py:22-26).

Built differently underneath:
  * one page-locked allocation for K and one for V across all layers;
  * ``set_kv_buffer`` with device tensors is a stream-ordered scatter kernel that stores
    straight into the pinned pool (no blocking device-to-host copy, no CPU scatter); host
    readers call ``synchronize()`` first.  CPU inputs take the host indexing path.
"""

from __future__ import annotations

import logging
from typing import Optional, Tuple

import torch

from .sglang_compat import KVCache, pinned_zeros

logger = logging.getLogger(__name__)


class DirectKVTokenToKVPool(KVCache):
    def __init__(
        self,
        size: int,
        page_size: int,
        dtype: torch.dtype,
        head_num: int,
        head_dim: int,
        layer_num: int,
        device: str = "cpu",
        enable_memory_saver: bool = False,
        v_head_dim: Optional[int] = None,
        start_layer: Optional[int] = None,
        end_layer: Optional[int] = None,
    ):
        if dtype not in (torch.float16, torch.bfloat16):
            # directkv/directkv_pool.py:68-72
            raise ValueError(
                f"DirectKVTokenToKVPool only supports float16 / bfloat16, got {dtype}. "
                "Pass --kv-cache-dtype auto or use a bf16/fp16 model."
            )
        super().__init__(size=size, page_size=page_size, dtype=dtype, layer_num=layer_num, device="cpu",
                         enable_memory_saver=False, start_layer=start_layer, end_layer=end_layer)
        self.head_num = head_num
        self.head_dim = head_dim
        self.v_head_dim = head_dim if v_head_dim is None else v_head_dim
        self._compute_device: Optional[torch.device] = None
        self._allocate()

    # ---- storage ------------------------------------------------------------
    @property
    def _n_layers(self) -> int:
        # The reference sizes by end_layer - start_layer + 1 (directkv/directkv_pool.py:98).
        return self.end_layer - self.start_layer + 1

    @property
    def n_slots(self) -> int:
        """Rows per layer: ``size`` token slots plus the reserved first page (row 0 for page_size 1)."""
        return self.size + max(1, self.page_size)

    def _allocate(self) -> None:
        nl, rows = self._n_layers, self.n_slots
        self._k_all = pinned_zeros((nl, rows, self.head_num, self.head_dim), self.dtype)
        self._v_all = pinned_zeros((nl, rows, self.head_num, self.v_head_dim), self.dtype)
        self.k_buffer = list(self._k_all.unbind(0))
        self.v_buffer = list(self._v_all.unbind(0))
        k_bytes, v_bytes = self.get_kv_size_bytes()
        self.mem_usage = (k_bytes + v_bytes) / 2**30
        self.token_stride = self.head_num * self.head_dim      # directkv/directkv_pool.py:139
        logger.info("[DirectKV] %d layers x (%d slots, %d KV heads, %d dim) page-locked: %.2f GiB",
                    nl, rows, self.head_num, self.head_dim, self.mem_usage)

    def get_kv_size_bytes(self) -> Tuple[int, int]:
        per = self._n_layers * self.n_slots * self.head_num * self.dtype.itemsize
        return per * self.head_dim, per * self.v_head_dim

    # ---- KVCache interface -------------------------------------------------------
    def _li(self, layer_id: int) -> int:
        return layer_id - self.start_layer                      # directkv/directkv_pool.py:165

    def get_key_buffer(self, layer_id: int) -> torch.Tensor:
        return self.k_buffer[self._li(layer_id)]

    def get_value_buffer(self, layer_id: int) -> torch.Tensor:
        return self.v_buffer[self._li(layer_id)]

    def get_kv_buffer(self, layer_id: int) -> Tuple[torch.Tensor, torch.Tensor]:
        return self.get_key_buffer(layer_id), self.get_value_buffer(layer_id)

    def set_kv_buffer(
        self,
        layer,
        loc: torch.Tensor,
        cache_k: torch.Tensor,
        cache_v: torch.Tensor,
        k_scale: Optional[float] = None,
        v_scale: Optional[float] = None,
        layer_id_override: Optional[int] = None,
    ) -> None:
        """Stores ``cache_k/v [n, H, D]`` at slots ``loc [n]`` of the layer's buffers.

        Device inputs: one scatter kernel per tensor on the current stream writes into the
        pinned pool directly.  CPU inputs: plain index assignment, as the reference does after
        its device-to-host copy (directkv/directkv_pool.py:196-209).
        """
        layer_id = layer_id_override if layer_id_override is not None else layer.layer_id
        li = self._li(layer_id)
        if cache_k.is_cuda:
            from . import _lib
            from .kernel import _ptr, _stream

            if loc.dtype not in (torch.int32, torch.int64):
                loc = loc.long()
            loc = loc.to(cache_k.device).contiguous()
            ck = cache_k.to(self.dtype).contiguous()
            cv = cache_v.to(self.dtype).contiguous()
            ctx = _lib.get_context(cache_k.device.index)
            self._compute_device = cache_k.device
            _lib.check(_lib.load().dkv_scatter_kv(
                ctx.handle, _ptr(self.k_buffer[li]), _ptr(self.v_buffer[li]), self.n_slots,
                self.head_num * self.head_dim * self.dtype.itemsize,
                self.head_num * self.v_head_dim * self.dtype.itemsize,
                _ptr(loc), 1 if loc.dtype == torch.int64 else 0, _ptr(ck), _ptr(cv), loc.numel(), _stream()))
            # ck / cv / loc must outlive the kernel: tie them to the stream.
            for t in (ck, cv, loc):
                t.record_stream(torch.cuda.current_stream(cache_k.device))
        else:
            idx = loc.cpu().long()
            self.k_buffer[li][idx] = cache_k.to(self.dtype)
            self.v_buffer[li][idx] = cache_v.to(self.dtype)

    def synchronize(self) -> None:
        """Makes earlier device-side stores visible to host readers of the buffers."""
        if self._compute_device is not None:
            torch.cuda.synchronize(self._compute_device)

    def get_v_head_dim(self) -> int:
        return self.v_head_dim

    @property
    def same_kv_dim(self) -> bool:
        return self.head_dim == self.v_head_dim

    @property
    def row_dim(self) -> int:
        return self.head_num * self.head_dim

    # ---- host-side block moves (directkv/directkv_pool.py:230-257) ---------------------
    def move_kv_cache(self, tgt_loc: torch.Tensor, src_loc: torch.Tensor):
        self.synchronize()
        tgt, src = tgt_loc.cpu().long(), src_loc.cpu().long()
        self._k_all[:, tgt] = self._k_all[:, src].clone()
        self._v_all[:, tgt] = self._v_all[:, src].clone()

    @staticmethod
    def _as_index(x) -> torch.Tensor:
        return (x if isinstance(x, torch.Tensor) else torch.as_tensor(x)).cpu().long()

    def load_from_host_per_layer(self, host_pool, host_indices, device_indices, layer_id, io_backend):
        src, dst = self._as_index(host_indices), self._as_index(device_indices)
        li, h_li = self._li(layer_id), layer_id - host_pool.start_layer
        self.k_buffer[li][dst] = host_pool.k_buffer[h_li][src]
        self.v_buffer[li][dst] = host_pool.v_buffer[h_li][src]

    def backup_to_host_all_layer(self, host_pool, host_indices, device_indices, io_backend):
        self.synchronize()
        h_idx, d_idx = self._as_index(host_indices), self._as_index(device_indices)
        for li in range(len(self.k_buffer)):
            h_li = self.start_layer + li - host_pool.start_layer
            host_pool.k_buffer[h_li][h_idx] = self.k_buffer[li][d_idx]
            host_pool.v_buffer[h_li][h_idx] = self.v_buffer[li][d_idx]

    def get_cpu_copy(self, indices: torch.Tensor):
        raise NotImplementedError("DirectKVTokenToKVPool: CPU is already the storage; no copy needed.")

    def load_cpu_copy(self, kv_cache_cpu, indices: torch.Tensor):
        raise NotImplementedError("DirectKVTokenToKVPool: CPU is already the storage; no load needed.")
