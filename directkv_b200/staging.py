"""Decode over a host-resident pool with the past rows brought in by the copy engines.

The streaming kernel reads a host-pinned pool with loads issued by the SMs (TMA); on the machines measured
such reads reach 51.5 GB/s whatever their size, while ``cudaMemcpyAsync`` from the same memory reaches
55.6 GB/s.  Where a request's past rows are one contiguous piece of host memory - the request pool's
``[row, position, head, 128]`` layout (directkv/directkv_request_pool.py:66-76 in the reference) - this helper
copies them with one ``cudaMemcpyAsync`` per request and tensor into a packed staging buffer in HBM and lets
``kernel.decode`` attend that copy (``kv_source_layer``); the new token is still projected with, and stored to,
the host pool.  The step then runs at the rate of the copy engines and leaves the SMs free while the rows are
in flight.  It needs the lengths on the host, so it is for eager steps; under CUDA-graph capture the
streaming kernel stays.
"""

from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from . import kernel

PAGE = 16                      # the packed copy is addressed in 16-token pages (one tile of the streaming kernel)
_STAGE_LAYER_BASE = 2_000_000  # engine ids of the staged copies


class DmaStagedDecode:
    """One staging buffer (K and V) per device, re-used by every layer of a step."""

    def __init__(self, device: torch.device, nh_kv: int, dtype: torch.dtype = torch.bfloat16):
        self.device = torch.device(device)
        self.nh_kv = int(nh_kv)
        self.dtype = dtype
        self._k: Optional[torch.Tensor] = None
        self._v: Optional[torch.Tensor] = None
        self._slots = 0
        self._engine_id = _STAGE_LAYER_BASE + (self.device.index or 0)
        self._table: Optional[torch.Tensor] = None
        self._table_key = None

    # -------------------------------------------------------------------------------------------------
    def _ensure(self, slots: int) -> None:
        if slots <= self._slots:
            return
        if self._k is not None:
            kernel.unregister_layer(self._engine_id)
        slots = int(slots * 1.25) // PAGE * PAGE + PAGE
        self._k = torch.empty(slots, self.nh_kv, 128, dtype=self.dtype, device=self.device)
        self._v = torch.empty_like(self._k)
        self._slots = slots
        kernel.register_layer(self._engine_id, self._k, self._v, page_size=PAGE, device=self.device.index)

    def _page_table(self, past: Sequence[int]) -> torch.Tensor:
        key = tuple(int(n) for n in past)
        if self._table_key == key:
            return self._table
        pages = [(n + PAGE - 1) // PAGE for n in key]
        width = max(1, max(pages))
        table = torch.zeros(len(key), width, dtype=torch.int32)
        at = 0
        for b, n in enumerate(pages):
            table[b, :n] = torch.arange(at, at + n, dtype=torch.int32)
            at += n
        self._table = table.pin_memory().to(self.device, non_blocking=True)
        self._table_key = key
        return self._table

    # -------------------------------------------------------------------------------------------------
    def decode(self, layer_id: int, k_rows: torch.Tensor, v_rows: torch.Tensor, rows: Sequence[int],
               seq_lens_host: Sequence[int], q: torch.Tensor, seq_lens: torch.Tensor, softmax_scale: float,
               row_map: torch.Tensor, x: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
               n_new: int = 1, **kw) -> torch.Tensor:
        """``k_rows`` / ``v_rows``: the layer's pinned pool ``[rows, positions, NH_kv, 128]``; request b lives in
        row ``rows[b]`` and has ``seq_lens_host[b]`` tokens including the ``n_new`` decoded now (0 when no token
        is added).  Everything else as in ``kernel.decode``."""
        past = [int(n) - n_new for n in seq_lens_host]
        starts: List[int] = []
        at = 0
        for n in past:
            starts.append(at)
            at += (n + PAGE - 1) // PAGE * PAGE
        self._ensure(at)
        for b, (r, n, s0) in enumerate(zip(rows, past, starts)):
            if n > 0:
                self._k[s0:s0 + n].copy_(k_rows[r, :n], non_blocking=True)      # one cudaMemcpyAsync each
                self._v[s0:s0 + n].copy_(v_rows[r, :n], non_blocking=True)
        table = self._page_table(past)
        return kernel.decode(layer_id, q, seq_lens, softmax_scale, row_map=row_map, x=x, out=out,
                             kv_source_layer=self._engine_id, src_page_table=table, **kw)
