"""Row-per-request host-pinned KV store for the B200 engine.

Public surface (class name, constructor arguments, method names, errors) follows the
reference's ``DirectKVRequestPool`` (directkv/directkv_request_pool.py:29-174) so that code
written against it keeps working: every live request owns one row of a
``[max_reqs, pad64(max_seqlen), NH_kv, head_dim]`` bf16 tensor per layer, rows are handed out
LIFO from a free-list, and position ``p`` of a request is ``[row, p, h, :]``.

Built differently underneath:
  * K and V of ALL layers live in two page-locked allocations ``[L, R, S, NH, D]``; the
    per-layer tensors in ``k_pool`` / ``v_pool`` are views of them.  One registration with the
    CUDA driver instead of 2*L, and slot arithmetic that is uniform across layers.
  * The engine reads and writes rows IN PLACE: ``row_table`` yields the int32 row map the
    kernels index with, so no per-step gather of rows is ever made.
  * Zero-filling a row on ``alloc`` is optional: the kernels mask by exact length and never
    read beyond a request's tokens.
"""

from __future__ import annotations

import logging
from typing import Dict, Iterable, List, Tuple

import torch

from .sglang_compat import pinned_zeros

logger = logging.getLogger(__name__)

_ALIGN = 64   # row lengths are multiples of 64 tokens (directkv/directkv_request_pool.py:22)


def _pad64(n: int) -> int:
    """Round up to a multiple of 64 (directkv/directkv_request_pool.py:25-26)."""
    return -(-int(n) // _ALIGN) * _ALIGN


class DirectKVRequestPool:
    def __init__(
        self,
        max_reqs: int,
        max_seqlen: int,
        num_kv_heads: int,
        head_dim: int,
        num_layers: int,
        start_layer: int = 0,
        dtype: torch.dtype = torch.bfloat16,
        zero_on_alloc: bool = True,
        spare_rows: int = 0,
    ):
        # spare_rows: rows behind the max_reqs allocatable ones that never enter the free-list.  The backend
        # keeps one as the target of the padded entries of a CUDA-graph replay (``pad_row``), whose stores
        # would otherwise land in some live request's row.
        self.spare_rows = int(spare_rows)
        self.max_reqs = max_reqs
        self.max_seqlen_pad = _pad64(max_seqlen)
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.num_layers = num_layers
        self.start_layer = start_layer
        self.dtype = dtype
        self.zero_on_alloc = zero_on_alloc

        full = (num_layers, max_reqs + self.spare_rows, self.max_seqlen_pad, num_kv_heads, head_dim)
        gib = 2 * torch.Size(full).numel() * dtype.itemsize / 2**30
        logger.info("[DirectKVPool] %d rows x %d layers x K,V [%d, %d, %d] page-locked: %.2f GiB",
                    max_reqs, num_layers, self.max_seqlen_pad, num_kv_heads, head_dim, gib)
        self._k_all = pinned_zeros(full, dtype)
        self._v_all = pinned_zeros(full, dtype)
        self.k_pool: List[torch.Tensor] = list(self._k_all.unbind(0))
        self.v_pool: List[torch.Tensor] = list(self._v_all.unbind(0))

        # LIFO free-list: row max_reqs-1 goes out first, a freed row is reused next
        # (directkv/directkv_request_pool.py:79-104).
        self._free: List[int] = [r for r in range(max_reqs)]
        self._req_to_row: Dict[int, int] = {}

    # ---- request lifecycle ------------------------------------------------
    def alloc(self, req_id: int) -> None:
        """Idempotent; raises RuntimeError when every row is taken."""
        if req_id in self._req_to_row:
            return
        if len(self._free) == 0:
            raise RuntimeError(
                f"[DirectKVPool] Out of rows (max_reqs={self.max_reqs}). "
                "Increase max_reqs or reduce --max-running-requests."
            )
        row = self._free.pop()
        self._req_to_row[req_id] = row
        if self.zero_on_alloc:
            self._k_all[:, row].zero_()
            self._v_all[:, row].zero_()

    def free(self, req_id: int) -> None:
        """Unknown ids are ignored."""
        row = self._req_to_row.pop(req_id, None)
        if row is not None:
            self._free.append(row)

    @property
    def free_rows(self) -> int:
        """Rows that ``alloc`` can still hand out."""
        return len(self._free)

    @property
    def pad_row(self) -> int:
        """First spare row (see ``spare_rows``); ValueError when the pool was built without one."""
        if self.spare_rows < 1:
            raise ValueError("the pool was built without spare rows")
        return self.max_reqs

    def row_of(self, req_id: int) -> int:
        """KeyError for an id that holds no row."""
        return self._req_to_row[req_id]

    def row_table(self, req_ids: Iterable[int], device=None) -> torch.Tensor:
        """int32 rows of ``req_ids`` in order: the engine's ``row_map`` argument."""
        t = torch.tensor([self._req_to_row[r] for r in req_ids], dtype=torch.int32)
        return t if device is None else t.to(device, non_blocking=True)

    # ---- tensor access ----------------------------------------------------
    def _layer(self, layer_id: int) -> int:
        return layer_id - self.start_layer

    def get_kv(self, req_id: int, layer_id: int, s_total: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Views ``[1, s_total, NH_kv, D]`` of the request's row (no copy)."""
        row, li = self._req_to_row[req_id], self._layer(layer_id)
        return (self.k_pool[li][row, :s_total].unsqueeze(0),
                self.v_pool[li][row, :s_total].unsqueeze(0))

    def get_row_tensor(self, layer_id: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """The whole ``[max_reqs, S, NH_kv, D]`` tensors of a layer: what the engine registers."""
        li = self._layer(layer_id)
        return self.k_pool[li], self.v_pool[li]

    def get_batch_kv(self, req_ids: List[int], layer_id: int, s_total: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """``[len(req_ids), s_total, NH_kv, D]`` gathered COPIES.

        The reference's method of this name also copies (a list index gathers,
        directkv/directkv_request_pool.py:148-152); the engine's decode path does not call it.
        """
        li = self._layer(layer_id)
        rows = torch.tensor([self._req_to_row[r] for r in req_ids], dtype=torch.long)
        return (self.k_pool[li].index_select(0, rows)[:, :s_total],
                self.v_pool[li].index_select(0, rows)[:, :s_total])

    def get_cuda_graph_kv(self, layer_id: int, max_bs: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """First ``max_bs`` rows, stable pointers (directkv/directkv_request_pool.py:158-166)."""
        li = self._layer(layer_id)
        return self.k_pool[li][:max_bs], self.v_pool[li][:max_bs]

    def __repr__(self) -> str:
        return (f"DirectKVRequestPool(max_reqs={self.max_reqs}, max_seqlen_pad={self.max_seqlen_pad}, "
                f"layers={self.num_layers}, free={len(self._free)})")
