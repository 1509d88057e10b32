"""Multi-GPU use of the engine: one process per GPU, ``torch.distributed`` for the plumbing.

Two partitionings, neither present in the reference (which is single-GPU; heads are only divided
by SGLang's tensor parallelism outside the backend, directkv/directkv_backend.py:68-72):

* **Head sharding** (the default): rank ``r`` of ``tp`` owns KV heads ``[r*NH_kv/tp, (r+1)*NH_kv/tp)``
  and the query heads that attend them, keeps its own host-pinned pool ``[slots, NH_kv/tp, 128]`` and
  a replica of the page table.  KV heads are independent, so attention needs no collective; the
  outputs are disjoint column blocks of the layer output.
* **Sequence split** (one very long request): rank ``r`` owns a contiguous, page-aligned token range
  in its own pool; every rank attends its range and produces the unnormalised ``(O, m, l)`` partial
  per query head (``NH_q x 132`` fp32, about 17 KB); one all-gather over NVLink (NCCL) exchanges them
  and each rank merges locally (``merge_rank_partials_kernel``).  The rank that owns the end of the
  sequence also projects and stores the new token.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

PARTIAL_STRIDE = 132


# --------------------------------------------------------------------------- head sharding
@dataclass(frozen=True)
class HeadShard:
    rank: int
    world: int
    nh_q: int
    nh_kv: int

    def __post_init__(self):
        if self.nh_kv % self.world != 0 or self.nh_q % self.nh_kv != 0:
            raise ValueError(f"cannot shard {self.nh_q} query / {self.nh_kv} KV heads over {self.world} ranks")

    @property
    def kv_heads(self) -> range:
        n = self.nh_kv // self.world
        return range(self.rank * n, (self.rank + 1) * n)

    @property
    def q_heads(self) -> range:
        g = self.nh_q // self.nh_kv
        return range(self.kv_heads.start * g, self.kv_heads.stop * g)

    def weights(self, wk: torch.Tensor, wv: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """This rank's rows of ``[NH_kv, 128, H]`` projection weights."""
        s = slice(self.kv_heads.start, self.kv_heads.stop)
        return wk[s].contiguous(), wv[s].contiguous()

    def queries(self, q: torch.Tensor) -> torch.Tensor:
        """This rank's heads of ``q [B, NH_q, 128]``."""
        return q[:, self.q_heads.start:self.q_heads.stop].contiguous()

    def pool(self, k_full: torch.Tensor) -> torch.Tensor:
        """This rank's heads of a full pool ``[slots, NH_kv, 128]`` (for building test shards)."""
        return k_full[:, self.kv_heads.start:self.kv_heads.stop].contiguous()


def gather_head_outputs(out_local: torch.Tensor, group=None) -> torch.Tensor:
    """Concatenates per-rank outputs ``[B, NH_q/tp, 128]`` along the head axis (parity checks only:
    in a model the following row-parallel projection consumes the shards directly)."""
    world = dist.get_world_size(group)
    parts = [torch.empty_like(out_local) for _ in range(world)]
    dist.all_gather(parts, out_local.contiguous(), group=group)
    return torch.cat(parts, dim=1)


# --------------------------------------------------------------------------- sequence split
def plan_sequence_split(n_tokens: int, world: int, page_size: int) -> List[Tuple[int, int]]:
    """Contiguous token ranges ``[start, end)`` per rank, cut at page boundaries, pages spread evenly.

    Ranks at the end may get empty ranges when there are fewer pages than ranks.
    """
    if n_tokens < 0 or world <= 0 or page_size <= 0:
        raise ValueError("bad arguments")
    pages = -(-n_tokens // page_size)
    base, extra = divmod(pages, world)
    out, p0 = [], 0
    for r in range(world):
        n = base + (1 if r < extra else 0)
        start = min(p0 * page_size, n_tokens)
        end = min((p0 + n) * page_size, n_tokens)
        out.append((start, end))
        p0 += n
    return out


def owner_of_new_token(plan: Sequence[Tuple[int, int]]) -> int:
    """Rank whose range ends the sequence (it projects and stores the token decoded next)."""
    last = 0
    for r, (s, e) in enumerate(plan):
        if e > s:
            last = r
    return last


def all_gather_partials(part_local: torch.Tensor, group=None) -> torch.Tensor:
    """``[rows, 132]`` per rank -> ``[world, rows, 132]`` on every rank (NCCL on GPUs, gloo on CPU)."""
    world = dist.get_world_size(group)
    flat = part_local.contiguous()
    out = torch.empty((world,) + tuple(flat.shape), dtype=flat.dtype, device=flat.device)
    if flat.is_cuda:
        dist.all_gather_into_tensor(out, flat, group=group)
    else:
        parts = [torch.empty_like(flat) for _ in range(world)]
        dist.all_gather(parts, flat, group=group)
        out = torch.stack(parts, dim=0)
    return out


class PartialExchange:
    """Peer-memory exchange for sequence-split decode on the GPUs of one box (at most 8 ranks).

    Each rank owns a device buffer ``[world, max_rows, 132]`` fp32 plus arrival counters; the buffers are
    mapped into every rank with CUDA IPC.  A decode step then needs no collective call: the merge kernel
    stores its partial records into every rank's buffer (plain stores over NVLink) and bumps that rank's
    counter; a second kernel waits - with a time limit - for all sources and merges from local memory.
    Every rank must make the same sequence of ``decode`` calls with the same ``B * NH_q``.
    """

    def __init__(self, max_rows: int, device: int, group=None):
        import ctypes as C

        from . import _lib

        self._lib = _lib
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.ctx = _lib.get_context(device)
        h = C.c_void_p()
        _lib.check(_lib.load().dkv_exchange_create(self.ctx.handle, self.rank, self.world, int(max_rows), C.byref(h)))
        self.handle = h
        mine = C.create_string_buffer(64)
        _lib.check(_lib.load().dkv_exchange_handle(self.handle, mine))
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(mine.raw), group=group)
        for r, hb in enumerate(handles):
            if r != self.rank:
                _lib.check(_lib.load().dkv_exchange_connect(self.handle, r, hb))
        dist.barrier(group=group)

    def decode(self, layer_id, q, local_seq_lens, softmax_scale, page_table, x=None, row_map=None, pos_offset=None,
               lse_out=None) -> torch.Tensor:
        """This rank's part of the step; returns the merged output ``[B, NH_q, 128]`` (same on every rank)."""
        from . import kernel

        out = kernel.decode(layer_id, q, local_seq_lens, softmax_scale, page_table=page_table, row_map=row_map, x=x,
                            pos_offset=pos_offset, lse_out=lse_out, exchange=self.handle)
        return out.view(q.size(0), -1, 128)

    def close(self) -> None:
        if self.handle:
            torch.cuda.synchronize()
            dist.barrier(group=self.group)      # nobody unmaps while a peer may still be storing
            self._lib.load().dkv_exchange_destroy(self.handle)
            self.handle = None


class PeerWatch:
    """Host-side liveness of the ranks of a partitioned group, over a c10d key-value store (``dist.TCPStore``,
    ``dist.FileStore``, ...).

    The reference is single-GPU and has no failure detection.  Here a rank that leaves (crash, eviction) would
    otherwise be noticed by its peers only inside their next collective - or, with the fused exchange, as a
    two-second device-side wait that runs out.  With a watch every rank publishes the step it is about to start
    (``beat``) and checks, BEFORE it launches, that every peer has published that step too (``require``): a rank
    that is gone shows up on the host, within ``timeout_s``, while no kernel or collective of the step is in flight.
    """

    def __init__(self, store, rank: int, world: int, prefix: str = "directkv_b200/alive"):
        self.store, self.rank, self.world, self.prefix = store, int(rank), int(world), prefix

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def beat(self, step: int) -> None:
        self.store.set(self._key(self.rank), str(int(step)))

    def _step_of(self, rank: int) -> int:
        key = self._key(rank)
        if not self.store.check([key]):
            return -1
        return int(self.store.get(key).decode())

    def missing(self, step: int, timeout_s: float = 1.0, poll_s: float = 0.01) -> List[int]:
        """Ranks that have not announced ``step`` (or a later one) within ``timeout_s``."""
        import time

        deadline = time.monotonic() + timeout_s
        pending = [r for r in range(self.world) if r != self.rank]
        while pending:
            pending = [r for r in pending if self._step_of(r) < step]
            if not pending or time.monotonic() >= deadline:
                break
            time.sleep(poll_s)
        return pending

    def require(self, step: int, timeout_s: float = 1.0) -> None:
        gone = self.missing(step, timeout_s)
        if gone:
            raise RuntimeError(f"directkv_b200: rank(s) {gone} did not reach step {step} within {timeout_s:.1f} s; "
                               "nothing of this step was launched")


def sequence_split_decode(
    layer_id: int,
    q: torch.Tensor,                       # [B, NH_q, 128] bf16 CUDA, replicated on every rank
    local_seq_lens: torch.Tensor,          # [B] int32 CUDA: tokens of each request in THIS rank's range
    softmax_scale: float,
    page_table: Optional[torch.Tensor],    # this rank's pages of its own pool
    x: Optional[torch.Tensor] = None,      # [B, H] on the rank that owns the new token, else None
    row_map: Optional[torch.Tensor] = None,
    group=None,
    lse_out: Optional[torch.Tensor] = None,
    pos_offset: Optional[torch.Tensor] = None,   # [B] int32: first global token position of this rank's range
) -> torch.Tensor:
    """Decode attention of requests whose tokens are spread over the ranks of ``group``.

    ``local_seq_lens`` counts the new token on the rank that passes ``x``; that rank also passes
    ``pos_offset`` (where its range starts in the sequence) so the token is rotated at its absolute
    position.  Returns the normalised output ``[B, NH_q, 128]`` on every rank.
    """
    from . import kernel

    b = q.size(0)
    nh_q = q.numel() // (b * 128)
    part = torch.empty(b * nh_q, PARTIAL_STRIDE, dtype=torch.float32, device=q.device)
    kernel.decode(layer_id, q, local_seq_lens, softmax_scale, page_table=page_table, row_map=row_map, x=x,
                  partial_out=part, normalized=False, pos_offset=pos_offset)
    gathered = all_gather_partials(part, group)
    out = kernel.merge_partials(gathered, lse_out=lse_out)
    return out.view(b, nh_q, 128)
