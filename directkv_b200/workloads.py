"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

These stand in for the serving traffic and model weights the reference measures with (neither
ships with it): layer shapes of Llama-3-8B, OPT-6.7B and OPT-30B, per-token hidden states
~N(0,1), W_k / W_v ~ N(0, 0.02), queries ~N(0,1), and a KV cache filled with N(0, (0.02^2 * H))
values - the distribution X.W^T has for those inputs - instead of being produced by a prefill
pass.  Everything is generated from fixed seeds so tests, the smoke check and the benchmark see
the same tensors.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

HEAD_DIM = 128


@dataclass(frozen=True)
class LayerShape:
    name: str
    hidden: int
    nh_q: int
    nh_kv: int
    rope_theta: Optional[float]   # None: no rotary embedding (OPT)

    @property
    def scale(self) -> float:
        return HEAD_DIM ** -0.5

    def kv_bytes_per_token(self, tp: int = 1) -> int:
        """K and V bytes one token occupies in one layer on one tensor-parallel rank."""
        return 2 * (self.nh_kv // tp) * HEAD_DIM * 2

    def shard(self, tp: int) -> "LayerShape":
        return LayerShape(f"{self.name}/tp{tp}", self.hidden, self.nh_q // tp, self.nh_kv // tp, self.rope_theta)


LLAMA3_8B = LayerShape("llama3-8b", 4096, 32, 8, 500000.0)
OPT_6_7B = LayerShape("opt-6.7b", 4096, 32, 32, None)
OPT_30B = LayerShape("opt-30b", 7168, 56, 56, None)


def build_cos_sin(max_pos: int, theta: float, device="cpu") -> torch.Tensor:
    """``[max_pos, 128]`` fp32 table ``[cos(p f_i) | sin(p f_i)]``, ``f_i = theta^(-i/64)``.

    The layout the reference derives from ``inv_freq`` (directkv/directkv_backend.py:299-304).
    """
    half = HEAD_DIM // 2
    inv_freq = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float32, device=device) / half))
    t = torch.arange(max_pos, dtype=torch.float32, device=device)
    fq = torch.outer(t, inv_freq)
    return torch.cat([fq.cos(), fq.sin()], dim=-1).contiguous()


def ragged_lengths_uniform(n: int, lo: int, hi: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi + 1, (n,), generator=g).tolist()


def ragged_lengths_lognormal(n: int, median: int, sigma: float, lo: int, hi: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    x = torch.exp(torch.randn(n, generator=g) * sigma + math.log(median))
    return x.clamp(lo, hi).round().long().tolist()


def permuted_page_table(seq_lens: Sequence[int], page_size: int, seed: int, slack_pages: int = 0):
    """Page table of a randomly permuted pool: request b gets the next ceil(len/page) entries of
    ``randperm(num_pages) + 1`` (page 0 is the reserved padding page).  Returns (table int32
    [B, max_pages], num_pages)."""
    pages = [(-(-int(s) // page_size)) for s in seq_lens]
    total = sum(pages) + slack_pages
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(total, generator=g) + 1
    table = torch.zeros(len(seq_lens), max(pages) if pages else 1, dtype=torch.int32)
    off = 0
    for b, n in enumerate(pages):
        table[b, :n] = perm[off:off + n].to(torch.int32)
        off += n
    return table, total


def _randn_bf16(shape, std: float, seed: int, device) -> torch.Tensor:
    g = torch.Generator(device=device).manual_seed(seed)
    return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std).to(torch.bfloat16)


def fill_pool_(pool: torch.Tensor, std: float, seed: int, device, chunk_rows: int = 1 << 16) -> None:
    """Fills a (host-pinned or device) pool [n_slots, NH, 128] with N(0, std^2) values, generated on
    ``device`` in chunks so that multi-GB host pools do not need host-side RNG."""
    n = pool.shape[0]
    for i, r0 in enumerate(range(0, n, chunk_rows)):
        r1 = min(n, r0 + chunk_rows)
        blk = _randn_bf16((r1 - r0,) + tuple(pool.shape[1:]), std, seed + 7919 * i, device)
        pool[r0:r1].copy_(blk)


def make_decode_case(
    shape: LayerShape,
    seq_lens: Sequence[int],           # lengths INCLUDING the token decoded in this step
    page_size: int,
    cfg_id: int,
    device,
    kv_on_host: bool = True,
    gen_device=None,
) -> Dict[str, torch.Tensor]:
    """One layer's decode inputs for a ragged batch over a paged pool.

    Seeds follow one scheme everywhere: X 1234+cfg, W 2234+cfg, Q 3234+cfg, page permutation
    5234+cfg, pool fill 6234+cfg.  Tensors that the engine reads on the device are created on
    ``device``; the pool is page-locked host memory when ``kv_on_host`` else device memory.
    """
    gen_device = gen_device or device
    b = len(seq_lens)
    x = _randn_bf16((b, shape.hidden), 1.0, 1234 + cfg_id, gen_device).to(device)
    wk = _randn_bf16((shape.nh_kv, HEAD_DIM, shape.hidden), 0.02, 2234 + cfg_id, gen_device).to(device)
    wv = _randn_bf16((shape.nh_kv, HEAD_DIM, shape.hidden), 0.02, 2235 + cfg_id + 1000, gen_device).to(device)
    q = _randn_bf16((b, shape.nh_q, HEAD_DIM), 1.0, 3234 + cfg_id, gen_device).to(device)
    table, num_pages = permuted_page_table(seq_lens, page_size, 5234 + cfg_id)
    n_slots = (num_pages + 1) * page_size
    pool_shape = (n_slots, shape.nh_kv, HEAD_DIM)
    if kv_on_host:
        pin = torch.device(device).type == "cuda"
        k_pool = torch.empty(pool_shape, dtype=torch.bfloat16, pin_memory=pin)
        v_pool = torch.empty(pool_shape, dtype=torch.bfloat16, pin_memory=pin)
    else:
        k_pool = torch.empty(pool_shape, dtype=torch.bfloat16, device=device)
        v_pool = torch.empty(pool_shape, dtype=torch.bfloat16, device=device)
    std = 0.02 * math.sqrt(shape.hidden)
    fill_pool_(k_pool, std, 6234 + cfg_id, gen_device)
    fill_pool_(v_pool, std, 7234 + cfg_id, gen_device)
    cos_sin = None
    if shape.rope_theta is not None:
        cos_sin = build_cos_sin(max(int(max(seq_lens)), 1) + 1, shape.rope_theta, device=device)
    return dict(
        x=x, wk=wk, wv=wv, q=q, k_pool=k_pool, v_pool=v_pool,
        page_table=table.to(device), seq_lens=torch.tensor(list(seq_lens), dtype=torch.int32, device=device),
        cos_sin=cos_sin, page_size=page_size, n_slots=n_slots,
    )


def kv_bytes(shape: LayerShape, seq_lens: Sequence[int], tp: int = 1) -> int:
    """Algorithmic KV bytes one decode step of one layer must read: exact token counts."""
    return shape.kv_bytes_per_token(tp) * int(sum(int(s) for s in seq_lens))
