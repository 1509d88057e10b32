"""CPU oracle for the DirectKV decode-attention hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain fp32 torch on the CPU, the arithmetic of the
reference's torch attention path and of its standalone kernel test oracle.  It is
imported only by tests, by the smoke check and by the CPU-baseline leg of the
benchmark; the product package never imports it and fails loudly when its CUDA
library is missing.

Parity status: pinned.  ``tests/golden/`` holds outputs of the reference's own
Python code (imported with stubbed third-party ``sglang`` base classes by
``tests/golden/make_golden.py``) and the oracle is checked against them in
``tests/test_oracle_golden.py``.  The reference keeps no stored golden files of
its own; its procedural known-answer cases (``tests/test_directkv_cpu_kv.cu:538-557``)
are re-generated from the same libc ``rand()`` streams in ``tests/``.

Every function cites the reference file:line it follows (paths relative to the
reference project's root).
"""

from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

TILE = 64          # directkv/directkv_backend.py:42, directkv_request_pool.py:22
HEAD_DIM = 128     # directkv/directkv_backend.py:163


# --------------------------------------------------------------------------
# Index arithmetic (bit-exact integer work)
# --------------------------------------------------------------------------
def pad64(n: int) -> int:
    """directkv/directkv_request_pool.py:25-26 and directkv_backend.py:45-46."""
    return math.ceil(n / TILE) * TILE


def decode_slot(s_past: int) -> int:
    """Row of the 64-row tile that holds the decode token: directkv_backend.py:602."""
    return s_past % TILE


def layer_index(layer_id: int, start_layer: int) -> int:
    """directkv/directkv_pool.py:165, directkv_request_pool.py:118."""
    return layer_id - start_layer


def token_slot(page_table_row: Sequence[int], t: int, page_size: int) -> int:
    """Slot of token ``t`` of one request under a paged table.

    With ``page_size == 1`` this is the reference's per-token lookup
    ``req_to_token[r, t]`` (directkv/directkv_backend.py:846-852); with larger
    pages the tokens of a page are consecutive slots.
    """
    return int(page_table_row[t // page_size]) * page_size + (t % page_size)


def request_slots(page_table_row: Sequence[int], n_tokens: int, page_size: int) -> torch.Tensor:
    t = torch.arange(n_tokens, dtype=torch.int64)
    pt = torch.as_tensor(page_table_row, dtype=torch.int64)
    return pt[t // page_size] * page_size + (t % page_size)


class RowFreeList:
    """Row assignment of directkv/directkv_request_pool.py:79-104 (LIFO free-list)."""

    def __init__(self, max_reqs: int):
        self.free: List[int] = list(range(max_reqs))
        self.req_to_row = {}

    def alloc(self, rid: int) -> None:
        if rid in self.req_to_row:
            return
        if not self.free:
            raise RuntimeError("out of rows")
        self.req_to_row[rid] = self.free.pop()

    def release(self, rid: int) -> None:
        row = self.req_to_row.pop(rid, None)
        if row is not None:
            self.free.append(row)


# --------------------------------------------------------------------------
# RoPE table and rotation
# --------------------------------------------------------------------------
def build_cos_sin(max_pos: int, head_dim: int = HEAD_DIM, theta: float = 500000.0) -> torch.Tensor:
    """[max_pos, head_dim] fp32, row p = [cos(p f_0..f_{D/2-1}) | sin(...)], f_i = theta^(-i/(D/2)).

    directkv/directkv_backend.py:299-304 (inv_freq branch) and
    benchmarks/bench_smpv2_perf.py:78-83.
    """
    half = head_dim // 2
    inv_freq = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float32) / half))
    t = torch.arange(max_pos, dtype=torch.float32)
    fq = torch.outer(t, inv_freq)
    return torch.cat([fq.cos(), fq.sin()], dim=-1)


def rope_neox(k_bf16: torch.Tensor, cos_sin: Optional[torch.Tensor], positions: torch.Tensor) -> torch.Tensor:
    """Neox rotation of ``k_bf16[..., T, NH, D]`` rows at absolute ``positions[T]``.

    csrc/directKV_kernel.cuh:504-518: read bf16, rotate in fp32
    (lo' = lo*cos - hi*sin, hi' = hi*cos + lo*sin), round to bf16.  ``cos_sin``
    None is the identity (OPT, csrc/directKV_kernel.cuh:165-171).
    """
    if cos_sin is None:
        return k_bf16
    d = k_bf16.shape[-1]
    half = d // 2
    cs = cos_sin[positions.long()].float()            # [T, D]
    cos = cs[:, :half].unsqueeze(1)                   # [T, 1, half]
    sin = cs[:, half:].unsqueeze(1)
    kf = k_bf16.float()
    lo, hi = kf[..., :half], kf[..., half:]
    out = torch.cat([lo * cos - hi * sin, hi * cos + lo * sin], dim=-1)
    return out.to(torch.bfloat16)


# --------------------------------------------------------------------------
# K/V projection of new tokens (over the FULL hidden dimension)
# --------------------------------------------------------------------------
def project_kv(x_bf16: torch.Tensor, wk_bf16: torch.Tensor, wv_bf16: torch.Tensor
               ) -> Tuple[torch.Tensor, torch.Tensor]:
    """K[t,h,d] = sum_hh X[t,hh] * Wk[h,d,hh] (fp32 accumulate) then bf16.

    tests/test_directkv_cpu_kv.cu:372-385 (projection oracle) and the bf16
    rounding point of csrc/directKV_kernel.cuh:496-499.  x: [T, H]; w: [NH, D, H].
    """
    x = x_bf16.float()
    nh, d, h = wk_bf16.shape
    k = x @ wk_bf16.float().reshape(nh * d, h).t()
    v = x @ wv_bf16.float().reshape(nh * d, h).t()
    return (k.reshape(-1, nh, d).to(torch.bfloat16), v.reshape(-1, nh, d).to(torch.bfloat16))


# --------------------------------------------------------------------------
# Attention (the parity target is the reference's torch SDPA path)
# --------------------------------------------------------------------------
def sdpa_decode(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
    """One decode token against ``k, v [S, NH_kv, D]``; q ``[NH_q, D]`` -> ``[NH_q, D]`` fp32.

    directkv/directkv_backend.py:813-825: permute to [1, NH, S, D], repeat_interleave
    KV heads to Q heads, scaled_dot_product_attention(is_causal=False, scale=scale).
    """
    nh_q, d = q.shape
    nh_kv = k.shape[1]
    k4 = k.float().permute(1, 0, 2).unsqueeze(0)
    v4 = v.float().permute(1, 0, 2).unsqueeze(0)
    if nh_q != nh_kv:
        k4 = k4.repeat_interleave(nh_q // nh_kv, dim=1)
        v4 = v4.repeat_interleave(nh_q // nh_kv, dim=1)
    q4 = q.float().view(1, 1, nh_q, d).permute(0, 2, 1, 3)
    o = F.scaled_dot_product_attention(q4, k4, v4, is_causal=False, scale=scale)
    return o.squeeze(0).squeeze(1)


def sdpa_extend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, sl_pre: int, scale: float,
                is_causal: bool = True) -> torch.Tensor:
    """``q [S_new, NH_q, D]`` against ``k, v [sl_pre + S_new, NH_kv, D]`` -> ``[S_new, NH_q, D]`` fp32.

    directkv/directkv_backend.py:876-889 and :910-924: additive mask
    triu(-inf, diagonal=sl_pre+1), i.e. query row i sees columns j <= sl_pre + i.
    """
    s_new, nh_q, d = q.shape
    s_tot, nh_kv, _ = k.shape
    k4 = k.float().permute(1, 0, 2).unsqueeze(0)
    v4 = v.float().permute(1, 0, 2).unsqueeze(0)
    if nh_q != nh_kv:
        g = nh_q // nh_kv
        k4 = k4.repeat_interleave(g, dim=1)
        v4 = v4.repeat_interleave(g, dim=1)
    q4 = q.float().permute(1, 0, 2).unsqueeze(0)
    mask = None
    if is_causal:
        mask = torch.triu(torch.full((s_new, s_tot), float("-inf")), diagonal=sl_pre + 1)
        mask = mask.unsqueeze(0).unsqueeze(0)
    o = F.scaled_dot_product_attention(q4, k4, v4, attn_mask=mask, scale=scale)
    return o.squeeze(0).permute(1, 0, 2)


def ref_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                  is_causal: bool, s_past: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Explicit max-subtracted softmax of tests/test_directkv_cpu_kv.cu:148-179.

    q [S_q, D], k/v [S_kv, D] fp32 for one (batch, head).  Returns (O, LSE) where
    LSE = max*1 + ln(sum) of the scaled scores (csrc/softmax.h:151).
    """
    scores = (q.float() @ k.float().t()) * scale
    if is_causal:
        i = torch.arange(q.shape[0]).unsqueeze(1)
        j = torch.arange(k.shape[0]).unsqueeze(0)
        scores = torch.where(j > s_past + i, torch.full_like(scores, -1e30), scores)
    mx = scores.max(dim=1, keepdim=True).values
    e = torch.exp(scores - mx)
    sm = e.sum(dim=1, keepdim=True)
    o = (e / sm) @ v.float()
    return o, (mx + torch.log(sm)).squeeze(1)


def lse_merge(o_parts: torch.Tensor, lse_parts: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Merge normalised partial outputs ``o_parts [N, ..., D]`` with ``lse_parts [N, ...]``.

    csrc/directKV_kernel.cuh:749-787 (running form) and kernel/kernel.cuh:640-736
    (combine form): w_n = exp(LSE_n - max), O = sum w_n O_n / sum w_n,
    LSE = max + ln(sum w_n); parts whose LSE is -inf contribute nothing.
    """
    mx = lse_parts.max(dim=0).values
    safe = torch.where(torch.isinf(mx), torch.zeros_like(mx), mx)
    w = torch.exp(lse_parts - safe)
    w = torch.where(torch.isinf(lse_parts), torch.zeros_like(w), w)
    z = w.sum(dim=0)
    o = (w.unsqueeze(-1) * o_parts).sum(dim=0) / z.clamp_min(1e-38).unsqueeze(-1)
    return o, safe + torch.log(z)


# --------------------------------------------------------------------------
# Whole-layer decode over a paged / slot-indexed host pool
# --------------------------------------------------------------------------
def decode_layer(
    x: Optional[torch.Tensor],            # [B, H] bf16 or None (k_new/v_new given instead)
    wk: Optional[torch.Tensor],           # [NH_kv, D, H] bf16
    wv: Optional[torch.Tensor],
    q: torch.Tensor,                      # [B, NH_q, D] bf16 (already rotated)
    k_pool: torch.Tensor,                 # [n_slots, NH_kv, D] bf16, modified in place
    v_pool: torch.Tensor,
    page_table: torch.Tensor,             # [B, max_pages] int
    seq_lens: Sequence[int],              # lengths INCLUDING the token decoded now
    page_size: int,
    cos_sin: Optional[torch.Tensor],
    scale: float,
    k_new: Optional[torch.Tensor] = None,  # [B, NH_kv, D] bf16 (used when x is None)
    v_new: Optional[torch.Tensor] = None,
    save_kv_cache: bool = True,
    return_lse: bool = False,
):
    """One decode step of one layer for a ragged batch.

    Follows directkv/directkv_backend.py:781-825 per request: the token's K/V
    (projected from X over the full hidden size and rotated at position S_past,
    or given) is written to the pool at position S_past, then SDPA runs over
    positions [0, S_past].  Slots come from the page table
    (directkv/directkv_backend.py:846-852).  Output [B, NH_q, D] fp32.
    """
    b = q.shape[0]
    nh_q, d = q.shape[1], q.shape[2]
    if x is not None:
        k_new, v_new = project_kv(x, wk, wv)                      # [B, NH_kv, D] bf16
        pos = torch.tensor([int(s) - 1 for s in seq_lens])
        if cos_sin is not None:
            k_new = torch.stack([rope_neox(k_new[i:i + 1], cos_sin, pos[i:i + 1])[0] for i in range(b)])
    outs, lses = [], []
    for i in range(b):
        sl = int(seq_lens[i])
        slots = request_slots(page_table[i].tolist(), sl, page_size)
        if k_new is not None:
            if save_kv_cache:
                k_pool[slots[sl - 1]] = k_new[i]
                v_pool[slots[sl - 1]] = v_new[i]
            k_i = torch.cat([k_pool[slots[: sl - 1]], k_new[i:i + 1]], dim=0)
            v_i = torch.cat([v_pool[slots[: sl - 1]], v_new[i:i + 1]], dim=0)
        else:
            k_i, v_i = k_pool[slots], v_pool[slots]
        outs.append(sdpa_decode(q[i], k_i, v_i, scale))
        if return_lse:
            g = nh_q // k_i.shape[1]
            kk = k_i.float().repeat_interleave(g, dim=1)          # [S, NH_q, D]
            sc = torch.einsum("hd,shd->hs", q[i].float(), kk) * scale
            lses.append(torch.logsumexp(sc, dim=1))
    o = torch.stack(outs, dim=0)
    if return_lse:
        return o, torch.stack(lses, dim=0)
    return o


def smpv2_fwd(
    x: torch.Tensor,        # [B, S_new, H] bf16
    wk: torch.Tensor,       # [NH_kv, D, H]
    wv: torch.Tensor,
    q: torch.Tensor,        # [B, S_new, NH_q, D]
    k_cpu: torch.Tensor,    # [B, S_total, NH_kv, D] bf16, new rows written in place
    v_cpu: torch.Tensor,
    cos_sin: Optional[torch.Tensor],
    softmax_scale: float,
    is_causal: bool,
    seqlen_past: int,
    q_pos_start: int = -1,
) -> torch.Tensor:
    """Oracle with the argument meaning of the reference's extension entry point.

    directkv/kernel/smpv2_extension.cu:574-637 (checks) and csrc/directKV_kernel.cuh
    :430-546 (project, rotate K at absolute positions, write back), :557-733
    (attention of the new rows over past + new rows, causal offset seqlen_past).
    ``q_pos_start >= 0`` rotates Q too (csrc/directKV_kernel.cuh:619-638).
    Returns O [B, S_new, NH_q, D] fp32.
    """
    bsz, s_new, _ = x.shape
    outs = []
    for b in range(bsz):
        k_new, v_new = project_kv(x[b], wk, wv)
        pos = torch.arange(seqlen_past, seqlen_past + s_new)
        k_new = rope_neox(k_new, cos_sin, pos)
        k_cpu[b, seqlen_past:seqlen_past + s_new] = k_new
        v_cpu[b, seqlen_past:seqlen_past + s_new] = v_new
        qb = q[b]
        if cos_sin is not None and q_pos_start >= 0:
            qb = rope_neox(qb, cos_sin, torch.arange(q_pos_start, q_pos_start + s_new))
        outs.append(sdpa_extend(qb, k_cpu[b], v_cpu[b], seqlen_past, softmax_scale, is_causal))
    return torch.stack(outs, dim=0)


# --------------------------------------------------------------------------
# Weight slicing (directkv/directkv_backend.py:243-271)
# --------------------------------------------------------------------------
def slice_qkv_weight(w_qkv: torch.Tensor, nh_q: int, nh_kv: int, d: int, h: int):
    q_s, k_s = nh_q * d, nh_kv * d
    wk = w_qkv[q_s:q_s + k_s].contiguous().view(nh_kv, d, h)
    wv = w_qkv[q_s + k_s:q_s + 2 * k_s].contiguous().view(nh_kv, d, h)
    return wk, wv
