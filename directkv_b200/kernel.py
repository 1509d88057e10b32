"""Python face of the engine: same entry points as the reference's ``directkv/kernel/__init__.py``
(``smpv2_fwd`` :225-257, ``smpv2_init_tma`` :260-279, ``smpv2_fwd_graph`` :282-314 and the
``directkv_*`` aliases the non-smpv2 backend asks for, directkv/directkv_backend.py:83-93), plus
the ragged, page-tabled decode call the B200 engine is built around.

Everything here only checks tensors, turns them into pointers and calls the C ABI; there is no
torch compute and no fallback.
"""

from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from . import _lib
from ._lib import DKV_NEW_GIVEN, DKV_NEW_NONE, DKV_NEW_PROJECT, PARTIAL_STRIDE, DecodeArgs, LayerDesc, get_context

HEAD_DIM = 128


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _chk(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _check_cuda_bf16(t: torch.Tensor, name: str) -> None:
    _chk(t.is_cuda, f"{name} must be a CUDA tensor")
    _chk(t.is_contiguous(), f"{name} must be contiguous")
    _chk(t.dtype == torch.bfloat16, f"{name} must be bfloat16")


def _check_kv(t: torch.Tensor, name: str) -> None:
    """KV storage: pinned host memory (the reference's only mode) or device memory (HBM-resident mode)."""
    _chk(t.is_contiguous(), f"{name} must be contiguous")
    _chk(t.dtype == torch.bfloat16, f"{name} must be bfloat16")
    if not t.is_cuda:
        _chk(t.is_pinned(), f"{name} must be a CPU tensor in pinned memory (or a CUDA tensor)")


def _check_cos_sin(cos_sin: Optional[torch.Tensor]) -> None:
    if cos_sin is None:
        return
    _chk(cos_sin.is_cuda, "cos_sin must be a CUDA tensor")
    _chk(cos_sin.dtype == torch.float32, "cos_sin must be float32")
    _chk(cos_sin.dim() == 2, "cos_sin must be 2D [max_pos, head_dim]")
    _chk(cos_sin.size(1) == HEAD_DIM, f"cos_sin.size(1) must equal head_dim={HEAD_DIM}, got {cos_sin.size(1)}")
    _chk(cos_sin.is_contiguous(), "cos_sin must be contiguous")


# ---------------------------------------------------------------------------
# Layer registration and the ragged decode call
# ---------------------------------------------------------------------------
def register_layer(
    layer_id: int,
    k_pool: torch.Tensor,            # [n_slots, NH_kv, 128] bf16 pinned-CPU or CUDA (any leading dims that flatten to slots)
    v_pool: torch.Tensor,
    wk: Optional[torch.Tensor] = None,   # [NH_kv, 128, H] bf16 CUDA
    wv: Optional[torch.Tensor] = None,
    cos_sin: Optional[torch.Tensor] = None,  # [max_pos, 128] fp32 CUDA
    page_size: int = 1,
    row_stride: int = 0,
    device: Optional[int] = None,
) -> None:
    """Builds and caches the TMA descriptors of one layer's KV pool and projection weights.

    Takes the place of ``smpv2_init_tma`` (directkv/kernel/smpv2_extension.cu:363-423).  The
    pool is used IN PLACE: nothing is copied, so what the engine stores for new tokens is
    visible to every later reader of the pool tensor.
    """
    _check_kv(k_pool, "k_pool")
    _check_kv(v_pool, "v_pool")
    _chk(k_pool.shape == v_pool.shape, "k_pool and v_pool must have the same shape")
    _chk(k_pool.dim() >= 3 and k_pool.size(-1) == HEAD_DIM, f"pool must be [..., NH_kv, {HEAD_DIM}]")
    nh_kv = k_pool.size(-2)
    n_slots = k_pool.numel() // (nh_kv * HEAD_DIM)
    hidden = 0
    if wk is not None:
        _check_cuda_bf16(wk, "Wk")
        _check_cuda_bf16(wv, "Wv")
        _chk(wk.dim() == 3 and wk.shape == wv.shape, "Wk/Wv must be 3D [NH, D, H] and equal in shape")
        _chk(wk.size(0) == nh_kv and wk.size(1) == HEAD_DIM, "Wk must be [NH_kv, 128, H] for this pool")
        hidden = wk.size(2)
    _check_cos_sin(cos_sin)
    ctx = get_context(device)
    d = LayerDesc(
        k_pool=_ptr(k_pool), v_pool=_ptr(v_pool), n_slots=n_slots, nh_kv=nh_kv, page_size=page_size,
        row_stride=row_stride, wk=_ptr(wk), wv=_ptr(wv), hidden=hidden, cos_sin=_ptr(cos_sin),
        max_pos=0 if cos_sin is None else cos_sin.size(0),
    )
    _lib.check(_lib.load().dkv_layer_register(ctx.handle, int(layer_id), C.byref(d)))
    ctx._keepalive[int(layer_id)] = (k_pool, v_pool, wk, wv, cos_sin)


def unregister_layer(layer_id: int, device: Optional[int] = None) -> None:
    ctx = get_context(device)
    _lib.check(_lib.load().dkv_layer_unregister(ctx.handle, int(layer_id)))
    ctx._keepalive.pop(int(layer_id), None)


def decode(
    layer_id: int,
    q: torch.Tensor,                      # [B, NH_q*128] or [B, NH_q, 128] bf16 CUDA
    seq_lens: torch.Tensor,               # [B] int32 CUDA, lengths INCLUDING the token decoded now
    softmax_scale: float,
    page_table: Optional[torch.Tensor] = None,   # [rows, max_pages] int32 CUDA; None = contiguous rows
    row_map: Optional[torch.Tensor] = None,      # [B] int32 CUDA
    x: Optional[torch.Tensor] = None,            # [B, H] bf16 CUDA -> project the new token's K/V
    k_new: Optional[torch.Tensor] = None,        # [B, NH_kv, 128] bf16 CUDA (already rotated)
    v_new: Optional[torch.Tensor] = None,
    save_kv_cache: bool = True,
    out: Optional[torch.Tensor] = None,
    lse_out: Optional[torch.Tensor] = None,
    partial_out: Optional[torch.Tensor] = None,  # [B, NH_q, 132] fp32: unnormalised (O, m, l)
    normalized: bool = True,
    pos_offset: Optional[torch.Tensor] = None,   # [B] int32 CUDA: added to seq_len-1 for the RoPE position
    exchange=None,                               # handle of a connected peer-memory exchange (sharding.PartialExchange)
    kv_source_layer: int = 0,                    # attend a copy of the past rows registered as this layer (0: off)
    src_page_table: Optional[torch.Tensor] = None,   # addressing of the copy (its page size) ...
    src_row_map: Optional[torch.Tensor] = None,      # ... or its rows
) -> Optional[torch.Tensor]:
    """One decode step of one registered layer for a ragged batch.  Returns O with q's shape.

    With ``exchange`` the call is this rank's part of a sequence-split decode: partial records go to
    every rank's exchange buffer over NVLink and ``out`` is the merged result of all ranks.
    """
    _check_cuda_bf16(q, "q")
    b = q.size(0)
    nh_q = q.numel() // (b * HEAD_DIM) if b else 0
    _chk(seq_lens.is_cuda and seq_lens.dtype == torch.int32 and seq_lens.is_contiguous(), "seq_lens must be int32 CUDA")
    _chk(seq_lens.numel() == b, "seq_lens must have one entry per request")
    if page_table is not None:
        _chk(page_table.is_cuda and page_table.dtype == torch.int32 and page_table.dim() == 2
             and page_table.stride(1) == 1, "page_table must be 2D int32 CUDA with unit inner stride")
    if row_map is not None:
        _chk(row_map.is_cuda and row_map.dtype == torch.int32 and row_map.numel() == b, "row_map must be [B] int32 CUDA")
    mode = DKV_NEW_NONE
    if x is not None:
        _check_cuda_bf16(x, "x")
        _chk(x.dim() == 2 and x.size(0) == b, "x must be [B, H]")
        mode = DKV_NEW_PROJECT
    elif k_new is not None:
        _check_cuda_bf16(k_new, "k_new")
        _check_cuda_bf16(v_new, "v_new")
        mode = DKV_NEW_GIVEN
    if normalized and out is None:
        out = torch.empty_like(q)
    if out is not None:
        _check_cuda_bf16(out, "out")
    if lse_out is not None:
        _chk(lse_out.is_cuda and lse_out.dtype == torch.float32 and lse_out.numel() == b * nh_q, "lse_out must be [B, NH_q] fp32 CUDA")
    if partial_out is not None:
        _chk(partial_out.is_cuda and partial_out.dtype == torch.float32 and partial_out.is_contiguous()
             and partial_out.numel() == b * nh_q * PARTIAL_STRIDE, "partial_out must be [B, NH_q, 132] fp32 CUDA")
    if pos_offset is not None:
        _chk(pos_offset.is_cuda and pos_offset.dtype == torch.int32 and pos_offset.numel() == b, "pos_offset must be [B] int32 CUDA")
    if src_page_table is not None:
        _chk(kv_source_layer != 0 and src_page_table.is_cuda and src_page_table.dtype == torch.int32
             and src_page_table.dim() == 2 and src_page_table.stride(1) == 1,
             "src_page_table needs kv_source_layer and must be 2D int32 CUDA with unit inner stride")
    if src_row_map is not None:
        _chk(kv_source_layer != 0 and src_row_map.is_cuda and src_row_map.dtype == torch.int32 and src_row_map.numel() == b,
             "src_row_map needs kv_source_layer and must be [B] int32 CUDA")
    if b == 0:
        return out
    a = DecodeArgs(
        layer_id=int(layer_id), batch=b, nh_q=nh_q, q=_ptr(q), q_stride=nh_q * HEAD_DIM,
        out=_ptr(out), out_stride=nh_q * HEAD_DIM, seq_lens=_ptr(seq_lens),
        page_table=_ptr(page_table), pt_stride=0 if page_table is None else page_table.stride(0),
        row_map=_ptr(row_map), new_mode=mode, x=_ptr(x), k_new=_ptr(k_new), v_new=_ptr(v_new),
        save_kv_cache=1 if save_kv_cache else 0, softmax_scale=float(softmax_scale),
        lse_out=_ptr(lse_out), partial_out=_ptr(partial_out), pos_offset=_ptr(pos_offset),
        kv_source_layer=int(kv_source_layer), src_page_table=_ptr(src_page_table),
        src_pt_stride=0 if src_page_table is None else src_page_table.stride(0), src_row_map=_ptr(src_row_map),
        pt_rows=0 if page_table is None else page_table.size(0),
    )
    ctx = get_context(q.device.index)
    if exchange is not None:
        _lib.check(_lib.load().dkv_decode_exchange(ctx.handle, exchange, C.byref(a), _ptr(out), _ptr(lse_out), _stream()))
    else:
        _lib.check(_lib.load().dkv_decode(ctx.handle, C.byref(a), _stream()))
    return out


def extend(
    layer_id: int,
    X: torch.Tensor,                  # [B, S_new, H] bf16 CUDA
    Q: torch.Tensor,                  # [B, S_new, NH_q, 128] bf16 CUDA
    softmax_scale: float,
    is_causal: bool,
    seqlen_past: int,
    q_pos_start: int = -1,
    row_map: Optional[torch.Tensor] = None,   # [B] int32 CUDA: pool row of each request
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Extend / chunked prefill on the rows of a registered layer (no descriptor rebuild).

    The kernel call of ``forward_extend`` (directkv/directkv_backend.py:681-697): the new rows'
    K/V are projected, rotated and stored at ``[row, seqlen_past + i]`` of the pool in place.
    """
    _check_cuda_bf16(X, "X")
    _check_cuda_bf16(Q, "Q")
    _chk(X.dim() == 3 and Q.dim() == 4 and Q.size(3) == HEAD_DIM, "X must be [B,S_new,H] and Q [B,S_new,NH_q,128]")
    B, S_new, _ = X.shape
    _chk(Q.size(0) == B and Q.size(1) == S_new, "Q must match X in batch and S_new")
    if row_map is not None:
        _chk(row_map.is_cuda and row_map.dtype == torch.int32 and row_map.numel() == B, "row_map must be [B] int32 CUDA")
    if out is None:
        out = torch.empty_like(Q)
    _check_cuda_bf16(out, "out")
    ctx = get_context(X.device.index)
    _lib.check(_lib.load().dkv_extend(
        ctx.handle, int(layer_id), _ptr(X), _ptr(Q), _ptr(out), B, S_new, Q.size(2), float(softmax_scale),
        1 if is_causal else 0, int(seqlen_past), int(q_pos_start), _ptr(row_map), _stream()))
    return out


def extend_attend(
    layer_id: int,
    Q: torch.Tensor,                  # [B, S_new, NH_q, 128] bf16 CUDA
    softmax_scale: float,
    is_causal: bool,
    seqlen_past: int,
    row_map: Optional[torch.Tensor] = None,      # [B] int32 CUDA: pool row / page-table row of each request
    page_table: Optional[torch.Tensor] = None,   # [rows, max_pages] int32 CUDA (page size of the registered layer)
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Attention of new rows that are already stored in the pool (``dkv_extend_attend``): the engine's form of
    ``_sdpa_extend_manual`` (directkv/directkv_backend.py:861-891) on the tensor-core extend kernel."""
    _check_cuda_bf16(Q, "Q")
    _chk(Q.dim() == 4 and Q.size(3) == HEAD_DIM, "Q must be [B,S_new,NH_q,128]")
    B, S_new = Q.size(0), Q.size(1)
    if row_map is not None:
        _chk(row_map.is_cuda and row_map.dtype == torch.int32 and row_map.numel() == B, "row_map must be [B] int32 CUDA")
    pt_stride = 0
    if page_table is not None:
        _chk(page_table.is_cuda and page_table.dtype == torch.int32 and page_table.dim() == 2 and page_table.stride(1) == 1,
             "page_table must be a 2-D int32 CUDA tensor with unit inner stride")
        pt_stride = page_table.stride(0)
    if out is None:
        out = torch.empty_like(Q)
    _check_cuda_bf16(out, "out")
    ctx = get_context(Q.device.index)
    _lib.check(_lib.load().dkv_extend_attend(
        ctx.handle, int(layer_id), _ptr(Q), _ptr(out), B, S_new, Q.size(2), float(softmax_scale),
        1 if is_causal else 0, int(seqlen_past), _ptr(row_map), _ptr(page_table), int(pt_stride), _stream()))
    return out


def extend_ragged(
    layer_id: int,
    X: Optional[torch.Tensor],        # [T, H] bf16 CUDA, or None when the new rows are stored already
    Q: torch.Tensor,                  # [T, NH_q, 128] bf16 CUDA: the requests' rows one after the other
    s_new: Sequence[int],             # new rows per request (host)
    past: Sequence[int],              # stored rows per request (host)
    rows: Sequence[int],              # pool row / page-table row per request (host)
    softmax_scale: float,
    is_causal: bool = True,
    page_table: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Extend of a ragged batch in one launch sequence (``dkv_extend_ragged``); the reference calls its kernel
    once per request (directkv/directkv_backend.py:681-697)."""
    import ctypes as C

    _check_cuda_bf16(Q, "Q")
    _chk(Q.dim() == 3 and Q.size(2) == HEAD_DIM, "Q must be [T,NH_q,128]")
    B = len(s_new)
    _chk(len(past) == B and len(rows) == B and B > 0, "s_new, past and rows must have one entry per request")
    _chk(int(sum(int(n) for n in s_new)) == Q.size(0), "sum(s_new) must equal the rows of Q")
    if X is not None:
        _check_cuda_bf16(X, "X")
        _chk(X.dim() == 2 and X.size(0) == Q.size(0), "X must be [T,H]")
    pt_stride = 0
    if page_table is not None:
        _chk(page_table.is_cuda and page_table.dtype == torch.int32 and page_table.dim() == 2 and page_table.stride(1) == 1,
             "page_table must be a 2-D int32 CUDA tensor with unit inner stride")
        pt_stride = page_table.stride(0)
    if out is None:
        out = torch.empty_like(Q)
    _check_cuda_bf16(out, "out")
    arr = C.c_int32 * B
    a_new, a_past, a_rows = arr(*[int(v) for v in s_new]), arr(*[int(v) for v in past]), arr(*[int(v) for v in rows])
    ctx = get_context(Q.device.index)
    _lib.check(_lib.load().dkv_extend_ragged(
        ctx.handle, int(layer_id), _ptr(X), _ptr(Q), _ptr(out), B, C.cast(a_new, C.c_void_p), C.cast(a_past, C.c_void_p),
        C.cast(a_rows, C.c_void_p), Q.size(1), float(softmax_scale), 1 if is_causal else 0, _ptr(page_table),
        int(pt_stride), _stream()))
    return out


def decode_noalloc(
    k_pool: torch.Tensor,        # [n_slots, NH_kv, 128] bf16, pinned CPU or CUDA
    v_pool: torch.Tensor,
    q: torch.Tensor,             # [B, NH_q, 128] or [B, NH_q*128] bf16 CUDA
    out: torch.Tensor,           # same shape as q, pre-allocated by the caller
    seq_lens: torch.Tensor,      # [B] int32 CUDA; every attended token is already in the pool
    page_table: torch.Tensor,    # [B, max_pages] int32 CUDA
    page_size: int,
    softmax_scale: float,
    lse_out: Optional[torch.Tensor] = None,
    sync_and_check: bool = False,
    status_out: Optional[torch.Tensor] = None,   # [1] int32 CUDA of the caller's: failure bits are OR-ed into it
) -> torch.Tensor:
    """Attention-only decode that allocates no device memory (``dkv_decode_noalloc``).

    For callers that cannot allocate when they call in: graph-capture regions, serving loops with
    a frozen memory plan, hosts that forbid ``cudaMalloc`` from plugins.  The caller passes every
    tensor, output included; scratch is a fixed 4 MiB array inside the library, shared by all
    calls, so calls that overlap on the GPU race and sizes beyond the array are rejected with
    ``RuntimeError``.  The first call on a device does a one-time set-up and should happen
    before any stream capture.  Needs no registered layer and no context.
    """
    _check_kv(k_pool, "k_pool")
    _check_kv(v_pool, "v_pool")
    _check_cuda_bf16(q, "q")
    _check_cuda_bf16(out, "out")
    _chk(out.shape == q.shape, "out must have q's shape")
    _chk(k_pool.dim() >= 3 and k_pool.size(-1) == HEAD_DIM and k_pool.shape == v_pool.shape, "pools must be [..., NH_kv, 128]")
    b = q.size(0)
    nh_q = q.numel() // (b * HEAD_DIM)
    nh_kv = k_pool.size(-2)
    _chk(seq_lens.is_cuda and seq_lens.dtype == torch.int32 and seq_lens.numel() == b, "seq_lens must be [B] int32 CUDA")
    _chk(page_table.is_cuda and page_table.dtype == torch.int32 and page_table.dim() == 2 and page_table.stride(1) == 1,
         "page_table must be 2D int32 CUDA with unit inner stride")
    if status_out is not None:
        _chk(status_out.is_cuda and status_out.dtype == torch.int32 and status_out.numel() >= 1,
             "status_out must be an int32 CUDA tensor")
    err = C.create_string_buffer(512)
    a = _lib.NoAllocArgs(
        k_pool=_ptr(k_pool), v_pool=_ptr(v_pool), n_slots=k_pool.numel() // (nh_kv * HEAD_DIM), nh_kv=nh_kv,
        page_size=int(page_size), batch=b, nh_q=nh_q, q=_ptr(q), q_stride=nh_q * HEAD_DIM, out=_ptr(out),
        out_stride=nh_q * HEAD_DIM, seq_lens=_ptr(seq_lens), page_table=_ptr(page_table),
        pt_stride=page_table.stride(0), softmax_scale=float(softmax_scale), lse_out=_ptr(lse_out),
        sync_and_check=1 if sync_and_check else 0, err_buf=C.cast(err, C.c_char_p), err_buf_len=512,
        status_out=_ptr(status_out),
    )
    with torch.cuda.device(q.device):
        rc = _lib.load().dkv_decode_noalloc(C.byref(a), _stream())
    if rc != _lib.DKV_OK:
        raise RuntimeError(f"directkv_b200 error {rc}: {err.value.decode()}")
    return out


def merge_partials(parts: torch.Tensor, out: Optional[torch.Tensor] = None,
                   lse_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Combines ``parts [R, rows, 132]`` (one unnormalised partial set per rank) into ``[rows, 128]`` bf16."""
    _chk(parts.is_cuda and parts.dtype == torch.float32 and parts.is_contiguous() and parts.dim() == 3
         and parts.size(2) == PARTIAL_STRIDE, "parts must be [R, rows, 132] fp32 CUDA contiguous")
    r, rows = parts.size(0), parts.size(1)
    if out is None:
        out = torch.empty(rows, HEAD_DIM, dtype=torch.bfloat16, device=parts.device)
    ctx = get_context(parts.device.index)
    _lib.check(_lib.load().dkv_merge_partials(ctx.handle, _ptr(parts), r, rows, _ptr(out), _ptr(lse_out), _stream()))
    return out


def stream_copy(dst: torch.Tensor, src: torch.Tensor) -> None:
    """SM-issued copy of ``src`` (pinned host or device) into ``dst`` (device): host-link probe."""
    nbytes = src.numel() * src.element_size()
    _chk(dst.is_cuda and dst.numel() * dst.element_size() >= nbytes, "dst must be a CUDA tensor at least as large as src")
    ctx = get_context(dst.device.index)
    _lib.check(_lib.load().dkv_stream_copy(ctx.handle, _ptr(dst), _ptr(src), nbytes, _stream()))


# ---------------------------------------------------------------------------
# Reference-shaped entry points
# ---------------------------------------------------------------------------
def smpv2_fwd(
    X: torch.Tensor,                  # [B, S_new, hidden_dim]      GPU bf16
    Wk: torch.Tensor,                 # [NH, head_dim, hidden_dim]  GPU bf16
    Wv: torch.Tensor,
    Q: torch.Tensor,                  # [B, S_new, NH_q, head_dim]  GPU bf16
    K_cpu: torch.Tensor,              # [B, S_total, NH, head_dim]  CPU-pinned bf16 (or CUDA: HBM mode)
    V_cpu: torch.Tensor,
    cos_sin: Optional[torch.Tensor],  # [max_pos, head_dim] GPU fp32, or None
    softmax_scale: float,
    is_causal: bool,
    seqlen_past: int,
    q_pos_start: int,
) -> torch.Tensor:
    """Fused forward: X->K,V projection + Neox RoPE + attention (directkv/kernel/__init__.py:225-257).

    Same arguments and result as the reference.  Unlike the reference, ``seqlen_past`` and
    ``S_new`` may be any positive sizes and the projection contracts the full hidden size.
    """
    _chk(X.dim() == 3, f"X must be 3D [B, S_new, H], got {X.dim()}D")
    _chk(Wk.dim() == 3, "Wk must be 3D [NH, D, H]")
    _chk(Wv.dim() == 3, "Wv must be 3D [NH, D, H]")
    _chk(Q.dim() == 4, "Q must be 4D [B, S_new, NH, D]")
    _chk(K_cpu.dim() == 4, "K_cpu must be 4D [B, S_total, NH, D]")
    _chk(V_cpu.dim() == 4, "V_cpu must be 4D [B, S_total, NH, D]")
    for t, n in ((X, "X"), (Wk, "Wk"), (Wv, "Wv"), (Q, "Q")):
        _check_cuda_bf16(t, n)
    _check_kv(K_cpu, "K_cpu")
    _check_kv(V_cpu, "V_cpu")
    _chk(Q.size(3) == HEAD_DIM, f"head_dim must be {HEAD_DIM}, got {Q.size(3)}")
    _chk(Q.size(2) % Wk.size(0) == 0,
         f"Q.size(2) (NH_q={Q.size(2)}) must be a multiple of Wk.size(0) (NH_kv={Wk.size(0)})")
    _check_cos_sin(cos_sin)
    B, S_new, H = X.shape
    nh_kv, nh_q = Wk.size(0), Q.size(2)
    S_total = K_cpu.size(1)
    _chk(Wk.size(1) == HEAD_DIM and Wk.size(2) == H and Wv.shape == Wk.shape, "Wk/Wv must be [NH, 128, H]")
    _chk(Q.size(0) == B and Q.size(1) == S_new, "Q must match X in batch and S_new")
    _chk(K_cpu.size(0) == B and K_cpu.size(2) == nh_kv and K_cpu.size(3) == HEAD_DIM and V_cpu.shape == K_cpu.shape,
         "K_cpu/V_cpu must be [B, S_total, NH_kv, 128]")
    O = torch.empty(B, S_new, nh_q, HEAD_DIM, dtype=torch.bfloat16, device=X.device)
    ctx = get_context(X.device.index)
    _lib.check(_lib.load().dkv_smpv2_fwd(
        ctx.handle, _ptr(X), _ptr(Wk), _ptr(Wv), _ptr(Q), _ptr(K_cpu), _ptr(V_cpu), _ptr(cos_sin),
        0 if cos_sin is None else cos_sin.size(0), B, S_new, H, nh_q, nh_kv, S_total,
        float(softmax_scale), 1 if is_causal else 0, int(seqlen_past), int(q_pos_start), _ptr(O), _stream()))
    return O


def smpv2_init_tma(
    layer_id: int,
    X_max: torch.Tensor,     # [max_bs, S_new_max, H]          GPU bf16
    Wk: torch.Tensor,        # [NH, D, H]                      GPU bf16
    Wv: torch.Tensor,
    Q_max: torch.Tensor,     # [max_bs, S_new_max, NH, D]      GPU bf16
    K_max: torch.Tensor,     # [n_pool, S_total_max, NH, D]    CPU-pinned bf16
    V_max: torch.Tensor,
    cos_sin: Optional[torch.Tensor] = None,
) -> None:
    """Per-layer set-up before graph capture (directkv/kernel/__init__.py:260-279).

    Registers the layer (descriptors for K_max/V_max rows and the weights) and pre-sizes
    scratch for ``max_bs * S_new_max`` query rows so that ``smpv2_fwd_graph`` allocates nothing.
    ``cos_sin`` is an addition: the reference passes the table on every call instead.
    """
    for t, n in ((X_max, "X_max"), (Wk, "Wk"), (Wv, "Wv"), (Q_max, "Q_max")):
        _check_cuda_bf16(t, n)
    _check_kv(K_max, "K_max")
    _check_kv(V_max, "V_max")
    _chk(K_max.dim() == 4 and X_max.dim() == 3 and Q_max.dim() == 4, "bad tensor ranks")
    register_layer(layer_id, K_max, V_max, Wk, Wv, cos_sin, page_size=1, row_stride=K_max.size(1),
                   device=X_max.device.index)
    ctx = get_context(X_max.device.index)
    ctx.reserve(X_max.size(0) * X_max.size(1), Q_max.size(2), Wk.size(0), X_max.size(2))


def smpv2_fwd_graph(
    layer_id: int,
    X_pad: torch.Tensor,         # [bs, S_new, H]        GPU bf16
    Q_pad: torch.Tensor,         # [bs, S_new, NH, D]    GPU bf16
    O_out: torch.Tensor,         # [bs, S_new, NH, D]    GPU bf16 (pre-allocated output)
    n_past_dev: torch.Tensor,    # [1] int32 GPU: number of past 64-token blocks for this step
    n_blks_dev: torch.Tensor,    # [1] int32 GPU (kept for signature compatibility; = n_past + S_new/64)
    cos_sin: Optional[torch.Tensor],
    softmax_scale: float,
    is_causal: bool,
    S_total_max: int,
    seqlen_past_max: int,
    req_pool_indices: Optional[torch.Tensor] = None,  # [bs] int32 GPU: batch_pos -> pool row
) -> torch.Tensor:
    """Graph-safe forward (directkv/kernel/__init__.py:282-314): loop bounds come from device memory."""
    for t, n in ((X_pad, "X_pad"), (Q_pad, "Q_pad"), (O_out, "O_out")):
        _check_cuda_bf16(t, n)
    _chk(n_past_dev.is_cuda and n_past_dev.dtype == torch.int32, "n_past_dev must be int32")
    _chk(n_blks_dev.is_cuda and n_blks_dev.dtype == torch.int32, "n_blks_dev must be int32")
    if req_pool_indices is not None:
        _chk(req_pool_indices.is_cuda and req_pool_indices.dtype == torch.int32, "req_pool_indices must be int32")
    B, S_new, _ = X_pad.shape
    ctx = get_context(X_pad.device.index)
    kept = ctx._keepalive.get(int(layer_id))
    if kept is not None and cos_sin is not None and (kept[4] is None or kept[4].data_ptr() != cos_sin.data_ptr()):
        # The reference passes the table per call; re-register (host-only work) when it changed.
        _check_cos_sin(cos_sin)
        register_layer(layer_id, kept[0], kept[1], kept[2], kept[3], cos_sin, page_size=1,
                       row_stride=kept[0].size(1), device=X_pad.device.index)
    _lib.check(_lib.load().dkv_smpv2_fwd_graph(
        ctx.handle, int(layer_id), _ptr(X_pad), _ptr(Q_pad), _ptr(O_out), _ptr(n_past_dev), B, S_new,
        Q_pad.size(2), float(softmax_scale), 1 if is_causal else 0, _ptr(req_pool_indices), _stream()))
    return O_out


# The plain ``directkv`` backend imports these names (directkv/directkv_backend.py:83-93).
directkv_fwd = smpv2_fwd
directkv_init_tma = smpv2_init_tma
directkv_fwd_graph = smpv2_fwd_graph
