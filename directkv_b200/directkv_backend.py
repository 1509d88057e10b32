"""SGLang attention backend over the B200 engine.

Same class name, constructor and method surface as the reference's ``DirectKVBackend``
(directkv/directkv_backend.py:63-928): ``init_forward_metadata``, ``forward_decode``,
``forward_extend`` and the four CUDA-graph hooks, reading the same fields of ``ForwardBatch``,
``RadixAttention`` and ``ModelRunner`` (:68-76, :159-196).

What is different underneath
  * One engine call per layer and step for the WHOLE ragged batch: no bucketing by 64-aligned
    length, no zero-padded 64-row tiles, no per-request SDPA fallback (the kernels take any
    length and any ``NH_q % NH_kv == 0``).
  * The request pool is read and written in place through a row map (the reference gathers a
    pageable copy per bucket, directkv/directkv_request_pool.py:148-152, so its kernel's write-back
    never reaches the pool).
  * Under CUDA graphs every request keeps its own length: lengths and rows live in device tensors
    that the replay hook refreshes (the reference forces one common padded length,
    directkv/directkv_backend.py:483-494).
  * When the layer's hidden states were not captured (no hook fired) the step runs over SGLang's
    token pool with the K/V SGLang computed - the data flow of the reference's
    ``_sdpa_decode_manual`` / ``_sdpa_extend_manual`` (:835-891) - still on the engine.
"""

from __future__ import annotations

import os

import logging
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from . import kernel
from ._lib import get_context
from .directkv_request_pool import DirectKVRequestPool
from .sglang_compat import AttentionBackend, get_attention_tp_size

logger = logging.getLogger(__name__)

_TILE = 64                       # directkv/directkv_backend.py:42
_TOKEN_POOL_LAYER_BASE = 1 << 20  # engine layer ids of the token-pool registrations


def _pad64(n: int) -> int:
    return -(-int(n) // _TILE) * _TILE


@dataclass
class _FwdMeta:
    """Host copies made once per step (directkv/directkv_backend.py:52-57) plus their device twins."""
    seq_lens_cpu: List[int]
    req_pool_indices_cpu: List[int]
    extend_seq_lens_cpu: Optional[List[int]]
    extend_prefix_lens_cpu: Optional[List[int]]
    seq_lens_dev: Optional[torch.Tensor] = None       # int32 [bs]
    rows_dev: Optional[torch.Tensor] = None           # int32 [bs] request-pool rows
    req_idx_dev: Optional[torch.Tensor] = None        # int32 [bs] rows of req_to_token
    graph: bool = False                               # made by a CUDA-graph hook: rows and lengths live in the static tensors


class DirectKVBackend(AttentionBackend):
    _NAME = "directkv"
    _TAG = "[DirectKV]"

    def __init__(self, model_runner):
        super().__init__()
        tp = get_attention_tp_size()
        cfg = model_runner.model_config
        self.num_q_heads = cfg.num_attention_heads // tp
        self.num_kv_heads = cfg.get_num_kv_heads(tp)
        self.head_dim = cfg.head_dim
        self.v_head_dim = getattr(cfg, "v_head_dim", None) or cfg.head_dim
        self.hidden_size = cfg.hidden_size
        self.device = model_runner.device
        self._check_args(model_runner)

        # The engine handles every grouping with NH_q % NH_kv == 0; anything else has no meaning for
        # grouped attention (the reference logs and falls back to a path that needs the same property).
        self._use_kernel = (self.num_q_heads % self.num_kv_heads == 0)
        if not self._use_kernel:
            raise ValueError(f"{self._NAME}: NH_q={self.num_q_heads} is not a multiple of NH_kv={self.num_kv_heads}")

        # The three entry points the reference binds in its constructor (:80-96)
        self._directkv_fwd = kernel.smpv2_fwd
        self._directkv_init_tma = kernel.smpv2_init_tma
        self._directkv_fwd_graph = kernel.smpv2_fwd_graph

        self._wk: Dict[int, torch.Tensor] = {}
        self._wv: Dict[int, torch.Tensor] = {}
        self._cos_sin: Optional[torch.Tensor] = None
        self._hidden: Dict[int, torch.Tensor] = {}
        self._hooks_ready = False
        self._model_runner = model_runner
        self._fwd_meta: Optional[_FwdMeta] = None
        self._pool_cls = DirectKVRequestPool
        self._pool: Optional[DirectKVRequestPool] = None
        self._registered: set = set()
        # Eager decode steps bring the past rows to HBM with the copy engines (DIRECTKV_B200_DMA_STAGING=0: stream
        # them with the SMs as under CUDA graphs).
        self._dma_staging = os.environ.get("DIRECTKV_B200_DMA_STAGING", "1") != "0"
        self._stager = None
        self._token_registered: Dict[int, int] = {}
        self._active_req_ids: set = set()
        self._last_seen: Dict[int, int] = {}
        self._last_len: Dict[int, int] = {}          # sequence length of each request at its latest step
        self._step_no = 0
        self._start_layer = 0
        # CUDA-graph state: device tensors with stable addresses, refreshed before each replay
        self._cg_max_bs = 0
        self._cg_seq_lens: Optional[torch.Tensor] = None
        self._cg_rows: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ checks
    def _check_args(self, runner) -> None:
        """Same three conditions as directkv/directkv_backend.py:159-169."""
        if not runner.server_args.disable_radix_cache:
            raise ValueError(f"{self._NAME} requires --disable-radix-cache")
        if self.head_dim != 128:
            raise ValueError(f"{self._NAME} requires head_dim=128, got {self.head_dim}. "
                             "Use a compatible model (e.g. OPT-6.7B, Llama-3-8B with GQA mod).")
        if runner.model_config.dtype not in (torch.bfloat16,):
            raise ValueError(f"{self._NAME} requires bfloat16 model weights.")

    # ------------------------------------------------------------------ pool
    def _ensure_pool(self) -> None:
        """Pool sizing of directkv/directkv_backend.py:174-197; layers are registered with the engine here."""
        if self._pool is None:
            mr = self._model_runner
            max_reqs = min(mr.req_to_token_pool.size, 64)
            context_len = getattr(mr.model_config, "context_len", 2048)
            max_seqlen = min(mr.req_to_token_pool.req_to_token.shape[1], context_len)
            self._start_layer = getattr(mr, "start_layer", 0)
            self._pool = self._pool_cls(
                max_reqs=max_reqs, max_seqlen=max_seqlen, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim,
                num_layers=mr.model_config.num_hidden_layers, start_layer=self._start_layer, spare_rows=1,
            )
            logger.info(f"{self._TAG} Pool: {self._pool}")
        for lid in self._wk:
            if lid not in self._registered:
                k_rows, v_rows = self._pool.get_row_tensor(lid)
                kernel.register_layer(lid, k_rows, v_rows, self._wk[lid], self._wv[lid], self._cos_sin, page_size=1,
                                      row_stride=self._pool.max_seqlen_pad, device=self._device_index())
                self._registered.add(lid)

    def _device_index(self) -> Optional[int]:
        d = torch.device(self.device)
        return d.index if d.index is not None else (torch.cuda.current_device() if torch.cuda.is_available() else None)

    # ------------------------------------------------------------------ hooks / weights
    def _setup_hooks(self) -> None:
        """Walks the model like directkv/directkv_backend.py:202-234: every module with an ``attn`` child that
        has a ``layer_id`` gives its K/V projection weights and gets a pre-hook that records its input."""
        model = self._model_runner.model
        self._start_layer = getattr(self._model_runner, "start_layer", 0)
        n = 0
        for _name, module in model.named_modules():
            layer_id = getattr(getattr(module, "attn", None), "layer_id", None)
            if layer_id is None:
                continue
            wk, wv = self._extract_weights(module, layer_id)
            if wk is None:
                continue
            self._wk[layer_id], self._wv[layer_id] = wk, wv
            if self._cos_sin is None:
                self._cos_sin = self._extract_cos_sin(module)
            module.register_forward_pre_hook(
                lambda _m, args, kwargs, _lid=layer_id: self._capture_hs(_lid, args, kwargs), with_kwargs=True)
            n += 1
        logger.info(f"{self._TAG} Hooked {n} layers; RoPE={'yes' if self._cos_sin is not None else 'no (OPT)'}.")
        self._hooks_ready = True

    def _capture_hs(self, layer_id: int, args, kwargs=None) -> None:
        if kwargs and "hidden_states" in kwargs:
            self._hidden[layer_id] = kwargs["hidden_states"]
        elif args:
            self._hidden[layer_id] = args[0]

    def _extract_weights(self, module, layer_id: int) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
        """K and V projection weights as [NH_kv, D, H] (directkv/directkv_backend.py:243-271).  As in the
        reference only ``.weight`` is used: a model with biased k/v projections (OPT) loses the bias."""
        nh_kv, nh_q, d, h = self.num_kv_heads, self.num_q_heads, self.head_dim, self.hidden_size
        qkv = getattr(module, "qkv_proj", None)
        if qkv is not None and hasattr(qkv, "weight"):
            w = qkv.weight.detach()
            k0 = nh_q * d
            k1 = k0 + nh_kv * d
            return (w[k0:k1].contiguous().view(nh_kv, d, h), w[k1:k1 + nh_kv * d].contiguous().view(nh_kv, d, h))
        kp, vp = getattr(module, "k_proj", None), getattr(module, "v_proj", None)
        if kp is not None and vp is not None and hasattr(kp, "weight") and hasattr(vp, "weight"):
            return (kp.weight.detach().contiguous().view(nh_kv, d, h), vp.weight.detach().contiguous().view(nh_kv, d, h))
        logger.warning(f"{self._TAG} Layer {layer_id}: cannot extract weights.")
        return None, None

    def _extract_cos_sin(self, module) -> Optional[torch.Tensor]:
        """[max_pos, D] fp32 table = [cos | sin] from whatever the rotary module offers
        (directkv/directkv_backend.py:273-305); None when the model has no rotary embedding."""
        rotary = getattr(module, "rotary_emb", None)
        if rotary is None:
            return None
        d = self.head_dim
        fused = getattr(rotary, "cos_sin_cache", None)
        if fused is not None and fused.shape[-1] == d:
            return fused.float().to(self.device).contiguous()
        for cname, sname in (("cos_cached", "sin_cached"), ("_cos_cached", "_sin_cached"), ("cos", "sin")):
            cos, sin = getattr(rotary, cname, None), getattr(rotary, sname, None)
            if cos is None or sin is None:
                continue
            while cos.dim() > 2:
                cos, sin = cos.squeeze(0), sin.squeeze(0)
            if cos.dim() == 2 and cos.shape[-1] in (d // 2, d):
                half = d // 2
                return torch.cat([cos[:, :half], sin[:, :half]], dim=-1).float().to(self.device).contiguous()
        inv_freq = getattr(rotary, "inv_freq", None)
        if inv_freq is not None:
            max_pos = getattr(rotary, "max_position_embeddings", 8192)
            t = torch.arange(max_pos, dtype=torch.float32, device=self.device)
            fq = torch.outer(t, inv_freq.float().to(self.device))
            return torch.cat([fq.cos(), fq.sin()], dim=-1).contiguous()
        return None

    # ------------------------------------------------------------------ per-step metadata
    def _sync_rows(self, req_ids: List[int], free_absent: bool = True) -> None:
        """Row lifecycle.  In a DECODE batch every running request is present, so a request that is
        absent has finished: its row is freed first, then new requests get rows - the reference's policy
        (directkv/directkv_backend.py:323-335).  An EXTEND batch carries only the requests being
        prefilled, so absence means nothing there (the reference frees - and later zero-fills - the rows
        of running requests in that case); rows are then only reclaimed, oldest first, when the pool
        is full."""
        current = set(req_ids)
        self._step_no += 1
        if free_absent:
            for rid in self._active_req_ids - current:
                self._pool.free(rid)
                self._last_seen.pop(rid, None)
                self._last_len.pop(rid, None)
            self._active_req_ids &= current
        for rid in req_ids:
            if rid not in self._active_req_ids:
                if self._pool.free_rows == 0:
                    idle = sorted((r for r in self._active_req_ids if r not in current), key=lambda r: self._last_seen.get(r, 0))
                    if idle:
                        self._pool.free(idle[0])
                        self._active_req_ids.discard(idle[0])
                        self._last_seen.pop(idle[0], None)
                        self._last_len.pop(idle[0], None)
                self._pool.alloc(rid)
                self._active_req_ids.add(rid)
            self._last_seen[rid] = self._step_no

    def init_forward_metadata(self, forward_batch) -> None:
        if forward_batch.forward_mode.is_idle():
            self._fwd_meta = None
            return
        if not self._hooks_ready:
            self._setup_hooks()
        # SGLang keeps a host copy of the lengths; use it and save one device-to-host synchronisation per step.
        sl_host = getattr(forward_batch, "seq_lens_cpu", None)
        seq_lens_cpu = sl_host.tolist() if sl_host is not None else forward_batch.seq_lens.cpu().tolist()
        req_ids_cpu = forward_batch.req_pool_indices.cpu().tolist()
        self._ensure_pool()
        self._sync_rows(req_ids_cpu, free_absent=forward_batch.forward_mode.is_decode())
        for rid, n in zip(req_ids_cpu, seq_lens_cpu):
            self._last_len[rid] = int(n)
        self._fwd_meta = _FwdMeta(
            seq_lens_cpu=seq_lens_cpu,
            req_pool_indices_cpu=req_ids_cpu,
            extend_seq_lens_cpu=getattr(forward_batch, "extend_seq_lens_cpu", None),
            extend_prefix_lens_cpu=getattr(forward_batch, "extend_prefix_lens_cpu", None),
            seq_lens_dev=forward_batch.seq_lens.to(device=self.device, dtype=torch.int32),
            rows_dev=self._pool.row_table(req_ids_cpu, self.device),
            req_idx_dev=forward_batch.req_pool_indices.to(device=self.device, dtype=torch.int32),
        )

    # ------------------------------------------------------------------ CUDA graphs
    def init_cuda_graph_state(self, max_bs: int, max_num_tokens: int) -> None:
        if not self._hooks_ready:
            self._setup_hooks()
        self._ensure_pool()
        self._cg_max_bs = max_bs
        self._cg_seq_lens = torch.ones(max_bs, dtype=torch.int32, device=self.device)
        self._cg_rows = torch.zeros(max_bs, dtype=torch.int32, device=self.device)
        # Scratch for max_bs requests is sized now: nothing is allocated while a graph is captured.
        get_context(self._device_index()).reserve(max_bs, self.num_q_heads, self.num_kv_heads, self.hidden_size)
        logger.info(f"{self._TAG} CUDA graph state: max_bs={max_bs}, layers={len(self._wk)}.")

    def _count_real(self, rid_list: List[int], seq_lens_cpu: List[int]) -> int:
        """Entries of a replayed batch that are requests.  SGLang pads a replay up to the captured batch size:
        the padded tail has the fill length and request indices that are stale or zero, so such an index may
        belong to a live request.  A tail entry counts as padding when its length is the fill value and its
        index repeats an earlier entry, holds no row, or belongs to a request whose previous length was not
        fill - 1 (a request that really has the fill length was one token shorter a step ago)."""
        fill = self.get_cuda_graph_seq_len_fill_value()
        n = len(rid_list)
        while n > 0:
            rid, length = rid_list[n - 1], int(seq_lens_cpu[n - 1])
            if length != fill:
                break
            if not (rid in rid_list[:n - 1] or rid not in self._active_req_ids or self._last_len.get(rid) != fill - 1):
                break
            n -= 1
        return n

    def _graph_meta(self, bs: int, req_pool_indices, seq_lens_cpu: List[int], n_real: Optional[int] = None) -> None:
        """Device-side lengths and rows of a captured or replayed batch.  Entries from ``n_real`` on are padding:
        they get the pool's spare row and length 1, so what the graph stores for them (the in-place write of
        the "new token") reaches no request's row, and they keep no row of their own."""
        rid_list = req_pool_indices[:bs].cpu().tolist()
        self._ensure_pool()
        if n_real is None:
            n_real = self._count_real(rid_list, seq_lens_cpu)
        real = rid_list[:n_real]
        if real:                       # a capture (placeholders only) changes no request's row
            self._sync_rows(real)
        for rid, n in zip(real, seq_lens_cpu):
            self._last_len[rid] = int(n)
        rows = [self._pool.row_of(r) for r in real] + [self._pool.pad_row] * (bs - n_real)
        self._cg_rows[:bs].copy_(torch.tensor(rows, dtype=torch.int32), non_blocking=False)
        if n_real < bs:
            self._cg_seq_lens[n_real:bs].fill_(1)
        self._fwd_meta = _FwdMeta(
            seq_lens_cpu=list(seq_lens_cpu[:n_real]) + [1] * (bs - n_real), req_pool_indices_cpu=rid_list,
            extend_seq_lens_cpu=None, extend_prefix_lens_cpu=None, seq_lens_dev=self._cg_seq_lens[:bs],
            rows_dev=self._cg_rows[:bs], req_idx_dev=req_pool_indices[:bs].to(torch.int32), graph=True,
        )

    def init_forward_metadata_capture_cuda_graph(self, bs, num_tokens, req_pool_indices, seq_lens, encoder_lens,
                                                 forward_mode, spec_info) -> None:
        # The batch of a capture is made of placeholders: all of it goes to the spare row.
        fill = self.get_cuda_graph_seq_len_fill_value()
        self._cg_seq_lens[:bs].fill_(fill)
        self._graph_meta(bs, req_pool_indices, [fill] * bs, n_real=0)

    def init_forward_metadata_replay_cuda_graph(self, bs, req_pool_indices, seq_lens, seq_lens_sum, encoder_lens,
                                                forward_mode, spec_info, seq_lens_cpu=None) -> None:
        sl_cpu = seq_lens_cpu.tolist() if seq_lens_cpu is not None else seq_lens[:bs].cpu().tolist()
        self._cg_seq_lens[:bs].copy_(seq_lens[:bs])          # every request keeps its OWN length
        self._graph_meta(bs, req_pool_indices, sl_cpu)

    def get_cuda_graph_seq_len_fill_value(self) -> int:
        return _TILE

    # ------------------------------------------------------------------ decode
    def forward_decode(self, q, k, v, layer, forward_batch, save_kv_cache: bool = True) -> torch.Tensor:
        lid, meta = layer.layer_id, self._fwd_meta
        bs = forward_batch.batch_size
        if meta is None:
            return torch.zeros(bs, self.num_q_heads * self.head_dim, dtype=q.dtype, device=self.device)
        x = self._hidden.pop(lid, None)
        q2 = q.reshape(bs, self.num_q_heads * self.head_dim).contiguous()
        if x is None or lid not in self._registered:
            return self._decode_token_pool(q2, k, v, layer, forward_batch)
        x2 = x.reshape(bs, self.hidden_size).contiguous()
        if self._dma_staging and save_kv_cache and not meta.graph and not torch.cuda.is_current_stream_capturing():
            # Eager step over the host-pinned request pool: the copy engines bring the past rows to HBM at the
            # full rate of the host link and the kernels attend that copy (directkv_b200/staging.py).
            if self._stager is None:
                from .staging import DmaStagedDecode

                self._stager = DmaStagedDecode(self.device, self.num_kv_heads, self._pool.dtype)
            li = lid - self._pool.start_layer
            rows = [self._pool.row_of(r) for r in meta.req_pool_indices_cpu[:bs]]
            return self._stager.decode(lid, self._pool.k_pool[li], self._pool.v_pool[li], rows, meta.seq_lens_cpu[:bs],
                                       q2, meta.seq_lens_dev[:bs], float(layer.scaling), meta.rows_dev[:bs], x=x2)
        return kernel.decode(lid, q2, meta.seq_lens_dev[:bs], float(layer.scaling), row_map=meta.rows_dev[:bs], x=x2,
                             save_kv_cache=save_kv_cache)

    def _token_layer(self, layer, forward_batch) -> int:
        """Engine registration of SGLang's token-indexed pool for this layer (page size 1 = per-token slots)."""
        lid = layer.layer_id
        pool = forward_batch.token_to_kv_pool
        k_buf, v_buf = pool.get_key_buffer(lid), pool.get_value_buffer(lid)
        eng = _TOKEN_POOL_LAYER_BASE + lid
        if self._token_registered.get(lid) != k_buf.data_ptr():
            kernel.register_layer(eng, k_buf, v_buf, page_size=1, device=self._device_index())
            self._token_registered[lid] = k_buf.data_ptr()
        return eng

    def _decode_token_pool(self, q2, k, v, layer, forward_batch) -> torch.Tensor:
        """Data flow of ``_sdpa_decode_manual`` (:835-859): store k, v at ``out_cache_loc``, attend the slots
        ``req_to_token[req, :seq_len]``."""
        meta = self._fwd_meta
        bs = forward_batch.batch_size
        forward_batch.token_to_kv_pool.set_kv_buffer(layer, forward_batch.out_cache_loc, k, v)
        eng = self._token_layer(layer, forward_batch)
        table = forward_batch.req_to_token_pool.req_to_token
        return kernel.decode(eng, q2, meta.seq_lens_dev[:bs], float(layer.scaling), page_table=table,
                             row_map=meta.req_idx_dev[:bs])

    # ------------------------------------------------------------------ extend
    def forward_extend(self, q, k, v, layer, forward_batch, save_kv_cache: bool = True) -> torch.Tensor:
        lid, meta = layer.layer_id, self._fwd_meta
        bs = forward_batch.batch_size
        nh_q, d = self.num_q_heads, self.head_dim
        if meta is None:
            return q.new_zeros(q.shape[0], nh_q * d)
        x_all = self._hidden.pop(lid, None)
        ext, pre = meta.extend_seq_lens_cpu, meta.extend_prefix_lens_cpu
        if x_all is None or lid not in self._registered or ext is None:
            return self._extend_token_pool(q, k, v, layer, forward_batch)
        # One launch sequence for the whole ragged batch (the reference calls its kernel once per request,
        # directkv/directkv_backend.py:681-697); requests without new rows take no part.
        live = [i for i in range(bs) if int(ext[i]) > 0]
        n_rows = sum(int(ext[i]) for i in live)
        if not live:
            return q.new_zeros(q.shape[0], nh_q * d)
        if n_rows != q.shape[0]:
            raise ValueError(f"{self._NAME}: extend_seq_lens sum to {n_rows} rows but q has {q.shape[0]}")
        out = kernel.extend_ragged(
            lid, x_all.reshape(n_rows, self.hidden_size).contiguous(), q.reshape(n_rows, nh_q, d).contiguous(),
            [int(ext[i]) for i in live], [int(pre[i]) if pre else 0 for i in live],
            [self._pool.row_of(meta.req_pool_indices_cpu[i]) for i in live], float(layer.scaling), True)
        return out.view(n_rows, nh_q * d)

    def _extend_token_pool(self, q, k, v, layer, forward_batch) -> torch.Tensor:
        """Data flow of ``_sdpa_extend_manual`` (:861-891) on the engine: store k, v, then every new row
        attends slots ``req_to_token[req, :prefix + i + 1]`` (the triu(diagonal=prefix+1) mask)."""
        meta = self._fwd_meta
        bs = forward_batch.batch_size
        nh_q, d = self.num_q_heads, self.head_dim
        forward_batch.token_to_kv_pool.set_kv_buffer(layer, forward_batch.out_cache_loc, k, v)
        eng = self._token_layer(layer, forward_batch)
        ext = meta.extend_seq_lens_cpu or [meta.seq_lens_cpu[i] for i in range(bs)]
        pre = meta.extend_prefix_lens_cpu or [0] * bs
        table = forward_batch.req_to_token_pool.req_to_token
        g_total = nh_q // self.num_kv_heads
        out = torch.empty(q.shape[0], nh_q * d, dtype=q.dtype, device=q.device)
        # A request whose new rows fill at least one 128-row query tile goes to the tensor-core extend kernel
        # (its rows are gathered through req_to_token once); shorter ones are batched as one virtual decode
        # request per new row.
        vlen, vrow, vidx = [], [], []
        long_req, long_idx = [], []
        off = 0
        for i in range(bs):
            n_new, n_pre = int(ext[i]), int(pre[i])
            if n_new * g_total >= 128:
                long_req.append((n_new, n_pre, meta.req_pool_indices_cpu[i]))
                long_idx.append((off, n_new))
            else:
                vlen += [n_pre + j + 1 for j in range(n_new)]
                vrow += [meta.req_pool_indices_cpu[i]] * n_new
                vidx += list(range(off, off + n_new))
            off += n_new
        if long_req:
            whole = len(long_req) == bs
            q_long = q if whole else torch.cat([q[o:o + n] for o, n in long_idx])
            o_long = kernel.extend_ragged(eng, None, q_long.reshape(-1, nh_q, d).contiguous(), [r[0] for r in long_req],
                                          [r[1] for r in long_req], [r[2] for r in long_req], float(layer.scaling), True,
                                          page_table=table).view(-1, nh_q * d)
            if whole:
                return o_long
            pos = 0
            for o, n in long_idx:
                out[o:o + n] = o_long[pos:pos + n]
                pos += n
        if vlen:
            vlen_t = torch.tensor(vlen, dtype=torch.int32).to(self.device, non_blocking=True)
            vrow_t = torch.tensor(vrow, dtype=torch.int32).to(self.device, non_blocking=True)
            q2 = q.reshape(-1, nh_q * d)
            if len(vidx) != q2.shape[0]:
                idx = torch.tensor(vidx, dtype=torch.long, device=q.device)
                o_small = kernel.decode(eng, q2[idx].contiguous(), vlen_t, float(layer.scaling), page_table=table, row_map=vrow_t)
                out[idx] = o_small
            else:
                out = kernel.decode(eng, q2.contiguous(), vlen_t, float(layer.scaling), page_table=table, row_map=vrow_t)
        return out
