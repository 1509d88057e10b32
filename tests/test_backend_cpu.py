"""Host-side logic of the attention backend (no GPU): argument checks, weight slicing and cos/sin
extraction against outputs of the reference's own methods, row bookkeeping."""

import os

import numpy as np
import pytest
import torch

from fake_sglang import FakeModel, make_runner

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def bf16(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def _backend(cls_name="DirectKVBackend", **kw):
    import directkv_b200

    model = FakeModel(2, 256, 8, 2, 10000.0, 128)
    runner = make_runner(model, 256, 8, 2, 2, "cpu", **kw)
    return getattr(directkv_b200, cls_name)(runner), runner


def test_constructor_checks_match_reference():
    # directkv/directkv_backend.py:159-169
    with pytest.raises(ValueError, match="directkv requires --disable-radix-cache"):
        _backend(disable_radix_cache=False)
    with pytest.raises(ValueError, match="directkv-smpv2 requires --disable-radix-cache"):
        _backend("DirectKVSmpV2Backend", disable_radix_cache=False)
    with pytest.raises(ValueError, match="head_dim=128"):
        _backend(head_dim=64)
    with pytest.raises(ValueError, match="bfloat16"):
        _backend(dtype=torch.float16)
    be, _ = _backend("DirectKVSmpV2Backend")
    assert be.num_q_heads == 8 and be.num_kv_heads == 2 and be.get_cuda_graph_seq_len_fill_value() == 64
    assert callable(be._smpv2_fwd) and callable(be._directkv_fwd_graph)


def test_weight_and_table_extraction_match_reference_outputs():
    g = np.load(os.path.join(GOLD, "torch_paths.npz"))
    be, _ = _backend()
    be.num_q_heads, be.num_kv_heads, be.head_dim, be.hidden_size = 8, 2, 32, 64   # the golden case's geometry

    class M:
        pass

    m = M()
    m.qkv_proj = M()
    m.qkv_proj.weight = bf16(g["w_qkv"])
    wk, wv = be._extract_weights(m, 0)
    assert torch.equal(wk, bf16(g["wk"])) and torch.equal(wv, bf16(g["wv"]))
    m2 = M()
    m2.k_proj, m2.v_proj = M(), M()
    m2.k_proj.weight = bf16(g["wk"]).reshape(-1, 64)
    m2.v_proj.weight = bf16(g["wv"]).reshape(-1, 64)
    wk2, wv2 = be._extract_weights(m2, 0)
    assert torch.equal(wk2, wk) and torch.equal(wv2, wv)
    assert be._extract_weights(M(), 0) == (None, None)
    be.head_dim = 128
    m.rotary_emb = M()
    m.rotary_emb.inv_freq = 1.0 / (float(g["cos_sin_theta"]) ** (torch.arange(0, 64, dtype=torch.float32) / 64))
    m.rotary_emb.max_position_embeddings = 96
    cs = be._extract_cos_sin(m)
    assert torch.allclose(cs, torch.from_numpy(g["cos_sin"]), atol=1e-6, rtol=0)
    # fused cache and separate cos/sin forms give the same table
    m3 = M()
    m3.rotary_emb = M()
    m3.rotary_emb.cos_sin_cache = cs.clone()
    assert torch.equal(be._extract_cos_sin(m3), cs)
    m4 = M()
    m4.rotary_emb = M()
    m4.rotary_emb.cos_cached, m4.rotary_emb.sin_cached = cs[None, :, :64], cs[None, :, 64:]
    assert torch.equal(be._extract_cos_sin(m4), cs)
    assert be._extract_cos_sin(M()) is None


def test_row_bookkeeping_frees_before_allocating():
    from directkv_b200.directkv_request_pool import DirectKVRequestPool

    be, _ = _backend()
    be._pool = DirectKVRequestPool(2, 64, 2, 128, 1)
    be._sync_rows([4, 7])
    rows = {4: be._pool.row_of(4), 7: be._pool.row_of(7)}
    be._sync_rows([7, 9])              # 4 finished: its row must be free again before 9 asks for one
    assert be._pool.row_of(7) == rows[7] and be._pool.row_of(9) == rows[4]
    with pytest.raises(RuntimeError, match="Out of rows"):
        be._sync_rows([7, 9, 11])
    # an EXTEND batch names only the requests being prefilled: running requests keep their rows,
    # and a row is reclaimed (oldest idle request first) only when the pool is full
    be2, _ = _backend()
    be2._pool = DirectKVRequestPool(3, 64, 2, 128, 1)
    be2._sync_rows([1, 2])
    r1 = be2._pool.row_of(1)
    be2._sync_rows([3], free_absent=False)
    assert be2._pool.row_of(1) == r1 and be2._pool.row_of(2) is not None and len(be2._pool._free) == 0
    be2._sync_rows([2, 3])                       # decode batch without 1: 1 has finished
    be2._sync_rows([4], free_absent=False)       # takes the row 1 left
    assert be2._pool.row_of(4) == r1
    be2._sync_rows([5], free_absent=False)       # pool full: the idle request seen longest ago (2) goes
    assert 2 not in be2._active_req_ids and 3 in be2._active_req_ids


def test_hooks_capture_hidden_states_by_kwarg_and_positional():
    be, runner = _backend()
    be._setup_hooks()
    assert sorted(be._wk) == [0, 1] and be._cos_sin is not None and be._cos_sin.shape == (128, 128)
    x = torch.randn(3, 256).to(torch.bfloat16)
    runner.model.layers[0](hidden_states=x)
    runner.model.layers[1](x)
    assert be._hidden[0] is x and be._hidden[1] is x


def test_padded_graph_replays_are_told_from_requests():
    """Host logic of the replay hook: SGLang pads a replayed batch up to the captured size with the fill length and a
    stale or zero request index.  Such a tail entry counts as padding when its index repeats an earlier entry, holds
    no row, or belongs to a request whose previous length was not fill - 1; the pool keeps a spare row for them."""
    be, _ = _backend("DirectKVSmpV2Backend")
    be._ensure_pool()
    assert be._pool.pad_row == be._pool.max_reqs and be._pool.free_rows == be._pool.max_reqs
    be._sync_rows([1, 2, 6])
    be._last_len.update({1: 90, 2: 63, 6: 10})
    fill = be.get_cuda_graph_seq_len_fill_value()
    assert be._count_real([1, 2, 6], [91, 64, 11]) == 3                 # nothing padded
    assert be._count_real([1, 2, 6, 0], [91, 64, 11, fill]) == 3        # index 0 holds no row
    assert be._count_real([1, 6, 2, 2], [91, 11, 64, fill]) == 3        # repeats an earlier entry
    assert be._count_real([6, 2, 1, 1], [11, 64, fill, fill]) == 2      # request 1 was 90 tokens long, not 63
    assert be._count_real([1, 6, 2], [91, 11, fill]) == 3               # request 2 was 63 long: really 64 now
    assert be._count_real([0, 0, 0, 0], [fill] * 4) == 0                # a capture's placeholders
    rows = {be._pool.row_of(r) for r in (1, 2, 6)}
    assert be._pool.pad_row not in rows


def test_request_pool_spare_rows_never_enter_the_free_list():
    from directkv_b200 import DirectKVRequestPool

    pool = DirectKVRequestPool(max_reqs=3, max_seqlen=70, num_kv_heads=2, head_dim=128, num_layers=1, spare_rows=1)
    assert pool.k_pool[0].shape[0] == 4 and pool.pad_row == 3
    for rid in (10, 11, 12):
        pool.alloc(rid)
    assert sorted(pool.row_of(r) for r in (10, 11, 12)) == [0, 1, 2] and pool.free_rows == 0
    with pytest.raises(RuntimeError, match="Out of rows"):
        pool.alloc(13)
    with pytest.raises(ValueError):
        DirectKVRequestPool(max_reqs=1, max_seqlen=64, num_kv_heads=1, head_dim=128, num_layers=1).pad_row
