"""Host-side pools against outputs of the reference's own pool classes (tests/golden) and the
reference's pool unit tests (tests/test_directkv_correctness.py:61-128).  No GPU needed."""

import os

import numpy as np
import pytest
import torch

from directkv_b200.directkv_pool import DirectKVTokenToKVPool
from directkv_b200.directkv_request_pool import DirectKVRequestPool, _pad64

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def bf16(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


class FakeLayer:
    layer_id = 1


def _make_pool(size=64, page_size=1, head_num=4, head_dim=32, layer_num=2, dtype=torch.float16):
    return DirectKVTokenToKVPool(size=size, page_size=page_size, dtype=dtype, head_num=head_num, head_dim=head_dim,
                                 layer_num=layer_num, v_head_dim=head_dim, start_layer=0, end_layer=layer_num)


def test_token_pool_matches_reference_outputs():
    g = np.load(os.path.join(GOLD, "pool_token.npz"))
    pool = DirectKVTokenToKVPool(size=40, page_size=1, dtype=torch.bfloat16, head_num=3, head_dim=16, layer_num=2,
                                 v_head_dim=16, start_layer=0, end_layer=2)
    assert list(pool.get_key_buffer(0).shape) == g["shape_k"].tolist()
    assert len(pool.k_buffer) == int(g["n_layers"])
    assert pool.token_stride == int(g["token_stride"]) and pool.row_dim == int(g["row_dim"])
    assert list(pool.get_kv_size_bytes()) == g["size_bytes"].tolist()
    pool.set_kv_buffer(FakeLayer(), torch.from_numpy(g["loc"]), bf16(g["k"]), bf16(g["v"]))
    assert torch.equal(pool.get_key_buffer(1), bf16(g["k_buf_l1"]))
    assert torch.equal(pool.get_value_buffer(1), bf16(g["v_buf_l1"]))
    assert pool.get_key_buffer(0).abs().sum() == 0
    pool.move_kv_cache(torch.tensor([30, 31]), torch.tensor([5, 17]))
    assert torch.equal(pool.get_key_buffer(1), bf16(g["k_buf_l1_after_move"]))
    assert int(g["fp32_raises"]) == 1
    with pytest.raises(ValueError):
        DirectKVTokenToKVPool(size=8, page_size=1, dtype=torch.float32, head_num=2, head_dim=16, layer_num=1)


def test_token_pool_reference_unit_cases():
    # tests/test_directkv_correctness.py:82-128
    pool = _make_pool()
    assert pool.get_key_buffer(0).device.type == "cpu"
    pool = _make_pool(size=32, head_num=2, head_dim=16, layer_num=1)

    class L0:
        layer_id = 0

    n = 10
    loc = torch.arange(n, dtype=torch.long)
    k = torch.randn(n, 2, 16, dtype=torch.float16)
    v = torch.randn(n, 2, 16, dtype=torch.float16)
    pool.set_kv_buffer(L0(), loc, k, v)
    assert (pool.get_key_buffer(0)[loc] - k).abs().max().item() == 0.0
    assert (pool.get_value_buffer(0)[loc] - v).abs().max().item() == 0.0
    pool = _make_pool(size=100, head_num=8, head_dim=64, layer_num=4)
    assert pool.get_key_buffer(0).shape == (101, 8, 64) and pool.get_value_buffer(3).shape == (101, 8, 64)
    assert _make_pool(dtype=torch.bfloat16).get_key_buffer(0).dtype == torch.bfloat16
    assert pool.get_v_head_dim() == 64 and pool.same_kv_dim
    with pytest.raises(NotImplementedError):
        pool.get_cpu_copy(torch.tensor([1]))


def test_token_pool_paged_rows_and_host_transfers():
    pool = DirectKVTokenToKVPool(size=64, page_size=16, dtype=torch.bfloat16, head_num=2, head_dim=128, layer_num=1)
    assert pool.get_key_buffer(0).shape[0] == 64 + 16   # one reserved page
    other = DirectKVTokenToKVPool(size=64, page_size=16, dtype=torch.bfloat16, head_num=2, head_dim=128, layer_num=1)
    other.k_buffer[0][5] = 1.0
    other.v_buffer[0][5] = 2.0
    pool.load_from_host_per_layer(other, torch.tensor([5]), torch.tensor([9]), 0, None)
    assert pool.k_buffer[0][9].float().mean() == 1.0 and pool.v_buffer[0][9].float().mean() == 2.0
    back = DirectKVTokenToKVPool(size=64, page_size=16, dtype=torch.bfloat16, head_num=2, head_dim=128, layer_num=1)
    pool.backup_to_host_all_layer(back, [3], [9], None)
    assert back.k_buffer[0][3].float().mean() == 1.0


def test_request_pool_matches_reference_outputs():
    g = np.load(os.path.join(GOLD, "pool_request.npz"))
    assert [_pad64(int(n)) for n in g["pad64_in"]] == g["pad64_out"].tolist()
    pool = DirectKVRequestPool(max_reqs=4, max_seqlen=100, num_kv_heads=2, head_dim=8, num_layers=2, start_layer=3)
    assert pool.max_seqlen_pad == int(g["max_seqlen_pad"])
    for (is_alloc, rid), (_, _, row, nfree) in zip(g["ops"].tolist(), g["trace"].tolist()):
        (pool.alloc if is_alloc else pool.free)(rid)
        assert pool._req_to_row.get(rid, -1) == row and len(pool._free) == nfree
    assert int(g["exhausted_raises"]) == 1
    with pytest.raises(RuntimeError, match="Out of rows"):
        pool.alloc(17)
    with pytest.raises(KeyError):
        pool.row_of(12345)
    assert [[r, pool.row_of(r)] for r in sorted(pool._req_to_row)] == g["rows_final"].tolist()
    pool.k_pool[0].copy_(bf16(g["k_l0"]))
    pool.k_pool[1].copy_(bf16(g["k_l1"]))
    pool.v_pool[1].copy_(bf16(g["v_l1"]))
    K, V = pool.get_kv(15, 4, 64)
    assert torch.equal(K, bf16(g["get_kv_K"])) and torch.equal(V, bf16(g["get_kv_V"]))
    assert K.data_ptr() == pool.k_pool[1][pool.row_of(15)].data_ptr()          # a view, not a copy
    Kb, _ = pool.get_batch_kv([16, 13], 3, 64)
    assert torch.equal(Kb, bf16(g["batch_K"]))
    assert list(pool.get_cuda_graph_kv(4, 2)[0].shape) == g["graph_K_shape"].tolist()
    assert pool.row_table([16, 13]).tolist() == [pool.row_of(16), pool.row_of(13)]
    assert pool.get_row_tensor(4)[0].data_ptr() == pool.k_pool[1].data_ptr()


def test_request_pool_zero_on_alloc_semantics():
    pool = DirectKVRequestPool(2, 64, 1, 8, 2)
    pool.alloc(1)
    r = pool.row_of(1)
    pool.k_pool[0][r].fill_(3.0)
    pool.v_pool[1][r].fill_(3.0)
    pool.free(1)
    pool.alloc(2)                       # LIFO: gets the same row back, zero-filled
    assert pool.row_of(2) == r and pool.k_pool[0][r].abs().sum() == 0 and pool.v_pool[1][r].abs().sum() == 0
    keep = DirectKVRequestPool(2, 64, 1, 8, 1, zero_on_alloc=False)
    keep.alloc(1)
    keep.k_pool[0][keep.row_of(1)].fill_(3.0)
    keep.free(1)
    keep.alloc(2)
    assert keep.k_pool[0][keep.row_of(2)].float().mean() == 3.0
    assert "free=1" in repr(keep)
