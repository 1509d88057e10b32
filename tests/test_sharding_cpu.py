"""Host-side logic of the multi-GPU partitionings, including a world_size-2 gloo run on the CPU:
sequence-split planning, head-shard slicing, and the partial exchange checked with the oracle's LSE merge."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dkv_testlib import orc
from directkv_b200 import sharding


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_plan_sequence_split_properties():
    for n, w, ps in [(0, 4, 16), (1, 4, 16), (1000, 2, 16), (1 << 20, 8, 16), (4097, 8, 16), (33, 4, 1), (100, 3, 64)]:
        plan = sharding.plan_sequence_split(n, w, ps)
        assert len(plan) == w and plan[0][0] == 0 and plan[-1][1] == n
        for (s0, e0), (s1, e1) in zip(plan, plan[1:]):
            assert e0 == s1 and s0 <= e0
        for s, e in plan:
            assert s % ps == 0 or s == n
        sizes = [-(-(e - s) // ps) for s, e in plan]
        assert max(sizes) - min(sizes) <= 1
        assert plan[sharding.owner_of_new_token(plan)][1] == n
    assert sharding.plan_sequence_split(1 << 20, 8, 16)[3] == (3 * 131072, 4 * 131072)
    with pytest.raises(ValueError):
        sharding.plan_sequence_split(10, 0, 16)


def test_head_shard_slices():
    sh = sharding.HeadShard(rank=3, world=8, nh_q=32, nh_kv=8)          # Llama-3-8B over 8 GPUs
    assert list(sh.kv_heads) == [3] and list(sh.q_heads) == [12, 13, 14, 15]
    sh = sharding.HeadShard(rank=7, world=8, nh_q=56, nh_kv=56)         # OPT-30B: 7 heads per GPU
    assert list(sh.kv_heads) == list(range(49, 56)) and sh.q_heads == sh.kv_heads
    wk = torch.arange(8 * 2 * 4).view(8, 2, 4)
    a, b = sharding.HeadShard(1, 4, 16, 8).weights(wk, wk + 100)
    assert torch.equal(a, wk[2:4]) and torch.equal(b, wk[2:4] + 100)
    q = torch.arange(2 * 16 * 3).view(2, 16, 3)
    assert torch.equal(sharding.HeadShard(1, 4, 16, 8).queries(q), q[:, 4:8])
    with pytest.raises(ValueError):
        sharding.HeadShard(0, 3, 32, 8)


def _partial(q, k, v, scale):
    """Unnormalised (O, m_log2, l) record as the engine emits it, from oracle math."""
    nh_q, d = q.shape
    g = nh_q // k.shape[1]
    out = torch.zeros(nh_q, sharding.PARTIAL_STRIDE)
    if k.shape[0] == 0:
        out[:, 128] = float("-inf")
        return out
    kk = k.float().repeat_interleave(g, dim=1)
    vv = v.float().repeat_interleave(g, dim=1)
    s = torch.einsum("hd,thd->ht", q.float(), kk) * scale * 1.4426950408889634
    m = s.max(dim=1).values
    p = torch.exp2(s - m[:, None])
    out[:, :128] = torch.einsum("ht,thd->hd", p, vv)
    out[:, 128] = m
    out[:, 129] = p.sum(dim=1)
    return out


def _gloo_worker(rank, world, port, n_tokens):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(5)                     # same tensors on every rank
        q = torch.randn(8, 128, generator=g).to(torch.bfloat16)
        k = torch.randn(n_tokens, 2, 128, generator=g).to(torch.bfloat16)
        v = torch.randn(n_tokens, 2, 128, generator=g).to(torch.bfloat16)
        scale = 128 ** -0.5
        s, e = sharding.plan_sequence_split(n_tokens, world, 16)[rank]
        part = _partial(q, k[s:e], v[s:e], scale)
        allp = sharding.all_gather_partials(part)
        assert allp.shape == (world, 8, sharding.PARTIAL_STRIDE)
        # merge (the algebra of merge_rank_partials_kernel) checked with the oracle's LSE merge
        m, l = allp[:, :, 128], allp[:, :, 129]
        lse = m * 0.6931471805599453 + torch.log(l)
        o_norm = allp[:, :, :128] / l.clamp_min(1e-38)[..., None]
        merged, _ = orc.lse_merge(o_norm, lse)
        full = orc.sdpa_decode(q, k, v, scale)
        assert torch.allclose(merged, full, atol=2e-5, rtol=1e-4), (merged - full).abs().max()
        # head sharding: outputs are disjoint head blocks
        sh = sharding.HeadShard(rank, world, 8, 2)
        o_local = orc.sdpa_decode(sh.queries(q[None])[0], sh.pool(k), sh.pool(v), scale)
        o_all = sharding.gather_head_outputs(o_local[None])
        assert torch.allclose(o_all[0], full, atol=2e-5, rtol=1e-4)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_tokens", [1000, 17])
def test_sequence_split_and_head_shard_over_gloo(n_tokens):
    mp.spawn(_gloo_worker, args=(2, _free_port(), n_tokens), nprocs=2, join=True)


# ---------------------------------------------------------------------------------------------------
# Failure detection, made on the host: a rank leaves BETWEEN steps (none of its collectives in flight).
# ---------------------------------------------------------------------------------------------------
def _leaving_worker(rank, world, port, store_port, results):
    from datetime import timedelta

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=5))
    store = dist.TCPStore("127.0.0.1", store_port, world, is_master=(rank == 0), timeout=timedelta(seconds=10))
    watch = sharding.PeerWatch(store, rank, world)
    part = torch.full((8, sharding.PARTIAL_STRIDE), float(rank))
    # step 0: everybody is there
    watch.beat(0)
    watch.require(0, timeout_s=5.0)
    allp = sharding.all_gather_partials(part)
    assert allp.shape[0] == world
    dist.barrier()
    if rank == 1:
        results.put((rank, "left after step 0"))
        os._exit(0)                                  # gone between steps; no collective of its own is pending
    # step 1: the watch reports the missing rank before anything is launched ...
    watch.beat(1)
    try:
        watch.require(1, timeout_s=0.5)
        results.put((rank, "watch saw nothing"))
    except RuntimeError as e:
        results.put((rank, "watch: " + str(e)))
    # ... and a rank that goes ahead anyway gets an error from the collective (short process-group timeout), not a hang
    try:
        sharding.all_gather_partials(part)
        results.put((rank, "collective returned"))
    except Exception as e:                            # gloo: connection closed by peer / timeout
        results.put((rank, "collective: " + type(e).__name__))
    os._exit(0)                                      # the group is broken: leave without the usual teardown


def test_a_rank_that_leaves_between_steps_is_noticed_on_the_host():
    ctx = mp.get_context("spawn")
    results = ctx.SimpleQueue()
    port, store_port = _free_port(), _free_port()
    procs = [ctx.Process(target=_leaving_worker, args=(r, 2, port, store_port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert not p.is_alive(), "a rank hung"
    got = {}
    while not results.empty():
        rank, msg = results.get()
        got.setdefault(rank, []).append(msg)
    assert got[1] == ["left after step 0"]
    assert any(m.startswith("watch: ") and "rank(s) [1]" in m and "step 1" in m for m in got[0]), got
    assert any(m.startswith("collective: ") for m in got[0]), got


def test_peer_watch_with_a_plain_store():
    """PeerWatch logic against an in-memory stand-in of the c10d store interface."""
    class Store:
        def __init__(self):
            self.d = {}

        def set(self, k, v):
            self.d[k] = v.encode() if isinstance(v, str) else v

        def get(self, k):
            return self.d[k]

        def check(self, keys):
            return all(k in self.d for k in keys)

    st = Store()
    w0, w1, w2 = (sharding.PeerWatch(st, r, 3) for r in range(3))
    w0.beat(4)
    w1.beat(4)
    assert w0.missing(4, timeout_s=0.05) == [2]
    w2.beat(5)                                       # a peer that is already a step ahead counts as present
    assert w0.missing(4, timeout_s=0.05) == []
    with pytest.raises(RuntimeError, match=r"rank\(s\) \[0, 1\] did not reach step 5"):
        w2.require(5, timeout_s=0.05)
