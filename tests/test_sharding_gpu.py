"""Two-GPU tests of head sharding and sequence split (NCCL); skipped on a single-GPU machine."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port):
    import sys

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from dkv_testlib import assert_close, orc
    from directkv_b200 import kernel, sharding, workloads
    from directkv_b200._lib import get_context

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        shape = workloads.LayerShape("t", 256, 8, 2, 10000.0)
        # ---- head sharding: full problem generated identically on every rank, each takes its heads ----
        lens = [5, 130, 1000, 64]
        full = workloads.make_decode_case(shape, lens, 16, 11, "cpu", kv_on_host=True)
        ref = orc.decode_layer(full["x"], full["wk"], full["wv"], full["q"], full["k_pool"].clone(), full["v_pool"].clone(),
                               full["page_table"], lens, 16, full["cos_sin"], shape.scale)
        sh = sharding.HeadShard(rank, world, shape.nh_q, shape.nh_kv)
        wk, wv = sh.weights(full["wk"], full["wv"])
        k_loc, v_loc = sh.pool(full["k_pool"]).pin_memory(), sh.pool(full["v_pool"]).pin_memory()
        kernel.register_layer(0, k_loc, v_loc, wk.to(dev), wv.to(dev), full["cos_sin"].to(dev), page_size=16, device=rank)
        out = kernel.decode(0, sh.queries(full["q"]).to(dev), full["seq_lens"].to(dev), shape.scale,
                            page_table=full["page_table"].to(dev), x=full["x"].to(dev))
        o_all = sharding.gather_head_outputs(out)
        get_context(rank).raise_on_status()
        assert_close(o_all, ref, f"head-sharded O (rank {rank})")
        # ---- sequence split: one request of 3000 tokens + the decoded one ----
        n = 3000
        one = workloads.make_decode_case(shape, [n + 1], 16, 12, "cpu", kv_on_host=True)
        ref1 = orc.decode_layer(one["x"], one["wk"], one["wv"], one["q"], one["k_pool"].clone(), one["v_pool"].clone(),
                                one["page_table"], [n + 1], 16, one["cos_sin"], shape.scale)
        plan = sharding.plan_sequence_split(n + 1, world, 16)
        owner = sharding.owner_of_new_token(plan)
        s, e = plan[rank]
        local_pages = one["page_table"][:, s // 16: -(-e // 16)].contiguous()
        kp, vp = one["k_pool"].pin_memory(), one["v_pool"].pin_memory()   # each rank reads only its own pages
        kernel.register_layer(1, kp, vp, one["wk"].to(dev), one["wv"].to(dev), one["cos_sin"].to(dev), page_size=16, device=rank)
        is_owner = rank == owner
        o = sharding.sequence_split_decode(
            1, one["q"].to(dev), torch.tensor([e - s], dtype=torch.int32, device=dev), shape.scale, local_pages.to(dev),
            x=one["x"].to(dev) if is_owner else None,
            pos_offset=torch.tensor([s], dtype=torch.int32, device=dev) if is_owner else None)
        get_context(rank).raise_on_status()
        assert_close(o, ref1, f"sequence-split O (rank {rank})")
        # ---- the same split with the exchange fused into the kernels (peer stores over NVLink, no NCCL call) ----
        ex = sharding.PartialExchange(max_rows=64, device=rank)
        lens_dev = torch.tensor([e - s], dtype=torch.int32, device=dev)
        off_dev = torch.tensor([s], dtype=torch.int32, device=dev)
        # 200 steps back to back with NO host synchronisation between them and a different query in each: a rank
        # may run a step ahead of its peer, so a record buffer that is reused too early, or a wait that lets a
        # later step's records through, shows up as a wrong output of some step.
        steps = 200
        g = torch.Generator().manual_seed(77)
        q_steps = torch.randn(steps, 1, shape.nh_q, 128, generator=g).to(torch.bfloat16)
        q_dev = q_steps.to(dev)
        outs = torch.empty(steps, 1, shape.nh_q, 128, dtype=torch.bfloat16, device=dev)
        x_dev = one["x"].to(dev) if is_owner else None
        pages_dev = local_pages.to(dev)
        for it in range(steps):
            kernel.decode(1, q_dev[it], lens_dev, shape.scale, page_table=pages_dev, x=x_dev,
                          pos_offset=off_dev if is_owner else None, out=outs[it], exchange=ex.handle)
        torch.cuda.synchronize()
        get_context(rank).raise_on_status()
        k_ref, v_ref = one["k_pool"].clone(), one["v_pool"].clone()
        for it in range(steps):
            ref_it = orc.decode_layer(one["x"], one["wk"], one["wv"], q_steps[it], k_ref, v_ref, one["page_table"], [n + 1],
                                      16, one["cos_sin"], shape.scale)
            assert_close(outs[it], ref_it, f"exchange O (rank {rank}, step {it} of {steps})")
        ex.close()
    finally:
        dist.destroy_process_group()


def test_two_gpu_head_shard_and_sequence_split():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    mp.spawn(_worker, args=(2, _free_port()), nprocs=2, join=True)
