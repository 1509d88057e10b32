"""Single-GPU tests of the peer-memory exchange: the one-rank case end to end, and the failure path - a
consumer whose peer never delivers runs into its (shortened) time limit, records that in the status word and
leaves the context usable.  Nothing here faults or hangs the GPU: the wait is bounded by design."""

import ctypes as C

import pytest
import torch

from dkv_testlib import assert_close, orc

pytestmark = pytest.mark.gpu

from directkv_b200 import _lib, kernel, sharding, workloads  # noqa: E402

DEV = "cuda:0"


def _pair(ctx, max_rows):
    lib = _lib.load()
    exs, bases = [], []
    for r in range(2):
        h = C.c_void_p()
        _lib.check(lib.dkv_exchange_create(ctx.handle, r, 2, max_rows, C.byref(h)))
        b = C.c_void_p()
        _lib.check(lib.dkv_exchange_base(h, C.byref(b)))
        exs.append(h)
        bases.append(b)
    _lib.check(lib.dkv_exchange_connect_ptr(exs[0], 1, bases[1]))
    _lib.check(lib.dkv_exchange_connect_ptr(exs[1], 0, bases[0]))
    return exs


def _split_case():
    shape = workloads.LayerShape("x", 128, 8, 2, None)
    n = 700
    case = workloads.make_decode_case(shape, [n], 16, 21, DEV)
    ref = orc.decode_layer(None, None, None, case["q"].cpu(), case["k_pool"].cpu(), case["v_pool"].cpu(),
                           case["page_table"].cpu(), [n], 16, None, shape.scale)
    plan = sharding.plan_sequence_split(n, 2, 16)
    return shape, case, ref, plan


def test_single_rank_exchange_matches_decode():
    """World size 1: producer and consumer of the same rank, three steps (cumulative counters).  The two-rank
    path needs two GPUs (tests/test_sharding_gpu.py): on one GPU a consumer kernel must never wait for a kernel
    launched after it."""
    ctx = _lib.get_context(0)
    shape, case, ref, plan = _split_case()
    kernel.register_layer(60, case["k_pool"], case["v_pool"], page_size=16)
    lib = _lib.load()
    h = C.c_void_p()
    _lib.check(lib.dkv_exchange_create(ctx.handle, 0, 1, 16, C.byref(h)))
    for step in range(3):
        lse = torch.empty(8, dtype=torch.float32, device=DEV)
        o = kernel.decode(60, case["q"], case["seq_lens"], shape.scale, page_table=case["page_table"], exchange=h,
                          lse_out=lse)
        ctx.raise_on_status()
        assert_close(o, ref, f"world-1 exchange step {step}")
    # 40 more steps without host synchronisation and with a different query each: consecutive steps alternate
    # between the two halves of the record buffer and carry their own sequence number.
    g = torch.Generator().manual_seed(5)
    qs = torch.randn(40, 1, 8, 128, generator=g).to(torch.bfloat16)
    qd, outs = qs.to(DEV), torch.empty(40, 1, 8, 128, dtype=torch.bfloat16, device=DEV)
    for i in range(40):
        kernel.decode(60, qd[i], case["seq_lens"], shape.scale, page_table=case["page_table"], exchange=h, out=outs[i])
    ctx.raise_on_status()
    for i in range(40):
        ref_i = orc.decode_layer(None, None, None, qs[i], case["k_pool"].cpu(), case["v_pool"].cpu(),
                                 case["page_table"].cpu(), [700], 16, None, shape.scale)
        assert_close(outs[i], ref_i, f"world-1 exchange, unsynchronised step {i}")
    with pytest.raises(RuntimeError, match="max_rows"):
        q_big = torch.zeros(3, 8 * 128, dtype=torch.bfloat16, device=DEV)
        kernel.decode(60, q_big, torch.ones(3, dtype=torch.int32, device=DEV), shape.scale,
                      page_table=case["page_table"].expand(3, -1).contiguous(), exchange=h)
    lib.dkv_exchange_destroy(h)
    kernel.unregister_layer(60)


def test_consumer_times_out_when_a_peer_never_delivers():
    ctx = _lib.get_context(0)
    shape, case, ref, plan = _split_case()
    kernel.register_layer(61, case["k_pool"], case["v_pool"], page_size=16)
    exs = _pair(ctx, 16)
    ctx.set("wait_limit_ms", 150)
    s, e = plan[0]
    lens = torch.tensor([e - s], dtype=torch.int32, device=DEV)
    pages = case["page_table"][:, s // 16: -(-e // 16)].contiguous()
    kernel.decode(61, case["q"], lens, shape.scale, page_table=pages, exchange=exs[0])   # rank 1 never calls
    st = ctx.read_status(clear=True)
    assert st & 1, f"expected the wait-timeout bit, got status {st:#x}"
    ctx.set("wait_limit_ms", 2000)
    # the context is still usable: an ordinary decode gives the right answer
    o = kernel.decode(61, case["q"], case["seq_lens"], shape.scale, page_table=case["page_table"])
    ctx.raise_on_status()
    assert_close(o, ref, "decode after the timeout")
    for x in exs:
        _lib.load().dkv_exchange_destroy(x)
    kernel.unregister_layer(61)
