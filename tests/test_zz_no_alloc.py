"""GPU test of dkv_decode_noalloc, the entry point for callers that may not allocate device memory
(graph-capture regions, serving loops with a frozen memory plan, hosts that forbid cudaMalloc in
plugins).  It is called through the C ABI twice in a row on different inputs - the scratch it uses
is one fixed array inside the library that keeps the previous call's contents - and each result is
compared with the regular entry point (dkv_decode, attention over tokens already in the pool)
and with the CPU oracle, within the suite's output tolerance.  The file sorts last so that a run
which stops at the first failure has already run every other test; it also passes alone in a fresh
process, because the entry point does its own per-device set-up and needs no context.
"""

import pytest
import torch

from dkv_testlib import assert_close, orc

pytestmark = pytest.mark.gpu

from directkv_b200 import kernel, workloads  # noqa: E402
from directkv_b200._lib import get_context  # noqa: E402

DEV = "cuda:0"


def _reference_entry_point(case, shape, page_size, lid):
    kernel.register_layer(lid, case["k_pool"], case["v_pool"], page_size=page_size)
    out = kernel.decode(lid, case["q"], case["seq_lens"], shape.scale, page_table=case["page_table"])
    get_context(0).raise_on_status()
    kernel.unregister_layer(lid)
    return out


@pytest.mark.parametrize("nh_q,nh_kv,kv_on_host", [(8, 8, True), (8, 2, False), (6, 3, True)])
def test_no_alloc_matches_regular_entry_point_twice(nh_q, nh_kv, kv_on_host):
    shape = workloads.LayerShape("na", 128, nh_q, nh_kv, None)
    first = workloads.make_decode_case(shape, [1, 16, 17, 300, 1500, 64], 16, 71, DEV, kv_on_host=kv_on_host)
    second = workloads.make_decode_case(shape, [900, 2, 33], 16, 72, DEV, kv_on_host=kv_on_host)
    mem_before = None
    for i, case in enumerate((first, second)):
        out = torch.empty_like(case["q"])
        torch.cuda.synchronize()
        if i == 1:
            mem_before = torch.cuda.mem_get_info()[0]      # after the one-time set-up of the first call
        kernel.decode_noalloc(case["k_pool"], case["v_pool"], case["q"], out, case["seq_lens"], case["page_table"],
                              16, shape.scale, sync_and_check=True)
        if i == 1:
            assert torch.cuda.mem_get_info()[0] == mem_before, "the call changed the amount of free device memory"
        ref = _reference_entry_point(case, shape, 16, 90 + i)
        assert_close(out, ref, f"call {i + 1}")
        lens = case["seq_lens"].tolist()
        oracle = orc.decode_layer(None, None, None, case["q"].cpu(), case["k_pool"].cpu(), case["v_pool"].cpu(),
                                  case["page_table"].cpu(), lens, 16, None, shape.scale)
        assert_close(out, oracle, f"call {i + 1} against the oracle")


def test_no_alloc_reports_device_side_trouble_in_the_callers_word():
    """Without sync_and_check the caller's own status word receives the failure bits: here a length that leads
    outside the page table (nothing outside the table is read; the call itself still returns DKV_OK)."""
    shape = workloads.LayerShape("na", 128, 4, 4, None)
    case = workloads.make_decode_case(shape, [40, 200], 16, 73, DEV, kv_on_host=False)
    out = torch.empty_like(case["q"])
    word = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernel.decode_noalloc(case["k_pool"], case["v_pool"], case["q"], out, case["seq_lens"], case["page_table"],
                          16, shape.scale, status_out=word)
    assert int(word.item()) == 0
    too_long = case["seq_lens"].clone()
    too_long[0] = case["page_table"].size(1) * 16 + 5
    kernel.decode_noalloc(case["k_pool"], case["v_pool"], case["q"], out, too_long, case["page_table"],
                          16, shape.scale, status_out=word)
    assert int(word.item()) & (1 << 5), f"expected the bad-page bit, got {int(word.item()):#x}"


def test_no_alloc_rejects_sizes_beyond_its_scratch():
    shape = workloads.LayerShape("na", 128, 32, 32, None)
    big = 400                                   # 32 MHA heads: the built-in scratch covers batch <= 173
    pool = torch.zeros(64, 32, 128, dtype=torch.bfloat16, device=DEV)
    q = torch.zeros(big, 32, 128, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError, match="built-in scratch"):
        kernel.decode_noalloc(pool, pool, q, torch.empty_like(q), torch.ones(big, dtype=torch.int32, device=DEV),
                              torch.ones(big, 1, dtype=torch.int32, device=DEV), 16, shape.scale)
    if torch.cuda.device_count() > 1:           # a pool that lives on another GPU is refused
        other = torch.zeros(64, 32, 128, dtype=torch.bfloat16, device="cuda:1")
        q1 = torch.zeros(1, 32, 128, dtype=torch.bfloat16, device=DEV)
        with pytest.raises(RuntimeError, match="lives on device"):
            kernel.decode_noalloc(other, other, q1, torch.empty_like(q1), torch.ones(1, dtype=torch.int32, device=DEV),
                                  torch.ones(1, 1, dtype=torch.int32, device=DEV), 16, shape.scale)
    with pytest.raises(RuntimeError, match="multiple of nh_kv"):
        q3 = torch.zeros(1, 3, 128, dtype=torch.bfloat16, device=DEV)
        kernel.decode_noalloc(pool[:, :2].contiguous(), pool[:, :2].contiguous(), q3, torch.empty_like(q3),
                              torch.ones(1, dtype=torch.int32, device=DEV),
                              torch.ones(1, 1, dtype=torch.int32, device=DEV), 16, shape.scale)
