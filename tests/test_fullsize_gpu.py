"""GPU parity at the FULL sizes of the benchmark workloads.

The oracle cannot redo a whole multi-GB batch in test time, but it can redo single requests of it: every case
below runs the engine on the complete batch (projection of the new tokens, RoPE, write-back, streamed attention,
merge) and compares the LONGEST request, the shortest and two seeded random ones with the CPU oracle - the long
ones are those that span many warps and many partial records.  Workloads:

  * OPT-6.7B layer, 16 requests with context U[512, 8192], 16-token permuted pages (pool in HBM);
  * Llama-3-8B layer, 64 requests with lognormal context (median 8K, clipped to [256, 128K]), three steps with
    10 % of the requests replaced before each later step (pool in HBM);
  * OPT-30B layer shard, 7 of 56 heads, hidden 7168, 32 requests of 16K (pool in HBM);
  * Llama-3-8B layer, one request of 32K and one of 128K tokens streamed from a pool in pinned HOST memory;
  * the single-request steps of the short-step probes with the pool in HBM (Llama-3-8B 4K and 128K, OPT-6.7B 4K, two
    Llama requests): one or two new tokens go through the matrix-vector projection, a 128K request through the widest
    merge.
"""

import pytest
import torch

from dkv_testlib import KV_ATOL, assert_close, orc

pytestmark = pytest.mark.gpu

from directkv_b200 import kernel, workloads  # noqa: E402
from directkv_b200._lib import get_context  # noqa: E402

DEV = "cuda:0"
PAGE = 16


def _picks(lens, seed):
    order = sorted(range(len(lens)), key=lambda i: lens[i])
    picks = [order[-1], order[0]]
    g = torch.Generator().manual_seed(977 + seed)
    for i in torch.randperm(len(lens), generator=g).tolist():
        if i not in picks and len(picks) < min(4, len(lens)):
            picks.append(i)
    return picks


def _check_full_batch(shape, lens, cfg_id, kv_on_host, lid, what):
    case = workloads.make_decode_case(shape, lens, PAGE, cfg_id, DEV, kv_on_host=kv_on_host)
    ctx = get_context(0)
    kernel.register_layer(lid, case["k_pool"], case["v_pool"], case["wk"], case["wv"], case["cos_sin"], page_size=PAGE)
    k_cpu = case["k_pool"].cpu() if case["k_pool"].is_cuda else case["k_pool"].clone()     # before the step stores into it
    v_cpu = case["v_pool"].cpu() if case["v_pool"].is_cuda else case["v_pool"].clone()
    out = kernel.decode(lid, case["q"], case["seq_lens"], shape.scale, page_table=case["page_table"], x=case["x"])
    ctx.raise_on_status()
    cs = None if case["cos_sin"] is None else case["cos_sin"].cpu()
    wk, wv = case["wk"].cpu(), case["wv"].cpu()
    for i in _picks(lens, cfg_id):
        sub = [i]
        ref = orc.decode_layer(case["x"][sub].cpu(), wk, wv, case["q"][sub].cpu(), k_cpu, v_cpu,
                               case["page_table"][sub].cpu(), [lens[i]], PAGE, cs, shape.scale)      # stores the new row into k_cpu
        assert_close(out[i], ref[0], f"{what}: request {i} ({lens[i]} tokens)")
        slot = orc.token_slot(case["page_table"][i].tolist(), lens[i] - 1, PAGE)
        assert_close(case["k_pool"][slot].cpu(), k_cpu[slot], f"{what}: stored K row of request {i}", atol=KV_ATOL, rtol=1e-2)
        assert_close(case["v_pool"][slot].cpu(), v_cpu[slot], f"{what}: stored V row of request {i}", atol=KV_ATOL, rtol=1e-2)
    kernel.unregister_layer(lid)
    del case, out, k_cpu, v_cpu
    torch.cuda.empty_cache()


def test_opt67b_ragged_batch_full_size():
    lens = [n + 1 for n in workloads.ragged_lengths_uniform(16, 512, 8192, seed=4235)]
    _check_full_batch(workloads.OPT_6_7B, lens, 1, False, 70, "opt-6.7b 16 ragged")


def test_llama3_continuous_batch_full_size_with_churn():
    base = workloads.ragged_lengths_lognormal(64, 8192, 1.0, 256, 131072, seed=4234 + 3)
    g = torch.Generator().manual_seed(99)
    for step in range(3):
        if step:                                   # 10 % of the requests leave; new ones with fresh seeded lengths join
            fresh = workloads.ragged_lengths_lognormal(6, 8192, 1.0, 256, 131072, seed=4234 + 3 + 17 * step)
            for j, i in enumerate(torch.randperm(64, generator=g)[:6].tolist()):
                base[i] = fresh[j]
        _check_full_batch(workloads.LLAMA3_8B, [n + 1 for n in base], 3 + step, False, 71, f"llama3-8b 64 ragged, step {step}")


def test_opt30b_shard_full_size():
    _check_full_batch(workloads.OPT_30B.shard(8), [16385] * 32, 5, False, 72, "opt-30b shard 32 x 16K")


@pytest.mark.parametrize("ctx_len", [32768, 131072])
def test_llama3_long_request_from_a_host_pool(ctx_len):
    _check_full_batch(workloads.LLAMA3_8B, [ctx_len + 1], 2, True, 73, f"llama3-8b one request of {ctx_len} from host memory")


@pytest.mark.parametrize("shape,lens", [(workloads.LLAMA3_8B, [4097]), (workloads.LLAMA3_8B, [131073]),
                                        (workloads.OPT_6_7B, [4097]), (workloads.LLAMA3_8B, [16385, 4097])])
def test_single_request_steps_with_the_pool_in_hbm(shape, lens):
    _check_full_batch(shape, lens, 6, False, 74, f"{shape.name} short step {lens}")
