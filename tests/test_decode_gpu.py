"""GPU parity of the decode path (dkv_decode through the C ABI) against the CPU oracle."""

import math

import pytest
import torch

from dkv_testlib import KV_ATOL, assert_close, orc

pytestmark = pytest.mark.gpu

from directkv_b200 import kernel, workloads  # noqa: E402
from directkv_b200._lib import PARTIAL_STRIDE, get_context  # noqa: E402

DEV = "cuda:0"


def _shape(hidden, nh_q, nh_kv, rope=True):
    return workloads.LayerShape(f"t{hidden}-{nh_q}-{nh_kv}", hidden, nh_q, nh_kv, 10000.0 if rope else None)


def _run_decode(shape, seq_lens, page_size, cfg_id, kv_on_host=True, mode="project", variant=-1, lid=7, mma=-1):
    case = workloads.make_decode_case(shape, seq_lens, page_size, cfg_id, DEV, kv_on_host=kv_on_host)
    k_ref, v_ref = case["k_pool"].cpu().clone(), case["v_pool"].cpu().clone()
    k_before = k_ref.clone()
    ctx = get_context(0)
    ctx.set("attn_variant", variant)
    ctx.set("attn_mma", mma)
    kernel.register_layer(lid, case["k_pool"], case["v_pool"], case["wk"], case["wv"], case["cos_sin"],
                          page_size=page_size)
    cs_cpu = None if case["cos_sin"] is None else case["cos_sin"].cpu()
    kw = {}
    if mode == "project":
        kw["x"] = case["x"]
        ref = orc.decode_layer(case["x"].cpu(), case["wk"].cpu(), case["wv"].cpu(), case["q"].cpu(), k_ref, v_ref,
                               case["page_table"].cpu(), seq_lens, page_size, cs_cpu, shape.scale)
    elif mode == "given":
        kn, vn = orc.project_kv(case["x"].cpu(), case["wk"].cpu(), case["wv"].cpu())
        kw["k_new"], kw["v_new"] = kn.to(DEV), vn.to(DEV)
        ref = orc.decode_layer(None, None, None, case["q"].cpu(), k_ref, v_ref, case["page_table"].cpu(), seq_lens,
                               page_size, None, shape.scale, k_new=kn, v_new=vn)
    else:
        ref = orc.decode_layer(None, None, None, case["q"].cpu(), k_ref, v_ref, case["page_table"].cpu(), seq_lens,
                               page_size, None, shape.scale)
    out = kernel.decode(lid, case["q"], case["seq_lens"], shape.scale, page_table=case["page_table"], **kw)
    ctx.raise_on_status()
    assert_close(out, ref.view_as(out), "O")
    ctx.set("attn_variant", -1)
    ctx.set("attn_mma", -1)
    if mode != "none":
        # Stored K/V of the new token: within the reference's write-back threshold; every other slot untouched.
        k_now, v_now = case["k_pool"].cpu(), case["v_pool"].cpu()
        touched = torch.zeros(k_now.shape[0], dtype=torch.bool)
        for b, sl in enumerate(seq_lens):
            slot = orc.token_slot(case["page_table"][b].tolist(), sl - 1, page_size)
            touched[slot] = True
            assert_close(k_now[slot], k_ref[slot], f"K write-back req {b}", atol=KV_ATOL, rtol=RTOL_KV)
            assert_close(v_now[slot], v_ref[slot], f"V write-back req {b}", atol=KV_ATOL, rtol=RTOL_KV)
        assert torch.equal(k_now[~touched], k_before[~touched]), "past K slots must be bit-identical"
    kernel.unregister_layer(lid)
    return out


RTOL_KV = 1e-2


@pytest.mark.parametrize("nh_q,nh_kv", [(4, 4), (8, 2), (6, 3), (7, 7), (8, 1), (12, 2)])
def test_head_groupings(nh_q, nh_kv):
    _run_decode(_shape(256, nh_q, nh_kv), [1, 2, 17, 40, 129, 300], 16, cfg_id=1)


@pytest.mark.parametrize("nh_q,nh_kv,variant", [(16, 1, 0), (16, 1, 2), (32, 1, 1), (9, 3, 2), (5, 1, 0), (28, 2, 1),
                                                (4, 4, 2), (8, 4, 0)])
def test_tensor_core_inner_product(nh_q, nh_kv, variant):
    """The mma form of the streaming kernel: 1..16 query rows per KV head pass (32 -> two passes of 16,
    28 per 2 -> 14 rows), forced on for the groupings the automatic choice leaves to the CUDA-core form."""
    _run_decode(_shape(128, nh_q, nh_kv), [1, 2, 16, 17, 40, 129, 300, 1025], 16, cfg_id=11, variant=variant, mma=1)


@pytest.mark.parametrize("page_size", [1, 4, 8, 16, 64])
@pytest.mark.parametrize("host", [True, False])
def test_tensor_core_inner_product_page_sizes(page_size, host):
    _run_decode(_shape(128, 8, 2), [1, 5, 16, 31, 64, 65, 200, 333], page_size, cfg_id=12, kv_on_host=host, mma=1)


def test_forms_of_the_streaming_kernel_agree():
    """Same inputs through the CUDA-core and the tensor-core form: outputs differ only by the bf16 rounding of
    the probabilities."""
    a = _run_decode(_shape(128, 8, 2), [700, 64, 3, 2048], 16, cfg_id=13, mma=0)
    b = _run_decode(_shape(128, 8, 2), [700, 64, 3, 2048], 16, cfg_id=13, mma=1)
    assert (a.float() - b.float()).abs().max().item() < 1e-2


@pytest.mark.parametrize("batch", [1, 15, 16, 17, 33, 64, 65, 128, 129, 257, 512, 513])
@pytest.mark.parametrize("hidden", [64, 320, 4096])
def test_projection_batch_sizes(batch, hidden):
    """Decode batches on both projection kernels: up to 512 tokens the swapped-operand kernel (tokens on the
    N side in chunks of up to 128, 16..128 padded columns, split-K per KV head and chunk), above that the
    128-token-tile kernel."""
    lens = [1 + (7 * i) % 40 for i in range(batch)]
    ctx = get_context(0)
    for flag in (1, 0):                      # 1: swapped-operand kernel whenever the batch fits; 0: never
        ctx.set("proj_decode", flag)
        try:
            _run_decode(_shape(hidden, 4, 2), lens, 16, cfg_id=20 + batch)
        finally:
            ctx.set("proj_decode", -1)


def test_projection_kernels_agree():
    ctx = get_context(0)
    outs = []
    for flag in (0, 1):
        ctx.set("proj_decode", flag)
        outs.append(_run_decode(_shape(1024, 8, 4), [30, 1, 17, 64, 5], 16, cfg_id=77))
    ctx.set("proj_decode", -1)
    assert (outs[0].float() - outs[1].float()).abs().max().item() < 1e-2


def test_long_single_request_merge():
    """One long request: every warp of the streaming grid leaves a partial record for the same few rows, which
    the merge kernel folds with eight warps per row."""
    _run_decode(_shape(128, 8, 2), [40000], 16, cfg_id=30, kv_on_host=False)
    _run_decode(_shape(128, 2, 2), [25000, 3], 16, cfg_id=31, kv_on_host=False, mma=0)


@pytest.mark.parametrize("page_size", [1, 2, 4, 8, 16, 32, 64])
def test_page_sizes(page_size):
    _run_decode(_shape(128, 4, 2), [1, 5, 16, 31, 64, 65, 200, 333], page_size, cfg_id=2)


@pytest.mark.parametrize("variant", [0, 1, 2])
def test_kernel_variants(variant):
    _run_decode(_shape(128, 8, 4), [3, 100, 257, 1000, 48, 16], 16, cfg_id=3, variant=variant)


@pytest.mark.parametrize("mode", ["project", "given", "none"])
def test_new_token_modes(mode):
    _run_decode(_shape(192, 4, 4, rope=(mode == "project")), [9, 77, 130, 16, 1 if mode != "none" else 2], 16,
                cfg_id=4, mode=mode)


def test_hbm_resident_pool():
    _run_decode(_shape(256, 8, 8, rope=False), [700, 64, 1, 15, 2048], 16, cfg_id=5, kv_on_host=False)


def test_config1_llama3_8b_layer():
    """Llama-3-8B layer, batch 1, 4096 cached tokens + the decoded one, RoPE theta 5e5."""
    _run_decode(workloads.LLAMA3_8B, [4097], 16, cfg_id=0)


def test_config2_shape_opt67b_ragged_small():
    """OPT-6.7B geometry (32 MHA heads, hidden 4096, 16-token permuted pages, 16 ragged requests) at short lengths."""
    lens = workloads.ragged_lengths_uniform(16, 8, 300, seed=4235)
    _run_decode(workloads.OPT_6_7B, lens, 16, cfg_id=1)


def test_config5_shape_opt30b_shard():
    """OPT-30B geometry on one GPU of eight: 7 MHA heads, hidden 7168."""
    _run_decode(workloads.OPT_30B.shard(8), [513, 1024, 37], 16, cfg_id=5)


def test_contiguous_rows_and_row_map():
    """Request-pool layout: slot = row * row_stride + position, with a row map."""
    shape = _shape(128, 4, 2)
    rows, s_pad = 5, 256
    g = torch.Generator().manual_seed(11)
    k_pool = (torch.randn(rows, s_pad, 2, 128, generator=g) * 0.5).to(torch.bfloat16).pin_memory()
    v_pool = (torch.randn(rows, s_pad, 2, 128, generator=g) * 0.5).to(torch.bfloat16).pin_memory()
    seq_lens = [200, 1, 64]
    row_map = [4, 0, 2]
    q = (torch.randn(3, 4, 128, generator=g)).to(torch.bfloat16)
    kn = (torch.randn(3, 2, 128, generator=g) * 0.5).to(torch.bfloat16)
    vn = (torch.randn(3, 2, 128, generator=g) * 0.5).to(torch.bfloat16)
    k_ref, v_ref = k_pool.clone().view(-1, 2, 128), v_pool.clone().view(-1, 2, 128)
    table = torch.tensor([[r * s_pad + t for t in range(s_pad)] for r in row_map], dtype=torch.int32)
    ref = orc.decode_layer(None, None, None, q, k_ref, v_ref, table, seq_lens, 1, None, shape.scale, k_new=kn, v_new=vn)
    kernel.register_layer(21, k_pool, v_pool, row_stride=s_pad)
    out = kernel.decode(21, q.to(DEV), torch.tensor(seq_lens, dtype=torch.int32, device=DEV), shape.scale,
                        row_map=torch.tensor(row_map, dtype=torch.int32, device=DEV), k_new=kn.to(DEV), v_new=vn.to(DEV))
    get_context(0).raise_on_status()
    assert_close(out, ref, "O")
    for b, (r, sl) in enumerate(zip(row_map, seq_lens)):
        assert torch.equal(k_pool[r, sl - 1], kn[b]) and torch.equal(v_pool[r, sl - 1], vn[b])
    kernel.unregister_layer(21)


def test_lse_and_sequence_split_merge():
    """Sequence split emulated on one GPU: two token ranges of one request produce unnormalised
    partials whose merge equals attention over the whole range (and the LSE matches)."""
    shape = _shape(128, 8, 2, rope=False)
    total = 1000
    case = workloads.make_decode_case(shape, [total], 16, 9, DEV)
    kernel.register_layer(31, case["k_pool"], case["v_pool"], page_size=16)
    q = case["q"]
    ref, lse_ref = orc.decode_layer(None, None, None, q.cpu(), case["k_pool"].cpu(), case["v_pool"].cpu(),
                                    case["page_table"].cpu(), [total], 16, None, shape.scale, return_lse=True)
    lse = torch.empty(1, 8, dtype=torch.float32, device=DEV)
    out = kernel.decode(31, q, case["seq_lens"], shape.scale, page_table=case["page_table"], lse_out=lse)
    assert_close(out, ref, "O")
    assert_close(lse, lse_ref, "LSE", atol=2e-3, rtol=1e-3)
    split = 512  # page aligned
    parts = torch.zeros(2, 8, PARTIAL_STRIDE, dtype=torch.float32, device=DEV)
    lens0 = torch.tensor([split], dtype=torch.int32, device=DEV)
    lens1 = torch.tensor([total - split], dtype=torch.int32, device=DEV)
    kernel.decode(31, q, lens0, shape.scale, page_table=case["page_table"], partial_out=parts[0], normalized=False)
    kernel.decode(31, q, lens1, shape.scale, page_table=case["page_table"][:, split // 16:].contiguous(),
                  partial_out=parts[1], normalized=False)
    lse2 = torch.empty(8, dtype=torch.float32, device=DEV)
    merged = kernel.merge_partials(parts, lse_out=lse2)
    get_context(0).raise_on_status()
    assert_close(merged.view(1, 8, 128), ref, "merged O")
    assert_close(lse2.view(1, 8), lse_ref, "merged LSE", atol=2e-3, rtol=1e-3)
    kernel.unregister_layer(31)


def test_larger_ragged_batch_balance():
    """64 requests with very uneven lengths (lognormal), GQA 4:1: exercises the even split of tiles over warps."""
    lens = workloads.ragged_lengths_lognormal(64, 600, 1.0, 1, 6000, seed=4238)
    _run_decode(_shape(128, 8, 2), lens, 16, cfg_id=6)


def test_config2_full_size_properties():
    """The OPT-6.7B ragged batch at its full size (16 requests, ctx U[512,8192], 32 MHA heads, 16-token pages, about
    1 GB of KV, pool in HBM), checked through properties that hold for every request at once (the comparison of
    single requests with the oracle at this size is tests/test_fullsize_gpu.py):
      * doubling V doubles O bit-exactly (powers of two are exact in bf16 and fp32);
      * moving every page to another slot (a different permutation of the same logical contents) leaves O
        bit-identical: tiles, their order and every rounding point are the same;
      * the two shortest requests agree with the oracle."""
    shape = workloads.OPT_6_7B
    lens = [n + 1 for n in workloads.ragged_lengths_uniform(16, 512, 8192, seed=4235)]
    page = 16
    case = workloads.make_decode_case(shape, lens, page, 1, DEV, kv_on_host=False)
    q, sl, table = case["q"], case["seq_lens"], case["page_table"]
    kernel.register_layer(61, case["k_pool"], case["v_pool"], page_size=page)
    out1 = kernel.decode(61, q, sl, shape.scale, page_table=table).clone()
    get_context(0).raise_on_status()

    short = sorted(range(len(lens)), key=lambda i: lens[i])[:2]
    ref = orc.decode_layer(None, None, None, q[short].cpu(), case["k_pool"].cpu(), case["v_pool"].cpu(),
                           table[short].cpu(), [lens[i] for i in short], page, None, shape.scale)
    assert_close(out1[short], ref.view_as(out1[short]), "O of the two shortest requests")

    case["v_pool"].mul_(2)
    out2 = kernel.decode(61, q, sl, shape.scale, page_table=table).clone()
    assert torch.equal(out2.float(), out1.float() * 2), "O must double bit-exactly with V"
    case["v_pool"].mul_(0.5)
    kernel.unregister_layer(61)

    # Same logical cache under another page permutation.
    n_pages = case["k_pool"].shape[0] // page
    g = torch.Generator().manual_seed(99)
    perm = torch.cat([torch.zeros(1, dtype=torch.long), torch.randperm(n_pages - 1, generator=g) + 1]).to(DEV)  # page 0 stays reserved
    k2 = torch.empty_like(case["k_pool"]).view(n_pages, page, shape.nh_kv, 128)
    v2 = torch.empty_like(case["v_pool"]).view(n_pages, page, shape.nh_kv, 128)
    k2[perm] = case["k_pool"].view(n_pages, page, shape.nh_kv, 128)
    v2[perm] = case["v_pool"].view(n_pages, page, shape.nh_kv, 128)
    table2 = perm[table.long()].to(torch.int32)
    kernel.register_layer(62, k2.view(-1, shape.nh_kv, 128), v2.view(-1, shape.nh_kv, 128), page_size=page)
    out3 = kernel.decode(62, q, sl, shape.scale, page_table=table2)
    get_context(0).raise_on_status()
    assert torch.equal(out3, out1), "O must not depend on where the pages live"
    kernel.unregister_layer(62)


def test_lengths_and_rows_that_lead_outside_the_page_table_are_reported_not_read():
    """seq_lens and row_map are device data the host never sees.  A length beyond the table's width, or a row beyond its
    rows, sets DKV_STATUS_BAD_PAGE (bit 5): the nearest entry is read instead (the request's output is then wrong, by
    construction), the new token of such a request is not stored, nothing outside the table is touched, and the context
    stays usable."""
    ctx = get_context(0)
    shape = _shape(128, 4, 4, rope=False)
    lens = [40, 200, 33]
    case = workloads.make_decode_case(shape, lens, 16, 77, DEV, kv_on_host=False)
    kernel.register_layer(64, case["k_pool"], case["v_pool"], case["wk"], case["wv"], None, page_size=16)
    good = kernel.decode(64, case["q"], case["seq_lens"], shape.scale, page_table=case["page_table"], save_kv_cache=False,
                         x=case["x"]).clone()
    assert ctx.read_status(clear=True) == 0
    k_before = case["k_pool"].clone()
    too_long = case["seq_lens"].clone()
    too_long[0] = case["page_table"].size(1) * 16 + 7                      # one page more than the table is wide
    out = kernel.decode(64, case["q"], too_long, shape.scale, page_table=case["page_table"], x=case["x"])
    st = ctx.read_status(clear=True)
    assert st & (1 << 5), f"expected the bad-page bit, got {st:#x}"
    assert torch.equal(out[1:], good[1:]), "the other requests are not affected"
    rows = torch.tensor([0, 7, 2], dtype=torch.int32, device=DEV)          # row 7 of a three-row table
    kernel.decode(64, case["q"], case["seq_lens"], shape.scale, page_table=case["page_table"], row_map=rows,
                  save_kv_cache=False, x=case["x"])
    st = ctx.read_status(clear=True)
    assert st & (1 << 5), f"expected the bad-page bit, got {st:#x}"
    # request 0 of the first bad call was not stored; requests 1 and 2 were
    changed = (case["k_pool"] != k_before).flatten(1).any(dim=1).nonzero().flatten().tolist()
    want = sorted(orc.token_slot(case["page_table"][b].tolist(), lens[b] - 1, 16) for b in (1, 2))
    assert changed == want, (changed, want)
    again = kernel.decode(64, case["q"], case["seq_lens"], shape.scale, page_table=case["page_table"], save_kv_cache=False,
                          x=case["x"])
    ctx.raise_on_status()
    assert torch.equal(again, good)
    kernel.unregister_layer(64)


@pytest.mark.parametrize("shape,lens", [(workloads.LLAMA3_8B, [300]), (workloads.LLAMA3_8B, [77, 1041]),
                                        (workloads.OPT_6_7B, [513]), (_shape(7168, 14, 7), [40, 2]),
                                        (_shape(1024, 4, 4, rope=False), [1, 130])])
def test_matrix_vector_projection_against_the_oracle_and_the_tensor_core_kernel(shape, lens):
    """One or two new tokens into a pool in HBM are projected by the matrix-vector kernel (proj_gemv = 1, default),
    larger batches and host pools by a tensor-core kernel.  Both forms: outputs, the stored K/V rows and the untouched
    slots against the oracle; the outputs of the two forms agree within the tolerance (the fp32 sums run in another
    order); each form gives the same bits when the same step runs twice."""
    ctx = get_context(0)
    outs = {}
    for gemv in (1, 0):
        ctx.set("proj_gemv", gemv)
        try:
            outs[gemv] = _run_decode(shape, lens, 16, cfg_id=5, kv_on_host=False, lid=66).clone()
            again = _run_decode(shape, lens, 16, cfg_id=5, kv_on_host=False, lid=66)
        finally:
            ctx.set("proj_gemv", 1)
        assert torch.equal(outs[gemv], again), f"gemv={gemv}: two runs of the same step differ"
    assert_close(outs[1], outs[0].float(), "matrix-vector against tensor-core projection")


def test_streaming_and_projection_kernels_fit_one_sm_together():
    """The decode projection runs under the 16-warp streaming kernels only while one CTA of each fits an SM's
    registers and shared memory at once (512 x 104 + 128 x 96 registers fill the file exactly); the library checks it
    from the compiled kernels' own attributes."""
    get_context(0).set("check_coresidency", 1)


def test_scratch_growth_is_refused_under_capture_and_allowed_outside():
    """A call recorded into a CUDA graph may not allocate: when its scratch need exceeds what the context holds, the
    entry point says so (size it with dkv_context_reserve or an eager call first) instead of calling cudaMalloc under
    capture; the same call outside capture grows the scratch and works."""
    shape = _shape(128, 8, 8, rope=False)
    big = 200000                                    # 200,000 short requests: about 850 MB of partial records
    pool = torch.zeros(64, 8, 128, dtype=torch.bfloat16, device=DEV)
    pool[16:32] = 1.0
    kernel.register_layer(63, pool, pool.clone(), page_size=16)
    q = torch.ones(big, 8, 128, dtype=torch.bfloat16, device=DEV)
    lens = torch.full((big,), 5, dtype=torch.int32, device=DEV)
    table = torch.ones(big, 1, dtype=torch.int32, device=DEV)
    out = torch.empty_like(q)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with pytest.raises(RuntimeError, match="before capturing"):
        with torch.cuda.graph(g):
            kernel.decode(63, q, lens, shape.scale, page_table=table, out=out)
    torch.cuda.synchronize()
    kernel.decode(63, q, lens, shape.scale, page_table=table, out=out)          # eager: grows, then runs
    get_context(0).raise_on_status()
    assert torch.equal(out.float(), torch.ones_like(out).float()), "attention over five identical rows returns that row"
    kernel.unregister_layer(63)


def test_dma_staged_decode_matches_streaming():
    """Request-pool layout in pinned host memory: the past rows copied to HBM by cudaMemcpyAsync and attended there
    give the same bits as streaming them from the host pool (same 16-token tiles in the same order), and the new
    token lands in the host pool either way."""
    from directkv_b200.staging import DmaStagedDecode

    shape = _shape(256, 8, 2)
    rows_total, s_pad = 5, 512
    g = torch.Generator().manual_seed(123)
    K = (torch.randn(rows_total, s_pad, 2, 128, generator=g) * 0.5).to(torch.bfloat16)
    V = (torch.randn(rows_total, s_pad, 2, 128, generator=g) * 0.5).to(torch.bfloat16)
    wk = (torch.randn(2, 128, 256, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    wv = (torch.randn(2, 128, 256, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    cs = orc.build_cos_sin(s_pad, 128, 10000.0).to(DEV)
    lens, rows = [200, 1, 65, 333], [4, 0, 2, 1]
    q = torch.randn(4, 8 * 128, generator=g).to(torch.bfloat16).to(DEV)
    x = torch.randn(4, 256, generator=g).to(torch.bfloat16).to(DEV)
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    rm = torch.tensor(rows, dtype=torch.int32, device=DEV)
    outs, pools = [], []
    # The copy lives in HBM, where four query heads per KV head would pick the tensor-core form of the streaming
    # kernel and short steps give each warp several tiles; with both switched off the two runs execute the same
    # arithmetic in the same order.
    get_context(0).set("attn_mma", 0)
    get_context(0).set("attn_min_units", 1)
    for staged in (False, True, True):
        if len(outs) == 2:
            get_context(0).set("attn_mma", -1)
            get_context(0).set("attn_min_units", 8)
        Kp, Vp = K.clone().pin_memory(), V.clone().pin_memory()
        kernel.register_layer(81, Kp, Vp, wk, wv, cs, row_stride=s_pad)
        if staged:
            st = DmaStagedDecode(torch.device(DEV), 2)
            o = st.decode(81, Kp, Vp, rows, lens, q, sl, shape.scale, rm, x=x)
        else:
            o = kernel.decode(81, q, sl, shape.scale, row_map=rm, x=x)
        torch.cuda.synchronize()
        get_context(0).raise_on_status()
        outs.append(o.clone())
        pools.append((Kp.clone(), Vp.clone()))
        kernel.unregister_layer(81)
    assert torch.equal(outs[0], outs[1])
    assert (outs[2].float() - outs[0].float()).abs().max().item() < 1e-2           # tensor-core form on the copy
    assert torch.equal(pools[0][0], pools[1][0]) and torch.equal(pools[0][1], pools[1][1])
    assert torch.equal(pools[0][0], pools[2][0])
    for b, (r, n) in enumerate(zip(rows, lens)):
        assert not torch.equal(pools[1][0][r, n - 1], K[r, n - 1])      # the new token was written to the host pool


@pytest.mark.parametrize("seed", range(24))
def test_randomised_configurations(seed):
    """Seeded random draws over head groupings, page sizes, batch sizes, lengths, where the pool lives, how the new
    token arrives and which forms of the kernels run; every draw is compared with the oracle."""
    import random

    rnd = random.Random(9000 + seed)
    nh_kv = rnd.choice([1, 2, 3, 4, 8])
    g = rnd.choice([1, 1, 2, 3, 4, 6, 8, 16])
    hidden = rnd.choice([64, 192, 512, 1024])
    page = rnd.choice([1, 2, 4, 8, 16, 32, 64])
    batch = rnd.choice([1, 2, 3, 7, 16, 40])
    hi = rnd.choice([20, 100, 700, 3000])
    lens = [rnd.randint(1, hi) for _ in range(batch)]
    mode = rnd.choice(["project", "project", "given", "none"])
    if mode == "none":
        lens = [max(2, n) for n in lens]
    ctx = get_context(0)
    ctx.set("proj_decode", rnd.choice([-1, 0, 1]))
    try:
        _run_decode(_shape(hidden, nh_kv * g, nh_kv, rope=(mode == "project" and rnd.random() < 0.7)), lens, page,
                    cfg_id=300 + seed, kv_on_host=rnd.random() < 0.5, mode=mode, variant=rnd.choice([-1, 0, 1, 2]),
                    mma=rnd.choice([-1, -1, 0, 1]) if g <= 16 else -1)
    finally:
        ctx.set("proj_decode", -1)


@pytest.mark.parametrize("seed", range(16))
def test_matrix_vector_projection_randomised(seed):
    """Seeded random draws of the shapes the matrix-vector projection takes (one or two requests, hidden size a
    multiple of 1024, pool in HBM): head counts, groupings, page sizes, lengths, with and without RoPE, every form of
    the streaming kernel; each compared with the oracle (output, stored rows, untouched slots)."""
    import random

    rnd = random.Random(7100 + seed)
    nh_kv = rnd.choice([1, 2, 3, 5, 8])
    g = rnd.choice([1, 1, 2, 4, 7, 8])
    hidden = rnd.choice([1024, 2048, 3072, 4096, 7168])
    page = rnd.choice([1, 4, 16, 64])
    batch = rnd.choice([1, 1, 2])
    hi = rnd.choice([1, 40, 700, 5000])
    lens = [rnd.randint(1, hi) for _ in range(batch)]
    _run_decode(_shape(hidden, nh_kv * g, nh_kv, rope=rnd.random() < 0.7), lens, page, cfg_id=700 + seed, kv_on_host=False,
                mode="project", variant=rnd.choice([-1, 0, 1, 2]), mma=rnd.choice([-1, -1, 0, 1]), lid=67)


@pytest.mark.parametrize("nh_q,nh_kv,host", [(8, 8, True), (8, 2, False), (8, 2, True), (16, 1, False)])
def test_results_do_not_depend_on_scheduling(nh_q, nh_kv, host):
    """Static split of the tiles over warps, fixed-order split-K sums and merges: repeated runs give the same bits
    (output and stored K/V)."""
    shape = _shape(1024, nh_q, nh_kv)
    lens = [1500, 37, 800, 2, 4097, 333]
    case = workloads.make_decode_case(shape, lens, 16, 41, DEV, kv_on_host=host)
    kernel.register_layer(91, case["k_pool"], case["v_pool"], case["wk"], case["wv"], case["cos_sin"], page_size=16)
    outs = []
    for _ in range(4):
        outs.append(kernel.decode(91, case["q"], case["seq_lens"], shape.scale, page_table=case["page_table"],
                                  x=case["x"]).clone())
        torch.cuda.synchronize()
    get_context(0).raise_on_status()
    kernel.unregister_layer(91)
    assert all(torch.equal(outs[0], o) for o in outs[1:])


@pytest.mark.parametrize("nh_q,nh_kv", [(4, 4), (8, 2), (16, 1)])
def test_units_per_warp_floor(nh_q, nh_kv):
    """Pools in HBM: below `attn_min_units` tiles per warp of the grid a step is split the short-step way (about 70 %
    of the warps, two tiles or more each, dealt out over the CTAs in turn).  Every threshold, from "never" to one that
    makes every step here a short one, gives the oracle's result."""
    ctx = get_context(0)
    outs = []
    try:
        for floor in (1, 3, 8, 64):
            ctx.set("attn_min_units", floor)
            outs.append(_run_decode(_shape(512, nh_q, nh_kv), [700, 33, 1, 2049], 16, cfg_id=55, kv_on_host=False))
    finally:
        ctx.set("attn_min_units", 5)
    for o in outs[1:]:
        assert (o.float() - outs[0].float()).abs().max().item() < 1e-2


@pytest.mark.parametrize("nh_q,nh_kv,host", [(4, 4, True), (8, 2, False), (16, 1, False), (8, 8, False)])
def test_small_batches_without_the_prep_launch(nh_q, nh_kv, host):
    """Batches of up to 32 requests run without attn_prep_kernel: the streaming and merge kernels scan the lengths
    themselves and the projection places its tokens itself.  Same bits as with the prep launch (knob off), for
    lengths that include empty pasts, and the same stored rows."""
    ctx = get_context(0)
    shape = _shape(256, nh_q, nh_kv)
    lens = [1, 1500, 37, 800, 2, 4097, 333, 16, 17] + [64] * 23          # 32 requests
    res = []
    try:
        for flag in (1, 0):
            ctx.set("attn_self_scan", flag)
            case = workloads.make_decode_case(shape, lens, 16, 43, DEV, kv_on_host=host)
            k0, v0 = case["k_pool"].cpu().clone(), case["v_pool"].cpu().clone()     # before the step stores into them
            kernel.register_layer(92, case["k_pool"], case["v_pool"], case["wk"], case["wv"], case["cos_sin"], page_size=16)
            lse = torch.empty(len(lens), nh_q, dtype=torch.float32, device=DEV)
            out = kernel.decode(92, case["q"], case["seq_lens"], shape.scale, page_table=case["page_table"], x=case["x"],
                                lse_out=lse)
            ctx.raise_on_status()
            res.append((out.clone(), lse.clone(), case["k_pool"].cpu().clone(), case["v_pool"].cpu().clone()))
            kernel.unregister_layer(92)
    finally:
        ctx.set("attn_self_scan", 1)
    for a, b in zip(res[0], res[1]):
        assert torch.equal(a, b)
    ref = orc.decode_layer(case["x"].cpu(), case["wk"].cpu(), case["wv"].cpu(), case["q"].cpu(), k0, v0,
                           case["page_table"].cpu(), lens, 16, case["cos_sin"].cpu(), shape.scale)
    assert_close(res[0][0], ref.view_as(res[0][0]), "O without the prep launch")


def test_errors():
    with pytest.raises(RuntimeError, match="not registered"):
        kernel.decode(999, torch.zeros(1, 128, dtype=torch.bfloat16, device=DEV),
                      torch.ones(1, dtype=torch.int32, device=DEV), 1.0)
    pool = torch.zeros(32, 2, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="pinned"):
        kernel.register_layer(1, pool, pool)
    pk = torch.zeros(32, 2, 128, dtype=torch.bfloat16).pin_memory()
    kernel.register_layer(41, pk, pk.clone().pin_memory(), page_size=16)
    with pytest.raises(RuntimeError, match="multiple"):
        kernel.decode(41, torch.zeros(1, 3 * 128, dtype=torch.bfloat16, device=DEV),
                      torch.ones(1, dtype=torch.int32, device=DEV), 1.0,
                      page_table=torch.ones(1, 1, dtype=torch.int32, device=DEV))
    kernel.unregister_layer(41)


def test_empty_batch():
    q = torch.zeros(0, 4 * 128, dtype=torch.bfloat16, device=DEV)
    out = kernel.decode(0, q, torch.zeros(0, dtype=torch.int32, device=DEV), 1.0)
    assert out.shape == q.shape
