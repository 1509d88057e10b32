"""GPU parity of the reference-shaped entry points (smpv2_fwd / smpv2_init_tma / smpv2_fwd_graph).

The first block replays the 12 seeded cases of the reference's kernel test
(tests/test_directkv_cpu_kv.cu:538-557) with its libc rand() input streams and its pass
criteria (:478-483); the second covers what that test never exercises: hidden sizes above 128
on the tensor-core projection, Neox RoPE, GQA, lengths that are not multiples of 64.
"""

import pytest
import torch

from dkv_testlib import KAT_CASES, KV_ATOL, assert_close, kat_inputs, orc

pytestmark = pytest.mark.gpu

from directkv_b200 import kernel  # noqa: E402
from directkv_b200._lib import get_context  # noqa: E402

DEV = "cuda:0"
SCALE = 128 ** -0.5


def _run_fwd(X, Wk, Wv, Q, K, V, cos_sin, causal, s_past, q_pos_start=-1, kv_on_host=True):
    K_ref, V_ref = K.clone(), V.clone()
    ref = orc.smpv2_fwd(X, Wk, Wv, Q, K_ref, V_ref, cos_sin, SCALE, causal, s_past, q_pos_start)
    Kd = K.clone().pin_memory() if kv_on_host else K.to(DEV)
    Vd = V.clone().pin_memory() if kv_on_host else V.to(DEV)
    cs = None if cos_sin is None else cos_sin.to(DEV)
    O = kernel.smpv2_fwd(X.to(DEV), Wk.to(DEV), Wv.to(DEV), Q.to(DEV), Kd, Vd, cs, SCALE, causal, s_past, q_pos_start)
    get_context(0).raise_on_status()
    o_err = assert_close(O, ref, "O")
    # K/V write-back of the new rows (reference thresholds), past rows bit-identical.
    assert_close(Kd.cpu()[:, s_past:], K_ref[:, s_past:], "K write-back", atol=KV_ATOL, rtol=1e-2)
    assert_close(Vd.cpu()[:, s_past:], V_ref[:, s_past:], "V write-back", atol=KV_ATOL, rtol=1e-2)
    if s_past > 0:
        assert torch.equal(Kd.cpu()[:, :s_past], K[:, :s_past]) and torch.equal(Vd.cpu()[:, :s_past], V[:, :s_past])
    return o_err


@pytest.mark.parametrize("name,B,NH,S_new,S_past,H,causal", KAT_CASES, ids=[c[0] for c in KAT_CASES])
def test_reference_kat_cases(oracle_clib, name, B, NH, S_new, S_past, H, causal):
    X, Wk, Wv, Q, K, V = kat_inputs(oracle_clib, B, NH, S_new, S_past, H)
    o_err = _run_fwd(X, Wk, Wv, Q, K, V, None, causal, S_past)
    assert o_err < 2e-2  # tests/test_directkv_cpu_kv.cu:478


def _rand_case(B, nh_q, nh_kv, S_new, S_past, H, seed, rope=True):
    g = torch.Generator().manual_seed(seed)
    X = torch.randn(B, S_new, H, generator=g).to(torch.bfloat16)
    Wk = (torch.randn(nh_kv, 128, H, generator=g) * 0.02).to(torch.bfloat16)
    Wv = (torch.randn(nh_kv, 128, H, generator=g) * 0.02).to(torch.bfloat16)
    Q = torch.randn(B, S_new, nh_q, 128, generator=g).to(torch.bfloat16)
    S_total = S_past + S_new
    K = torch.zeros(B, S_total, nh_kv, 128, dtype=torch.bfloat16)
    V = torch.zeros(B, S_total, nh_kv, 128, dtype=torch.bfloat16)
    std = 0.02 * H ** 0.5
    K[:, :S_past] = (torch.randn(B, S_past, nh_kv, 128, generator=g) * std).to(torch.bfloat16)
    V[:, :S_past] = (torch.randn(B, S_past, nh_kv, 128, generator=g) * std).to(torch.bfloat16)
    cs = orc.build_cos_sin(S_total + 8, 128, 500000.0) if rope else None
    return X, Wk, Wv, Q, K, V, cs


@pytest.mark.parametrize("H", [64, 128, 1024, 4096, 7168])
def test_projection_full_hidden_with_rope(H):
    """The projection contracts ALL hidden columns (tcgen05, split-K) and rotates K at absolute positions."""
    X, Wk, Wv, Q, K, V, cs = _rand_case(2, 8, 2, 40, 24, H, seed=100 + H)
    _run_fwd(X, Wk, Wv, Q, K, V, cs, True, 24)


@pytest.mark.parametrize("S_new,S_past", [(1, 0), (1, 333), (130, 0), (257, 70), (64, 64), (32, 500), (33, 96), (96, 31)])
def test_unaligned_lengths_gqa(S_new, S_past):
    X, Wk, Wv, Q, K, V, cs = _rand_case(2, 8, 2, S_new, S_past, 256, seed=7 + S_new)
    _run_fwd(X, Wk, Wv, Q, K, V, cs, True, S_past)


def test_many_token_tiles_no_split_k():
    """More than one 128-token tile per head and enough tiles that split-K is off."""
    X, Wk, Wv, Q, K, V, cs = _rand_case(1, 32, 32, 300, 0, 512, seed=55, rope=False)
    _run_fwd(X, Wk, Wv, Q, K, V, cs, True, 0)


@pytest.mark.parametrize("S_new", [600, 700])
def test_projection_wide_tiles(S_new):
    """More 128-token tiles than SMs: the projection takes 256 tokens per CTA (two accumulators in TMEM); the last
    CTA of a head holds one partial sub-tile (600 = 4 x 128 + 88) or two (700 = 5 x 128 + 60).  Compared with the
    128-token form as well."""
    ctx = get_context(0)
    X, Wk, Wv, Q, K, V, cs = _rand_case(1, 32, 32, S_new, 0, 256, seed=61 + S_new)
    _run_fwd(X, Wk, Wv, Q, K, V, cs, True, 0, kv_on_host=False)
    pools = []
    for wide in (1, 0):
        ctx.set("proj_wide", wide)
        Kd, Vd = K.clone().to(DEV), V.clone().to(DEV)
        kernel.smpv2_fwd(X.to(DEV), Wk.to(DEV), Wv.to(DEV), Q.to(DEV), Kd, Vd, cs.to(DEV), SCALE, True, 0, -1)
        pools.append((Kd.cpu(), Vd.cpu()))
    ctx.set("proj_wide", 1)
    ctx.raise_on_status()
    assert torch.equal(pools[0][0], pools[1][0]) and torch.equal(pools[0][1], pools[1][1])


def test_q_rotation_and_hbm_pool():
    X, Wk, Wv, Q, K, V, cs = _rand_case(1, 4, 4, 48, 80, 128, seed=77)
    _run_fwd(X, Wk, Wv, Q, K, V, cs, True, 80, q_pos_start=80, kv_on_host=False)


def test_checks_match_reference_messages():
    X, Wk, Wv, Q, K, V, cs = _rand_case(1, 4, 4, 16, 16, 128, seed=3, rope=False)
    Xd, Wkd, Wvd, Qd = X.to(DEV), Wk.to(DEV), Wv.to(DEV), Q.to(DEV)
    Kp, Vp = K.pin_memory(), V.pin_memory()
    with pytest.raises(RuntimeError, match="S_total"):
        kernel.smpv2_fwd(Xd, Wkd, Wvd, Qd, Kp, Vp, None, SCALE, True, 8, -1)
    with pytest.raises(RuntimeError, match="bfloat16"):
        kernel.smpv2_fwd(Xd.float(), Wkd, Wvd, Qd, Kp, Vp, None, SCALE, True, 16, -1)
    with pytest.raises(RuntimeError, match="3D"):
        kernel.smpv2_fwd(Xd[0], Wkd, Wvd, Qd, Kp, Vp, None, SCALE, True, 16, -1)
    with pytest.raises(RuntimeError, match="multiple"):
        kernel.smpv2_fwd(Xd, Wkd[:3].contiguous(), Wvd[:3].contiguous(), Qd, Kp[:, :, :3].contiguous().pin_memory(),
                         Vp[:, :, :3].contiguous().pin_memory(), None, SCALE, True, 16, -1)
    with pytest.raises(RuntimeError, match="not initialized"):
        kernel.smpv2_fwd_graph(12345, Xd, Qd, torch.empty_like(Qd), torch.zeros(1, dtype=torch.int32, device=DEV),
                               torch.zeros(1, dtype=torch.int32, device=DEV), None, SCALE, True, 64, 0)


def test_graph_entry_points_replay():
    """smpv2_init_tma + smpv2_fwd_graph: loop bounds come from device memory, pool rows from
    req_pool_indices; captured once in a CUDA graph and replayed with a different past length."""
    nh, H, S_new, rows, S_max = 4, 128, 64, 3, 256
    g = torch.Generator().manual_seed(5)
    Wk = (torch.randn(nh, 128, H, generator=g) * 0.05).to(torch.bfloat16)
    Wv = (torch.randn(nh, 128, H, generator=g) * 0.05).to(torch.bfloat16)
    K_pool = (torch.randn(rows, S_max, nh, 128, generator=g) * 0.3).to(torch.bfloat16).pin_memory()
    V_pool = (torch.randn(rows, S_max, nh, 128, generator=g) * 0.3).to(torch.bfloat16).pin_memory()
    bs = 2
    X = torch.randn(bs, S_new, H, generator=g).to(torch.bfloat16).to(DEV)
    Q = torch.randn(bs, S_new, nh, 128, generator=g).to(torch.bfloat16).to(DEV)
    O = torch.empty_like(Q)
    n_past = torch.zeros(1, dtype=torch.int32, device=DEV)
    n_blks = torch.zeros(1, dtype=torch.int32, device=DEV)
    rpi = torch.tensor([2, 0], dtype=torch.int32, device=DEV)
    kernel.smpv2_init_tma(50, X, Wk.to(DEV), Wv.to(DEV), Q, K_pool, V_pool)

    def oracle(past):
        Kr, Vr = K_pool.clone(), V_pool.clone()
        outs = []
        for b, r in enumerate([2, 0]):
            kb, vb = Kr[r:r + 1, :past + S_new].clone(), Vr[r:r + 1, :past + S_new].clone()
            outs.append(orc.smpv2_fwd(X[b:b + 1].cpu(), Wk, Wv, Q[b:b + 1].cpu(), kb, vb, None, SCALE, True, past)[0])
        return torch.stack(outs)

    n_past.fill_(1)
    ref1 = oracle(64)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        kernel.smpv2_fwd_graph(50, X, Q, O, n_past, n_blks, None, SCALE, True, S_max, S_max - 64, rpi)  # warm-up
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    assert_close(O, ref1, "eager O")
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        kernel.smpv2_fwd_graph(50, X, Q, O, n_past, n_blks, None, SCALE, True, S_max, S_max - 64, rpi)
    n_past.fill_(2)
    ref2 = oracle(128)
    graph.replay()
    torch.cuda.synchronize()
    get_context(0).raise_on_status()
    assert_close(O, ref2, "replayed O")
    kernel.unregister_layer(50)


@pytest.mark.parametrize("nh_q,nh_kv,S_new,S_past,host", [
    (32, 8, 600, 1000, True),      # Llama-3-8B grouping: 4 query heads x 32 tokens per CTA, staged host pool
    (8, 8, 300, 0, True),          # MHA, first chunk
    (16, 1, 130, 70, False),       # 16 query heads on one KV head: 8 tokens per CTA
    (12, 2, 200, 333, True),       # ratio 6 = 2 x 3 sub-groups
    (4, 4, 128, 128, False),       # exactly one tile of each
])
def test_tensor_core_extend_shapes(nh_q, nh_kv, S_new, S_past, host):
    X, Wk, Wv, Q, K, V, cs = _rand_case(2, nh_q, nh_kv, S_new, S_past, 256, seed=900 + S_new)
    _run_fwd(X, Wk, Wv, Q, K, V, cs, True, S_past, kv_on_host=host)


@pytest.mark.parametrize("causal", [True, False])
def test_extend_kernel_forms_agree(causal):
    """Two query tiles per CTA with specialised warps (O kept in TMEM, lazily rescaled) against the one-tile form."""
    ctx = get_context(0)
    X, Wk, Wv, Q, K, V, cs = _rand_case(2, 8, 2, 700, 300, 128, seed=41)
    outs = []
    for pp in (1, 0):
        ctx.set("extend_pingpong", pp)
        Kd, Vd = K.clone().to(DEV), V.clone().to(DEV)
        outs.append(kernel.smpv2_fwd(X.to(DEV), Wk.to(DEV), Wv.to(DEV), Q.to(DEV), Kd, Vd, cs.to(DEV), SCALE, causal,
                                     300, -1).float().cpu())
    ctx.set("extend_pingpong", 1)
    ctx.raise_on_status()
    assert (outs[0] - outs[1]).abs().max() < 2e-2


def test_extend_large_scores_rescale():
    """Scores that keep growing along the keys force the lazy rescale of O (steps of more than 2^8) many times."""
    B, nh, S_new, S_past, H = 1, 4, 512, 0, 128
    X, Wk, Wv, Q, K, V, cs = _rand_case(B, nh, nh, S_new, S_past, H, seed=43, rope=False)
    ramp = torch.linspace(0.2, 6.0, S_new).view(1, S_new, 1)
    X = (X.float() * ramp).to(torch.bfloat16)
    Q = (Q.float() * 3.0).to(torch.bfloat16)
    Wk = (Wk.float() * 8.0).to(torch.bfloat16)
    _run_fwd(X, Wk, Wv, Q, K, V, cs, True, S_past, kv_on_host=False)


@pytest.mark.parametrize("spike", [60.0, 400.0, 3000.0])
def test_extend_scores_that_outgrow_the_row_reference(spike):
    """Half-tiles off the diagonal form their probabilities against the reference maximum the row already has and take
    no maximum of their own; a key whose score lies far above everything before it (2^60 ... beyond what exp2 can
    hold) sends that half-tile back for its maximum.  Spikes at several places of the past, one in the first
    half-tile, one right before the diagonal, and rows that never see one."""
    nh_q, nh_kv, S_new, S_past = 8, 2, 300, 1500
    total = S_past + S_new
    g = torch.Generator().manual_seed(77)
    Q = torch.randn(1, S_new, nh_q, 128, generator=g).to(torch.bfloat16)
    K = (torch.randn(1, total, nh_kv, 128, generator=g) * 0.5).to(torch.bfloat16)
    V = torch.randn(1, total, nh_kv, 128, generator=g).to(torch.bfloat16)
    # a key parallel to one query scores |q|^2 * c * scale with that query and something random with the others
    for key, qrow, head in ((5, 10, 0), (700, 10, 0), (701, 40, 3), (1290, 250, 5), (1499, 299, 7), (1600, 120, 1)):
        q = Q[0, qrow, head].float()
        c = spike / (float(q @ q) * SCALE * 1.4426950408889634)
        K[0, key, head // (nh_q // nh_kv)] = (q * c).to(torch.bfloat16)
    kernel.register_layer(73, K.to(DEV), V.to(DEV), row_stride=total)
    out = kernel.extend_attend(73, Q.to(DEV), SCALE, True, S_past)
    get_context(0).raise_on_status()
    ref = orc.sdpa_extend(Q[0], K[0], V[0], S_past, SCALE)
    assert torch.isfinite(out.float()).all()
    assert_close(out[0], ref, f"spike {spike}")
    kernel.unregister_layer(73)


@pytest.mark.parametrize("page_size,host", [(1, True), (1, False), (16, True), (64, False)])
@pytest.mark.parametrize("S_new,S_past", [(200, 0), (130, 333)])
def test_extend_attend_paged_pool(page_size, host, S_new, S_past):
    """Attention of rows already stored in a paged pool (the token pool with page size 1 is SGLang's req_to_token):
    the rows are gathered through the page table into a contiguous staging tensor, then the tensor-core kernel."""
    nh_q, nh_kv, B = 8, 2, 2
    total = S_past + S_new
    pages_per_req = (total + page_size - 1) // page_size
    n_pages = B * pages_per_req + 3
    g = torch.Generator().manual_seed(500 + page_size + S_new)
    perm = (torch.randperm(n_pages - 1, generator=g) + 1).int()                   # page 0 stays unused
    table = torch.zeros(B + 1, pages_per_req + 2, dtype=torch.int32)
    rows = [2, 0]                                                                 # page-table row of each request
    for b, r in enumerate(rows):
        table[r, :pages_per_req] = perm[b * pages_per_req:(b + 1) * pages_per_req]
    k_pool = (torch.randn(n_pages * page_size, nh_kv, 128, generator=g) * 0.5).to(torch.bfloat16)
    v_pool = (torch.randn(n_pages * page_size, nh_kv, 128, generator=g) * 0.5).to(torch.bfloat16)
    Q = torch.randn(B, S_new, nh_q, 128, generator=g).to(torch.bfloat16)
    kd, vd = (k_pool.pin_memory(), v_pool.pin_memory()) if host else (k_pool.to(DEV), v_pool.to(DEV))
    kernel.register_layer(71, kd, vd, page_size=page_size)
    out = kernel.extend_attend(71, Q.to(DEV), SCALE, True, S_past, row_map=torch.tensor(rows, dtype=torch.int32, device=DEV),
                               page_table=table.to(DEV))
    get_context(0).raise_on_status()
    for b, r in enumerate(rows):
        pos = torch.arange(total)
        slots = table[r, pos // page_size].long() * page_size + pos % page_size
        ref = orc.sdpa_extend(Q[b], k_pool[slots], v_pool[slots], S_past, SCALE)
        assert_close(out[b], ref, f"request {b}")
    kernel.unregister_layer(71)


def test_extend_attend_contiguous_rows_and_errors():
    nh_q, nh_kv, rows, s_pad, S_new, S_past = 4, 4, 3, 512, 140, 60
    g = torch.Generator().manual_seed(77)
    K = (torch.randn(rows, s_pad, nh_kv, 128, generator=g) * 0.5).to(torch.bfloat16)
    V = (torch.randn(rows, s_pad, nh_kv, 128, generator=g) * 0.5).to(torch.bfloat16)
    Q = torch.randn(1, S_new, nh_q, 128, generator=g).to(torch.bfloat16)
    kernel.register_layer(72, K.to(DEV), V.to(DEV), row_stride=s_pad)
    out = kernel.extend_attend(72, Q.to(DEV), SCALE, True, S_past, row_map=torch.tensor([1], dtype=torch.int32, device=DEV))
    get_context(0).raise_on_status()
    ref = orc.sdpa_extend(Q[0], K[1, :S_past + S_new], V[1, :S_past + S_new], S_past, SCALE)
    assert_close(out[0], ref, "O")
    with pytest.raises(RuntimeError, match="exceeds the pool row"):
        kernel.extend_attend(72, Q.to(DEV), SCALE, True, s_pad, row_map=torch.tensor([1], dtype=torch.int32, device=DEV))
    kernel.unregister_layer(72)
    with pytest.raises(RuntimeError, match="not registered"):
        kernel.extend_attend(72, Q.to(DEV), SCALE, True, 0)


@pytest.mark.parametrize("host", [True, False])
def test_extend_ragged_batch(host):
    """Three requests with different new / past lengths in ONE launch sequence (projection + RoPE + write-back +
    attention), each compared with the oracle run on that request alone; rows of the pool that no request writes
    stay bit-identical."""
    nh_q, nh_kv, H, s_pad = 8, 2, 256, 640
    s_new, past, rows = [200, 70, 333], [0, 130, 64], [3, 0, 2]
    g = torch.Generator().manual_seed(4321)
    Wk = (torch.randn(nh_kv, 128, H, generator=g) * 0.05).to(torch.bfloat16)
    Wv = (torch.randn(nh_kv, 128, H, generator=g) * 0.05).to(torch.bfloat16)
    K = (torch.randn(4, s_pad, nh_kv, 128, generator=g) * 0.4).to(torch.bfloat16)
    V = (torch.randn(4, s_pad, nh_kv, 128, generator=g) * 0.4).to(torch.bfloat16)
    T = sum(s_new)
    X = torch.randn(T, H, generator=g).to(torch.bfloat16)
    Q = torch.randn(T, nh_q, 128, generator=g).to(torch.bfloat16)
    cs = orc.build_cos_sin(s_pad, 128, 10000.0)
    Kd, Vd = (K.clone().pin_memory(), V.clone().pin_memory()) if host else (K.to(DEV), V.to(DEV))
    kernel.register_layer(73, Kd, Vd, Wk.to(DEV), Wv.to(DEV), cs.to(DEV), row_stride=s_pad)
    out = kernel.extend_ragged(73, X.to(DEV), Q.to(DEV), s_new, past, rows, SCALE, True)
    get_context(0).raise_on_status()
    Kc, Vc = Kd.cpu(), Vd.cpu()
    off = 0
    for n, p, r in zip(s_new, past, rows):
        kb, vb = K[r:r + 1, :p + n].clone(), V[r:r + 1, :p + n].clone()
        ref = orc.smpv2_fwd(X[off:off + n].unsqueeze(0), Wk, Wv, Q[off:off + n].unsqueeze(0), kb, vb, cs, SCALE, True, p)
        assert_close(out[off:off + n], ref[0], f"O of the request in row {r}")
        assert_close(Kc[r, p:p + n], kb[0, p:], "K write-back", atol=KV_ATOL, rtol=1e-2)
        assert_close(Vc[r, p:p + n], vb[0, p:], "V write-back", atol=KV_ATOL, rtol=1e-2)
        assert torch.equal(Kc[r, :p], K[r, :p]) and torch.equal(Kc[r, p + n:], K[r, p + n:])
        off += n
    assert torch.equal(Kc[1], K[1]) and torch.equal(Vc[1], V[1])
    kernel.unregister_layer(73)


@pytest.mark.parametrize("s_new,past", [(1105, 4096), (1487, 6144), (70, 2048)])
def test_back_to_back_extends_when_the_second_query_tile_is_empty(s_new, past):
    """The last pair of query tiles of a chunk may hold only ONE tile (here s_new leaves fewer than 32 rows for the
    pair with 4 query heads per KV head), which then reads no key at all while its partner walks past + s_new of
    them.  Several layers' calls are issued back to back without host synchronisation, as a model does: every output
    must match the oracle and no wait may run out."""
    nh_q, nh_kv, H, layers = 8, 2, 256, 4
    s_pad = past + s_new + 23
    g = torch.Generator().manual_seed(977)
    X = torch.randn(s_new, H, generator=g).to(torch.bfloat16)
    Q = torch.randn(s_new, nh_q, 128, generator=g).to(torch.bfloat16)
    cs = orc.build_cos_sin(s_pad, 128, 10000.0)
    Xd, Qd = X.to(DEV), Q.to(DEV)
    pools, weights = [], []
    for li in range(layers):
        Wk = (torch.randn(nh_kv, 128, H, generator=g) * 0.05).to(torch.bfloat16)
        Wv = (torch.randn(nh_kv, 128, H, generator=g) * 0.05).to(torch.bfloat16)
        K = (torch.randn(1, s_pad, nh_kv, 128, generator=g) * 0.4).to(torch.bfloat16)
        V = (torch.randn(1, s_pad, nh_kv, 128, generator=g) * 0.4).to(torch.bfloat16)
        Kd, Vd = K.clone().pin_memory(), V.clone().pin_memory()
        kernel.register_layer(80 + li, Kd, Vd, Wk.to(DEV), Wv.to(DEV), cs.to(DEV), row_stride=s_pad)
        pools.append((K, V, Kd, Vd))
        weights.append((Wk, Wv))
    outs = []
    for rep in range(3):
        for li in range(layers):
            outs.append(kernel.extend_ragged(80 + li, Xd, Qd, [s_new], [past], [0], SCALE, True))
    get_context(0).raise_on_status()
    for li in range(layers):
        K, V, Kd, Vd = pools[li]
        kb, vb = K[:, :past + s_new].clone(), V[:, :past + s_new].clone()
        ref = orc.smpv2_fwd(X.unsqueeze(0), weights[li][0], weights[li][1], Q.unsqueeze(0), kb, vb, cs, SCALE, True, past)
        for rep in range(3):
            assert_close(outs[rep * layers + li], ref[0], f"O of layer {li}, pass {rep}")
        assert_close(Kd[0, past:past + s_new], kb[0, past:], "K write-back", atol=KV_ATOL, rtol=1e-2)
        kernel.unregister_layer(80 + li)


def test_extend_ragged_attend_paged():
    """Rows already stored in a token pool (page size 1): ragged attention through the page table."""
    nh_q, nh_kv = 8, 2
    s_new, past, rows = [150, 40, 260], [90, 0, 10], [1, 3, 0]
    g = torch.Generator().manual_seed(99)
    n_slots = 1200
    k_pool = (torch.randn(n_slots, nh_kv, 128, generator=g) * 0.5).to(torch.bfloat16)
    v_pool = (torch.randn(n_slots, nh_kv, 128, generator=g) * 0.5).to(torch.bfloat16)
    perm = (torch.randperm(n_slots - 1, generator=g) + 1).int()
    table = torch.zeros(4, 300, dtype=torch.int32)
    at = 0
    for n, p, r in zip(s_new, past, rows):
        table[r, :n + p] = perm[at:at + n + p]
        at += n + p
    Q = torch.randn(sum(s_new), nh_q, 128, generator=g).to(torch.bfloat16)
    kernel.register_layer(74, k_pool.pin_memory(), v_pool.pin_memory(), page_size=1)
    out = kernel.extend_ragged(74, None, Q.to(DEV), s_new, past, rows, SCALE, True, page_table=table.to(DEV))
    get_context(0).raise_on_status()
    off = 0
    for n, p, r in zip(s_new, past, rows):
        slots = table[r, :n + p].long()
        ref = orc.sdpa_extend(Q[off:off + n], k_pool[slots], v_pool[slots], p, SCALE)
        assert_close(out[off:off + n], ref, f"request in table row {r}")
        off += n
    kernel.unregister_layer(74)
    with pytest.raises(RuntimeError, match="sum"):
        kernel.extend_ragged(74, None, Q.to(DEV), [1], [0], [0], SCALE)


def test_extend_is_reproducible():
    X, Wk, Wv, Q, K, V, cs = _rand_case(1, 8, 2, 900, 200, 512, seed=71)
    outs = []
    for _ in range(3):
        Kd, Vd = K.clone().to(DEV), V.clone().to(DEV)
        outs.append(kernel.smpv2_fwd(X.to(DEV), Wk.to(DEV), Wv.to(DEV), Q.to(DEV), Kd, Vd, cs.to(DEV), SCALE, True, 200, -1).clone())
        torch.cuda.synchronize()
    get_context(0).raise_on_status()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


def test_extend_paths_agree():
    """The tensor-core extend kernel and the row-streamed path (decode kernels, one virtual request per new
    row) implement the same function: compare them directly, non-causal included."""
    ctx = get_context(0)
    for causal in (True, False):
        X, Wk, Wv, Q, K, V, cs = _rand_case(1, 8, 2, 257, 100, 128, seed=31)
        outs = []
        for rowwise in (0, 1):
            ctx.set("extend_rowwise", rowwise)
            Kd, Vd = K.clone().pin_memory(), V.clone().pin_memory()
            outs.append(kernel.smpv2_fwd(X.to(DEV), Wk.to(DEV), Wv.to(DEV), Q.to(DEV), Kd, Vd, cs.to(DEV), SCALE, causal,
                                         100, -1).float().cpu())
        ctx.set("extend_rowwise", 0)
        ctx.raise_on_status()
        assert (outs[0] - outs[1]).abs().max() < 2e-2
