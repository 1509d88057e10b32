"""End-to-end GPU test of the attention backend with stand-ins for SGLang's runner, model and batch:
chunked prefill through forward_extend, ragged decode steps with request churn, the CUDA-graph hooks
with per-request lengths, and the token-pool path, each against the CPU oracle."""

import pytest
import torch

from dkv_testlib import assert_close, orc
from fake_sglang import DECODE, EXTEND, FakeModel, make_batch, make_runner

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
H, NH_Q, NH_KV, D, LAYERS = 256, 8, 2, 128, 2


class OracleState:
    """Per layer and request: the K/V rows the reference's torch path would hold."""

    def __init__(self, model, cos_sin):
        self.cos_sin = cos_sin
        self.w = []
        for layer in model.layers:
            w = layer.qkv_proj.weight.detach().cpu()
            self.w.append(orc.slice_qkv_weight(w, NH_Q, NH_KV, D, H))
        self.kv = {}

    def extend(self, lid, rid, x, q, n_pre):
        wk, wv = self.w[lid]
        n_new = x.shape[0]
        k_old, v_old = self.kv.get((lid, rid), (torch.zeros(0, NH_KV, D, dtype=torch.bfloat16),) * 2)
        K = torch.cat([k_old[:n_pre], torch.zeros(n_new, NH_KV, D, dtype=torch.bfloat16)])[None]
        V = torch.cat([v_old[:n_pre], torch.zeros(n_new, NH_KV, D, dtype=torch.bfloat16)])[None]
        o = orc.smpv2_fwd(x[None], wk, wv, q.view(1, n_new, NH_Q, D), K, V, self.cos_sin, D ** -0.5, True, n_pre)
        self.kv[(lid, rid)] = (K[0], V[0])
        return o[0].reshape(n_new, NH_Q * D)


def _setup(theta=500000.0, max_reqs=8):
    import directkv_b200

    torch.manual_seed(0)
    model = FakeModel(LAYERS, H, NH_Q, NH_KV, theta, 512).to(DEV)
    runner = make_runner(model, H, NH_Q, NH_KV, LAYERS, DEV, max_reqs=max_reqs, context_len=512)
    be = directkv_b200.DirectKVSmpV2Backend(runner)
    cs = orc.build_cos_sin(512, 128, theta) if theta else None
    return be, runner, model, OracleState(model, cs)


def _rand(shape, g, std=1.0):
    return (torch.randn(shape, generator=g) * std).to(torch.bfloat16)


def test_prefill_then_ragged_decode_with_churn():
    be, runner, model, ref = _setup()
    g = torch.Generator().manual_seed(42)
    # ---- chunked prefill: request 3 in two chunks (64 + 6), request 5 in one (33) ----
    plan = [([64, 33], [0, 0], [3, 5]), ([6], [64], [3])]
    totals = {}
    for ext, pre, rids in plan:
        fb = make_batch(EXTEND, [p + e for p, e in zip(pre, ext)], rids, DEV, extend_lens=ext, prefix_lens=pre)
        be.init_forward_metadata(fb)
        for lid, layer in enumerate(model.layers):
            x = _rand((sum(ext), H), g)
            q = _rand((sum(ext), NH_Q * D), g)
            layer(hidden_states=x.to(DEV))
            out = be.forward_extend(q.to(DEV), None, None, layer.attn, fb)
            off = 0
            for e, p, rid in zip(ext, pre, rids):
                exp = ref.extend(lid, rid, x[off:off + e], q[off:off + e], p)
                assert_close(out[off:off + e], exp, f"extend layer {lid} req {rid}")
                off += e
        for e, p, rid in zip(ext, pre, rids):
            totals[rid] = p + e
    # ---- decode steps; request 5 finishes after step 2 and request 9 (fresh prefill) joins ----
    active = [3, 5]
    for step in range(4):
        if step == 2:
            active = [3, 9]
            # the batch carries every running request (request 3 with nothing new) plus the newcomer
            fb = make_batch(EXTEND, [totals[3], 17], [3, 9], DEV, extend_lens=[0, 17], prefix_lens=[totals[3], 0])
            be.init_forward_metadata(fb)
            for lid, layer in enumerate(model.layers):
                x, q = _rand((17, H), g), _rand((17, NH_Q * D), g)
                layer(hidden_states=x.to(DEV))
                out = be.forward_extend(q.to(DEV), None, None, layer.attn, fb)
                assert_close(out, ref.extend(lid, 9, x, q, 0), f"late prefill layer {lid}")
            totals[9] = 17
        lens = [totals[r] + 1 for r in active]
        fb = make_batch(DECODE, lens, active, DEV)
        be.init_forward_metadata(fb)
        for lid, layer in enumerate(model.layers):
            x, q = _rand((len(active), H), g), _rand((len(active), NH_Q * D), g)
            layer(hidden_states=x.to(DEV))
            out = be.forward_decode(q.to(DEV), None, None, layer.attn, fb)
            for i, rid in enumerate(active):
                exp = ref.extend(lid, rid, x[i:i + 1], q[i:i + 1], totals[rid])
                assert_close(out[i:i + 1], exp, f"decode step {step} layer {lid} req {rid}")
        for r in active:
            totals[r] += 1
    from directkv_b200._lib import get_context

    get_context(0).raise_on_status()
    # the pool rows hold exactly what the oracle holds (in place, no copies)
    for (lid, rid), (K, _) in ref.kv.items():
        if rid in active:
            row = be._pool.row_of(rid)
            got = be._pool.k_pool[lid][row, :K.shape[0]]
            assert_close(got, K, f"pool row layer {lid} req {rid}", atol=1e-2, rtol=1e-2)


def test_cuda_graph_hooks_keep_per_request_lengths():
    be, runner, model, ref = _setup(theta=None)
    g = torch.Generator().manual_seed(7)
    rids, pre = [1, 2, 6], [80, 5, 131]
    fb = make_batch(EXTEND, pre, rids, DEV, extend_lens=pre, prefix_lens=[0, 0, 0])
    be.init_forward_metadata(fb)
    layer = model.layers[0]
    x, q = _rand((sum(pre), H), g), _rand((sum(pre), NH_Q * D), g)
    layer(hidden_states=x.to(DEV))
    be.forward_extend(q.to(DEV), None, None, layer.attn, fb)
    off = 0
    for n, rid in zip(pre, rids):
        ref.extend(0, rid, x[off:off + n], q[off:off + n], 0)
        off += n
    # ---- capture one decode step of layer 0 for a batch of 4 (one more than there are requests) ----
    be.init_cuda_graph_state(4, 4)
    bs = 4
    x_s = torch.zeros(bs, H, dtype=torch.bfloat16, device=DEV)
    q_s = torch.zeros(bs, NH_Q * D, dtype=torch.bfloat16, device=DEV)
    fill = be.get_cuda_graph_seq_len_fill_value()
    rpi = torch.zeros(bs, dtype=torch.int64, device=DEV)                       # placeholders, as SGLang passes them
    sl = torch.full((bs,), fill, dtype=torch.int64, device=DEV)
    torch.cuda.synchronize()
    before = [(be._pool.k_pool[0][be._pool.row_of(r)].clone(), be._pool.v_pool[0][be._pool.row_of(r)].clone()) for r in rids]
    be.init_forward_metadata_capture_cuda_graph(bs, bs, rpi, sl, None, DECODE, None)
    fbd = make_batch(DECODE, [fill] * bs, [0] * bs, DEV)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        layer(hidden_states=x_s)
        be.forward_decode(q_s, None, None, layer.attn, fbd)
    torch.cuda.current_stream().wait_stream(s)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        layer(hidden_states=x_s)
        out_s = be.forward_decode(q_s, None, None, layer.attn, fbd)
    torch.cuda.synchronize()
    # warm-up and capture ran on placeholders: they stored to the pool's spare row, no request's row changed
    for r, (kb, vb) in zip(rids, before):
        assert torch.equal(be._pool.k_pool[0][be._pool.row_of(r)], kb), f"capture touched the K row of request {r}"
        assert torch.equal(be._pool.v_pool[0][be._pool.row_of(r)], vb), f"capture touched the V row of request {r}"
    # A prefill AFTER the capture makes the engine's scratch grow; the graph must keep working on the memory it
    # recorded (the outgrown allocation is retired, not freed).
    n_big = 400
    fb2 = make_batch(EXTEND, [n_big], [7], DEV, extend_lens=[n_big], prefix_lens=[0])
    be.init_forward_metadata(fb2)
    xb, qb = _rand((n_big, H), g), _rand((n_big, NH_Q * D), g)
    layer(hidden_states=xb.to(DEV))
    ob = be.forward_extend(qb.to(DEV), None, None, layer.attn, fb2)
    assert_close(ob, ref.extend(0, 7, xb, qb, 0), "prefill after the capture")
    # ---- replays with ragged lengths: three requests in a batch padded to four.  The padded entry carries the
    # fill length and a stale request index that collides with live request 1 (80+ tokens): nothing may be
    # stored into that request's row at position fill - 1. ----
    lens = list(pre)
    for step in range(3):
        cur = [n + 1 for n in lens]
        xs, qs = _rand((bs, H), g), _rand((bs, NH_Q * D), g)
        x_s.copy_(xs)
        q_s.copy_(qs)
        rpi.copy_(torch.tensor(rids + [1], dtype=torch.int64))
        sl_now = torch.tensor(cur + [fill], dtype=torch.int64, device=DEV)
        row1 = be._pool.row_of(1)
        k63 = be._pool.k_pool[0][row1, fill - 1].clone()
        be.init_forward_metadata_replay_cuda_graph(bs, rpi, sl_now, sum(cur) + fill, None, DECODE, None,
                                                   seq_lens_cpu=sl_now.cpu())
        graph.replay()
        torch.cuda.synchronize()
        from directkv_b200._lib import get_context
        get_context(0).raise_on_status()
        assert torch.equal(be._pool.k_pool[0][row1, fill - 1], k63), "a padded entry stored into a live request's row"
        for i, rid in enumerate(rids):
            exp = ref.extend(0, rid, xs[i:i + 1], qs[i:i + 1], lens[i])
            assert_close(out_s[i:i + 1], exp, f"replay {step} req {rid}")
        lens = cur


def test_padding_detection_of_graph_replays():
    """Which tail entries of a replayed batch are padding (host logic of the replay hook)."""
    be, runner, model, ref = _setup(theta=None)
    be._ensure_pool()
    be._sync_rows([1, 2, 6])
    be._last_len.update({1: 90, 2: 63, 6: 10})
    fill = be.get_cuda_graph_seq_len_fill_value()
    assert be._count_real([1, 2, 6], [91, 64, 11]) == 3                 # nothing padded
    assert be._count_real([1, 2, 6, 0], [91, 64, 11, fill]) == 3        # index 0 holds no row
    assert be._count_real([1, 6, 2, 2], [91, 11, 64, fill]) == 3        # repeats an earlier entry
    assert be._count_real([6, 2, 1, 1], [11, 64, fill, fill]) == 2      # request 1 was 90 tokens long, not 63
    assert be._count_real([1, 6, 2], [91, 11, fill]) == 3               # request 2 was 63 long: really 64 now


def test_token_pool_path_when_no_hidden_states():
    """No pre-hook fired: K/V computed by the model are stored through set_kv_buffer and attention
    runs over req_to_token slots (reference data flow: directkv_backend.py:835-891)."""
    from directkv_b200 import DirectKVTokenToKVPool

    be, runner, model, _ = _setup(theta=None)
    g = torch.Generator().manual_seed(9)
    pool = DirectKVTokenToKVPool(size=400, page_size=1, dtype=torch.bfloat16, head_num=NH_KV, head_dim=D,
                                 layer_num=LAYERS, start_layer=0, end_layer=LAYERS - 1)
    perm = (torch.randperm(400, generator=g) + 1).int()
    r2t = runner.req_to_token_pool
    lens = {2: 50, 4: 21}
    r2t.req_to_token[2, :60] = perm[:60].to(DEV)
    r2t.req_to_token[4, :60] = perm[100:160].to(DEV)
    layer = model.layers[1]
    k_ref = torch.zeros(401, NH_KV, D, dtype=torch.bfloat16)
    v_ref = torch.zeros(401, NH_KV, D, dtype=torch.bfloat16)
    # extend both requests
    ext = [lens[2], lens[4]]
    loc = torch.cat([r2t.req_to_token[2, :50], r2t.req_to_token[4, :21]]).long()
    fb = make_batch(EXTEND, ext, [2, 4], DEV, extend_lens=ext, prefix_lens=[0, 0], token_pool=pool,
                    req_to_token_pool=r2t, out_cache_loc=loc)
    be.init_forward_metadata(fb)
    q, k, v = _rand((71, NH_Q * D), g), _rand((71, NH_KV * D), g, 0.5), _rand((71, NH_KV * D), g, 0.5)
    out = be.forward_extend(q.to(DEV), k.to(DEV), v.to(DEV), layer.attn, fb)
    k_ref[loc.cpu()], v_ref[loc.cpu()] = k.view(-1, NH_KV, D), v.view(-1, NH_KV, D)
    off = 0
    for rid, n in zip([2, 4], ext):
        slots = r2t.req_to_token[rid, :n].long().cpu()
        exp = orc.sdpa_extend(q[off:off + n].view(n, NH_Q, D), k_ref[slots], v_ref[slots], 0, D ** -0.5)
        assert_close(out[off:off + n], exp.reshape(n, -1), f"token-pool extend req {rid}")
        off += n
    # one decode step
    loc = torch.stack([r2t.req_to_token[2, 50], r2t.req_to_token[4, 21]]).long()
    fb = make_batch(DECODE, [51, 22], [2, 4], DEV, token_pool=pool, req_to_token_pool=r2t, out_cache_loc=loc)
    be.init_forward_metadata(fb)
    q, k, v = _rand((2, NH_Q * D), g), _rand((2, NH_KV * D), g, 0.5), _rand((2, NH_KV * D), g, 0.5)
    out = be.forward_decode(q.to(DEV), k.to(DEV), v.to(DEV), layer.attn, fb)
    k_ref[loc.cpu()], v_ref[loc.cpu()] = k.view(-1, NH_KV, D), v.view(-1, NH_KV, D)
    for i, (rid, n) in enumerate(zip([2, 4], [51, 22])):
        slots = r2t.req_to_token[rid, :n].long().cpu()
        exp = orc.sdpa_decode(q[i].view(NH_Q, D), k_ref[slots], v_ref[slots], D ** -0.5)
        assert_close(out[i].view(NH_Q, D), exp, f"token-pool decode req {rid}")
    pool.synchronize()
    assert torch.equal(pool.get_key_buffer(1)[loc.cpu()], k.view(-1, NH_KV, D))


def test_token_pool_chunked_prefill():
    """Token pool, one request prefilled in two chunks (200 rows, then 100 more on a prefix of 200): both chunks are
    long enough for the tensor-core kernel, which reads the rows through req_to_token."""
    from directkv_b200 import DirectKVTokenToKVPool

    be, runner, model, _ = _setup(theta=None)
    g = torch.Generator().manual_seed(19)
    pool = DirectKVTokenToKVPool(size=700, page_size=1, dtype=torch.bfloat16, head_num=NH_KV, head_dim=D,
                                 layer_num=LAYERS, start_layer=0, end_layer=LAYERS - 1)
    r2t = runner.req_to_token_pool
    perm = (torch.randperm(700, generator=g) + 1).int()
    r2t.req_to_token[3, :300] = perm[:300].to(DEV)
    layer = model.layers[0]
    k_ref = torch.zeros(701, NH_KV, D, dtype=torch.bfloat16)
    v_ref = torch.zeros(701, NH_KV, D, dtype=torch.bfloat16)
    for pre, n in ((0, 200), (200, 100)):
        loc = r2t.req_to_token[3, pre:pre + n].long()
        fb = make_batch(EXTEND, [pre + n], [3], DEV, extend_lens=[n], prefix_lens=[pre], token_pool=pool,
                        req_to_token_pool=r2t, out_cache_loc=loc)
        be.init_forward_metadata(fb)
        q, k, v = _rand((n, NH_Q * D), g), _rand((n, NH_KV * D), g, 0.5), _rand((n, NH_KV * D), g, 0.5)
        out = be.forward_extend(q.to(DEV), k.to(DEV), v.to(DEV), layer.attn, fb)
        k_ref[loc.cpu()], v_ref[loc.cpu()] = k.view(-1, NH_KV, D), v.view(-1, NH_KV, D)
        slots = r2t.req_to_token[3, :pre + n].long().cpu()
        exp = orc.sdpa_extend(q.view(n, NH_Q, D), k_ref[slots], v_ref[slots], pre, D ** -0.5)
        assert_close(out, exp.reshape(n, -1), f"chunk at prefix {pre}")


def test_set_kv_buffer_scatter_kernel_matches_host_path():
    from directkv_b200 import DirectKVTokenToKVPool

    class L:
        layer_id = 0

    g = torch.Generator().manual_seed(3)
    a = DirectKVTokenToKVPool(size=64, page_size=1, dtype=torch.bfloat16, head_num=3, head_dim=64, layer_num=1)
    b = DirectKVTokenToKVPool(size=64, page_size=1, dtype=torch.bfloat16, head_num=3, head_dim=64, layer_num=1)
    loc = torch.tensor([5, 64, 1, 33], dtype=torch.int32)
    k, v = _rand((4, 3, 64), g), _rand((4, 3, 64), g)
    a.set_kv_buffer(L(), loc, k, v)                                   # host path
    b.set_kv_buffer(L(), loc.to(DEV), k.to(DEV), v.to(DEV))          # scatter kernel into pinned memory
    b.synchronize()
    assert torch.equal(a.get_key_buffer(0), b.get_key_buffer(0)) and torch.equal(a.get_value_buffer(0), b.get_value_buffer(0))
