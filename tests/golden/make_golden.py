"""Generates tests/golden/*.npz by running the REFERENCE's own Python code on the CPU.

Run where the reference checkout is present:

    python tests/golden/make_golden.py /path/to/reference

The reference modules import the third-party ``sglang`` package at module top
(directkv/directkv_backend.py:32-33, directkv/directkv_pool.py:39), which is not installable
here, so minimal stand-ins for the two base classes it derives from are placed in
``sys.modules`` first, and ``pin_memory=True`` allocations are turned into pageable ones (there
is no CUDA driver on the generating machine).  Nothing of the reference's arithmetic or index
logic is replaced: the vectors written here are outputs of its code.

What is captured
  pool_token.npz    DirectKVTokenToKVPool: shapes, set/get round trip, move_kv_cache
  pool_request.npz  DirectKVRequestPool: pad64, LIFO row assignment trace, views, batch gather
  torch_paths.npz   DirectKVBackend torch attention paths (_sdpa_decode_directkv,
                    _sdpa_decode_manual, _sdpa_extend_manual, _sdpa_single), weight slicing and
                    the cos/sin table, on small seeded inputs (fp32 on the CPU)
bf16 tensors are stored as their uint16 bit patterns.
"""

from __future__ import annotations

import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def install_stubs():
    """Stand-ins for the sglang names the reference imports."""
    class AttentionBackend:
        def __init__(self):
            pass

    class KVCache:
        def __init__(self, size, page_size, dtype, layer_num, device, enable_memory_saver,
                     start_layer=None, end_layer=None):
            self.size, self.page_size, self.dtype, self.layer_num = size, page_size, dtype, layer_num
            self.device = device
            self.start_layer = start_layer or 0
            self.end_layer = end_layer or layer_num - 1

    def mod(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        sys.modules[name] = m
        return m

    for name in ["sglang", "sglang.srt", "sglang.srt.layers", "sglang.srt.layers.attention",
                 "sglang.srt.mem_cache", "sglang.srt.model_executor"]:
        mod(name)
    mod("sglang.srt.layers.attention.base_attn_backend", AttentionBackend=AttentionBackend)
    mod("sglang.srt.layers.dp_attention", get_attention_tp_size=lambda: 1)
    mod("sglang.srt.mem_cache.memory_pool", KVCache=KVCache)

    # No CUDA driver here: page-locked allocations become pageable ones.
    real_zeros, real_empty = torch.zeros, torch.empty

    def zeros(*a, **k):
        k.pop("pin_memory", None)
        return real_zeros(*a, **k)

    def empty(*a, **k):
        k.pop("pin_memory", None)
        return real_empty(*a, **k)

    torch.zeros, torch.empty = zeros, empty


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()
    return t.contiguous().numpy().copy()


def gen_token_pool(ref_dir, out):
    sys.path.insert(0, os.path.join(ref_dir, "directkv"))
    import directkv_pool as rp

    class FakeLayer:
        layer_id = 1

    g = torch.Generator().manual_seed(101)
    pool = rp.DirectKVTokenToKVPool(size=40, page_size=1, dtype=torch.bfloat16, head_num=3, head_dim=16,
                                    layer_num=2, v_head_dim=16, start_layer=0, end_layer=2)
    loc = torch.tensor([5, 1, 17, 40, 9, 2], dtype=torch.int64)
    k = torch.randn(6, 3, 16, generator=g).to(torch.bfloat16)
    v = torch.randn(6, 3, 16, generator=g).to(torch.bfloat16)
    pool.set_kv_buffer(FakeLayer(), loc, k, v)
    res = dict(shape_k=np.array(pool.get_key_buffer(0).shape), n_layers=np.array(len(pool.k_buffer)),
               loc=loc.numpy(), k=bits(k), v=bits(v),
               k_buf_l1=bits(pool.get_key_buffer(1)), v_buf_l1=bits(pool.get_value_buffer(1)),
               token_stride=np.array(pool.token_stride), row_dim=np.array(pool.row_dim),
               size_bytes=np.array(pool.get_kv_size_bytes()))
    pool.move_kv_cache(torch.tensor([30, 31]), torch.tensor([5, 17]))
    res["k_buf_l1_after_move"] = bits(pool.get_key_buffer(1))
    try:
        rp.DirectKVTokenToKVPool(size=8, page_size=1, dtype=torch.float32, head_num=2, head_dim=16, layer_num=1)
        res["fp32_raises"] = np.array(0)
    except ValueError:
        res["fp32_raises"] = np.array(1)
    np.savez_compressed(os.path.join(out, "pool_token.npz"), **res)


def gen_request_pool(ref_dir, out):
    import directkv_request_pool as rq

    pool = rq.DirectKVRequestPool(max_reqs=4, max_seqlen=100, num_kv_heads=2, head_dim=8, num_layers=2, start_layer=3)
    trace = []
    ops = [("alloc", 10), ("alloc", 11), ("alloc", 10), ("free", 10), ("alloc", 12), ("alloc", 13), ("alloc", 14),
           ("free", 99), ("free", 12), ("free", 11), ("alloc", 15), ("alloc", 16)]
    for op, rid in ops:
        getattr(pool, op)(rid)
        trace.append([1 if op == "alloc" else 0, rid, pool._req_to_row.get(rid, -1), len(pool._free)])
    raised = 0
    try:
        pool.alloc(17)
    except RuntimeError:
        raised = 1
    g = torch.Generator().manual_seed(7)
    for li in range(2):
        pool.k_pool[li].copy_(torch.randn(pool.k_pool[li].shape, generator=g).to(torch.bfloat16))
        pool.v_pool[li].copy_(torch.randn(pool.v_pool[li].shape, generator=g).to(torch.bfloat16))
    K, V = pool.get_kv(15, 4, 64)
    Kb, Vb = pool.get_batch_kv([16, 13], 3, 64)
    Kg, _ = pool.get_cuda_graph_kv(4, 2)
    np.savez_compressed(
        os.path.join(out, "pool_request.npz"),
        pad64_in=np.array([0, 1, 63, 64, 65, 100, 128, 4097]),
        pad64_out=np.array([rq._pad64(n) for n in [0, 1, 63, 64, 65, 100, 128, 4097]]),
        max_seqlen_pad=np.array(pool.max_seqlen_pad), ops=np.array([[1 if o == "alloc" else 0, r] for o, r in ops]),
        trace=np.array(trace), exhausted_raises=np.array(raised),
        rows_final=np.array([[r, pool.row_of(r)] for r in sorted(pool._req_to_row)]),
        k_l0=bits(pool.k_pool[0]), k_l1=bits(pool.k_pool[1]), v_l1=bits(pool.v_pool[1]),
        get_kv_K=bits(K), get_kv_V=bits(V), batch_K=bits(Kb), batch_V=bits(Vb), graph_K_shape=np.array(Kg.shape),
    )


def gen_torch_paths(ref_dir, out):
    import directkv_backend as rb
    import directkv_request_pool as rq

    NH_q, NH_kv, D, H = 8, 2, 32, 64
    g = torch.Generator().manual_seed(2024)
    be = object.__new__(rb.DirectKVBackend)
    be.num_q_heads, be.num_kv_heads, be.head_dim, be.v_head_dim, be.hidden_size = NH_q, NH_kv, D, D, H
    be.device = torch.device("cpu")

    class Layer:
        layer_id = 0
        scaling = D ** -0.5

    res = {}
    # ---- _sdpa_decode_directkv: request pool, token appended at S_past --------------------------
    pool = rq.DirectKVRequestPool(max_reqs=3, max_seqlen=128, num_kv_heads=NH_kv, head_dim=D, num_layers=1)
    pool.alloc(5)
    pool.alloc(6)
    seq_lens = [38, 101]
    for li in range(1):
        pool.k_pool[li].copy_((torch.randn(pool.k_pool[li].shape, generator=g) * 0.7).to(torch.bfloat16).float())
        pool.v_pool[li].copy_((torch.randn(pool.v_pool[li].shape, generator=g) * 0.7).to(torch.bfloat16).float())
    # run the reference in fp32 on bf16-representable values: cast pool to float32 copies
    pool.k_pool = [t.float() for t in pool.k_pool]
    pool.v_pool = [t.float() for t in pool.v_pool]
    be._pool = pool
    q = torch.randn(2, NH_q * D, generator=g).to(torch.bfloat16).float()
    k = (torch.randn(2, NH_kv * D, generator=g) * 0.7).to(torch.bfloat16).float()
    v = (torch.randn(2, NH_kv * D, generator=g) * 0.7).to(torch.bfloat16).float()
    meta = rb._FwdMeta(seq_lens_cpu=seq_lens, req_pool_indices_cpu=[5, 6], extend_seq_lens_cpu=None,
                       extend_prefix_lens_cpu=None)
    res["dec_k_pool_before"] = pool.k_pool[0].to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16).copy()
    res["dec_v_pool_before"] = pool.v_pool[0].to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16).copy()
    outs = [be._sdpa_decode_directkv(i, q, k, v, Layer(), meta) for i in range(2)]
    res.update(dec_q=bits(q.to(torch.bfloat16)), dec_k=bits(k.to(torch.bfloat16)), dec_v=bits(v.to(torch.bfloat16)),
               dec_seq_lens=np.array(seq_lens), dec_rows=np.array([pool.row_of(5), pool.row_of(6)]),
               dec_out=torch.stack(outs).numpy(),
               dec_k_pool_after=bits(pool.k_pool[0].to(torch.bfloat16)))

    # ---- _sdpa_decode_manual / _sdpa_extend_manual: token pool + req_to_token ------------------
    n_slots = 300
    k_buf = (torch.randn(n_slots, NH_kv, D, generator=g) * 0.7).to(torch.bfloat16).float()
    v_buf = (torch.randn(n_slots, NH_kv, D, generator=g) * 0.7).to(torch.bfloat16).float()
    perm = torch.randperm(n_slots - 1, generator=g) + 1
    req_to_token = torch.zeros(4, 120, dtype=torch.int32)
    req_to_token[2, :77] = perm[:77].int()
    req_to_token[0, :120] = perm[100:220].int()

    class TokPool:
        def set_kv_buffer(self, layer, loc, ck, cv):
            k_buf[loc.long()] = ck.view(-1, NH_kv, D)
            v_buf[loc.long()] = cv.view(-1, NH_kv, D)

        def get_key_buffer(self, lid):
            return k_buf

        def get_value_buffer(self, lid):
            return v_buf

    class R2T:
        pass

    r2t = R2T()
    r2t.req_to_token = req_to_token

    class FB:
        pass

    fb = FB()
    fb.batch_size = 2
    fb.seq_lens = torch.tensor([77, 120])
    fb.req_pool_indices = torch.tensor([2, 0])
    fb.token_to_kv_pool = TokPool()
    fb.req_to_token_pool = r2t
    fb.out_cache_loc = torch.tensor([int(req_to_token[2, 76]), int(req_to_token[0, 119])])
    be._fwd_meta = rb._FwdMeta(seq_lens_cpu=[77, 120], req_pool_indices_cpu=[2, 0], extend_seq_lens_cpu=None,
                               extend_prefix_lens_cpu=None)
    q2 = torch.randn(2, NH_q * D, generator=g).to(torch.bfloat16).float()
    k2 = (torch.randn(2, NH_kv * D, generator=g) * 0.7).to(torch.bfloat16).float()
    v2 = (torch.randn(2, NH_kv * D, generator=g) * 0.7).to(torch.bfloat16).float()
    res["man_k_buf_before"] = bits(k_buf.to(torch.bfloat16)).copy()
    res["man_v_buf_before"] = bits(v_buf.to(torch.bfloat16)).copy()
    o_man = be._sdpa_decode_manual(q2, k2, v2, Layer(), fb)
    res.update(man_q=bits(q2.to(torch.bfloat16)), man_k=bits(k2.to(torch.bfloat16)), man_v=bits(v2.to(torch.bfloat16)),
               man_req_to_token=req_to_token.numpy(), man_seq_lens=np.array([77, 120]), man_req_idx=np.array([2, 0]),
               man_out=o_man.numpy())

    # extend over the token pool: 2 requests, prefix 40 / 0, new 24 / 50
    ext, pre = [24, 50], [40, 0]
    fb.seq_lens = torch.tensor([64, 50])
    be._fwd_meta = rb._FwdMeta(seq_lens_cpu=[64, 50], req_pool_indices_cpu=[2, 0], extend_seq_lens_cpu=ext,
                               extend_prefix_lens_cpu=pre)
    tot = sum(ext)
    q3 = torch.randn(tot, NH_q * D, generator=g).to(torch.bfloat16).float()
    k3 = (torch.randn(tot, NH_kv * D, generator=g) * 0.7).to(torch.bfloat16).float()
    v3 = (torch.randn(tot, NH_kv * D, generator=g) * 0.7).to(torch.bfloat16).float()
    fb.out_cache_loc = torch.cat([req_to_token[2, 40:64], req_to_token[0, 0:50]]).long()
    res["ext_k_buf_before"] = bits(k_buf.to(torch.bfloat16)).copy()
    res["ext_v_buf_before"] = bits(v_buf.to(torch.bfloat16)).copy()
    o_ext = be._sdpa_extend_manual(q3, k3, v3, Layer(), fb)
    res.update(ext_q=bits(q3.to(torch.bfloat16)), ext_k=bits(k3.to(torch.bfloat16)), ext_v=bits(v3.to(torch.bfloat16)),
               ext_lens=np.array(ext), ext_pre=np.array(pre), ext_out=o_ext.numpy(),
               ext_out_cache_loc=fb.out_cache_loc.numpy())

    # ---- _sdpa_single on the request pool (misaligned extend) ---------------------------------------
    pool2 = rq.DirectKVRequestPool(max_reqs=2, max_seqlen=128, num_kv_heads=NH_kv, head_dim=D, num_layers=1)
    pool2.alloc(1)
    pool2.k_pool = [(torch.randn(pool2.k_pool[0].shape, generator=g) * 0.7).to(torch.bfloat16).float()]
    pool2.v_pool = [(torch.randn(pool2.v_pool[0].shape, generator=g) * 0.7).to(torch.bfloat16).float()]
    be._pool = pool2
    be._fwd_meta = rb._FwdMeta(seq_lens_cpu=[50], req_pool_indices_cpu=[1], extend_seq_lens_cpu=[20],
                               extend_prefix_lens_cpu=[30])
    res["single_k_pool_before"] = bits(pool2.k_pool[0].to(torch.bfloat16)).copy()
    res["single_v_pool_before"] = bits(pool2.v_pool[0].to(torch.bfloat16)).copy()
    q4 = torch.randn(20, NH_q * D, generator=g).to(torch.bfloat16).float()
    k4 = (torch.randn(20, NH_kv * D, generator=g) * 0.7).to(torch.bfloat16).float()
    v4 = (torch.randn(20, NH_kv * D, generator=g) * 0.7).to(torch.bfloat16).float()
    o_single = be._sdpa_single(q4, k4, v4, 20, 30, Layer(), None, 0, 0, True)
    res.update(single_q=bits(q4.to(torch.bfloat16)), single_k=bits(k4.to(torch.bfloat16)),
               single_v=bits(v4.to(torch.bfloat16)), single_out=o_single.numpy(), single_row=np.array(pool2.row_of(1)))

    # ---- weight slicing and cos/sin table ---------------------------------------------------------------
    class Lin:
        pass

    class Rot:
        pass

    class Mod:
        pass

    w = torch.randn(NH_q * D + 2 * NH_kv * D, H, generator=g).to(torch.bfloat16)
    m = Mod()
    m.qkv_proj = Lin()
    m.qkv_proj.weight = w
    wk, wv = be._extract_weights(m, 0)
    rot = Rot()
    rot.inv_freq = 1.0 / (500000.0 ** (torch.arange(0, 64, dtype=torch.float32) / 64))
    rot.max_position_embeddings = 96
    m.rotary_emb = rot
    cs = be._extract_cos_sin(m)
    res.update(w_qkv=bits(w), wk=bits(wk), wv=bits(wv), cos_sin=cs.numpy(), cos_sin_theta=np.array(500000.0))
    np.savez_compressed(os.path.join(out, "torch_paths.npz"), **res)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <checkout of the reference project>")
    ref = sys.argv[1]
    install_stubs()
    gen_token_pool(ref, HERE)
    gen_request_pool(ref, HERE)
    gen_torch_paths(ref, HERE)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")
