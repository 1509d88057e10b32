"""Pins the CPU oracle: against outputs of the reference's own Python code (tests/golden/*.npz,
made by tests/golden/make_golden.py) and against the plain-C restatement of the reference's
kernel-test oracle on its seeded cases.  No GPU needed."""

import ctypes
import os

import numpy as np
import pytest
import torch

from dkv_testlib import KAT_CASES, kat_inputs, libc_rand_stream, orc

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


@pytest.fixture(scope="module")
def paths():
    return np.load(os.path.join(GOLD, "torch_paths.npz"))


def test_decode_request_pool_path(paths):
    """directkv_backend.py:781-825 (_sdpa_decode_directkv): token written at S_past, SDPA over [0, S_past]."""
    g = paths
    k_pool, v_pool = bf16(g["dec_k_pool_before"]), bf16(g["dec_v_pool_before"])     # [rows, S, NH_kv, D]
    rows, S, nh_kv, d = k_pool.shape
    q = bf16(g["dec_q"]).view(2, -1, d)
    kn, vn = bf16(g["dec_k"]).view(2, nh_kv, d), bf16(g["dec_v"]).view(2, nh_kv, d)
    seq_lens = (g["dec_seq_lens"] ).tolist()
    # the reference's S_past = seq_len - 1 and the token lands at [row, S_past]
    table = torch.tensor([[int(r) * S + t for t in range(S)] for r in g["dec_rows"]], dtype=torch.int32)
    kp, vp = k_pool.view(-1, nh_kv, d).clone(), v_pool.view(-1, nh_kv, d).clone()
    out = orc.decode_layer(None, None, None, q, kp, vp, table, seq_lens, 1, None, d ** -0.5, k_new=kn, v_new=vn)
    ref = torch.from_numpy(g["dec_out"]).view(2, -1, d)
    assert torch.allclose(out, ref, atol=2e-6, rtol=1e-5)
    assert torch.equal(kp.view(rows, S, nh_kv, d), bf16(g["dec_k_pool_after"]))


def test_decode_token_pool_path(paths):
    """directkv_backend.py:835-859 (_sdpa_decode_manual): slots gathered through req_to_token."""
    g = paths
    k_buf, v_buf = bf16(g["man_k_buf_before"]), bf16(g["man_v_buf_before"])
    nh_kv, d = k_buf.shape[1], k_buf.shape[2]
    q = bf16(g["man_q"]).view(2, -1, d)
    kn, vn = bf16(g["man_k"]).view(2, nh_kv, d), bf16(g["man_v"]).view(2, nh_kv, d)
    r2t = torch.from_numpy(g["man_req_to_token"])
    table = r2t[torch.from_numpy(g["man_req_idx"]).long()]
    out = orc.decode_layer(None, None, None, q, k_buf.clone(), v_buf.clone(), table, g["man_seq_lens"].tolist(), 1,
                           None, d ** -0.5, k_new=kn, v_new=vn)
    ref = torch.from_numpy(g["man_out"]).view(2, -1, d)
    assert torch.allclose(out, ref, atol=2e-6, rtol=1e-5)


def test_extend_token_pool_path(paths):
    """directkv_backend.py:861-891 (_sdpa_extend_manual): triu(-inf, diagonal=sl_pre+1) mask."""
    g = paths
    k_buf, v_buf = bf16(g["ext_k_buf_before"]).clone(), bf16(g["ext_v_buf_before"]).clone()
    nh_kv, d = k_buf.shape[1], k_buf.shape[2]
    q = bf16(g["ext_q"])
    kn, vn = bf16(g["ext_k"]).view(-1, nh_kv, d), bf16(g["ext_v"]).view(-1, nh_kv, d)
    loc = torch.from_numpy(g["ext_out_cache_loc"]).long()
    k_buf[loc], v_buf[loc] = kn, vn
    r2t = torch.from_numpy(g["man_req_to_token"])
    ref = torch.from_numpy(g["ext_out"])
    off = 0
    for (rid, sl_new, sl_pre) in zip([2, 0], g["ext_lens"].tolist(), g["ext_pre"].tolist()):
        slots = r2t[rid, :sl_pre + sl_new].long()
        o = orc.sdpa_extend(q[off:off + sl_new].view(sl_new, -1, d), k_buf[slots], v_buf[slots], sl_pre, d ** -0.5)
        assert torch.allclose(o.reshape(sl_new, -1), ref[off:off + sl_new], atol=2e-6, rtol=1e-5)
        off += sl_new


def test_extend_request_pool_path(paths):
    """directkv_backend.py:893-924 (_sdpa_single)."""
    g = paths
    k_pool, v_pool = bf16(g["single_k_pool_before"]).clone(), bf16(g["single_v_pool_before"]).clone()
    nh_kv, d = k_pool.shape[2], k_pool.shape[3]
    row = int(g["single_row"])
    kn, vn = bf16(g["single_k"]).view(20, nh_kv, d), bf16(g["single_v"]).view(20, nh_kv, d)
    k_pool[row, 30:50], v_pool[row, 30:50] = kn, vn
    q = bf16(g["single_q"]).view(20, -1, d)
    o = orc.sdpa_extend(q, k_pool[row, :50], v_pool[row, :50], 30, d ** -0.5)
    assert torch.allclose(o.reshape(20, -1), torch.from_numpy(g["single_out"]), atol=2e-6, rtol=1e-5)


def test_weight_slices_and_cos_sin_table(paths):
    """directkv_backend.py:243-271 and :299-304."""
    g = paths
    w = bf16(g["w_qkv"])
    wk, wv = orc.slice_qkv_weight(w, 8, 2, 32, 64)
    assert torch.equal(wk, bf16(g["wk"])) and torch.equal(wv, bf16(g["wv"]))
    cs = orc.build_cos_sin(96, 128, float(g["cos_sin_theta"]))
    assert torch.allclose(cs, torch.from_numpy(g["cos_sin"]), atol=1e-6, rtol=0)
    from directkv_b200 import workloads

    assert torch.allclose(workloads.build_cos_sin(96, float(g["cos_sin_theta"])), torch.from_numpy(g["cos_sin"]),
                          atol=1e-6, rtol=0)


def test_index_maps_bit_exact():
    g = np.load(os.path.join(GOLD, "pool_request.npz"))
    assert [orc.pad64(int(n)) for n in g["pad64_in"]] == g["pad64_out"].tolist()
    fl = orc.RowFreeList(4)
    for (is_alloc, rid), (_, _, row, nfree) in zip(g["ops"].tolist(), g["trace"].tolist()):
        (fl.alloc if is_alloc else fl.release)(rid)
        assert fl.req_to_row.get(rid, -1) == row and len(fl.free) == nfree
    assert orc.decode_slot(63) == 63 and orc.decode_slot(64) == 0 and orc.layer_index(5, 3) == 2
    assert orc.token_slot([7, 3], 17, 16) == 3 * 16 + 1 and orc.token_slot([9, 4, 2], 2, 1) == 2


def test_rope_matches_kernel_formula():
    """csrc/directKV_kernel.cuh:504-518 written out element by element."""
    g = torch.Generator().manual_seed(1)
    k = torch.randn(3, 2, 128, generator=g).to(torch.bfloat16)
    cs = orc.build_cos_sin(50, 128, 10000.0)
    pos = torch.tensor([0, 7, 49])
    out = orc.rope_neox(k, cs, pos)
    for t in range(3):
        for d in (0, 5, 63):
            c, s = cs[pos[t], d].item(), cs[pos[t], 64 + d].item()
            lo, hi = k[t, 1, d].float().item(), k[t, 1, d + 64].float().item()
            assert out[t, 1, d].item() == torch.tensor(lo * c - hi * s).to(torch.bfloat16).item()
            assert out[t, 1, d + 64].item() == torch.tensor(hi * c + lo * s).to(torch.bfloat16).item()
    assert torch.equal(orc.rope_neox(k, None, pos), k)


def test_lse_merge_equals_full_softmax():
    g = torch.Generator().manual_seed(3)
    q, k, v = torch.randn(4, 32, generator=g), torch.randn(90, 32, generator=g), torch.randn(90, 32, generator=g)
    full, lse = orc.ref_attention(q, k, v, 0.3, False, 0)
    parts = [orc.ref_attention(q, k[a:b], v[a:b], 0.3, False, 0) for a, b in [(0, 17), (17, 64), (64, 90)]]
    o, l2 = orc.lse_merge(torch.stack([p[0] for p in parts]), torch.stack([p[1] for p in parts]))
    assert torch.allclose(o, full, atol=1e-5) and torch.allclose(l2, lse, atol=1e-5)


@pytest.mark.parametrize("case", [c for c in KAT_CASES if c[3] <= 128 and c[4] <= 512], ids=lambda c: c[0])
def test_c_oracle_agrees_on_reference_kat_cases(oracle_clib, case):
    """The plain-C restatement of tests/test_directkv_cpu_kv.cu:148-179/:372-385 and the torch oracle agree on
    the reference's own seeded cases (projection over H, attention with the s_past causal offset)."""
    name, B, NH, S_new, S_past, H, causal = case
    X, Wk, Wv, Q, K, V = kat_inputs(oracle_clib, B, NH, S_new, S_past, H)
    Kt, Vt = K.clone(), V.clone()
    O_t = orc.smpv2_fwd(X, Wk, Wv, Q, Kt, Vt, None, 128 ** -0.5, causal, S_past)
    lib = oracle_clib
    lib.dkv_ref_project.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 4
    lib.dkv_ref_attention.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int] * 3 + [ctypes.c_float, ctypes.c_int, ctypes.c_int]
    S_total = S_past + S_new
    for b in range(B):
        Yk = np.empty((S_new, NH, 128), dtype=np.float32)
        Yv = np.empty((S_new, NH, 128), dtype=np.float32)
        xb = X[b].contiguous().view(torch.int16).numpy()
        lib.dkv_ref_project(Yk.ctypes.data, xb.ctypes.data, Wk.view(torch.int16).numpy().ctypes.data, S_new, NH, 128, H)
        lib.dkv_ref_project(Yv.ctypes.data, xb.ctypes.data, Wv.view(torch.int16).numpy().ctypes.data, S_new, NH, 128, H)
        Kf = torch.cat([K[b, :S_past].float(), torch.from_numpy(Yk)], 0)
        Vf = torch.cat([V[b, :S_past].float(), torch.from_numpy(Yv)], 0)
        for h in range(NH):
            qh = Q[b, :, h].float().contiguous().numpy()
            kh, vh = Kf[:, h].contiguous().numpy(), Vf[:, h].contiguous().numpy()
            o = np.empty((S_new, 128), dtype=np.float32)
            lib.dkv_ref_attention(o.ctypes.data, qh.ctypes.data, kh.ctypes.data, vh.ctypes.data, S_new, S_total, 128,
                                  128 ** -0.5, int(causal), S_past)
            # the C oracle keeps K/V unrounded (as the reference test does); bf16 rounding of K/V moves O by < 2e-3
            assert np.abs(o - O_t[b, :, h].numpy()).max() < 2e-3, name


def test_c_oracle_paged_decode_agrees(oracle_clib):
    from directkv_b200 import workloads

    shape = workloads.LayerShape("t", 128, 8, 2, None)
    lens = [5, 33, 100]
    case = workloads.make_decode_case(shape, lens, 4, 3, "cpu")
    ref = orc.decode_layer(None, None, None, case["q"], case["k_pool"], case["v_pool"], case["page_table"], lens, 4,
                           None, shape.scale)
    out = np.empty((3, 8, 128), dtype=np.float32)
    lib = oracle_clib
    lib.dkv_ref_decode_paged.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int, ctypes.c_void_p] + [ctypes.c_int] * 5 + [ctypes.c_float]
    pt = case["page_table"].contiguous()
    sl = torch.tensor(lens, dtype=torch.int32)
    lib.dkv_ref_decode_paged(out.ctypes.data, case["q"].view(torch.int16).numpy().ctypes.data,
                             case["k_pool"].view(torch.int16).numpy().ctypes.data,
                             case["v_pool"].view(torch.int16).numpy().ctypes.data, pt.numpy().ctypes.data, pt.shape[1],
                             sl.numpy().ctypes.data, 3, 8, 2, 128, 4, shape.scale)
    assert np.abs(out - ref.numpy()).max() < 1e-4


def test_libc_stream_is_the_reference_formula(oracle_clib):
    a = libc_rand_stream(oracle_clib, 8, 0.2, 42)
    libc = ctypes.CDLL(None)
    libc.srand(42)
    rmax = 2147483647
    exp = [(np.float32(libc.rand()) / np.float32(rmax) - np.float32(0.5)) * np.float32(0.2) for _ in range(8)]
    assert np.allclose(a.numpy(), np.array(exp, dtype=np.float32), atol=1e-9)
