"""Shared helpers of the test-suite: tolerance check, oracle wrappers, libc rand() streams."""

from __future__ import annotations

import ctypes
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from oracle import directkv_oracle as orc  # noqa: E402

# Parity bar for outputs: |out - oracle| <= 2e-2 + 1e-2 * |oracle| (bf16 storage, fp32 accumulate).
ATOL, RTOL = 2e-2, 1e-2
# Stored K/V rows: the reference's own threshold (tests/test_directkv_cpu_kv.cu:478-480).
KV_ATOL = 1e-2


def assert_close(out: torch.Tensor, ref: torch.Tensor, what: str = "O", atol: float = ATOL, rtol: float = RTOL):
    out = out.detach().float().cpu()
    ref = ref.detach().float().cpu()
    assert out.shape == ref.shape, f"{what}: shape {tuple(out.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(out).all(), f"{what}: non-finite values"
    err = (out - ref).abs()
    bound = atol + rtol * ref.abs()
    bad = err > bound
    assert not bad.any(), (f"{what}: {int(bad.sum())} of {bad.numel()} elements outside tolerance; "
                           f"max abs err {err.max().item():.4e}")
    return err.max().item()


def libc_rand_stream(clib, n: int, mul: float, seed: int, reseed: bool = True) -> torch.Tensor:
    """(rand()/RAND_MAX - 0.5) * mul for n draws (tests/test_directkv_cpu_kv.cu:184-188, :252-254)."""
    out = np.empty(n, dtype=np.float32)
    clib.dkv_ref_rand_stream.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_float, ctypes.c_uint, ctypes.c_int]
    clib.dkv_ref_rand_stream.restype = None
    clib.dkv_ref_rand_stream(out.ctypes.data, n, mul, seed, 1 if reseed else 0)
    return torch.from_numpy(out)


def kat_inputs(clib, B, NH, S_new, S_past, H, D=128):
    """Inputs of one case of the reference's kernel test (tests/test_directkv_cpu_kv.cu:230-275)."""
    S_total = S_past + S_new
    X = libc_rand_stream(clib, B * S_new * H, 0.2, 42).view(B, S_new, H).to(torch.bfloat16)
    Wk = libc_rand_stream(clib, NH * D * H, 0.2, 43).view(NH, D, H).to(torch.bfloat16)
    Wv = libc_rand_stream(clib, NH * D * H, 0.2, 44).view(NH, D, H).to(torch.bfloat16)
    Q = libc_rand_stream(clib, B * S_new * NH * D, 0.2, 45).view(B, S_new, NH, D).to(torch.bfloat16)
    K = torch.zeros(B, S_total, NH, D, dtype=torch.bfloat16)
    V = torch.zeros(B, S_total, NH, D, dtype=torch.bfloat16)
    if S_past > 0:
        n = B * S_past * NH * D
        kp = libc_rand_stream(clib, n, 0.2, 99, reseed=True).view(B, S_past, NH, D)
        vp = libc_rand_stream(clib, n, 0.2, 99, reseed=False).view(B, S_past, NH, D)
        K[:, :S_past] = kp.to(torch.bfloat16)
        V[:, :S_past] = vp.to(torch.bfloat16)
    return X, Wk, Wv, Q, K, V


# The 12 seeded configurations of tests/test_directkv_cpu_kv.cu:538-557
KAT_CASES = [
    # name, B, NH, S_new, S_past, H, causal
    ("pf-tiny", 1, 2, 64, 0, 128, False),
    ("pf-tiny-causal", 1, 2, 64, 0, 128, True),
    ("pf-small-causal", 1, 8, 512, 0, 128, True),
    ("pf-1k-causal", 1, 8, 1024, 0, 128, True),
    ("pf-1k-noncausal", 1, 8, 1024, 0, 128, False),
    ("pf-b4", 4, 8, 512, 0, 128, True),
    ("dec-tiny", 1, 2, 64, 128, 128, True),
    ("dec-small", 1, 8, 64, 512, 128, True),
    ("dec-medium", 1, 8, 128, 1024, 128, True),
    ("dec-noncausal", 1, 4, 128, 512, 128, False),
    ("dec-b4", 4, 8, 64, 256, 128, True),
    ("dec-longctx", 1, 8, 64, 4096, 128, True),
]
