"""Test doubles for the SGLang objects the attention backend talks to (SGLang is not installed):
a model whose attention modules look like SGLang's (``qkv_proj`` / ``k_proj``+``v_proj``, ``rotary_emb``,
``attn`` with ``layer_id`` and ``scaling``), a model runner, and a forward batch."""

from __future__ import annotations

import types

import torch
import torch.nn as nn

from directkv_b200.sglang_compat import ForwardMode


class FakeRadixAttention(nn.Module):
    def __init__(self, layer_id: int, scaling: float):
        super().__init__()
        self.layer_id = layer_id
        self.scaling = scaling


class FakeRotary:
    def __init__(self, theta: float, max_pos: int):
        self.inv_freq = 1.0 / (theta ** (torch.arange(0, 64, dtype=torch.float32) / 64))
        self.max_position_embeddings = max_pos


class FakeSelfAttention(nn.Module):
    def __init__(self, layer_id, hidden, nh_q, nh_kv, theta, max_pos, fused_qkv=True, seed=0):
        super().__init__()
        g = torch.Generator().manual_seed(1000 + seed + layer_id)
        d = 128
        if fused_qkv:
            self.qkv_proj = nn.Linear(hidden, (nh_q + 2 * nh_kv) * d, bias=False, dtype=torch.bfloat16)
            self.qkv_proj.weight.data = (torch.randn(self.qkv_proj.weight.shape, generator=g) * 0.02).to(torch.bfloat16)
        else:
            self.k_proj = nn.Linear(hidden, nh_kv * d, bias=False, dtype=torch.bfloat16)
            self.v_proj = nn.Linear(hidden, nh_kv * d, bias=False, dtype=torch.bfloat16)
            self.k_proj.weight.data = (torch.randn(self.k_proj.weight.shape, generator=g) * 0.02).to(torch.bfloat16)
            self.v_proj.weight.data = (torch.randn(self.v_proj.weight.shape, generator=g) * 0.02).to(torch.bfloat16)
        if theta is not None:
            self.rotary_emb = FakeRotary(theta, max_pos)
        self.attn = FakeRadixAttention(layer_id, d ** -0.5)

    def forward(self, hidden_states=None):
        return hidden_states


class FakeModel(nn.Module):
    def __init__(self, n_layers, hidden, nh_q, nh_kv, theta, max_pos, fused_qkv=True):
        super().__init__()
        self.layers = nn.ModuleList(
            [FakeSelfAttention(i, hidden, nh_q, nh_kv, theta, max_pos, fused_qkv) for i in range(n_layers)])


def make_runner(model, hidden, nh_q, nh_kv, n_layers, device, max_reqs=8, context_len=512, head_dim=128,
                dtype=torch.bfloat16, disable_radix_cache=True):
    cfg = types.SimpleNamespace(
        num_attention_heads=nh_q, head_dim=head_dim, hidden_size=hidden, dtype=dtype, context_len=context_len,
        num_hidden_layers=n_layers, get_num_kv_heads=lambda tp: nh_kv // tp)
    r2t = types.SimpleNamespace(size=max_reqs,
                                req_to_token=torch.zeros(max_reqs, context_len, dtype=torch.int32, device=device))
    return types.SimpleNamespace(model_config=cfg, server_args=types.SimpleNamespace(disable_radix_cache=disable_radix_cache),
                                 req_to_token_pool=r2t, model=model, device=device)


def make_batch(mode, seq_lens, req_ids, device, extend_lens=None, prefix_lens=None, token_pool=None, req_to_token_pool=None,
               out_cache_loc=None):
    return types.SimpleNamespace(
        forward_mode=mode, batch_size=len(seq_lens),
        seq_lens=torch.tensor(seq_lens, dtype=torch.int64, device=device),
        req_pool_indices=torch.tensor(req_ids, dtype=torch.int64, device=device),
        extend_seq_lens_cpu=extend_lens, extend_prefix_lens_cpu=prefix_lens,
        token_to_kv_pool=token_pool, req_to_token_pool=req_to_token_pool, out_cache_loc=out_cache_loc)


DECODE, EXTEND, IDLE = ForwardMode.DECODE, ForwardMode.EXTEND, ForwardMode.IDLE
