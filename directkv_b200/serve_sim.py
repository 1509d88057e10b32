"""Closed-loop serving simulation over the attention backend, for the serving-level benchmarks of the reference.

The reference measures token latency with an HTTP client against a running SGLang server
(benchmarks/bench_offload_serving.py, benchmarks/bench_offload_longctx.py).  Neither SGLang nor model weights
exist on the machines this package is measured on, so this module drives the backend the way SGLang's model
runner does - ``init_forward_metadata``, a forward pre-hook per attention module that hands over the layer's
hidden states, ``forward_extend`` for chunked prefill, ``forward_decode`` per layer and step, the CUDA-graph hooks -
with stand-ins for the runner, the model and the batch, and reports the reference's columns: time per output
token (mean / p50 / p90 / p99), tokens per second, time to first token.  Only the ATTENTION layers run (random
weights; no MLP, norm, sampling, scheduler or network), and arrivals are closed-loop (a fixed batch with a fraction of
the requests replaced per step), not Poisson: the rows are labelled accordingly.

The stand-ins are also what the test-suite uses (tests/fake_sglang.py re-exports them).
"""

from __future__ import annotations

import statistics
import time
import types
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn as nn

from .sglang_compat import ForwardMode
from .workloads import LayerShape

DECODE, EXTEND, IDLE = ForwardMode.DECODE, ForwardMode.EXTEND, ForwardMode.IDLE

# Columns of the reference's serving benchmark (benchmarks/bench_offload_serving.py:71-79).
SERVING_CSV_HEADER = [
    "system", "model", "dataset", "request_rate",
    "mean_latency", "p50_latency", "p90_latency", "p99_latency",
    "throughput_tps", "mean_ttft", "p99_ttft",
    "mean_e2e_latency", "p50_e2e_latency", "p90_e2e_latency", "p99_e2e_latency",
    "output_len",
    "num_completed", "num_failed",
]


# --------------------------------------------------------------------------- stand-ins for SGLang objects
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
    """An attention module as SGLang's models build it: ``qkv_proj`` (or ``k_proj`` + ``v_proj``), ``rotary_emb``,
    ``attn`` with ``layer_id`` and ``scaling``; its input is the layer's hidden states."""

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


# --------------------------------------------------------------------------- the simulation
def _host_memory_available() -> Optional[int]:
    try:
        with open("/proc/meminfo") as f:
            for line in f:
                if line.startswith("MemAvailable:"):
                    return int(line.split()[1]) * 1024
    except OSError:
        pass
    return None


def _pct(xs: Sequence[float], q: float) -> float:
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(round(q * (len(xs) - 1))))]


class ServeSim:
    """A fixed batch of requests served by the ``directkv-smpv2`` backend over a host-pinned request pool.

    ``layers`` attention layers are built (weights and pool rows of their own); one token passes through them
    ``layer_repeats`` times, so a 32-layer model is ``layers=4, layer_repeats=8`` with an eighth of the pinned
    memory (the KV of every pass still crosses the host link; what is shared is only the storage).  The backend
    keeps at most 64 request rows, like the reference (directkv/directkv_backend.py:174-197).
    """

    def __init__(self, shape: LayerShape, max_reqs: int, context_len: int, device, layers: int = 4,
                 layer_repeats: int = 8, chunk: int = 4096, seed: int = 0):
        import directkv_b200

        self.shape, self.device, self.chunk = shape, torch.device(device), int(chunk)
        self.layers, self.repeats = layers, layer_repeats
        self.model = FakeModel(layers, shape.hidden, shape.nh_q, shape.nh_kv, shape.rope_theta, context_len,
                               fused_qkv=shape.rope_theta is not None).to(self.device)
        self.runner = make_runner(self.model, shape.hidden, shape.nh_q, shape.nh_kv, layers, self.device,
                                  max_reqs=max_reqs, context_len=context_len)
        self.backend = directkv_b200.DirectKVSmpV2Backend(self.runner)
        self.gen = torch.Generator(device=self.device).manual_seed(4321 + seed)
        self.lengths: Dict[int, int] = {}
        self._graphs: Dict[int, tuple] = {}

    def _rand(self, rows: int, cols: int) -> torch.Tensor:
        return torch.randn(rows, cols, generator=self.gen, device=self.device, dtype=torch.float32).to(torch.bfloat16)

    def _layer_passes(self):
        for _ in range(self.repeats):
            for layer in self.model.layers:
                yield layer

    # ---- prefill ----------------------------------------------------------------------------------------
    def prefill(self, rid: int, n_tokens: int) -> float:
        """Chunked prefill of one request; returns the seconds it took (its time to first token)."""
        torch.cuda.synchronize(self.device)
        t0 = time.perf_counter()
        done = 0
        while done < n_tokens:
            n = min(self.chunk, n_tokens - done)
            fb = make_batch(EXTEND, [done + n], [rid], self.device, extend_lens=[n], prefix_lens=[done])
            self.backend.init_forward_metadata(fb)
            x = self._rand(n, self.shape.hidden)
            q = self._rand(n, self.shape.nh_q * 128)
            for layer in self._layer_passes():
                layer(hidden_states=x)
                self.backend.forward_extend(q, None, None, layer.attn, fb)
            done += n
        torch.cuda.synchronize(self.device)
        self.lengths[rid] = n_tokens
        return time.perf_counter() - t0

    # ---- decode -----------------------------------------------------------------------------------------
    def decode_step(self, rids: List[int]) -> float:
        """One decoded token for every request of the batch, eager launches; returns the seconds it took."""
        bs = len(rids)
        lens = [self.lengths[r] + 1 for r in rids]
        x = self._rand(bs, self.shape.hidden)
        q = self._rand(bs, self.shape.nh_q * 128)
        torch.cuda.synchronize(self.device)
        t0 = time.perf_counter()
        fb = make_batch(DECODE, lens, rids, self.device)
        fb.seq_lens_cpu = torch.tensor(lens, dtype=torch.int64)
        self.backend.init_forward_metadata(fb)
        for layer in self._layer_passes():
            layer(hidden_states=x)
            self.backend.forward_decode(q, None, None, layer.attn, fb)
        torch.cuda.synchronize(self.device)
        dt = time.perf_counter() - t0
        for r in rids:
            self.lengths[r] += 1
        return dt

    def _graph_for(self, bs: int):
        if bs in self._graphs:
            return self._graphs[bs]
        be, dev = self.backend, self.device
        if not self._graphs:
            be.init_cuda_graph_state(max(bs, self.runner.req_to_token_pool.size), max(bs, self.runner.req_to_token_pool.size))
        x_s = torch.zeros(bs, self.shape.hidden, dtype=torch.bfloat16, device=dev)
        q_s = torch.zeros(bs, self.shape.nh_q * 128, dtype=torch.bfloat16, device=dev)
        fill = be.get_cuda_graph_seq_len_fill_value()
        rpi = torch.zeros(bs, dtype=torch.int64, device=dev)
        sl = torch.full((bs,), fill, dtype=torch.int64, device=dev)
        be.init_forward_metadata_capture_cuda_graph(bs, bs, rpi, sl, None, DECODE, None)
        fb = make_batch(DECODE, [fill] * bs, [0] * bs, dev)

        def body():
            for layer in self._layer_passes():
                layer(hidden_states=x_s)
                be.forward_decode(q_s, None, None, layer.attn, fb)

        s = torch.cuda.Stream(device=dev)
        s.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(s):
            body()
        torch.cuda.current_stream(dev).wait_stream(s)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            body()
        torch.cuda.synchronize(dev)
        self._graphs[bs] = (graph, x_s, q_s, rpi)
        return self._graphs[bs]

    def decode_step_graph(self, rids: List[int]) -> float:
        """The same step replayed from a CUDA graph of all layer passes (captured once per batch size)."""
        bs = len(rids)
        graph, x_s, q_s, rpi = self._graph_for(bs)
        lens = [self.lengths[r] + 1 for r in rids]
        x_s.copy_(self._rand(bs, self.shape.hidden))
        q_s.copy_(self._rand(bs, self.shape.nh_q * 128))
        rpi.copy_(torch.tensor(rids, dtype=torch.int64))
        sl = torch.tensor(lens, dtype=torch.int64)
        sl_dev = sl.to(self.device)
        torch.cuda.synchronize(self.device)
        t0 = time.perf_counter()
        self.backend.init_forward_metadata_replay_cuda_graph(bs, rpi, sl_dev, sum(lens), None, DECODE, None, seq_lens_cpu=sl)
        graph.replay()
        torch.cuda.synchronize(self.device)
        dt = time.perf_counter() - t0
        for r in rids:
            self.lengths[r] += 1
        return dt


def run_config(name: str, shape: LayerShape, ctx_lens: Sequence[int], device, decode_steps: int = 12, churn: float = 0.0,
               fresh_lens: Optional[Sequence[int]] = None, use_graph: bool = False, layers: int = 4, layer_repeats: int = 8,
               chunk: int = 4096, seed: int = 0, check_each_step: bool = False) -> dict:
    """Prefills ``ctx_lens`` requests, then decodes ``decode_steps`` tokens for the whole batch; with ``churn`` that
    fraction of the requests is replaced before every step after the first by new ones (lengths from
    ``fresh_lens`` in turn), whose prefill counts as their time to first token.  Returns one row in the reference's
    serving columns plus the raw figures."""
    from ._lib import get_context

    dev = torch.device(device)
    n_req = len(ctx_lens)
    max_ctx = max(list(ctx_lens) + list(fresh_lens or [0])) + decode_steps + 64
    # The request pool is page-locked host memory: refuse a configuration that would take more than half of what
    # the machine has free rather than push it into swapping.
    n_swap = int(round(churn * n_req)) if fresh_lens else 0
    pool_rows = min(n_req + n_swap + 1, 64) + 1
    pool_bytes = 2 * layers * pool_rows * (-(-max_ctx // 64) * 64) * shape.nh_kv * 128 * 2
    avail = _host_memory_available()
    if avail is not None and pool_bytes > avail // 2:
        raise RuntimeError(f"serve_sim: the request pool of '{name}' needs {pool_bytes / 2**30:.1f} GiB of pinned host memory, "
                           f"more than half of the {avail / 2**30:.1f} GiB available")
    # Rows: the batch, the requests that join before those they replace are seen to be gone, and the warm-up request.
    sim = ServeSim(shape, max_reqs=n_req + n_swap + 1, context_len=max_ctx, device=dev, layers=layers,
                   layer_repeats=layer_repeats, chunk=chunk, seed=seed)
    sim.prefill(n_req, 16)                        # untimed: allocates the pool, registers the layers, first launches
    sim.lengths.pop(n_req, None)                  # (its row is released at the first decode step, where it is absent)
    ttft = []
    rids = list(range(n_req))
    for rid, n in zip(rids, ctx_lens):
        ttft.append(sim.prefill(rid, int(n)))
    step = sim.decode_step_graph if use_graph else sim.decode_step
    ctx = get_context(dev.index)

    def check(what):
        if check_each_step:                       # find the step a device-side failure belongs to (synchronises)
            st = ctx.read_status(clear=False)
            if st:
                raise RuntimeError(f"serve_sim: device status {st:#x} after {what}")

    check("the prefill of the batch")
    step(rids)                                    # untimed warm-up step (graph capture, first-use set-up)
    check("the warm-up decode step")
    tpot, next_rid, fresh_i = [], n_req + 1, 0
    g = torch.Generator().manual_seed(99 + seed)
    for s in range(decode_steps):
        if s and n_swap and fresh_lens:
            for i in torch.randperm(n_req, generator=g)[:n_swap].tolist():
                # the leaving request's row is released by the backend at the next decode step (it is absent)
                old = rids[i]
                sim.lengths.pop(old, None)
                rids[i] = next_rid
                ttft.append(sim.prefill(next_rid, int(fresh_lens[fresh_i % len(fresh_lens)])))
                check(f"the prefill of request {next_rid} ({fresh_lens[fresh_i % len(fresh_lens)]} tokens) before step {s}")
                next_rid += 1
                fresh_i += 1
        tpot.append(step(rids))
        check(f"decode step {s}")
    ctx.raise_on_status()
    mean = statistics.mean(tpot)
    layers_total = layers * layer_repeats
    row = {
        "system": f"directkv-b200 ({'cuda-graph' if use_graph else 'eager'}; attention layers only, synthetic weights)",
        "model": f"{shape.name}, {layers_total} attention layers ({layers} stored, passed {layer_repeats}x)",
        "dataset": f"synthetic: {name}", "request_rate": "closed loop",
        "mean_latency": mean, "p50_latency": _pct(tpot, 0.5), "p90_latency": _pct(tpot, 0.9), "p99_latency": _pct(tpot, 0.99),
        "throughput_tps": n_req / mean, "mean_ttft": statistics.mean(ttft), "p99_ttft": _pct(ttft, 0.99),
        "output_len": decode_steps, "num_completed": n_req, "num_failed": 0,
    }
    kv_bytes = sum(sim.lengths[r] for r in rids) * shape.kv_bytes_per_token() * layers_total
    row_extra = {"config": name, "requests": n_req, "tokens_in_batch": int(sum(sim.lengths[r] for r in rids)),
                 "kv_gbs": kv_bytes / _pct(tpot, 0.5) / 1e9, "graph": use_graph}
    del sim
    torch.cuda.empty_cache()
    return {**row, **row_extra}
