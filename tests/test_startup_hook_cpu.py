"""Registration of the backends in SGLang (directkv/directkv_startup_hook.py:84-229 in the reference), against
stand-ins for the SGLang modules it touches: both API generations, the factories' errors, the pool swap, and the
deferred registration that fires when SGLang is imported later."""

import importlib
import sys
import types

import pytest
import torch

from directkv_b200 import directkv_startup_hook as hook
from directkv_b200.directkv_pool import DirectKVTokenToKVPool


def _mod(monkeypatch, name, **attrs):
    m = types.ModuleType(name)
    for k, v in attrs.items():
        setattr(m, k, v)
    monkeypatch.setitem(sys.modules, name, m)
    return m


def _parents(monkeypatch, dotted):
    parts = dotted.split(".")
    for i in range(1, len(parts)):
        name = ".".join(parts[:i])
        if name not in sys.modules:
            m = _mod(monkeypatch, name)
            m.__path__ = []  # a package


def _runner(backend="directkv", radix_off=True, graph_off=True, mla=False):
    sa = types.SimpleNamespace(attention_backend=backend, disable_radix_cache=radix_off, disable_cuda_graph=graph_off,
                               enable_memory_saver=False)
    cfg = types.SimpleNamespace(head_dim=128, context_len=256, get_num_kv_heads=lambda tp: 4)
    return types.SimpleNamespace(server_args=sa, model_config=cfg, use_mla_backend=mla, max_total_num_tokens=64,
                                 page_size=1, kv_cache_dtype=torch.bfloat16, num_effective_layers=2, start_layer=0,
                                 end_layer=1, device="cpu", max_running_requests=4, req_to_token_pool=None)


class _Allocator:
    def __init__(self, size, dtype=None, device=None, kvcache=None, **extra):
        self.size, self.kvcache, self.extra = size, kvcache, extra


class _ReqToTokenPool:
    def __init__(self, size, max_context_len, device, enable_memory_saver):
        self.size, self.max_context_len = size, max_context_len


@pytest.fixture
def fake_backends(monkeypatch):
    """The factories build these instead of engines that need a GPU."""
    import directkv_b200.directkv_backend as b1
    import directkv_b200.directkv_smpv2_backend as b2

    class A:
        def __init__(self, runner):
            self.runner = runner

    class B(A):
        pass

    monkeypatch.setattr(b1, "DirectKVBackend", A)
    monkeypatch.setattr(b2, "DirectKVSmpV2Backend", B)
    return A, B


@pytest.fixture
def registry_sglang(monkeypatch):
    """SGLang >= 0.5: attention_registry, server_args choices, ModelRunnerKVCacheMixin._init_pools."""
    _parents(monkeypatch, hook.REGISTRY_MODULE)
    backends = {}

    def register_attention_backend(name):
        def deco(fn):
            backends[name] = fn
            return fn
        return deco

    reg = _mod(monkeypatch, hook.REGISTRY_MODULE, ATTENTION_BACKENDS=backends,
               register_attention_backend=register_attention_backend)
    sa = _mod(monkeypatch, "sglang.srt.server_args", ATTENTION_BACKEND_CHOICES=["flashinfer", "triton"])
    calls = []

    class ModelRunnerKVCacheMixin:
        def _init_pools(self, *a, **k):
            calls.append("original")

    _parents(monkeypatch, "sglang.srt.model_executor.model_runner_kv_cache_mixin")
    mixin = _mod(monkeypatch, "sglang.srt.model_executor.model_runner_kv_cache_mixin",
                 ModelRunnerKVCacheMixin=ModelRunnerKVCacheMixin)
    _parents(monkeypatch, "sglang.srt.mem_cache.allocator")
    _mod(monkeypatch, "sglang.srt.mem_cache.allocator", TokenToKVPoolAllocator=_Allocator)
    _mod(monkeypatch, "sglang.srt.mem_cache.memory_pool", ReqToTokenPool=_ReqToTokenPool)
    return types.SimpleNamespace(reg=reg, sa=sa, mixin=mixin, calls=calls, backends=backends)


def test_registry_route(registry_sglang, fake_backends):
    A, B = fake_backends
    assert hook.register() == "registry" and hook.route_taken() == "registry"
    assert set(hook.BACKEND_NAMES) <= set(registry_sglang.backends)
    assert registry_sglang.sa.ATTENTION_BACKEND_CHOICES[-2:] == ["directkv", "directkv-smpv2"]
    assert isinstance(registry_sglang.backends["directkv"](_runner()), A)
    assert isinstance(registry_sglang.backends["directkv-smpv2"](_runner("directkv-smpv2", graph_off=False)), B)
    # Registering twice changes nothing.
    patched = registry_sglang.mixin.ModelRunnerKVCacheMixin._init_pools
    hook.register()
    assert registry_sglang.mixin.ModelRunnerKVCacheMixin._init_pools is patched
    assert registry_sglang.sa.ATTENTION_BACKEND_CHOICES.count("directkv") == 1


def test_factory_errors(registry_sglang, fake_backends):
    hook.register()
    mk = registry_sglang.backends
    with pytest.raises(ValueError, match="--disable-radix-cache"):
        mk["directkv"](_runner(radix_off=False))
    with pytest.raises(ValueError, match="--disable-cuda-graph"):
        mk["directkv"](_runner(graph_off=False))
    with pytest.raises(ValueError, match="MLA"):
        mk["directkv"](_runner(mla=True))
    with pytest.raises(ValueError, match="directkv-smpv2 requires --disable-radix-cache"):
        mk["directkv-smpv2"](_runner("directkv-smpv2", radix_off=False))
    with pytest.raises(ValueError, match="MLA"):
        mk["directkv-smpv2"](_runner("directkv-smpv2", mla=True))


def test_registry_route_pool_init(registry_sglang):
    hook.register()
    cls = registry_sglang.mixin.ModelRunnerKVCacheMixin
    other = _runner(backend="flashinfer")
    cls._init_pools(other)
    assert registry_sglang.calls == ["original"] and not hasattr(other, "token_to_kv_pool")
    r = _runner(backend="directkv-smpv2")
    cls._init_pools(r)
    assert registry_sglang.calls == ["original"]
    assert isinstance(r.token_to_kv_pool, DirectKVTokenToKVPool)
    assert r.token_to_kv_pool.get_key_buffer(0).shape[1:] == (4, 128)
    assert isinstance(r.req_to_token_pool, _ReqToTokenPool) and r.req_to_token_pool.max_context_len == 260
    assert r.token_to_kv_pool_allocator.kvcache is r.token_to_kv_pool
    assert r.token_to_kv_pool_allocator.extra == {"need_sort": False}


@pytest.fixture
def legacy_sglang(monkeypatch):
    """SGLang 0.4.x: ModelRunner._get_attention_backend_from_str and ModelRunner.init_memory_pool."""
    _parents(monkeypatch, hook.MODEL_RUNNER_MODULE)
    calls = []

    class ModelRunner:
        def _get_attention_backend_from_str(self, backend_str):
            calls.append(("backend", backend_str))
            return backend_str

        def init_memory_pool(self, total_gpu_memory, max_num_reqs=None, max_total_tokens=None):
            calls.append(("pool", total_gpu_memory, max_num_reqs, max_total_tokens))
            self.token_to_kv_pool = "gpu pool"

    mr = _mod(monkeypatch, hook.MODEL_RUNNER_MODULE, ModelRunner=ModelRunner)
    _parents(monkeypatch, "sglang.srt.mem_cache.allocator")
    _mod(monkeypatch, "sglang.srt.mem_cache.allocator", TokenToKVPoolAllocator=_Allocator)
    return types.SimpleNamespace(mr=mr, calls=calls)


def test_model_runner_route(legacy_sglang, fake_backends):
    A, B = fake_backends
    assert hook.register() == "model_runner"
    cls = legacy_sglang.mr.ModelRunner

    def runner(**kw):
        r = cls()
        r.__dict__.update(_runner(**kw).__dict__)
        return r

    r = runner()
    assert isinstance(r._get_attention_backend_from_str("directkv"), A)
    assert isinstance(r._get_attention_backend_from_str("directkv-smpv2"), B)
    assert r._get_attention_backend_from_str("triton") == "triton" and legacy_sglang.calls == [("backend", "triton")]
    with pytest.raises(ValueError, match="--disable-cuda-graph"):
        runner(graph_off=False)._get_attention_backend_from_str("directkv")

    r.init_memory_pool(0.5, 8, 64)
    assert legacy_sglang.calls[-1] == ("pool", 0.5, 8, 64)
    assert isinstance(r.token_to_kv_pool, DirectKVTokenToKVPool)
    assert r.token_to_kv_pool_allocator.kvcache is r.token_to_kv_pool
    other = runner(backend="flashinfer")
    other.init_memory_pool(0.5)
    assert other.token_to_kv_pool == "gpu pool"
    # Idempotent.
    patched = cls.init_memory_pool
    hook.register()
    assert cls.init_memory_pool is patched


def test_deferred_registration(tmp_path, monkeypatch, fake_backends):
    """install() before SGLang is imported: the finder registers right after the module body ran and removes itself."""
    for name in [n for n in sys.modules if n == "sglang" or n.startswith("sglang.")]:
        monkeypatch.delitem(sys.modules, name)
    pkg = tmp_path / "sglang" / "srt" / "model_executor"
    pkg.mkdir(parents=True)
    for d in (tmp_path / "sglang", tmp_path / "sglang" / "srt", pkg):
        (d / "__init__.py").write_text("")
    (pkg / "model_runner.py").write_text(
        "class ModelRunner:\n"
        "    def _get_attention_backend_from_str(self, s):\n        return s\n"
        "    def init_memory_pool(self, total_gpu_memory, max_num_reqs=None, max_total_tokens=None):\n        pass\n")
    monkeypatch.syspath_prepend(str(tmp_path))
    importlib.invalidate_caches()
    try:
        assert hook.install() is None
        assert any(isinstance(f, hook._RegisterAfterImport) for f in sys.meta_path)
        importlib.import_module("sglang.srt")                       # other SGLang modules pass through untouched
        assert any(isinstance(f, hook._RegisterAfterImport) for f in sys.meta_path)
        mr = importlib.import_module(hook.MODEL_RUNNER_MODULE)
        assert getattr(mr.ModelRunner.init_memory_pool, "_directkv_patched", False)
        assert not any(isinstance(f, hook._RegisterAfterImport) for f in sys.meta_path)
        assert hook.route_taken() == "model_runner"
    finally:
        hook.uninstall()
        for name in [n for n in sys.modules if n == "sglang" or n.startswith("sglang.")]:
            monkeypatch.delitem(sys.modules, name, raising=False)
