"""Registration of the ``directkv`` and ``directkv-smpv2`` attention backends in SGLang.

Same effect as the reference's startup hook (directkv/directkv_startup_hook.py:84-229): after it ran,
``--attention-backend directkv`` / ``directkv-smpv2`` select :class:`DirectKVBackend` /
:class:`DirectKVSmpV2Backend`, and the model runner's KV pool is a host-pinned
:class:`DirectKVTokenToKVPool`.  Both SGLang API generations are handled:

* 0.5 and later: ``attention_registry.register_attention_backend`` plus
  ``ModelRunnerKVCacheMixin._init_pools`` (directkv_startup_hook.py:115-168, 264-320);
* 0.4.x: ``ModelRunner._get_attention_backend_from_str`` and ``ModelRunner.init_memory_pool``
  (directkv_startup_hook.py:175-229, 232-262).

The factories raise the reference's ``ValueError`` for a radix cache that is not disabled, for CUDA graphs with
``directkv``, and for MLA models.

Differences in mechanism, not in effect: nothing is done at interpreter start-up and ``builtins.__import__`` is
left alone.  Call :func:`register` once SGLang's modules are imported (it returns which route it took), or
:func:`install` earlier: that puts a finder on ``sys.meta_path`` which registers as soon as one of the two SGLang
modules finishes importing, then removes itself.
"""

from __future__ import annotations

import importlib.abc
import importlib.util
import logging
import sys
from typing import Callable, Optional

log = logging.getLogger(__name__)

BACKEND_NAMES = ("directkv", "directkv-smpv2")
REGISTRY_MODULE = "sglang.srt.layers.attention.attention_registry"
MODEL_RUNNER_MODULE = "sglang.srt.model_executor.model_runner"
_PATCH_MARK = "_directkv_patched"

_route_taken: Optional[str] = None


# ---------------------------------------------------------------------------------------------------------
# Backend factories (checks and messages of directkv_startup_hook.py:120-137, 184-214)
# ---------------------------------------------------------------------------------------------------------
def _check_server_args(runner, name: str) -> None:
    sa = runner.server_args
    if not sa.disable_radix_cache:
        raise ValueError(f"{name} requires --disable-radix-cache. Add this flag when launching the server.")
    if name == "directkv" and not sa.disable_cuda_graph:
        raise ValueError("directkv requires --disable-cuda-graph. Add this flag when launching the server.")
    if getattr(runner, "use_mla_backend", False):
        raise ValueError(f"{name} does not support MLA models.")


def create_directkv_backend(runner):
    _check_server_args(runner, "directkv")
    from .directkv_backend import DirectKVBackend

    log.info("Using DirectKV attention backend (host-pinned KV cache)")
    return DirectKVBackend(runner)


def create_directkv_smpv2_backend(runner):
    _check_server_args(runner, "directkv-smpv2")
    from .directkv_smpv2_backend import DirectKVSmpV2Backend

    log.info("Using DirectKV-SMPv2 backend (fused projection)")
    return DirectKVSmpV2Backend(runner)


_FACTORIES = {"directkv": create_directkv_backend, "directkv-smpv2": create_directkv_smpv2_backend}


# ---------------------------------------------------------------------------------------------------------
# Pool swap
# ---------------------------------------------------------------------------------------------------------
def _selected(runner) -> bool:
    return getattr(runner.server_args, "attention_backend", None) in BACKEND_NAMES


def _make_token_pool(runner):
    from .directkv_pool import DirectKVTokenToKVPool
    from .sglang_compat import get_attention_tp_size

    cfg = runner.model_config
    head_dim = cfg.head_dim
    return DirectKVTokenToKVPool(
        size=runner.max_total_num_tokens,
        page_size=runner.page_size,
        dtype=runner.kv_cache_dtype,
        head_num=cfg.get_num_kv_heads(get_attention_tp_size()),
        head_dim=head_dim,
        layer_num=runner.num_effective_layers,
        v_head_dim=getattr(cfg, "v_head_dim", None) or head_dim,
        start_layer=runner.start_layer,
        end_layer=runner.end_layer,
    )


def _make_allocator(runner, **extra):
    """SGLang's token allocator over the new pool (directkv_startup_hook.py:253-258, 311-318); ``None`` when this
    SGLang has no such class."""
    try:
        from sglang.srt.mem_cache.allocator import TokenToKVPoolAllocator  # type: ignore
    except ImportError:
        return None
    return TokenToKVPoolAllocator(runner.max_total_num_tokens, dtype=runner.kv_cache_dtype, device=runner.device,
                                  kvcache=runner.token_to_kv_pool, **extra)


def replace_pool(runner) -> None:
    """0.4.x route: SGLang built its GPU pool already; put the host-pinned one in its place."""
    runner.token_to_kv_pool = _make_token_pool(runner)
    alloc = _make_allocator(runner)
    if alloc is not None:
        runner.token_to_kv_pool_allocator = alloc
    log.info("DirectKV pool: %d tokens in host-pinned memory", runner.max_total_num_tokens)


def init_pools(runner) -> None:
    """0.5 route: build the request-to-token table (when absent), the host-pinned pool and its allocator."""
    if getattr(runner, "req_to_token_pool", None) is None:
        from sglang.srt.mem_cache.memory_pool import ReqToTokenPool  # type: ignore

        runner.req_to_token_pool = ReqToTokenPool(
            size=runner.max_running_requests,
            max_context_len=runner.model_config.context_len + 4,
            device=runner.device,
            enable_memory_saver=runner.server_args.enable_memory_saver,
        )
    runner.token_to_kv_pool = _make_token_pool(runner)
    alloc = _make_allocator(runner, need_sort=False)
    if alloc is not None:
        runner.token_to_kv_pool_allocator = alloc


# ---------------------------------------------------------------------------------------------------------
# The two registration routes
# ---------------------------------------------------------------------------------------------------------
def _already(fn: Callable) -> bool:
    return bool(getattr(fn, _PATCH_MARK, False))


def _register_via_registry(reg_mod) -> None:
    backends = reg_mod.ATTENTION_BACKENDS
    for name, factory in _FACTORIES.items():
        if name not in backends:
            reg_mod.register_attention_backend(name)(factory)
    sa_mod = sys.modules.get("sglang.srt.server_args")
    choices = getattr(sa_mod, "ATTENTION_BACKEND_CHOICES", None) if sa_mod is not None else None
    if choices is not None:
        for name in BACKEND_NAMES:
            if name not in choices:
                choices.append(name)
    try:
        mixin_mod = importlib.import_module("sglang.srt.model_executor.model_runner_kv_cache_mixin")
        cls = mixin_mod.ModelRunnerKVCacheMixin
        original = cls._init_pools
    except (ImportError, AttributeError):
        return
    if _already(original):
        return

    def _init_pools(self, *args, **kwargs):
        if _selected(self):
            init_pools(self)
        else:
            original(self, *args, **kwargs)

    setattr(_init_pools, _PATCH_MARK, True)
    cls._init_pools = _init_pools


def _register_via_model_runner(mr_mod) -> None:
    runner_cls = mr_mod.ModelRunner
    get_backend = getattr(runner_cls, "_get_attention_backend_from_str", None)
    if get_backend is not None and not _already(get_backend):

        def _get_attention_backend_from_str(self, backend_str):
            factory = _FACTORIES.get(backend_str)
            return factory(self) if factory is not None else get_backend(self, backend_str)

        setattr(_get_attention_backend_from_str, _PATCH_MARK, True)
        runner_cls._get_attention_backend_from_str = _get_attention_backend_from_str

    init_pool = getattr(runner_cls, "init_memory_pool", None)
    if init_pool is not None and not _already(init_pool):

        def init_memory_pool(self, total_gpu_memory, max_num_reqs=None, max_total_tokens=None):
            init_pool(self, total_gpu_memory, max_num_reqs, max_total_tokens)
            if _selected(self):
                replace_pool(self)

        setattr(init_memory_pool, _PATCH_MARK, True)
        runner_cls.init_memory_pool = init_memory_pool


def register() -> Optional[str]:
    """Registers with whichever SGLang API is loaded.  Returns ``"registry"``, ``"model_runner"`` or ``None`` when
    neither module has been imported yet.  Idempotent."""
    global _route_taken
    reg_mod = sys.modules.get(REGISTRY_MODULE)
    if reg_mod is not None and hasattr(reg_mod, "ATTENTION_BACKENDS"):
        _register_via_registry(reg_mod)
        _route_taken = "registry"
        return _route_taken
    mr_mod = sys.modules.get(MODEL_RUNNER_MODULE)
    if mr_mod is not None and hasattr(mr_mod, "ModelRunner"):
        _register_via_model_runner(mr_mod)
        _route_taken = "model_runner"
        return _route_taken
    return None


def route_taken() -> Optional[str]:
    return _route_taken


# ---------------------------------------------------------------------------------------------------------
# Deferred registration: a finder that watches for the two SGLang modules
# ---------------------------------------------------------------------------------------------------------
class _RegisterAfterImport(importlib.abc.MetaPathFinder):
    """Delegates to the other finders; when the found module is one of the two SGLang modules, its loader is
    wrapped so that :func:`register` runs right after the module body."""

    def find_spec(self, fullname, path=None, target=None):
        if fullname not in (REGISTRY_MODULE, MODEL_RUNNER_MODULE):
            return None
        for finder in sys.meta_path:
            if finder is self or not hasattr(finder, "find_spec"):
                continue
            spec = finder.find_spec(fullname, path, target)
            if spec is None or spec.loader is None:
                continue
            spec.loader = _LoaderThenRegister(spec.loader)
            return spec
        return None


class _LoaderThenRegister(importlib.abc.Loader):
    def __init__(self, inner):
        self._inner = inner

    def create_module(self, spec):
        return self._inner.create_module(spec)

    def exec_module(self, module):
        self._inner.exec_module(module)
        if register() is not None:
            uninstall()


_finder: Optional[_RegisterAfterImport] = None


def install() -> Optional[str]:
    """Registers now when SGLang is already imported, else arms the deferred registration."""
    global _finder
    route = register()
    if route is None and _finder is None:
        _finder = _RegisterAfterImport()
        sys.meta_path.insert(0, _finder)
    return route


def uninstall() -> None:
    global _finder
    if _finder is not None and _finder in sys.meta_path:
        sys.meta_path.remove(_finder)
    _finder = None
