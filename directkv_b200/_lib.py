"""ctypes binding of libdirectkv_b200.so (the C ABI declared in include/directkv_b200.h).

There is no CPU or PyTorch fallback: if the shared library is missing or cannot be loaded the
import of any compute entry point raises, and every non-zero status becomes ``RuntimeError``
(what the reference's ``TORCH_CHECK`` failures surface as in Python,
directkv/kernel/smpv2_extension.cu:587-631).
"""

from __future__ import annotations

import ctypes as C
import threading
from pathlib import Path
from typing import Dict, Optional

LIB_PATH = Path(__file__).resolve().parent / "_lib" / "libdirectkv_b200.so"

DKV_OK = 0
DKV_ERR_INVALID = 1
DKV_ERR_CUDA = 2
DKV_ERR_UNSUPPORTED = 3
DKV_ERR_NOT_REGISTERED = 4
DKV_ERR_DEVICE_STATUS = 5

DKV_NEW_NONE = 0
DKV_NEW_PROJECT = 1
DKV_NEW_GIVEN = 2

STATUS_BITS = {
    1 << 0: "a bounded device-side wait ran out of time",
    1 << 1: "a write-back slot was outside the KV pool",
    1 << 2: "a RoPE position was outside the cos/sin table",
    1 << 3: "the tensor-core completion barrier ran out of time",
    1 << 4: "the sequence-split exchange found a record of another step (the ranks' calls do not line up)",
    1 << 5: "a sequence length or row led outside the page table",
    1 << 8: "(in the KV-streaming kernel)",
    1 << 9: "(in the projection's load pipeline)",
    1 << 10: "(in the projection's tensor-core pipeline)",
    1 << 11: "(in the extend attention kernel)",
    1 << 12: "(in the sequence-split exchange)",
}

PARTIAL_STRIDE = 132  # floats per unnormalised partial row: O[128], m (log2 domain), l, 2 pad


class LayerDesc(C.Structure):
    _fields_ = [
        ("k_pool", C.c_void_p),
        ("v_pool", C.c_void_p),
        ("n_slots", C.c_int64),
        ("nh_kv", C.c_int),
        ("page_size", C.c_int),
        ("row_stride", C.c_int64),
        ("wk", C.c_void_p),
        ("wv", C.c_void_p),
        ("hidden", C.c_int),
        ("cos_sin", C.c_void_p),
        ("max_pos", C.c_int),
    ]


class DecodeArgs(C.Structure):
    _fields_ = [
        ("layer_id", C.c_int),
        ("batch", C.c_int),
        ("nh_q", C.c_int),
        ("q", C.c_void_p),
        ("q_stride", C.c_int64),
        ("out", C.c_void_p),
        ("out_stride", C.c_int64),
        ("seq_lens", C.c_void_p),
        ("page_table", C.c_void_p),
        ("pt_stride", C.c_int),
        ("row_map", C.c_void_p),
        ("new_mode", C.c_int),
        ("x", C.c_void_p),
        ("k_new", C.c_void_p),
        ("v_new", C.c_void_p),
        ("save_kv_cache", C.c_int),
        ("softmax_scale", C.c_float),
        ("lse_out", C.c_void_p),
        ("partial_out", C.c_void_p),
        ("pos_offset", C.c_void_p),
        ("kv_source_layer", C.c_int),
        ("src_page_table", C.c_void_p),
        ("src_pt_stride", C.c_int),
        ("src_row_map", C.c_void_p),
        ("pt_rows", C.c_int),
    ]


class NoAllocArgs(C.Structure):
    _fields_ = [
        ("k_pool", C.c_void_p),
        ("v_pool", C.c_void_p),
        ("n_slots", C.c_int64),
        ("nh_kv", C.c_int),
        ("page_size", C.c_int),
        ("batch", C.c_int),
        ("nh_q", C.c_int),
        ("q", C.c_void_p),
        ("q_stride", C.c_int64),
        ("out", C.c_void_p),
        ("out_stride", C.c_int64),
        ("seq_lens", C.c_void_p),
        ("page_table", C.c_void_p),
        ("pt_stride", C.c_int),
        ("softmax_scale", C.c_float),
        ("lse_out", C.c_void_p),
        ("sync_and_check", C.c_int),
        ("err_buf", C.c_char_p),
        ("err_buf_len", C.c_int),
        ("status_out", C.c_void_p),
    ]


# name -> (restype, argtypes); also the list of symbols include/directkv_b200.h declares.
SIGNATURES = {
    "dkv_version": (C.c_int, []),
    "dkv_last_error": (C.c_char_p, []),
    "dkv_context_create": (C.c_int, [C.c_int, C.POINTER(C.c_void_p)]),
    "dkv_context_destroy": (C.c_int, [C.c_void_p]),
    "dkv_context_reserve": (C.c_int, [C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_int]),
    "dkv_context_set": (C.c_int, [C.c_void_p, C.c_char_p, C.c_int]),
    "dkv_profile_read": (C.c_int, [C.c_void_p, C.POINTER(C.c_double), C.POINTER(C.c_longlong),
                                   C.POINTER(C.c_longlong), C.c_int]),
    "dkv_read_status": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint), C.c_int]),
    "dkv_layer_register": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(LayerDesc)]),
    "dkv_layer_unregister": (C.c_int, [C.c_void_p, C.c_int]),
    "dkv_decode": (C.c_int, [C.c_void_p, C.POINTER(DecodeArgs), C.c_void_p]),
    "dkv_exchange_create": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int64, C.POINTER(C.c_void_p)]),
    "dkv_exchange_handle": (C.c_int, [C.c_void_p, C.c_char_p]),
    "dkv_exchange_connect": (C.c_int, [C.c_void_p, C.c_int, C.c_char_p]),
    "dkv_exchange_base": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "dkv_exchange_connect_ptr": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "dkv_exchange_destroy": (C.c_int, [C.c_void_p]),
    "dkv_decode_exchange": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(DecodeArgs), C.c_void_p, C.c_void_p, C.c_void_p]),
    "dkv_merge_partials": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]),
    "dkv_smpv2_fwd": (C.c_int, [C.c_void_p] + [C.c_void_p] * 6 + [C.c_void_p, C.c_int] + [C.c_int] * 6
                      + [C.c_float, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "dkv_smpv2_fwd_graph": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                      C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, C.c_void_p, C.c_void_p]),
    "dkv_extend": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                             C.c_float, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "dkv_extend_attend": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float,
                                    C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "dkv_extend_ragged": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p,
                                    C.c_void_p, C.c_int, C.c_float, C.c_int, C.c_void_p, C.c_int64, C.c_void_p]),
    "dkv_scatter_kv": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p,
                                 C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "dkv_decode_noalloc": (C.c_int, [C.POINTER(NoAllocArgs), C.c_void_p]),
    "dkv_stream_copy": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
}

_lib = None
_lock = threading.Lock()
_contexts: Dict[int, "Context"] = {}


def load() -> C.CDLL:
    """Loads the shared library (once).  Raises RuntimeError when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"directkv_b200: {LIB_PATH} is missing. Build it with `python -m directkv_b200.build` "
                "(nvcc, sm_100a). There is no CPU or PyTorch fallback."
            )
        lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError here means the library is stale
            fn.restype = res
            fn.argtypes = args
        _lib = lib
        return lib


def check(rc: int) -> None:
    if rc != DKV_OK:
        msg = load().dkv_last_error()
        raise RuntimeError(f"directkv_b200 error {rc}: {msg.decode() if msg else '?'}")


class Context:
    """Per-device engine context (scratch, status word, registered layers)."""

    def __init__(self, device: int):
        lib = load()
        h = C.c_void_p()
        check(lib.dkv_context_create(device, C.byref(h)))
        self.handle = h
        self.device = device
        self._keepalive = {}

    def set(self, key: str, value: int) -> None:
        check(load().dkv_context_set(self.handle, key.encode(), int(value)))

    def reserve(self, max_rows: int, nh_q: int, nh_kv: int, hidden: int) -> None:
        check(load().dkv_context_reserve(self.handle, max_rows, nh_q, nh_kv, hidden))

    def read_status(self, clear: bool = True) -> int:
        st = C.c_uint(0)
        check(load().dkv_read_status(self.handle, C.byref(st), 1 if clear else 0))
        return st.value

    def profile_read(self, reset: bool = True):
        """(summed ms of the bracketed streaming-kernel launches, their count, all launches)."""
        ms, n, tot = C.c_double(0), C.c_longlong(0), C.c_longlong(0)
        check(load().dkv_profile_read(self.handle, C.byref(ms), C.byref(n), C.byref(tot), 1 if reset else 0))
        return ms.value, n.value, tot.value

    def raise_on_status(self) -> None:
        """Synchronises the device and raises if any kernel recorded a failure."""
        st = self.read_status(clear=True)
        if st:
            why = "; ".join(v for k, v in STATUS_BITS.items() if st & k)
            raise RuntimeError(f"directkv_b200 device status 0x{st:x}: {why}")

    def close(self) -> None:
        if self.handle:
            load().dkv_context_destroy(self.handle)
            self.handle = None


def get_context(device: Optional[int] = None) -> Context:
    """The context of a CUDA device (the current one by default), created on first use."""
    import torch

    if not torch.cuda.is_available():
        raise RuntimeError("directkv_b200 needs a CUDA device (B200, sm_100a); there is no CPU path")
    if device is None:
        device = torch.cuda.current_device()
    ctx = _contexts.get(device)
    if ctx is None:
        ctx = Context(device)
        _contexts[device] = ctx
    return ctx
