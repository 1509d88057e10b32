"""The C-ABI library loads without a GPU and exports every symbol include/*.h declares."""

import ctypes
import glob
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = []
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = open(h).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"\b(dkv_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_header_declares_the_boundary():
    names = declared_symbols()
    for must in ("dkv_decode", "dkv_smpv2_fwd", "dkv_smpv2_fwd_graph", "dkv_layer_register", "dkv_extend",
                 "dkv_merge_partials", "dkv_scatter_kv", "dkv_context_create"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from directkv_b200 import _lib, build

    build.build_library()
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
    # the ctypes table covers the same set
    assert sorted(_lib.SIGNATURES) == declared_symbols()
    assert _lib.load().dkv_version() >= 100


def test_no_compute_without_gpu_is_loud():
    import torch

    if torch.cuda.is_available():
        pytest.skip("GPU present")
    from directkv_b200 import _lib, kernel

    with pytest.raises(RuntimeError, match="no CPU path"):
        _lib.get_context(0)
    with pytest.raises(RuntimeError):
        kernel.decode(0, torch.zeros(1, 128, dtype=torch.bfloat16), torch.ones(1, dtype=torch.int32), 1.0)


def test_struct_layouts_match_header_field_order():
    from directkv_b200 import _lib

    text = open(os.path.join(ROOT, "include", "directkv_b200.h")).read()

    def fields(struct_name):
        body = re.search(r"typedef struct \{([^}]*)\} " + struct_name + ";", text).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        return re.findall(r"([a-z_0-9]+)\s*;", body)

    assert fields("dkv_layer_desc") == [f[0] for f in _lib.LayerDesc._fields_]
    assert fields("dkv_decode_args") == [f[0] for f in _lib.DecodeArgs._fields_]
    assert fields("dkv_noalloc_args") == [f[0] for f in _lib.NoAllocArgs._fields_]
