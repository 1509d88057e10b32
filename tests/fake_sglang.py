"""Test doubles for the SGLang objects the attention backend talks to (SGLang is not installed): a model whose
attention modules look like SGLang's, a model runner and a forward batch.  They live in the package
(directkv_b200/serve_sim.py, which also drives the backend for the serving-level benchmark); this module re-exports
them for the tests."""

from directkv_b200.serve_sim import (DECODE, EXTEND, IDLE, FakeModel, FakeRadixAttention, FakeRotary,  # noqa: F401
                                     FakeSelfAttention, make_batch, make_runner)
