"""The C-ABI library loads and exports every symbol include/see_cuda.h declares.
No compute is called: this runs without a GPU."""

import ctypes
import os
import re

import pytest

from see_ai_b200 import backend as B
from see_ai_b200 import engine as E

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "see_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(see_(?:cuda|engine)_\w+)\s*\(", text)))


def test_header_and_binding_agree():
    assert declared_symbols() == sorted(B.EXPORTED_SYMBOLS + E.ENGINE_SYMBOLS)


def test_library_exports_every_declared_symbol():
    if not os.path.exists(B.LIB_PATH):
        from see_ai_b200 import build
        build.build()
    lib = ctypes.CDLL(B.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(lib, name), name


def test_create_fails_loudly_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(B.BackendError) as e:
        B.CudaBackend(0)
    assert "no CPU fallback" in str(e.value) or "cuda" in str(e.value)
    with pytest.raises(B.BackendError):
        E.Engine(0)
