"""CPU checks of the boundary: the shared library loads, exports every symbol the header declares, and the
product refuses to run without a GPU instead of falling back."""
import ctypes
import os
import re

import pytest
import torch

import _capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    text = open(os.path.join(ROOT, "include", "vla_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vla_[a-z_0-9]+)\s*\(", text)))


def test_header_and_binding_agree():
    assert header_functions() == sorted(_capi.EXPORTS)


def test_library_exports_every_symbol():
    if not os.path.exists(_capi.LIB_PATH):
        pytest.skip("library not built")
    lib = ctypes.CDLL(_capi.LIB_PATH)
    for name in header_functions():
        assert hasattr(lib, name), name


def test_no_cpu_fallback():
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    from pi0_infer import Pi0Inference
    with pytest.raises(RuntimeError):
        Pi0Inference({"language_embeds": torch.zeros(0, 2048)}, 1, 50)
    if os.path.exists(_capi.LIB_PATH):
        cfg = _capi.VlaConfig(model=0, num_views=1, chunk_size=50, prompt_len=0, batch=1, device=0)
        h = ctypes.c_void_p()
        rc = _capi.lib().vla_create(ctypes.byref(cfg), ctypes.byref(h))
        assert rc == 1 and not h.value
        assert b"no CPU path" in _capi.lib().vla_last_error(None)


def test_product_does_not_import_oracle():
    pkg = os.path.join(ROOT, "realtime-vla_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                assert "oracle" not in open(os.path.join(dirpath, f)).read(), f
