"""No-GPU checks of the boundary: the C-ABI library loads and exports every declared symbol."""
import ctypes
import os
import re

import pytest

import kalosm_b200 as kb

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "fusor_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fb200_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    assert _declared_symbols() == sorted(kb.EXPORTS)


def test_library_exports_every_declared_symbol():
    assert os.path.exists(kb.LIB_PATH), "libfusor_b200.so is not built (python -m kalosm_b200.build)"
    lib = ctypes.CDLL(kb.LIB_PATH)
    missing = [s for s in _declared_symbols() if not hasattr(lib, s)]
    assert not missing, missing


def test_no_device_means_error_not_fallback():
    """Without a CUDA device the library reports an error; nothing computes on the CPU."""
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        pytest.skip("a GPU is present")
    with pytest.raises(kb.FusorError) as e:
        kb.Device(0)
    assert e.value.code == kb.ERR_CUDA
    assert "no CPU fallback" in str(e.value)


def test_product_never_imports_the_oracle():
    for dirpath, _dirs, files in os.walk(os.path.join(ROOT, "kalosm_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower() or f == "__init__.py" and "oracle" not in text, (dirpath, f)
