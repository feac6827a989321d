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


def test_binding_refuses_buffers_the_library_would_overrun():
    # caller-supplied outputs and residuals are checked on the host before the C call: the library
    # trusts their size, so an undersized buffer would become an out-of-bounds device write
    import types
    import numpy as np
    dev = types.SimpleNamespace(lib=None, h=1)
    w = types.SimpleNamespace(shape=(64, 128), h=2)
    x = kb.Tensor(dev, (4, 128), np.float32, ptr=1)
    cases = {
        "small": kb.Tensor(dev, (4, 32), np.float32, ptr=1),
        "wrong dtype": kb.Tensor(dev, (4, 64), np.float16, ptr=1),
        "other device": kb.Tensor(types.SimpleNamespace(lib=None, h=3), (4, 64), np.float32, ptr=1),
    }
    for what, bad in cases.items():
        for call in (lambda: x.q_mat_mul(w, out=bad), lambda: x.q_mat_mul_noalloc(w, bad),
                     lambda: x.q_mat_mul(w, epilogue=kb.EPI_RESIDUAL, r1=bad)):
            try:
                call()
            except kb.FusorError as e:
                assert e.code == kb.ERR_INVALID_SHAPE, what
            else:
                raise AssertionError(f"{what}: not refused")


def test_missing_nccl_is_an_error_code():
    # FB200_NCCL_LIB points the run-time loader at a file that does not exist: the communicator
    # entry points answer FB200_ERR_NCCL instead of crashing (fresh process: the lookup is cached)
    import subprocess
    import sys
    code = ("import kalosm_b200 as kb, ctypes as C; L = kb.load_library(); "
            "buf = (C.c_uint8 * kb.COMM_ID_BYTES)(); print(L.fb200_comm_unique_id(buf, kb.COMM_ID_BYTES))")
    out = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, FB200_NCCL_LIB="/nonexistent/libnccl.so.2"),
                         capture_output=True, text=True, cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert out.returncode == 0, out.stderr
    assert int(out.stdout.strip().splitlines()[-1]) == kb.ERR_NCCL
