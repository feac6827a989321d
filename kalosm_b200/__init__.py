"""kalosm_b200 — host-side mirror of Fusor's operator API over ``libfusor_b200.so``.

The shared library (hand-written sm_100a CUDA behind a C ABI, ``include/fusor_b200.h``) is the
product; this module is the thin Python binding the tests and the benchmark drive it with.
Class and method names follow the ``fusor`` crate of floneum/kalosm: ``Device``, ``Tensor``,
``QMatrix.from_raw_bytes``, ``Tensor.q_mat_mul``, ``KvCache.append``, ``flash_attention`` …
There is no CPU fallback: importing works anywhere, but creating a ``Device`` without the
compiled library or without a CUDA GPU raises ``FusorError``.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
# FB200_LIB_PATH selects another build of the library (a deployment's own location, or a variant under test)
LIB_PATH = os.environ.get("FB200_LIB_PATH") or os.path.join(_HERE, "libfusor_b200.so")

# ggml type ids (fusor-ml/gguf/src/lib.rs:35-50)
F32, F16, Q4_0, Q5_0, Q8_0, Q4_K, Q5_K, Q6_K = 0, 1, 2, 6, 8, 12, 13, 14
BLOCK = {F32: (1, 4), F16: (1, 2), Q4_0: (32, 18), Q5_0: (32, 22), Q8_0: (32, 34),
         Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210)}

OK = 0
ERR_INVALID_SHAPE, ERR_UNSUPPORTED_DTYPE, ERR_CAPACITY, ERR_CUDA = -1, -2, -3, -4
ERR_INVALID_ARGUMENT, ERR_TIMEOUT, ERR_DEVICE_MISMATCH, ERR_NCCL = -5, -6, -7, -8
COMM_ID_BYTES = 128
IPC_HANDLE_BYTES = 64
EPI_NONE, EPI_RESIDUAL, EPI_SWIGLU, EPI_BIAS = 0, 1, 2, 3
MASK_NONE, MASK_CAUSAL, MASK_QK, MASK_BATCH_KEY = 0, 1, 2, 3


class FusorError(RuntimeError):
    """An fb200_* call returned a negative status (mirrors fusor::Error, fusor/src/error.rs:4-15)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"fb200 status {code}: {message}")
        self.code = code


class SamplerConfig(C.Structure):
    """fb200_sampler_config; fields as GpuSamplerConfig (models/kalosm-llama/src/lib.rs:477-488)."""
    _fields_ = [("strategy", C.c_int), ("temperature", C.c_float), ("repetition_penalty", C.c_float),
                ("repetition_penalty_range", C.c_int), ("top_k", C.c_int), ("top_p", C.c_float),
                ("min_p", C.c_float), ("tau", C.c_float), ("eta", C.c_float), ("mu", C.c_float),
                ("seed", C.c_uint64)]

    def __init__(self, strategy=0, temperature=1.0, repetition_penalty=1.0, repetition_penalty_range=64,
                 top_k=64, top_p=float("nan"), min_p=float("nan"), tau=5.0, eta=0.1, mu=10.0, seed=0):
        super().__init__(strategy, temperature, repetition_penalty, repetition_penalty_range, top_k, top_p,
                         min_p, tau, eta, mu, seed)


SAMPLER_STANDARD, SAMPLER_MIROSTAT2 = 0, 1
SAMPLER_MAX_TOP_K = 1024


class _Epilogue(C.Structure):
    _fields_ = [("kind", C.c_int), ("r1", C.c_void_p), ("r2", C.c_void_p)]


class LlamaConfig(C.Structure):
    """fb200_llama_config; field meanings follow the GGUF keys of kalosm-llama raw/mod.rs:377-415."""
    _fields_ = [("n_layer", C.c_int), ("hidden", C.c_int), ("ffn", C.c_int), ("n_head", C.c_int),
                ("n_kv_head", C.c_int), ("head_dim", C.c_int), ("vocab", C.c_int),
                ("max_seq_len", C.c_int), ("max_batch", C.c_int), ("rms_eps", C.c_float),
                ("rope_theta", C.c_float), ("rope_factor", C.c_float),
                ("rope_low_freq_factor", C.c_float), ("rope_high_freq_factor", C.c_float),
                ("rope_original_ctx", C.c_int)]


EXPORTS = [
    "fb200_device_create", "fb200_device_destroy", "fb200_device_synchronize", "fb200_last_error",
    "fb200_launch_count", "fb200_device_status", "fb200_device_clear_status",
    "fb200_device_set_scratch_limit", "fb200_device_set_poison", "fb200_malloc", "fb200_free", "fb200_upload",
    "fb200_download", "fb200_memset", "fb200_qmatrix_from_raw_bytes", "fb200_qmatrix_free",
    "fb200_qmatrix_shape", "fb200_qmatrix_ggml_type", "fb200_qmatrix_nbytes",
    "fb200_qmatrix_dequantize", "fb200_qmatrix_concat_rows", "fb200_q_mat_mul",
    "fb200_q_mat_mul_host", "fb200_q_mat_mul_noalloc", "fb200_rms_norm_q_mat_mul", "fb200_rms_norm", "fb200_silu_mul", "fb200_rope_tables",
    "fb200_rope_pair", "fb200_embedding_lookup", "fb200_argmax", "fb200_top_k", "fb200_sample",
    "fb200_llama_generate_sampled", "fb200_kv_cache_create",
    "fb200_kv_cache_free", "fb200_kv_cache_reset", "fb200_kv_cache_truncate", "fb200_kv_cache_len", "fb200_kv_cache_append",
    "fb200_kv_cache_buffers", "fb200_flash_attention", "fb200_llama_create", "fb200_llama_free",
    "fb200_llama_set_tensor", "fb200_llama_set_rope_freqs", "fb200_llama_reset", "fb200_llama_truncate", "fb200_llama_position", "fb200_llama_forward",
    "fb200_llama_generate_greedy", "fb200_llama_logits_dev", "fb200_llama_set_tensor_parallel",
    "fb200_comm_unique_id", "fb200_comm_create", "fb200_comm_destroy", "fb200_comm_all_reduce_sum",
    "fb200_comm_exchange_handle", "fb200_comm_exchange_attach", "fb200_exchange_wait_check",
]

_lib = None


def load_library():
    """dlopen libfusor_b200.so and declare the signatures. Raises FusorError if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FusorError(ERR_CUDA, f"{LIB_PATH} is not built (run `python -m kalosm_b200.build`); "
                                   "there is no CPU fallback")
    L = C.CDLL(LIB_PATH)
    vp, sz, i32, u32, u64, f32 = C.c_void_p, C.c_size_t, C.c_int, C.c_uint32, C.c_uint64, C.c_float
    pp = C.POINTER(C.c_void_p)
    sig = {
        "fb200_device_create": (i32, [i32, vp, pp]),
        "fb200_device_destroy": (i32, [vp]),
        "fb200_device_synchronize": (i32, [vp]),
        "fb200_last_error": (C.c_char_p, [vp]),
        "fb200_launch_count": (u64, [vp]),
        "fb200_device_status": (i32, [vp, C.POINTER(i32)]),
        "fb200_device_clear_status": (i32, [vp]),
        "fb200_device_set_scratch_limit": (i32, [vp, sz]),
        "fb200_device_set_poison": (i32, [vp, i32]),
        "fb200_malloc": (i32, [vp, sz, pp]),
        "fb200_free": (i32, [vp, vp]),
        "fb200_upload": (i32, [vp, vp, vp, sz]),
        "fb200_download": (i32, [vp, vp, vp, sz]),
        "fb200_memset": (i32, [vp, vp, i32, sz]),
        "fb200_qmatrix_from_raw_bytes": (i32, [vp, C.POINTER(u64), i32, vp, sz, u32, pp]),
        "fb200_qmatrix_free": (i32, [vp]),
        "fb200_qmatrix_shape": (i32, [vp, C.POINTER(u64), C.POINTER(u64)]),
        "fb200_qmatrix_ggml_type": (i32, [vp, C.POINTER(u32)]),
        "fb200_qmatrix_nbytes": (i32, [vp, C.POINTER(u64)]),
        "fb200_qmatrix_dequantize": (i32, [vp, vp]),
        "fb200_qmatrix_concat_rows": (i32, [pp, i32, pp]),
        "fb200_q_mat_mul": (i32, [vp, vp, sz, vp, vp, C.POINTER(_Epilogue)]),
        "fb200_q_mat_mul_host": (i32, [vp, vp, sz, vp, vp]),
        "fb200_q_mat_mul_noalloc": (i32, [vp, vp, sz, vp, vp]),
        "fb200_rms_norm_q_mat_mul": (i32, [vp, vp, vp, vp, f32, sz, vp, vp, C.POINTER(_Epilogue)]),
        "fb200_rms_norm": (i32, [vp, vp, vp, vp, vp, f32, sz, sz, vp]),
        "fb200_silu_mul": (i32, [vp, vp, vp, sz, vp]),
        "fb200_rope_tables": (i32, [vp, i32, i32, f32, f32, f32, f32, i32, vp, vp]),
        "fb200_rope_pair": (i32, [vp, vp, vp, i32, i32, i32, i32, i32, vp, vp, i32, i32]),
        "fb200_embedding_lookup": (i32, [vp, vp, vp, sz, vp]),
        "fb200_argmax": (i32, [vp, vp, sz, sz, vp, vp]),
        "fb200_top_k": (i32, [vp, vp, sz, sz, i32, vp, vp]),
        "fb200_sample": (i32, [vp, vp, sz, sz, C.POINTER(SamplerConfig), vp, sz, i32, u64, vp, vp]),
        "fb200_llama_generate_sampled": (i32, [vp, vp, i32, i32, C.POINTER(SamplerConfig), vp]),
        "fb200_kv_cache_create": (i32, [vp, i32, i32, i32, i32, pp]),
        "fb200_kv_cache_free": (i32, [vp]),
        "fb200_kv_cache_reset": (i32, [vp]),
        "fb200_kv_cache_truncate": (i32, [vp, i32]),
        "fb200_kv_cache_len": (i32, [vp, C.POINTER(i32), C.POINTER(i32)]),
        "fb200_kv_cache_append": (i32, [vp, vp, vp, i32]),
        "fb200_kv_cache_buffers": (i32, [vp, pp, pp]),
        "fb200_flash_attention": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, f32, vp,
                                        i32, vp]),
        "fb200_llama_create": (i32, [vp, C.POINTER(LlamaConfig), pp]),
        "fb200_llama_free": (i32, [vp]),
        "fb200_llama_set_tensor": (i32, [vp, i32, i32, u32, u64, u64, vp, sz]),
        "fb200_llama_set_rope_freqs": (i32, [vp, vp, sz]),
        "fb200_llama_reset": (i32, [vp]),
        "fb200_llama_truncate": (i32, [vp, i32]),
        "fb200_llama_position": (i32, [vp, C.POINTER(i32)]),
        "fb200_llama_forward": (i32, [vp, vp, i32, i32, vp, vp]),
        "fb200_llama_generate_greedy": (i32, [vp, vp, i32, i32, vp]),
        "fb200_llama_logits_dev": (i32, [vp, pp]),
        "fb200_llama_set_tensor_parallel": (i32, [vp, vp]),
        "fb200_comm_unique_id": (i32, [vp, sz]),
        "fb200_comm_create": (i32, [vp, i32, i32, vp, sz, pp]),
        "fb200_comm_destroy": (i32, [vp]),
        "fb200_comm_all_reduce_sum": (i32, [vp, vp, sz]),
        "fb200_comm_exchange_handle": (i32, [vp, sz, vp, sz]),
        "fb200_comm_exchange_attach": (i32, [vp, vp, sz]),
        "fb200_exchange_wait_check": (i32, [vp, i32]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


def _hp(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data


class Tensor:
    """A contiguous row-major device buffer with a shape and dtype (fusor::Tensor::Gpu)."""

    def __init__(self, device: "Device", shape: Sequence[int], dtype=np.float32, ptr: Optional[int] = None):
        self.device = device
        self.shape = tuple(int(s) for s in shape)
        self.dtype = np.dtype(dtype)
        self.nbytes = int(np.prod(self.shape, dtype=np.int64)) * self.dtype.itemsize
        self._owned = ptr is None
        if ptr is None:
            out = C.c_void_p()
            device._check(device.lib.fb200_malloc(device.h, max(self.nbytes, 1), C.byref(out)))
            ptr = out.value
        self.ptr = ptr

    @classmethod
    def from_slice(cls, device: "Device", array, dtype=None) -> "Tensor":
        """Tensor::from_slice (fusor/src/lib.rs:356-362): upload a host array."""
        a = np.ascontiguousarray(array, dtype=dtype)
        t = cls(device, a.shape, a.dtype)
        device._check(device.lib.fb200_upload(device.h, t.ptr, _hp(a), a.nbytes))
        return t

    def as_slice(self) -> np.ndarray:
        """Tensor::as_slice (fusor/src/lib.rs:364-368): the synchronising read-back."""
        out = np.empty(self.shape, dtype=self.dtype)
        self.device._check(self.device.lib.fb200_download(self.device.h, _hp(out), self.ptr, self.nbytes))
        return out

    def fill_bytes(self, value: int) -> None:
        self.device._check(self.device.lib.fb200_memset(self.device.h, self.ptr, value, self.nbytes))

    def q_mat_mul(self, w: "QMatrix", epilogue: int = EPI_NONE, r1: "Tensor" = None,
                  r2: "Tensor" = None, out: "Tensor" = None) -> "Tensor":
        """Tensor::q_mat_mul (fusor/src/lib.rs:1132-1223): self [.., K] . W[N, K]^T."""
        k = self.shape[-1]
        n, wk = w.shape
        if k != wk:
            raise FusorError(ERR_INVALID_SHAPE, f"lhs columns ({k}) != weight in_features ({wk})")
        m = int(np.prod(self.shape[:-1], dtype=np.int64)) if len(self.shape) > 1 else 1
        n_out = n // 2 if epilogue == EPI_SWIGLU else n
        out_shape = (self.shape[:-1] if len(self.shape) > 1 else ()) + (n_out,)
        for name, t in (("out", out), ("r1", r1), ("r2", r2)):
            self._require_f32(name, t, n_out if name == "r1" and epilogue == EPI_BIAS else m * n_out)
        y = out if out is not None else Tensor(self.device, out_shape, np.float32)
        ep = _Epilogue(epilogue, r1.ptr if r1 is not None else None, r2.ptr if r2 is not None else None)
        d = self.device
        d._check(d.lib.fb200_q_mat_mul(d.h, self.ptr, m, w.h, y.ptr, C.byref(ep)))
        return y

    def _require_f32(self, name: str, t: Optional["Tensor"], elems: int) -> None:
        """Refuses a caller-supplied buffer the library would otherwise write or read out of bounds."""
        if t is None:
            return
        if t.dtype != np.float32 or t.nbytes < elems * 4 or t.device is not self.device:
            raise FusorError(ERR_INVALID_SHAPE, f"{name} must be an f32 tensor of at least {elems} elements on the "
                                                f"same device handle (got {t.dtype}, {t.nbytes} bytes)")

    def q_mat_mul_noalloc(self, w: "QMatrix", out: "Tensor") -> "Tensor":
        """self [M <= 32, K] . W^T into the caller's `out`, through the entry point that never
        allocates (its scratch is a fixed array inside the library). Both tensors must exist
        before the call; see fb200_q_mat_mul_noalloc in include/fusor_b200.h for the limits."""
        k = self.shape[-1]
        if k != w.shape[1]:
            raise FusorError(ERR_INVALID_SHAPE, f"lhs columns ({k}) != weight in_features ({w.shape[1]})")
        m = int(np.prod(self.shape[:-1], dtype=np.int64)) if len(self.shape) > 1 else 1
        self._require_f32("out", out, m * w.shape[0])
        d = self.device
        d._check(d.lib.fb200_q_mat_mul_noalloc(d.h, self.ptr, m, w.h, out.ptr))
        return out

    def rms_norm_q_mat_mul(self, norm_weight: "Tensor", eps: float, w: "QMatrix",
                           residual: "Tensor" = None, epilogue: int = EPI_NONE, r1: "Tensor" = None,
                           r2: "Tensor" = None) -> "Tensor":
        """rms_norm(self (+ residual)) . W^T with the norm fused into the product where possible."""
        k = self.shape[-1]
        n, wk = w.shape
        if k != wk:
            raise FusorError(ERR_INVALID_SHAPE, f"lhs columns ({k}) != weight in_features ({wk})")
        m = int(np.prod(self.shape[:-1], dtype=np.int64)) if len(self.shape) > 1 else 1
        n_out = n // 2 if epilogue == EPI_SWIGLU else n
        y = Tensor(self.device, (self.shape[:-1] if len(self.shape) > 1 else ()) + (n_out,), np.float32)
        ep = _Epilogue(epilogue, r1.ptr if r1 is not None else None, r2.ptr if r2 is not None else None)
        d = self.device
        d._check(d.lib.fb200_rms_norm_q_mat_mul(d.h, self.ptr, residual.ptr if residual is not None else None,
                                                norm_weight.ptr, eps, m, w.h, y.ptr, C.byref(ep)))
        return y

    def free(self) -> None:
        if self._owned and self.ptr:
            self.device.lib.fb200_free(self.device.h, self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Device:
    """fusor::Device::gpu() (fusor/src/device.rs:29-40): one CUDA device and stream."""

    def __init__(self, ordinal: int = 0, stream: Optional[int] = None):
        self.lib = load_library()
        out = C.c_void_p()
        rc = self.lib.fb200_device_create(ordinal, stream, C.byref(out))
        if rc:
            raise FusorError(rc, self.lib.fb200_last_error(None).decode())
        self.h = out.value
        self.ordinal = ordinal

    def _check(self, rc: int) -> None:
        if rc:
            raise FusorError(rc, self.lib.fb200_last_error(self.h).decode())

    def synchronize(self) -> None:
        self._check(self.lib.fb200_device_synchronize(self.h))

    @property
    def launch_count(self) -> int:
        return int(self.lib.fb200_launch_count(self.h))

    def status(self) -> int:
        s = C.c_int()
        self._check(self.lib.fb200_device_status(self.h, C.byref(s)))
        return s.value

    def clear_status(self) -> None:
        """Resets the device status word after a reported time-out."""
        self._check(self.lib.fb200_device_clear_status(self.h))

    def set_scratch_limit(self, nbytes: int) -> None:
        """Budget of the handle's scratch buffers (0 = unlimited): growing beyond it fails with ERR_CAPACITY."""
        self._check(self.lib.fb200_device_set_scratch_limit(self.h, int(nbytes)))

    def set_poison(self, enable: bool) -> None:
        """Fill freshly allocated scratch with NaN bytes (debug aid)."""
        self._check(self.lib.fb200_device_set_poison(self.h, 1 if enable else 0))

    def exchange_wait_check(self, poll_limit: int) -> None:
        """Bounded arrival wait of the tensor-parallel peer exchange on a word nothing sets: raises
        FusorError(ERR_TIMEOUT) after `poll_limit` polls and leaves the code in `status()`."""
        self._check(self.lib.fb200_exchange_wait_check(self.h, poll_limit))

    def tensor(self, array, dtype=None) -> Tensor:
        return Tensor.from_slice(self, array, dtype)

    def empty(self, shape, dtype=np.float32) -> Tensor:
        return Tensor(self, shape, dtype)

    # ---- composite ops -------------------------------------------------------------------
    def rms_norm(self, x: Tensor, weight: Tensor, eps: float, residual: Tensor = None,
                 bias: Tensor = None) -> Tensor:
        n = x.shape[-1]
        rows = x.nbytes // 4 // n
        y = Tensor(self, x.shape)
        self._check(self.lib.fb200_rms_norm(self.h, x.ptr, residual.ptr if residual else None,
                                            weight.ptr, bias.ptr if bias else None, eps, rows, n, y.ptr))
        return y

    def silu_mul(self, gate: Tensor, up: Tensor) -> Tensor:
        y = Tensor(self, gate.shape)
        self._check(self.lib.fb200_silu_mul(self.h, gate.ptr, up.ptr, gate.nbytes // 4, y.ptr))
        return y

    def argmax(self, logits: Tensor):
        n = logits.shape[-1]
        rows = logits.nbytes // 4 // n
        ids, vals = Tensor(self, (rows,), np.uint32), Tensor(self, (rows,), np.float32)
        self._check(self.lib.fb200_argmax(self.h, logits.ptr, rows, n, ids.ptr, vals.ptr))
        return ids, vals

    def top_k(self, logits: Tensor, k: int):
        """Tensor::top_k_pairs (fusor/src/lib.rs:416-453): (ids [rows, k], values [rows, k]), descending,
        ties -> higher id."""
        n = logits.shape[-1]
        rows = logits.nbytes // 4 // n
        ids, vals = Tensor(self, (rows, k), np.uint32), Tensor(self, (rows, k), np.float32)
        self._check(self.lib.fb200_top_k(self.h, logits.ptr, rows, n, k, ids.ptr, vals.ptr))
        return ids, vals

    def sample(self, logits: Tensor, cfg: "SamplerConfig", previous: Tensor = None, counter: int = 0,
               mu: Tensor = None) -> Tensor:
        """One step of the on-device sampler over logits [rows, n]; previous [rows, L] u32."""
        n = logits.shape[-1]
        rows = logits.nbytes // 4 // n
        ids = Tensor(self, (rows,), np.uint32)
        plen = previous.shape[-1] if previous is not None else 0
        self._check(self.lib.fb200_sample(self.h, logits.ptr, rows, n, C.byref(cfg),
                                          previous.ptr if previous is not None else None, plen, plen, counter,
                                          mu.ptr if mu is not None else None, ids.ptr))
        return ids

    def flash_attention(self, q: Tensor, k: Tensor, v: Tensor, scale: float, skv: int = None,
                        mask: Tensor = None, mask_kind: int = MASK_NONE, out: Tensor = None) -> Tensor:
        """Tensor::flash_attention (fusor/src/composite/flash_attention.rs:58-109).
        q f32 [B,H,Sq,D]; k, v fp16 [B,Hkv,cap,D] of which the first `skv` rows are valid."""
        b, h, sq, d = q.shape
        _, hkv, cap, _ = k.shape
        skv = cap if skv is None else skv
        out = Tensor(self, q.shape) if out is None else out
        self._check(self.lib.fb200_flash_attention(self.h, q.ptr, k.ptr, v.ptr, b, h, hkv, sq, skv,
                                                   cap, d, scale, mask.ptr if mask else None,
                                                   mask_kind, out.ptr))
        return out

    def close(self) -> None:
        if self.h:
            self.lib.fb200_device_destroy(self.h)
            self.h = None


class QMatrix:
    """fusor::QMatrix (fusor/src/quantized.rs:80-284) on the device."""

    def __init__(self, device: Device, handle: int):
        self.device, self.h = device, handle
        n, k = C.c_uint64(), C.c_uint64()
        device.lib.fb200_qmatrix_shape(handle, C.byref(n), C.byref(k))
        self.shape = (n.value, k.value)

    @classmethod
    def from_raw_bytes(cls, device: Device, shape: Sequence[int], raw, ggml_type: int) -> "QMatrix":
        raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
        shp = (C.c_uint64 * len(shape))(*[int(s) for s in shape])
        out = C.c_void_p()
        device._check(device.lib.fb200_qmatrix_from_raw_bytes(device.h, shp, len(shape), _hp(raw),
                                                              raw.size, ggml_type, C.byref(out)))
        return cls(device, out.value)

    @classmethod
    def concat_rows(cls, mats: Sequence["QMatrix"]) -> Optional["QMatrix"]:
        arr = (C.c_void_p * len(mats))(*[m.h for m in mats])
        out = C.c_void_p()
        rc = mats[0].device.lib.fb200_qmatrix_concat_rows(arr, len(mats), C.byref(out))
        if rc == ERR_INVALID_SHAPE:
            return None  # the reference returns None for mismatched parts
        mats[0].device._check(rc)
        return cls(mats[0].device, out.value)

    @property
    def ggml_type(self) -> int:
        t = C.c_uint32()
        self.device.lib.fb200_qmatrix_ggml_type(self.h, C.byref(t))
        return t.value

    @property
    def nbytes(self) -> int:
        n = C.c_uint64()
        self.device.lib.fb200_qmatrix_nbytes(self.h, C.byref(n))
        return n.value

    def dequantize(self) -> Tensor:
        out = Tensor(self.device, self.shape, np.float32)
        self.device._check(self.device.lib.fb200_qmatrix_dequantize(self.h, out.ptr))
        return out

    def embedding(self, ids: Tensor) -> Tensor:
        n_ids = ids.nbytes // 4
        out = Tensor(self.device, ids.shape + (self.shape[1],), np.float32)
        d = self.device
        d._check(d.lib.fb200_embedding_lookup(d.h, self.h, ids.ptr, n_ids, out.ptr))
        return out

    def q_mat_mul_host(self, x: np.ndarray) -> np.ndarray:
        """Product with host buffers (copies inside the call)."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        m = x.size // self.shape[1]
        y = np.empty(x.shape[:-1] + (self.shape[0],), dtype=np.float32)
        d = self.device
        d._check(d.lib.fb200_q_mat_mul_host(d.h, _hp(x), m, self.h, _hp(y)))
        return y

    def free(self) -> None:
        if self.h:
            self.device.lib.fb200_qmatrix_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class RopeCache:
    """fusor::RopeCache (fusor/src/composite/rope.rs:233-340): cos/sin tables on the device."""

    def __init__(self, device: Device, head_dim: int, ctx: int, theta: float, scaling=None):
        self.device, self.head_dim, self.ctx = device, head_dim, ctx
        self.cos = Tensor(device, (ctx, head_dim // 2))
        self.sin = Tensor(device, (ctx, head_dim // 2))
        factor, low, high, orig = (0.0, 1.0, 4.0, ctx) if scaling is None else scaling
        device._check(device.lib.fb200_rope_tables(device.h, head_dim, ctx, theta, factor, low, high,
                                                   orig, self.cos.ptr, self.sin.ptr))

    def forward(self, q: Tensor, k: Tensor, start_pos: int = 0, interleaved: bool = False):
        """In place on q [B,H,S,D] and k [B,Hkv,S,D]."""
        b, h, s, d = q.shape
        hkv = k.shape[1]
        dv = self.device
        dv._check(dv.lib.fb200_rope_pair(dv.h, q.ptr, k.ptr, b, h, hkv, s, d, self.cos.ptr,
                                         self.sin.ptr, start_pos, 1 if interleaved else 0))
        return q, k

    def forward_interleaved(self, q: Tensor, k: Tensor, start_pos: int = 0):
        return self.forward(q, k, start_pos, True)


class KvCache:
    """fusor::KvCache (fusor/src/cache/kv_cache.rs:12-68) with an fp16 device buffer."""

    def __init__(self, device: Device, batch: int, n_kv_head: int, head_dim: int, max_seq_len: int):
        self.device = device
        self.batch, self.n_kv_head, self.head_dim = batch, n_kv_head, head_dim
        out = C.c_void_p()
        device._check(device.lib.fb200_kv_cache_create(device.h, batch, n_kv_head, head_dim,
                                                       max_seq_len, C.byref(out)))
        self.h = out.value

    def append(self, k: Tensor, v: Tensor):
        """Appends k, v [B,Hkv,S,D]; returns (K, V) views of the whole buffers plus the length."""
        self.device._check(self.device.lib.fb200_kv_cache_append(self.h, k.ptr, v.ptr, k.shape[2]))
        kp, vp = C.c_void_p(), C.c_void_p()
        self.device.lib.fb200_kv_cache_buffers(self.h, C.byref(kp), C.byref(vp))
        shape = (self.batch, self.n_kv_head, self.capacity, self.head_dim)
        return (Tensor(self.device, shape, np.float16, kp.value),
                Tensor(self.device, shape, np.float16, vp.value), self.current_seq_len)

    def reset(self):
        self.device.lib.fb200_kv_cache_reset(self.h)

    def truncate(self, length: int) -> None:
        """Keeps the first `length` positions."""
        self.device._check(self.device.lib.fb200_kv_cache_truncate(self.h, length))

    @property
    def current_seq_len(self) -> int:
        n, c = C.c_int(), C.c_int()
        self.device.lib.fb200_kv_cache_len(self.h, C.byref(n), C.byref(c))
        return n.value

    @property
    def capacity(self) -> int:
        n, c = C.c_int(), C.c_int()
        self.device.lib.fb200_kv_cache_len(self.h, C.byref(n), C.byref(c))
        return c.value

    def __del__(self):
        try:
            if self.h:
                self.device.lib.fb200_kv_cache_free(self.h)
                self.h = None
        except Exception:
            pass


class Comm:
    """Tensor-parallel communicator: one rank per process and GPU (NCCL). `unique_id()` on rank 0,
    the id travels to the other ranks by any host channel (e.g. a torch.distributed broadcast),
    then every rank constructs its Comm; the constructor returns when all ranks have joined."""

    @staticmethod
    def unique_id() -> bytes:
        buf = (C.c_uint8 * COMM_ID_BYTES)()
        rc = load_library().fb200_comm_unique_id(buf, COMM_ID_BYTES)
        if rc:
            raise FusorError(rc, "NCCL is not available (libnccl.so.2)")
        return bytes(buf)

    def __init__(self, device: Device, size: int, rank: int, unique_id: bytes):
        self.device, self.size, self.rank = device, size, rank
        buf = (C.c_uint8 * COMM_ID_BYTES).from_buffer_copy(unique_id)
        out = C.c_void_p()
        device._check(device.lib.fb200_comm_create(device.h, size, rank, buf, COMM_ID_BYTES, C.byref(out)))
        self.h = out.value

    def all_reduce_sum(self, t: Tensor) -> Tensor:
        """In-place sum of an f32 tensor over the ranks."""
        self.device._check(self.device.lib.fb200_comm_all_reduce_sum(self.h, t.ptr, int(np.prod(t.shape))))
        return t

    def enable_peer_exchange(self, row_floats: int, all_gather) -> None:
        """Maps every rank's exchange buffer into every other rank (CUDA IPC), so that the
        single-sequence decode kernel sums its partial rows over NVLink itself instead of calling
        NCCL. `row_floats` = the model's hidden size; `all_gather(obj)` returns the list of every
        rank's `obj` in rank order (any host channel). Call on all ranks, before the first decode
        step of a model that uses this communicator."""
        buf = (C.c_uint8 * IPC_HANDLE_BYTES)()
        self.device._check(self.device.lib.fb200_comm_exchange_handle(self.h, row_floats, buf, IPC_HANDLE_BYTES))
        handles = all_gather(bytes(buf))
        if len(handles) != self.size:
            raise FusorError(ERR_INVALID_ARGUMENT, "all_gather must return one handle per rank")
        packed = (C.c_uint8 * (IPC_HANDLE_BYTES * self.size)).from_buffer_copy(b"".join(handles))
        self.device._check(self.device.lib.fb200_comm_exchange_attach(self.h, packed, IPC_HANDLE_BYTES))

    def destroy(self) -> None:
        if self.h:
            self.device.lib.fb200_comm_destroy(self.h)
            self.h = None


class Llama:
    """Llama-architecture decoder (kalosm-llama Model::forward, raw/mod.rs:851-1049).

    With `comm` the model is one rank of a tensor-parallel group: pass the WHOLE model's head and
    FFN sizes; the local counts (divided by comm.size) go to the library, and `set_tensor` expects
    this rank's shards (see `kalosm_b200.tp`)."""

    TENSORS = {"token_embd": 0, "output": 1, "attn_q": 2, "attn_k": 3, "attn_v": 4,
               "attn_output": 5, "ffn_gate": 6, "ffn_up": 7, "ffn_down": 8, "attn_norm": 9,
               "ffn_norm": 10, "output_norm": 11}

    def __init__(self, device: Device, *, n_layer, hidden, ffn, n_head, n_kv_head, head_dim, vocab,
                 max_seq_len, max_batch=1, rms_eps=1e-5, rope_theta=500000.0, rope_scaling=None, comm=None):
        self.device = device
        self.comm = comm
        tp = comm.size if comm is not None else 1
        if n_head % tp or n_kv_head % tp or ffn % tp or vocab % tp:
            raise FusorError(ERR_INVALID_SHAPE, f"heads {n_head}/{n_kv_head}, ffn {ffn} and vocab {vocab} must be "
                                                f"divisible by the {tp} tensor-parallel ranks")
        n_head, n_kv_head, ffn = n_head // tp, n_kv_head // tp, ffn // tp
        factor, low, high, orig = (0.0, 1.0, 4.0, max_seq_len) if rope_scaling is None else rope_scaling
        self.cfg = LlamaConfig(n_layer, hidden, ffn, n_head, n_kv_head, head_dim, vocab, max_seq_len,
                               max_batch, rms_eps, rope_theta, factor, low, high, orig)
        out = C.c_void_p()
        device._check(device.lib.fb200_llama_create(device.h, C.byref(self.cfg), C.byref(out)))
        self.h = out.value
        self.vocab = vocab // tp  # rows of the output head on this rank = width of the logits it returns
        if comm is not None:
            device._check(device.lib.fb200_llama_set_tensor_parallel(self.h, comm.h))

    def set_tensor(self, name: str, layer: int, ggml_type: int, shape, raw) -> None:
        raw = np.ascontiguousarray(raw)
        raw8 = raw.view(np.uint8).reshape(-1)
        n = int(shape[0])
        k = int(shape[1]) if len(shape) > 1 else 1
        d = self.device
        d._check(d.lib.fb200_llama_set_tensor(self.h, layer, self.TENSORS[name], ggml_type, n, k,
                                              _hp(raw8), raw8.size))

    def set_rope_freqs(self, weights) -> None:
        """rope_freqs.weight of a checkpoint: per-frequency factors multiplied into the inverse frequencies."""
        w = np.ascontiguousarray(weights, dtype=np.float32).reshape(-1)
        self.device._check(self.device.lib.fb200_llama_set_rope_freqs(self.h, _hp(w), w.size))

    def reset(self) -> None:
        self.device._check(self.device.lib.fb200_llama_reset(self.h))

    def truncate(self, length: int) -> None:
        """Rewinds the KV caches to the first `length` positions."""
        self.device._check(self.device.lib.fb200_llama_truncate(self.h, length))

    @property
    def position(self) -> int:
        p = C.c_int()
        self.device.lib.fb200_llama_position(self.h, C.byref(p))
        return p.value

    def forward(self, tokens, want_logits: bool = True):
        """tokens [batch, seq] -> (logits [batch, vocab] or None, greedy ids [batch])."""
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        if t.ndim == 1:
            t = t[None, :]
        batch, seq = t.shape
        logits = np.empty((batch, self.vocab), dtype=np.float32) if want_logits else None
        nxt = np.empty(batch, dtype=np.uint32)
        d = self.device
        d._check(d.lib.fb200_llama_forward(self.h, _hp(t), batch, seq, _hp(logits), _hp(nxt)))
        return logits, nxt

    def generate_greedy(self, tokens, steps: int) -> np.ndarray:
        t = np.ascontiguousarray(tokens, dtype=np.uint32).reshape(-1)
        out = np.empty((t.size, steps), dtype=np.uint32)
        d = self.device
        d._check(d.lib.fb200_llama_generate_greedy(self.h, _hp(t), t.size, steps, _hp(out)))
        return out

    def generate_sampled(self, tokens, steps: int, cfg: "SamplerConfig") -> np.ndarray:
        """Sampled decode on the device (run-ahead: no logits or ids cross PCIe until the end)."""
        t = np.ascontiguousarray(tokens, dtype=np.uint32).reshape(-1)
        out = np.empty((t.size, steps), dtype=np.uint32)
        d = self.device
        d._check(d.lib.fb200_llama_generate_sampled(self.h, _hp(t), t.size, steps, C.byref(cfg), _hp(out)))
        return out

    def free(self) -> None:
        if self.h:
            self.device.lib.fb200_llama_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass
