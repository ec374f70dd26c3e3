"""ctypes access to the in-tree native libraries (plain C ABI, no torch headers).

``host()`` returns libr4dxb_host.so (C++: container, quantizers, sampler, planners).
``cuda()`` returns libr4dxb_cuda.so (sm_100a kernels).  On a machine with a CUDA device the kernel
library is mandatory: ops never fall back to eager PyTorch when it is missing.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

_HERE = Path(__file__).resolve().parent
_LOCK = threading.Lock()
_HOST = None
_CUDA = None


class NativeLibraryError(RuntimeError):
    pass


def _load(name: str, kind: str) -> ctypes.CDLL:
    path = _HERE / "lib" / name
    if not path.exists():
        if os.environ.get("R4DXB_NO_AUTOBUILD"):
            raise NativeLibraryError(f"{path} is missing; run `python -m r4dx_b200.native.build`")
        from . import build as _build
        _build.build(cuda=(kind == "cuda"), host=(kind == "host"))
    if not path.exists():
        raise NativeLibraryError(f"{path} is missing after build")
    return ctypes.CDLL(str(path))


def host() -> ctypes.CDLL:
    global _HOST
    with _LOCK:
        if _HOST is None:
            _HOST = _load("libr4dxb_host.so", "host")
            _declare_host(_HOST)
        return _HOST


def cuda() -> ctypes.CDLL:
    global _CUDA
    with _LOCK:
        if _CUDA is None:
            _CUDA = _load("libr4dxb_cuda.so", "cuda")
            _declare_cuda(_CUDA)
        return _CUDA


def cuda_loaded() -> bool:
    return _CUDA is not None


c_i64 = ctypes.c_int64
c_u64 = ctypes.c_uint64
c_int = ctypes.c_int
c_f32 = ctypes.c_float
c_f64 = ctypes.c_double
c_ptr = ctypes.c_void_p
c_str = ctypes.c_char_p


def _sig(lib, name, restype, argtypes):
    fn = getattr(lib, name)
    fn.restype = restype
    fn.argtypes = argtypes


def _declare_host(L):
    _sig(L, "r4dxb_trellis_code_f16", ctypes.c_uint16, [ctypes.c_uint32])
    _sig(L, "r4dxb_trellis_decode", None, [c_ptr, c_i64, c_i64, c_int, c_ptr])
    _sig(L, "r4dxb_trellis_packed_words", c_i64, [c_i64, c_i64, c_int])
    _sig(L, "r4dxb_trellis_quantize", c_f64, [c_ptr, c_i64, c_i64, c_int, c_u64, c_int, c_ptr, c_ptr, c_ptr])
    _sig(L, "r4dxb_bpe_new", c_ptr, [c_ptr, c_i64])
    _sig(L, "r4dxb_bpe_free", None, [c_ptr])
    _sig(L, "r4dxb_bpe_encode", c_i64, [c_ptr, c_ptr, c_i64, c_ptr])
    _sig(L, "r4dxb_trellis_quantize_ldlq", c_f64, [c_ptr, c_ptr, c_i64, c_i64, c_int, c_u64, c_int, c_f32, c_ptr, c_ptr, c_ptr, c_ptr])
    _sig(L, "r4dxb_trellis_reconstruct", None, [c_ptr, c_ptr, c_ptr, c_i64, c_i64, c_int, c_int, c_ptr])
    _sig(L, "r4dxb_trellis_encode_tile", c_f32, [c_ptr, c_int, c_ptr])
    _sig(L, "r4dxb_trellis_random_fill", None, [c_ptr, c_i64, c_u64])
    _sig(L, "r4dxb_w4a16_quantize", c_int, [c_ptr, c_i64, c_i64, c_int, c_ptr, c_ptr])
    _sig(L, "r4dxb_w4a16_dequantize", c_int, [c_ptr, c_ptr, c_i64, c_i64, c_int, c_ptr])
    _sig(L, "r4dxb_w8a16_quantize", c_int, [c_ptr, c_i64, c_i64, c_int, c_ptr, c_ptr])
    _sig(L, "r4dxb_w8a16_dequantize", c_int, [c_ptr, c_ptr, c_i64, c_i64, c_int, c_ptr])
    _sig(L, "r4dxb_container_open", c_ptr, [c_str, c_ptr, c_int])
    _sig(L, "r4dxb_container_close", None, [c_ptr])
    _sig(L, "r4dxb_container_count", c_i64, [c_ptr])
    _sig(L, "r4dxb_container_name", c_str, [c_ptr, c_i64])
    _sig(L, "r4dxb_container_dtype", c_str, [c_ptr, c_i64])
    _sig(L, "r4dxb_container_rank", c_int, [c_ptr, c_i64])
    _sig(L, "r4dxb_container_dim", c_i64, [c_ptr, c_i64, c_int])
    _sig(L, "r4dxb_container_data", c_ptr, [c_ptr, c_i64])
    _sig(L, "r4dxb_container_nbytes", c_u64, [c_ptr, c_i64])
    _sig(L, "r4dxb_container_find", c_i64, [c_ptr, c_str])
    _sig(L, "r4dxb_container_meta_count", c_i64, [c_ptr])
    _sig(L, "r4dxb_container_meta_key", c_str, [c_ptr, c_i64])
    _sig(L, "r4dxb_container_meta_get", c_str, [c_ptr, c_str])
    _sig(L, "r4dxb_writer_new", c_ptr, [c_str])
    _sig(L, "r4dxb_writer_free", None, [c_ptr])
    _sig(L, "r4dxb_writer_meta", None, [c_ptr, c_str, c_str])
    _sig(L, "r4dxb_writer_plan", c_int, [c_ptr, c_str, c_str, c_ptr, c_int, c_u64])
    _sig(L, "r4dxb_writer_begin", c_int, [c_ptr])
    _sig(L, "r4dxb_writer_write", c_int, [c_ptr, c_int, c_ptr, c_u64])
    _sig(L, "r4dxb_writer_finish", c_int, [c_ptr])
    _sig(L, "r4dxb_writer_error", c_str, [c_ptr])
    for name, (res, args) in _HOST_EXTRA.items():
        if hasattr(L, name):
            _sig(L, name, res, args)


# filled by modules that add host entry points (sampler, planners, ...)
_HOST_EXTRA: dict = {}
_CUDA_SIGS: dict = {}


def _declare_cuda(L):
    for name, (res, args) in _CUDA_SIGS.items():
        if not hasattr(L, name):
            raise NativeLibraryError(f"kernel library lacks {name}; rebuild with python -m r4dx_b200.native.build")
        _sig(L, name, res, args)


def register_cuda_sig(name: str, restype, argtypes) -> None:
    _CUDA_SIGS[name] = (restype, argtypes)
    if _CUDA is not None:
        _sig(_CUDA, name, restype, argtypes)


def register_host_sig(name: str, restype, argtypes) -> None:
    _HOST_EXTRA[name] = (restype, argtypes)
    if _HOST is not None and hasattr(_HOST, name):
        _sig(_HOST, name, restype, argtypes)
