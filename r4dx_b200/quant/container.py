"""Weight container reader/writer (C++ mmap reader, two-phase writer) as torch tensors.

The file is a safetensors-compatible shell; ``__metadata__`` carries ``model_config`` (JSON),
``quant`` (JSON: per-tensor layout, kb / group) and provenance strings.
"""
from __future__ import annotations

import ctypes
import json
from typing import Dict, Iterable, Tuple

import numpy as np
import torch

from .. import native

_DTYPES = {
    "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "I32": torch.int32,
    "U8": torch.uint8, "I8": torch.int8, "I64": torch.int64, "F8_E4M3": torch.float8_e4m3fn,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class Container:
    """Read-only view of a container file; tensors are zero-copy views of the mapping."""

    def __init__(self, path: str):
        L = native.host()
        err = ctypes.create_string_buffer(512)
        self._L = L
        self._h = L.r4dxb_container_open(path.encode(), err, 512)
        if not self._h:
            raise IOError(f"cannot open container {path}: {err.value.decode()}")
        self.path = path
        self.names = [L.r4dxb_container_name(self._h, i).decode() for i in range(L.r4dxb_container_count(self._h))]
        self._index = {n: i for i, n in enumerate(self.names)}
        self.metadata = {}
        for i in range(L.r4dxb_container_meta_count(self._h)):
            k = L.r4dxb_container_meta_key(self._h, i)
            self.metadata[k.decode()] = L.r4dxb_container_meta_get(self._h, k).decode()

    def close(self):
        if self._h:
            self._L.r4dxb_container_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __contains__(self, name: str) -> bool:
        return name in self._index

    def info(self, name: str) -> Tuple[str, Tuple[int, ...], int]:
        i = self._index[name]
        L = self._L
        shape = tuple(L.r4dxb_container_dim(self._h, i, d) for d in range(L.r4dxb_container_rank(self._h, i)))
        return L.r4dxb_container_dtype(self._h, i).decode(), shape, L.r4dxb_container_nbytes(self._h, i)

    def tensor(self, name: str) -> torch.Tensor:
        dtype, shape, nbytes = self.info(name)
        i = self._index[name]
        ptr = self._L.r4dxb_container_data(self._h, i)
        buf = (ctypes.c_uint8 * nbytes).from_address(ptr)
        arr = np.frombuffer(buf, dtype=np.uint8)
        t = torch.from_numpy(arr)          # read-only mapping: callers copy (.to(device)) before writing
        td = _DTYPES[dtype]
        if td != torch.uint8:
            t = t.view(td)
        return t.view(*shape) if shape else t.view(())

    def byte_view(self, name: str) -> torch.Tensor:
        _, _, nbytes = self.info(name)
        i = self._index[name]
        ptr = self._L.r4dxb_container_data(self._h, i)
        buf = (ctypes.c_uint8 * nbytes).from_address(ptr)
        return torch.from_numpy(np.frombuffer(buf, dtype=np.uint8))

    def model_config(self):
        from ..config import ModelConfig
        return ModelConfig.from_json(self.metadata["model_config"])

    def quant_info(self) -> dict:
        return json.loads(self.metadata.get("quant", "{}"))


def write_container(path: str, tensors: Iterable[Tuple[str, torch.Tensor]], metadata: Dict[str, str]) -> None:
    """Two-phase write: plan every tensor, then stream bytes; lands atomically via ``.partial``."""
    import warnings
    L = native.host()
    tensors = list(tensors)
    w = L.r4dxb_writer_new(path.encode())
    try:
        for k, v in metadata.items():
            L.r4dxb_writer_meta(w, k.encode(), v.encode())
        for name, t in tensors:
            shape = (ctypes.c_int64 * t.dim())(*t.shape)
            idx = L.r4dxb_writer_plan(w, name.encode(), _NAMES[t.dtype].encode(), shape, t.dim(),
                                      t.numel() * t.element_size())
            if idx < 0:
                raise IOError(L.r4dxb_writer_error(w).decode())
        if L.r4dxb_writer_begin(w) != 0:
            raise IOError(L.r4dxb_writer_error(w).decode())
        for idx, (name, t) in enumerate(tensors):
            t = t.detach().cpu().contiguous()
            if L.r4dxb_writer_write(w, idx, t.data_ptr(), t.numel() * t.element_size()) != 0:
                raise IOError(L.r4dxb_writer_error(w).decode())
        if L.r4dxb_writer_finish(w) != 0:
            raise IOError(L.r4dxb_writer_error(w).decode())
    finally:
        L.r4dxb_writer_free(w)
