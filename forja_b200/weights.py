"""Weight sources: safetensors files and shard indexes (mirror of crates/forja-host/src/weights.rs
`Safetensors` / `WeightTensor` / `WeightError` over the C ABI's fj_safetensors_* entry points)."""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Optional, Tuple

from . import _lib
from .backend import DTYPE_SIZE, BackendError, Layout, Tensor

IO, NOT_REGULAR_FILE, MAPPING, TRUNCATED, INVALID_HEADER, INVALID_INDEX, HEADER_TOO_LARGE, UNSUPPORTED_DTYPE, INVALID_RANGE, OVERLAPPING_RANGES = range(20, 30)
_NAMES = {IO: "Io", NOT_REGULAR_FILE: "NotRegularFile", MAPPING: "Mapping", TRUNCATED: "Truncated", INVALID_HEADER: "InvalidHeader", INVALID_INDEX: "InvalidIndex",
          HEADER_TOO_LARGE: "HeaderTooLarge", UNSUPPORTED_DTYPE: "UnsupportedDtype", INVALID_RANGE: "InvalidRange", OVERLAPPING_RANGES: "OverlappingRanges"}


class WeightError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"{_NAMES.get(status, status)}: {message}")
        self.status, self.kind, self.message = status, _NAMES.get(status), message


def _check(lib, status: int):
    if status == 0:
        return
    message = (lib.fj_weights_last_error() or b"").decode("utf-8", "replace")
    if status in _NAMES:
        raise WeightError(status, message)
    raise BackendError(status)


class WeightTensor:
    def __init__(self, raw: "_lib.FjWeightTensor"):
        self.name = raw.name.decode("utf-8")
        self.dtype, self.shape = raw.dtype, tuple(raw.shape[:raw.rank])
        self.byte_offset, self.byte_len, self.is_dtype_aligned = raw.byte_offset, raw.byte_len, bool(raw.dtype_aligned)


class Safetensors:
    """One validated safetensors file. ``open_all`` also takes a ``*.json`` shard index."""

    def __init__(self, handle, lib):
        self._h, self._lib = handle, lib

    @staticmethod
    def open(path) -> "Safetensors":
        lib = _lib.load()
        handle = C.c_void_p()
        _check(lib, lib.fj_safetensors_open(os.fsencode(path), C.byref(handle)))
        return Safetensors(handle, lib)

    @staticmethod
    def open_all(path) -> List["Safetensors"]:
        lib = _lib.load()
        count = C.c_uint32(0)
        handles = (C.c_void_p * 1024)()
        _check(lib, lib.fj_safetensors_open_all(os.fsencode(path), handles, 1024, C.byref(count)))
        return [Safetensors(C.c_void_p(handles[i]), lib) for i in range(count.value)]

    def close(self):
        if self._h:
            self._lib.fj_safetensors_close(self._h)
        self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001 - interpreter shutdown
            pass

    @property
    def shard_name(self) -> Optional[str]:
        name = self._lib.fj_safetensors_shard_name(self._h)
        return None if name is None else name.decode("utf-8")

    @property
    def file_len(self) -> int:
        return self._lib.fj_safetensors_file_len(self._h)

    @property
    def data_start(self) -> int:
        return self._lib.fj_safetensors_data_start(self._h)

    def tensors(self) -> List[WeightTensor]:
        out = []
        for i in range(self._lib.fj_safetensors_tensor_count(self._h)):
            raw = _lib.FjWeightTensor()
            _check(self._lib, self._lib.fj_safetensors_tensor(self._h, i, C.byref(raw)))
            out.append(WeightTensor(raw))
        return out

    def import_into(self, backend) -> "ImportedWeights":
        """Maps the file and imports its data region as one read-only buffer of ``backend``."""
        buf = C.c_uint64(0)
        _check(self._lib, self._lib.fj_safetensors_import(backend._h, self._h, C.byref(buf)))
        return ImportedWeights(self, backend, buf.value, self.file_len - self.data_start)


class ImportedWeights:
    def __init__(self, source: Safetensors, backend, buffer: int, byte_len: int):
        self.source, self.backend, self.buffer, self.byte_len = source, backend, buffer, byte_len

    def _tensor(self, raw: "_lib.FjTensor") -> Tensor:
        shape = tuple(raw.shape[:raw.rank])
        return Tensor(raw.buffer, Layout(raw.dtype, raw.offset, shape, tuple(raw.strides[:raw.rank])), self.byte_len, False)

    def tensor(self, name: str) -> Tensor:
        raw = _lib.FjTensor()
        _check(self.source._lib, self.source._lib.fj_safetensors_view(self.source._h, name.encode("utf-8"), self.buffer, C.byref(raw)))
        return self._tensor(raw)

    def quant(self, prefix: str, bits: int = 4, group_size: int = 64) -> Tuple[Tensor, Tensor, Tensor]:
        """(packed, scales, biases) of the MLX affine-quantised matrix stored under ``prefix``."""
        p, s, b = _lib.FjTensor(), _lib.FjTensor(), _lib.FjTensor()
        _check(self.source._lib, self.source._lib.fj_safetensors_quant_views(self.source._h, prefix.encode("utf-8"), self.buffer, bits, group_size,
                                                                              C.byref(p), C.byref(s), C.byref(b)))
        return self._tensor(p), self._tensor(s), self._tensor(b)
