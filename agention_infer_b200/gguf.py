"""GGUF container access over the C ABI (`agn_gguf_*`): header, metadata, tensor directory and
the upload of a tensor to the device — the host-side counterpart of the reference's
`parser::parse` (src/parser.rs:9-66), `loader::load` (src/loader.rs:14-19) and `GgufFile`
accessors (src/types.rs).  Parsing needs no GPU."""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Union

from . import _abi
from .backend import BackendError, CudaBackend, DeviceBuffer


class GgufError(RuntimeError):
    """`GgufError` (src/error.rs:3-42) with the ABI status code."""

    def __init__(self, status: int, message: str):
        super().__init__(f"[agn status {status}] {message}")
        self.status = status


class TensorInfo:
    """`TensorInfo` (src/types.rs:373-403) plus derived row geometry."""

    def __init__(self, raw: _abi.TensorInfo):
        self.name = raw.name.decode()
        self.ggml_type = int(raw.ggml_type)
        self.dims = [int(raw.dims[i]) for i in range(raw.n_dims)]
        self.byte_offset, self.file_offset = int(raw.byte_offset), int(raw.file_offset)
        self.n_rows, self.row_len = int(raw.n_rows), int(raw.row_len)
        self.row_bytes, self.n_bytes = int(raw.row_bytes), int(raw.n_bytes)

    def __repr__(self):
        return f"TensorInfo({self.name!r}, type={self.ggml_type}, dims={self.dims}, offset={self.byte_offset})"


def split_index(name: str):
    """`parse_split_index` (src/loader.rs:25-38): (file_index, total_files) of "name-00001-of-00004.gguf", else None."""
    lib = _abi.load()
    i, n = C.c_uint64(), C.c_uint64()
    if lib.agn_gguf_split_index(name.encode(), C.byref(i), C.byref(n)) != _abi.AGN_OK:
        return None
    return int(i.value), int(n.value)


class GgufFile:
    """A parsed GGUF file: `GgufFile(path)` memory-maps it, `GgufFile(data=bytes)` parses a buffer."""

    def __init__(self, path: Optional[str] = None, data: Optional[Union[bytes, bytearray]] = None):
        self._lib = _abi.load()
        self._g = C.c_void_p()
        err = C.create_string_buffer(256)
        if (path is None) == (data is None):
            raise ValueError("give either a path or data")
        if path is not None:
            st = self._lib.agn_gguf_open(str(path).encode(), C.byref(self._g), err, len(err))
        else:
            self._keep = (C.c_uint8 * len(data)).from_buffer_copy(data)  # the parser reads tensor bytes from it later
            st = self._lib.agn_gguf_parse(self._keep, len(data), C.byref(self._g), err, len(err))
        if st != _abi.AGN_OK:
            self._g = C.c_void_p()
            raise GgufError(st, err.value.decode())

    def close(self) -> None:
        if self._g:
            self._lib.agn_gguf_close(self._g)
            self._g = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def version(self) -> int:
        return int(self._lib.agn_gguf_version(self._g))

    @property
    def tensor_count(self) -> int:
        return int(self._lib.agn_gguf_tensor_count(self._g))

    @property
    def metadata_count(self) -> int:
        return int(self._lib.agn_gguf_metadata_count(self._g))

    @property
    def data_offset(self) -> int:
        return int(self._lib.agn_gguf_data_offset(self._g))

    def get_u64(self, key: str) -> Optional[int]:
        """`GgufFile::get_u64`: unsigned integer metadata of any width, else None."""
        v = C.c_uint64()
        return int(v.value) if self._lib.agn_gguf_get_u64(self._g, key.encode(), C.byref(v)) == _abi.AGN_OK else None

    def get_f32(self, key: str) -> Optional[float]:
        v = C.c_float()
        return float(v.value) if self._lib.agn_gguf_get_f32(self._g, key.encode(), C.byref(v)) == _abi.AGN_OK else None

    def get_string(self, key: str) -> Optional[str]:
        v = C.c_char_p()
        return v.value.decode() if self._lib.agn_gguf_get_string(self._g, key.encode(), C.byref(v)) == _abi.AGN_OK else None

    def get_array_info(self, key: str):
        """(element type id, length) of array metadata, else None."""
        t, n = C.c_uint32(), C.c_uint64()
        if self._lib.agn_gguf_get_array_info(self._g, key.encode(), C.byref(t), C.byref(n)) != _abi.AGN_OK:
            return None
        return int(t.value), int(n.value)

    def tensors(self) -> List[TensorInfo]:
        out = []
        raw = _abi.TensorInfo()
        for i in range(self.tensor_count):
            if self._lib.agn_gguf_tensor_at(self._g, i, C.byref(raw)) == _abi.AGN_OK:
                out.append(TensorInfo(raw))
        return out

    def find(self, name: str) -> Optional[TensorInfo]:
        raw = _abi.TensorInfo()
        if self._lib.agn_gguf_find_tensor(self._g, name.encode(), C.byref(raw)) != _abi.AGN_OK:
            return None
        return TensorInfo(raw)

    def upload(self, backend: CudaBackend, name: str):
        """Copies the tensor to the device: (DeviceBuffer, TensorInfo) — the `table` of get_rows."""
        raw = _abi.TensorInfo()
        p = C.c_void_p()
        st = self._lib.agn_gguf_upload_tensor(backend._ctx, self._g, name.encode(), C.byref(p), C.byref(raw))
        if st != _abi.AGN_OK:
            raise BackendError(st, self._lib.agn_last_error(backend._ctx).decode())
        info = TensorInfo(raw)
        return DeviceBuffer(backend, p.value, info.n_bytes), info
