"""GGUF container access over the C ABI (`agn_gguf_*`): header, metadata, tensor directory and
the upload of a tensor to the device — the host-side counterpart of the reference's
`parser::parse` (src/parser.rs:9-66), `loader::load` (src/loader.rs:14-19) and `GgufFile`
accessors (src/types.rs).  Parsing needs no GPU."""
from __future__ import annotations

import ctypes as C
import dataclasses
import warnings
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


def rope_freq_scale(scaling_type: Optional[str], factor: Optional[float]) -> Optional[float]:
    """`compute_rope_freq_scale` (src/model/llama/cpu_path.rs:34-40): the freq_scale of the rope entry points, or None
    for a scheme that is not applied (e.g. "yarn")."""
    out = C.c_float()
    st = _abi.load().agn_rope_freq_scale(None if scaling_type is None else scaling_type.encode(), 0 if factor is None else 1,
                                         0.0 if factor is None else float(factor), C.byref(out))
    return float(out.value) if st == _abi.AGN_OK else None


@dataclasses.dataclass
class ModelConfig:
    """`ModelConfig::from_gguf` (src/model/mod.rs:196-286): the hyper-parameters the layer ops take, read from the GGUF
    metadata under the architecture's prefix, with the reference's defaults."""
    architecture: str
    context_length: int
    embedding_length: int
    block_count: int
    head_count: int
    head_count_kv: int
    head_dim: int
    feed_forward_length: int
    rope_freq_base: float
    rope_scaling_type: Optional[str]
    rope_scaling_factor: Optional[float]
    layer_norm_rms_epsilon: float
    vocab_size: int

    @property
    def freq_scale(self) -> float:
        """`LlamaModel::rope_freq_scale` (src/model/llama/cpu_path.rs:44-60): 1.0 with a warning for an unapplied scheme."""
        s = rope_freq_scale(self.rope_scaling_type, self.rope_scaling_factor)
        if s is None:
            warnings.warn(f"rope scaling type '{self.rope_scaling_type}' is not applied; positions are used unscaled")
            return 1.0
        return s


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

    def get_i64_array(self, key: str) -> Optional[List[int]]:
        """`GgufFile::get_i64_array` (src/types.rs:451-454): an integer array of any element width, else None."""
        n = C.c_uint64()
        if self._lib.agn_gguf_get_array_i64(self._g, key.encode(), None, 0, C.byref(n)) != _abi.AGN_OK:
            return None
        buf = (C.c_int64 * max(int(n.value), 1))()
        self._lib.agn_gguf_get_array_i64(self._g, key.encode(), buf, n.value, C.byref(n))
        return [int(buf[i]) for i in range(int(n.value))]

    def tensors(self) -> List[TensorInfo]:
        out = []
        raw = _abi.TensorInfo()
        for i in range(self.tensor_count):
            st = self._lib.agn_gguf_tensor_at(self._g, i, C.byref(raw))
            if st == _abi.AGN_EFORMAT:
                raise GgufError(st, f"tensor {i}: dimensions or offset overflow 64 bits")
            if st == _abi.AGN_OK:
                out.append(TensorInfo(raw))
        return out

    def find(self, name: str) -> Optional[TensorInfo]:
        raw = _abi.TensorInfo()
        st = self._lib.agn_gguf_find_tensor(self._g, name.encode(), C.byref(raw))
        if st == _abi.AGN_EFORMAT:
            raise GgufError(st, f"tensor '{name}': dimensions or offset overflow 64 bits")
        if st != _abi.AGN_OK:
            return None
        return TensorInfo(raw)

    def model_config(self) -> ModelConfig:
        """`ModelConfig::from_gguf` (src/model/mod.rs:213-286); a per-layer `head_count_kv` array (0 for layers without
        attention) is reduced to its largest positive entry, as the reference does (:236-246)."""
        arch = self.get_string("general.architecture")
        if arch is None:
            raise GgufError(_abi.AGN_ENOTFOUND, "missing metadata: general.architecture")

        def need(field):
            v = self.get_u64(f"{arch}.{field}")
            if v is None:
                raise GgufError(_abi.AGN_ENOTFOUND, f"missing metadata: {arch}.{field}")
            return v

        head_count, embedding_length = need("attention.head_count"), need("embedding_length")
        key_length = self.get_u64(f"{arch}.attention.key_length")
        emb = self.find("token_embd.weight")
        if emb is None:
            raise GgufError(_abi.AGN_ENOTFOUND, "missing metadata: token_embd.weight tensor")
        u = lambda f, d: d if self.get_u64(f"{arch}.{f}") is None else self.get_u64(f"{arch}.{f}")
        head_count_kv = self.get_u64(f"{arch}.attention.head_count_kv")
        if head_count_kv is None:
            per_layer = [v for v in (self.get_i64_array(f"{arch}.attention.head_count_kv") or []) if v > 0]
            head_count_kv = max(per_layer) if per_layer else head_count
        fl = lambda f, d: d if self.get_f32(f"{arch}.{f}") is None else self.get_f32(f"{arch}.{f}")
        return ModelConfig(
            architecture=arch, context_length=u("context_length", 4096), embedding_length=embedding_length,
            block_count=u("block_count", 32), head_count=head_count, head_count_kv=head_count_kv,
            head_dim=key_length if key_length is not None else embedding_length // head_count,
            feed_forward_length=u("feed_forward_length", 0), rope_freq_base=fl("rope.freq_base", 10000.0),
            rope_scaling_type=self.get_string(f"{arch}.rope.scaling.type"),
            rope_scaling_factor=self.get_f32(f"{arch}.rope.scaling.factor"),
            layer_norm_rms_epsilon=fl("attention.layer_norm_rms_epsilon", 1e-5),
            vocab_size=emb.dims[1] if len(emb.dims) >= 2 else emb.dims[0])

    def upload(self, backend: CudaBackend, name: str):
        """Copies the tensor to the device: (DeviceBuffer, TensorInfo) — the `table` of get_rows."""
        raw = _abi.TensorInfo()
        p = C.c_void_p()
        st = self._lib.agn_gguf_upload_tensor(backend._ctx, self._g, name.encode(), C.byref(p), C.byref(raw))
        if st != _abi.AGN_OK:
            raise BackendError(st, self._lib.agn_last_error(backend._ctx).decode())
        info = TensorInfo(raw)
        return DeviceBuffer(backend, p.value, info.n_bytes), info

    def tensor_bytes(self, name: str) -> bytes:
        """A copy of the tensor's bytes as the file holds them (`&raw_data[byte_offset ..]`, src/quant/mod.rs:97-135)."""
        p, n = C.c_void_p(), C.c_uint64(0)
        st = self._lib.agn_gguf_tensor_data(self._g, name.encode(), C.byref(p), C.byref(n))
        if st != _abi.AGN_OK:
            raise GgufError(st, f"tensor {name!r}")
        return C.string_at(p.value, n.value)

    def upload_tensors(self, backend: CudaBackend, names, release_pages: bool = True):
        """`pre_upload_gpu` (src/model/llama/gpu_resident.rs:112-152): uploads the named tensors in ascending file-offset
        order and (release_pages) drops the consumed part of the mapping from the page cache as it goes.
        Returns ({name: (DeviceBuffer, TensorInfo)}, bytes of page cache released)."""
        names = list(names)
        n = len(names)
        c_names = (C.c_char_p * n)(*[s.encode() for s in names])
        ptrs = (C.c_void_p * n)()
        infos = (_abi.TensorInfo * n)()
        released = C.c_uint64(0)
        st = self._lib.agn_gguf_upload_tensors(backend._ctx, self._g, c_names, n, ptrs, infos, 1 if release_pages else 0,
                                               C.byref(released))
        if st != _abi.AGN_OK:
            raise BackendError(st, self._lib.agn_last_error(backend._ctx).decode())
        out = {}
        for i, name in enumerate(names):
            info = TensorInfo(infos[i])
            out[name] = (DeviceBuffer(backend, ptrs[i], info.n_bytes), info)
        return out, int(released.value)

    def release_pages(self, start: int, end: int) -> int:
        """Drops the whole pages inside file bytes [start, end) from the page cache; returns the bytes released."""
        released = C.c_uint64(0)
        st = self._lib.agn_gguf_release_pages(self._g, start, end, C.byref(released))
        if st != _abi.AGN_OK:
            raise GgufError(st, "release_pages")
        return int(released.value)

    def dequant_tensor(self, backend: CudaBackend, name: str):
        """`WeightMap::dequant_tensor` (src/model/mod.rs:318-345): the whole tensor as f32 [n_rows, row_len] on the device
        (every row through the get_rows kernel).  Returns (DeviceBuffer, TensorInfo)."""
        import numpy as np
        table, info = self.upload(backend, name)
        ids = backend.upload(np.arange(info.n_rows, dtype=np.uint32))
        out = backend.get_rows(info.ggml_type, table, info.n_bytes, info.n_rows, info.row_len, ids, info.n_rows)
        backend.sync()
        table.free(); ids.free()
        return out, info
