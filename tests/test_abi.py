"""The C-ABI library loads without a GPU, exports every symbol include/agention_b200.h
declares, and refuses to create a context when no device is present (no CPU fallback)."""
import ctypes as C
import re
from pathlib import Path

import pytest

from agention_infer_b200 import _abi
from agention_infer_b200.build import build_library

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    build_library()
    return _abi.load()


def declared_symbols():
    text = (ROOT / "include" / "agention_b200.h").read_text()
    return sorted(set(re.findall(r"AGN_API[^;(]*?\b(agn_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_typed(lib):
    names = declared_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert set(names) == set(_abi.SIGNATURES), "ctypes signatures out of step with the header"


def test_no_oracle_or_torch_dependency():
    import subprocess
    out = subprocess.run(["ldd", str(_abi.LIB_PATH)], capture_output=True, text=True).stdout
    assert "oracle" not in out and "torch" not in out


def test_type_size_matches_reference_table(lib):  # src/types.rs:88-168
    assert lib.agn_type_size(_abi.AGN_Q8_0, 2048) == 2176
    assert lib.agn_type_size(_abi.AGN_Q4_K, 3584) == 2016
    assert lib.agn_type_size(_abi.AGN_Q6_K, 4096) == 3360
    assert lib.agn_type_size(_abi.AGN_Q8_0, 33) == 68
    assert lib.agn_type_size(_abi.AGN_BF16, 5) == 10
    assert lib.agn_type_size(_abi.AGN_Q5_K, 512) == 352
    assert lib.agn_type_size(_abi.AGN_Q5_0, 64) == 44
    assert lib.agn_type_size(_abi.AGN_Q2_K, 512) == 168  # the codec's 84-byte block, src/quant/q2_k.rs:24
    assert lib.agn_type_size(11, 256) == 0  # Q3_K: no kernel


def test_status_strings_and_name(lib):
    assert lib.agn_backend_name() == b"cuda-sm100a"
    assert lib.agn_status_string(_abi.AGN_OK) == b"ok"
    assert b"out of range" in lib.agn_status_string(_abi.AGN_EOOB_ID)
    assert lib.agn_last_error(None) == b"null context"


def test_null_context_is_rejected(lib):
    assert lib.agn_sync(None) == _abi.AGN_EINVAL
    assert lib.agn_silu_mul_f32(None, None, None, None, 4) == _abi.AGN_EINVAL
    assert lib.agn_ctx_create(0, None) == _abi.AGN_EINVAL
    assert lib.agn_quantize_rows_q8_k_f32(None, None, 1, 256, None, None, None) == _abi.AGN_EINVAL
    assert lib.agn_rms_norm_q8_k_f32(None, None, None, 1, 256, 1e-6, None, None, None) == _abi.AGN_EINVAL
    assert lib.agn_host_quantize_rows_q8_k_f32(None, None, 1, 256, None, None, None) == _abi.AGN_EINVAL


def test_host_side_helpers_need_no_gpu(lib):
    assert [lib.agn_q8_k_blocks(n) for n in (-5, 0, 1, 255, 256, 257, 3584)] == [0, 0, 1, 1, 1, 2, 14]
    released = C.c_uint64(7)
    assert lib.agn_gguf_release_pages(None, 0, 10, C.byref(released)) == _abi.AGN_EINVAL and released.value == 0


def test_context_creation_fails_loudly_without_a_gpu(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present; the no-device path is exercised on CPU-only hosts")
    ctx = C.c_void_p()
    assert lib.agn_ctx_create(0, C.byref(ctx)) == _abi.AGN_ECUDA
    assert not ctx.value
    from agention_infer_b200 import BackendError, CudaBackend
    with pytest.raises(BackendError):
        CudaBackend(0)
