"""B200-native (sm_100a) CUDA backend for the layer-op hot path of the gguf-rs engine:
RMSNorm, rotary embedding, SwiGLU silu*mul, row softmax and quantised-embedding
get_rows, behind the C ABI of include/agention_b200.h.

Importing the package does not load the CUDA library; constructing `CudaBackend`
does, and fails loudly when the library or a GPU is missing (no fallback path).
"""
from ._abi import (AGN_BF16, AGN_KV_Q8_0_WORDS, AGN_F16, AGN_F32, AGN_Q2_K, AGN_Q4_K, AGN_Q5_0, AGN_Q5_K, AGN_Q6_K, AGN_Q8_0, AGN_ROPE_NEOX,
                   AGN_ROPE_NORMAL, LIB_PATH)
from .backend import BackendError, CudaBackend, DeviceBuffer

__all__ = ["CudaBackend", "DeviceBuffer", "BackendError", "LIB_PATH", "AGN_F32", "AGN_F16", "AGN_BF16", "AGN_KV_Q8_0_WORDS",
           "AGN_Q8_0", "AGN_Q2_K", "AGN_Q4_K", "AGN_Q5_0", "AGN_Q5_K", "AGN_Q6_K", "AGN_ROPE_NEOX", "AGN_ROPE_NORMAL"]
