"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations (real GGUF model files are not available, so these stand in for model
activations and quantised embedding tables).

Every array is produced on the host by numpy `Generator(PCG64(seed))` with
seed = 20261125 + 1000 * config + stream, so the CPU oracle and the GPU see identical bytes.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np

from ._abi import AGN_Q2_K, AGN_Q4_K, AGN_Q5_0, AGN_Q5_K, AGN_Q6_K, AGN_Q8_0

BASE_SEED = 20261125
STREAMS = {name: i for i, name in enumerate(
    ["x", "w", "q", "k", "gate", "up", "scores", "ids", "pos", "table", "logits", "wq", "wk", "delta"])}


@dataclass(frozen=True)
class LayerConfig:
    """Shapes of one benchmark configuration (names follow GGUF metadata keys)."""
    index: int
    name: str
    T: int
    hidden: int
    head_dim: int
    n_q_heads: int
    n_kv_heads: int
    ffn: int
    eps: float
    theta: float
    vocab: int
    embd_dtype: int
    random_pos: bool = False
    n_experts: int = 0

    @property
    def n_rot(self) -> int:
        return self.head_dim


CONFIGS = {
    "c1": LayerConfig(1, "llama-3.2-1b-shaped T=512", 512, 2048, 64, 32, 8, 8192, 1e-5, 500000.0, 128256, AGN_Q8_0),
    "c2": LayerConfig(2, "qwen2.5-7b-shaped prefill T=4096", 4096, 3584, 128, 28, 4, 18944, 1e-6, 1e6, 152064,
                      AGN_Q4_K),
    "c3": LayerConfig(3, "qwen2.5-7b-shaped decode sweep", 64, 3584, 128, 28, 4, 18944, 1e-6, 1e6, 152064, AGN_Q4_K,
                      random_pos=True),
    "c4": LayerConfig(4, "llama-3-8b-shaped prefill T=65536", 65536, 4096, 128, 32, 8, 14336, 1e-5, 500000.0, 128256,
                      AGN_Q6_K),
    "c5": LayerConfig(5, "mixtral-8x7b-shaped MoE T=8192", 8192, 4096, 128, 32, 8, 14336, 1e-5, 1e6, 32000, AGN_Q4_K,
                      n_experts=8),
}


def rng_for(config_index: int, stream: str, salt: int = 0) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(BASE_SEED + 1000 * config_index + STREAMS[stream] + 100000 * salt))


def activations(cfg_index: int, stream: str, shape, std: float = 1.0, salt: int = 0) -> np.ndarray:
    """f32 ~ N(0, std^2)."""
    r = rng_for(cfg_index, stream, salt)
    a = r.standard_normal(size=shape, dtype=np.float32)
    if std != 1.0:
        a *= np.float32(std)
    return a


def norm_weight(cfg_index: int, stream: str, n: int) -> np.ndarray:
    """RMSNorm weight ~ N(1, 0.02)."""
    r = rng_for(cfg_index, stream)
    return (1.0 + 0.02 * r.standard_normal(size=n)).astype(np.float32)


def token_ids(cfg_index: int, T: int, vocab: int, salt: int = 0) -> np.ndarray:
    return rng_for(cfg_index, "ids", salt).integers(0, vocab, size=T, dtype=np.uint32)


def positions(cfg_index: int, T: int, random_pos: bool, hi: int = 32768) -> np.ndarray:
    if random_pos:
        return rng_for(cfg_index, "pos").integers(0, hi, size=T, dtype=np.int32)
    return np.arange(T, dtype=np.int32)


def _f16_scales(r: np.random.Generator, n: int) -> np.ndarray:
    return np.abs(r.normal(0.0, 0.01, size=n)).astype(np.float16)


def quant_table(dtype: int, n_rows: int, row_len: int, cfg_index: int = 0, salt: int = 0) -> np.ndarray:
    """A [n_rows, type_size(row_len)] uint8 table of random quant blocks:
    Q8_0: f16 |N(0,.01)| scale + 32 int8 uniform[-127,127];
    Q4_K: f16 d, dmin |N(0,.01)|, 12 uniform scale bytes, 128 uniform nibble bytes;
    Q6_K: 128 uniform ql, 64 uniform qh, 16 int8 uniform scales, f16 d |N(0,.01)|."""
    r = rng_for(cfg_index, "table", salt)
    if dtype == AGN_Q8_0:
        nb = n_rows * ((row_len + 31) // 32)
        t = np.empty((nb, 34), dtype=np.uint8)
        t[:, 0:2] = _f16_scales(r, nb).view(np.uint8).reshape(nb, 2)
        t[:, 2:] = r.integers(-127, 128, size=(nb, 32), dtype=np.int8).view(np.uint8)
    elif dtype == AGN_Q4_K:
        nb = n_rows * ((row_len + 255) // 256)
        t = r.integers(0, 256, size=(nb, 144), dtype=np.uint8)
        t[:, 0:2] = _f16_scales(r, nb).view(np.uint8).reshape(nb, 2)
        t[:, 2:4] = _f16_scales(r, nb).view(np.uint8).reshape(nb, 2)
    elif dtype == AGN_Q5_K:  # f16 d, dmin, 12 scale bytes, 32 high-bit bytes, 128 nibble bytes
        nb = n_rows * ((row_len + 255) // 256)
        t = r.integers(0, 256, size=(nb, 176), dtype=np.uint8)
        t[:, 0:2] = _f16_scales(r, nb).view(np.uint8).reshape(nb, 2)
        t[:, 2:4] = _f16_scales(r, nb).view(np.uint8).reshape(nb, 2)
    elif dtype == AGN_Q5_0:  # f16 d, 4 bytes of high bits, 16 nibble bytes
        nb = n_rows * ((row_len + 31) // 32)
        t = r.integers(0, 256, size=(nb, 22), dtype=np.uint8)
        t[:, 0:2] = _f16_scales(r, nb).view(np.uint8).reshape(nb, 2)
    elif dtype == AGN_Q2_K:  # 16 scale/min nibble bytes, 64 bytes of 2-bit values, f16 d, f16 dmin
        nb = n_rows * ((row_len + 255) // 256)
        t = r.integers(0, 256, size=(nb, 84), dtype=np.uint8)
        t[:, 80:82] = _f16_scales(r, nb).view(np.uint8).reshape(nb, 2)
        t[:, 82:84] = _f16_scales(r, nb).view(np.uint8).reshape(nb, 2)
    elif dtype == AGN_Q6_K:
        nb = n_rows * ((row_len + 255) // 256)
        t = r.integers(0, 256, size=(nb, 210), dtype=np.uint8)
        t[:, 208:210] = _f16_scales(r, nb).view(np.uint8).reshape(nb, 2)
    else:
        raise ValueError(f"no synthetic generator for ggml type {dtype}")
    return t.reshape(n_rows, -1)


def causal_scores(cfg_index: int, n_heads: int, L: int) -> np.ndarray:
    """Attention scores [n_heads, L, L] ~ N(0, 4); row i of each head has i+1 valid entries."""
    return activations(cfg_index, "scores", (n_heads, L, L), std=2.0)


def scale_of_rows(ref: np.ndarray) -> np.ndarray:
    """Row scale used by the parity tolerance: max |reference| over the last axis."""
    s = np.max(np.abs(ref), axis=-1, keepdims=True)
    return np.maximum(s, np.float32(1e-30))


def rel_to_row_scale(got: np.ndarray, ref: np.ndarray) -> np.ndarray:
    """|got - ref| / scale(row), element by element."""
    got = got.reshape(ref.shape)
    return np.abs(got.astype(np.float64) - ref.astype(np.float64)) / scale_of_rows(ref)


def max_rel_to_row_scale(got: np.ndarray, ref: np.ndarray) -> float:
    """max_i |got - ref| / scale(row) — the parity figure for the float ops."""
    err = rel_to_row_scale(got, ref)
    return float(err.max()) if err.size else 0.0


def p999_rel_to_row_scale(got: np.ndarray, ref: np.ndarray) -> float:
    """The 99.9th percentile of the same figure (how far the bulk of the elements sits below the maximum)."""
    err = rel_to_row_scale(got, ref)
    return float(np.quantile(err, 0.999)) if err.size else 0.0
