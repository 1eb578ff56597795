"""Seeded synthetic inputs for the attention path.

The reference ships no model files or datasets, so every workload here is
standard-normal data drawn from a fixed seed, generated in fp32 (Q first, then
K, then V, each row-major) and cast ONCE, round-to-nearest-even, to the storage
dtype; the cast values are the ground truth that both the CUDA path and the CPU
checker receive. Shapes follow the Llama-family configurations the reference
targets (GQA, KV cache laid out [seq][kv_head][head_dim] as in
include/model/block.hpp:66-67).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class DecodeShape:
    name: str
    seed: int
    batch: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    kv_len: int
    q_dtype: str  # "f32" | "f16" | "bf16"
    kv_dtype: str  # "f16" | "bf16"

    @property
    def kv_bytes(self) -> int:
        return 2 * self.batch * self.kv_len * self.n_kv_heads * self.head_dim * 2

    def algorithmic_bytes(self, o_bytes: int = 4) -> int:
        """K and V read once + Q read + O written (each K/V element counted once, whatever the GQA factor)."""
        qb = {"f32": 4, "f16": 2, "bf16": 2}[self.q_dtype]
        qo = self.batch * self.n_heads * self.head_dim
        return self.kv_bytes + qo * qb + qo * o_bytes


@dataclass(frozen=True)
class PrefillShape:
    name: str
    seed: int
    batch: int
    seq: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    dtype: str  # "bf16" | "f16"

    @property
    def causal_flops(self) -> int:
        """QK^T and PV, 2 flop per multiply-add, unmasked entries only."""
        return 4 * self.head_dim * self.batch * self.n_heads * self.seq * (self.seq + 1) // 2


# TinyLlama-1.1B-shaped single-layer decode (the CPU-runnable case).
C1 = DecodeShape("C1-tinyllama-decode", 0, 1, 32, 4, 64, 512, "f32", "f16")
# Llama-3-8B-shaped batched decode, the configuration the headline metric is quoted on.
C2 = DecodeShape("C2-llama3-8b-decode-b16-kv4096", 1, 16, 32, 8, 128, 4096, "f16", "f16")
# Llama-3-8B-shaped causal prefill.
C3 = PrefillShape("C3-llama3-8b-prefill-b4-s2048", 2, 4, 2048, 32, 8, 128, "bf16")
# Long-context decode, KV sequence sharded over the GPUs of one box.
C4 = DecodeShape("C4-llama3-8b-decode-b1-kv131072", 3, 1, 32, 8, 128, 131072, "f16", "f16")


def _normal(rng: np.random.Generator, shape) -> np.ndarray:
    return rng.standard_normal(size=shape, dtype=np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    lsb = (u >> 16) & 1
    return ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def cast_storage(x: np.ndarray, dtype: str) -> np.ndarray:
    """fp32 -> storage array: float32, float16, or uint16 bf16 bit patterns."""
    if dtype == "f32":
        return x
    if dtype == "f16":
        return x.astype(np.float16)  # numpy rounds to nearest even, like _cvtss_sh(x, 0)
    if dtype == "bf16":
        return f32_to_bf16_bits(x)
    raise ValueError(dtype)


def widen(x: np.ndarray, dtype: str) -> np.ndarray:
    """storage array -> fp32 (exact)."""
    if dtype == "bf16":
        return bf16_bits_to_f32(x)
    return x.astype(np.float32)


def as_f16_for_oracle(x: np.ndarray, dtype: str) -> np.ndarray:
    """K/V storage -> fp16 array for the CPU checker, which only reads fp16.

    A bf16 value with |x| >= 2^-14 is exactly representable in fp16 as long as it
    is below 65504; smaller magnitudes land on fp16's subnormal grid with an
    error below 2^-25, five orders under the parity tolerance.
    """
    if dtype == "f16":
        return x
    return bf16_bits_to_f32(x).astype(np.float16)


def decode_inputs(shape: DecodeShape, kv_len: int | None = None, batch: int | None = None):
    """-> q [B,H,D], k [B,T,Hkv,D], v [B,T,Hkv,D] in storage dtypes."""
    rng = np.random.Generator(np.random.PCG64(shape.seed))
    B = shape.batch if batch is None else batch
    T = shape.kv_len if kv_len is None else kv_len
    q = _normal(rng, (B, shape.n_heads, shape.head_dim))
    k = _normal(rng, (B, T, shape.n_kv_heads, shape.head_dim))
    k = cast_storage(k, shape.kv_dtype)
    v = _normal(rng, (B, T, shape.n_kv_heads, shape.head_dim))
    v = cast_storage(v, shape.kv_dtype)
    return cast_storage(q, shape.q_dtype), k, v


def prefill_inputs(shape: PrefillShape, seq: int | None = None, batch: int | None = None):
    """-> q [B,S,H,D], k [B,S,Hkv,D], v [B,S,Hkv,D] in the shape's storage dtype."""
    rng = np.random.Generator(np.random.PCG64(shape.seed))
    B = shape.batch if batch is None else batch
    S = shape.seq if seq is None else seq
    q = cast_storage(_normal(rng, (B, S, shape.n_heads, shape.head_dim)), shape.dtype)
    k = cast_storage(_normal(rng, (B, S, shape.n_kv_heads, shape.head_dim)), shape.dtype)
    v = cast_storage(_normal(rng, (B, S, shape.n_kv_heads, shape.head_dim)), shape.dtype)
    return q, k, v


def error_metrics(got: np.ndarray, want: np.ndarray):
    """(max_abs, max_rel). rel = |a-b| / max(|b|, 1e-2 * rms(b)): attention outputs at
    long context have magnitude ~1e-2 and pass through zero, so the denominator
    is floored at one percent of the tensor's RMS value."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    diff = np.abs(got - want)
    rms = float(np.sqrt(np.mean(want * want))) if want.size else 0.0
    den = np.maximum(np.abs(want), max(1e-2 * rms, 1e-30))
    return float(diff.max(initial=0.0)), float((diff / den).max(initial=0.0))


ABS_TOL = 2e-3
REL_TOL = 1e-2
