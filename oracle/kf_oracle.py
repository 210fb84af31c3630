"""CPU oracle for the KernelForge hot paths -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

This module restates, in plain numpy, the arithmetic that the reference project
defines for its two inference paths.  It exists so the CUDA kernels can be
checked against an independent implementation; nothing in the shipped package
imports it.  Only the test-suite, the smoke check and the `cpu_baseline` /
`--impl reference` legs of the benchmark may call it.

Parity status: PINNED.  The functions here are checked (tests/test_oracle_golden.py)
against fixtures that were produced by importing the reference's own Python
package and test oracles on CPU (tests/golden/make_golden.py), and against the
reference's known-answer nibble layout (tests/test_quantize.py:16-25).

Reference locations followed by each function are given in its docstring as
`path:line` inside the reference project.
"""

from __future__ import annotations

import math

import numpy as np

GROUP_SIZES = (64, 128)
# nibble position i (bits 4i..4i+3) stores the weight at k-offset NIBBLE_K[i]
# (kernelforge/quantize.py:34, csrc/micro/sanitize_gemm.cu:27)
NIBBLE_K = (0, 2, 4, 6, 1, 3, 5, 7)
FP16_TINY = np.float32(6.103515625e-05)  # smallest normal fp16


# --------------------------------------------------------------------------
# INT4 weight format
# --------------------------------------------------------------------------

def quantize_int4(weight: np.ndarray, group_size: int = 128):
    """Symmetric per-(row, group) INT4 quantiser.  kernelforge/quantize.py:61-71.

    weight: [N, K] any float dtype.  Returns (q int8 [N, K] in [-8, 7],
    scales fp16 [N, K/G]).  All arithmetic is IEEE fp32: absmax / 7, clamp to
    the smallest normal fp16, one round-to-nearest-even to fp16; a group whose
    absmax is 0 gets scale exactly 1; q = clamp(rint(w / scale32), -8, 7).
    """
    if weight.ndim != 2:
        raise ValueError("weight must be 2-D [N, K]")
    if group_size not in GROUP_SIZES:
        raise ValueError(f"group_size must be one of {GROUP_SIZES}")
    n, k = weight.shape
    if k % group_size:
        raise ValueError(f"K={k} is not a multiple of group_size={group_size}")
    w = weight.astype(np.float32).reshape(n, k // group_size, group_size)
    absmax = np.abs(w).max(axis=-1, keepdims=True)
    s = np.maximum(absmax / np.float32(7.0), FP16_TINY).astype(np.float16)
    s32 = s.astype(np.float32)
    s32 = np.where(absmax == 0, np.float32(1.0), s32)
    q = np.clip(np.rint(w / s32), -8, 7).astype(np.int8).reshape(n, k)
    return q, s32.astype(np.float16).reshape(n, k // group_size)


def pack_int4(q: np.ndarray) -> np.ndarray:
    """int8 [N, K] in [-8, 7] -> int32 [N, K/8].  kernelforge/quantize.py:74-85."""
    if q.ndim != 2 or q.shape[1] % 8:
        raise ValueError("q must be [N, K] with K a multiple of 8")
    if q.size and (q.min() < -8 or q.max() > 7):
        raise ValueError("q values must lie in [-8, 7]")
    n, k = q.shape
    u = (q.astype(np.int64) + 8).reshape(n, k // 8, 8).astype(np.uint32)
    word = np.zeros((n, k // 8), dtype=np.uint32)
    for pos, koff in enumerate(NIBBLE_K):
        word |= u[..., koff] << np.uint32(4 * pos)
    return word.view(np.int32)


def unpack_int4(packed: np.ndarray) -> np.ndarray:
    """int32 [N, K/8] -> int8 [N, K].  kernelforge/quantize.py:88-97."""
    n, kw = packed.shape
    w = np.ascontiguousarray(packed).view(np.uint32)
    out = np.empty((n, kw, 8), dtype=np.int8)
    for pos, koff in enumerate(NIBBLE_K):
        out[..., koff] = ((w >> np.uint32(4 * pos)) & np.uint32(0xF)).astype(np.int8) - 8
    return out.reshape(n, kw * 8)


def quantize_weight(weight: np.ndarray, group_size: int = 128):
    """(packed int32 [N, K/8], scales fp16 [N, K/G]).  kernelforge/quantize.py:100-105."""
    q, s = quantize_int4(weight, group_size)
    return pack_int4(q), s


def dequantize(packed: np.ndarray, scales: np.ndarray, group_size: int, dtype=np.float32) -> np.ndarray:
    """W_hat = q * scale, [N, K].  kernelforge/quantize.py:108-114.

    fp32: the exact product float(q) * float(scale).  fp16: ONE fp16 multiply
    half(q) * scale (round to nearest even), as the reference does.
    """
    n, kw = packed.shape
    k = kw * 8
    q = unpack_int4(packed).reshape(n, k // group_size, group_size)
    if dtype == np.float16:
        prod = q.astype(np.float32) * scales.astype(np.float32)[..., None]  # exact in fp32
        return prod.astype(np.float16).reshape(n, k)
    return (q.astype(np.float32) * scales.astype(np.float32)[..., None]).reshape(n, k).astype(dtype)


def int4_linear(x: np.ndarray, packed: np.ndarray, scales: np.ndarray, group_size: int = 128,
                acc=np.float32) -> np.ndarray:
    """y = x.float() @ dequantize(qw, fp32).T, the reference's FP32 oracle for both
    INT4 kernels (tests/test_gemm.py:32, bench/bench_gemm.py:79).  Returns `acc` dtype
    (fp32 by default, fp64 on request for error analysis); the caller rounds."""
    w = dequantize(packed, scales, group_size, np.float32).astype(acc)
    return x.astype(acc) @ w.T


# --------------------------------------------------------------------------
# Attention
# --------------------------------------------------------------------------

def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, causal: bool, scale: float | None = None,
              acc=np.float32) -> np.ndarray:
    """FP32 attention with grouped-query heads and Nq <= Nk bottom-right causal mask.

    q [B, H, Nq, D], k/v [B, Hk, Nk, D].  Follows `reference_general`
    (tests/test_attention.py:217-226) and `reference_attention` (:33-41): K/V heads are
    repeated H/Hk times, s = q k^T * scale, key j is hidden from query i when
    j > i + (Nk - Nq), softmax over keys, times v.  Default scale 1/sqrt(D)
    (kernelforge/ops.py:53-58).
    """
    b, h, nq, d = q.shape
    hk, nk = k.shape[1], k.shape[2]
    g = h // hk
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    out = np.empty((b, h, nq, d), dtype=acc)
    rows = np.arange(nq)[:, None] + (nk - nq)
    hidden = np.arange(nk)[None, :] > rows
    for bi in range(b):
        for hi in range(h):
            qf = q[bi, hi].astype(acc)
            kf = k[bi, hi // g].astype(acc)
            vf = v[bi, hi // g].astype(acc)
            s = (qf @ kf.T) * acc(scale)
            if causal:
                s = np.where(hidden, -np.inf, s)
            s = s - s.max(axis=-1, keepdims=True)
            p = np.exp(s)
            p /= p.sum(axis=-1, keepdims=True)
            out[bi, hi] = p @ vf
    return out


def attention_flops(b: int, h: int, nq: int, nk: int, d: int, causal: bool) -> float:
    """4*B*H*Nq*Nk*D, halved when causal (kernelforge/bench_utils.py:193-196)."""
    f = 4.0 * b * h * nq * nk * d
    return f / 2 if causal else f


def int4_bytes(m: int, n: int, k: int, group: int) -> int:
    """packed + scales + x + y bytes (bench/bench_gemm.py:80,98)."""
    return n * k // 2 + 2 * n * (k // group) + 2 * m * k + 2 * m * n


def decode_attn_bytes(b: int, h: int, hk: int, nk: int, d: int) -> int:
    """K and V read once plus q and o, fp16."""
    return 2 * b * hk * nk * d * 2 + 2 * b * h * d * 2
