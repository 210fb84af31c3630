"""Python entry points of the B200 kernels: the operator surface of KernelForge's two inference paths.

Public names, argument meaning, validation rules, exception types and message wording follow the
reference's stable API (kernelforge/ops.py:171-302): `flash_attn`, `int4_linear`, `int4_matmul`,
`int4_gemv`, `int4_gemm`, `GEMV_MAX_M`, and the two `torch.library` custom ops
`kernelforge::flash_attn` / `kernelforge::int4_matmul` with their fake (meta) kernels, so the ops
trace under torch.compile and capture in CUDA graphs.  Below the operator surface everything is
new: tensors are handed as raw pointers to libkfb200.so (include/kfb200.h), hand-written sm_100a
kernels.  Inference only: no backward pass is defined.  There is no CPU or PyTorch fallback.
"""

from __future__ import annotations

import ctypes
import math

import torch

from . import _capi

ATTN_HEAD_DIMS = (64, 128)
ATTN_V1_HEAD_DIMS = ATTN_HEAD_DIMS  # the reference's name for the same tuple (kernelforge/modules.py:87 reads it)
TC_ATTN_DTYPES = (torch.float16, torch.bfloat16)
INT4_GROUP_SIZES = (64, 128)


def _resolve_scale(scale: float | None, head_dim: int) -> float:
    if scale is None:
        return 1.0 / math.sqrt(head_dim)
    if scale <= 0:
        raise ValueError(f"scale must be positive, got {scale}")
    return float(scale)


# ---------------------------------------------------------------------------
# INT4 weight-only linear
# ---------------------------------------------------------------------------

INT4_ACT_DTYPES = (torch.float16, torch.bfloat16)   # the reference takes fp16 only (README.md:103); bf16 is served by the GEMM


def _check_int4(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, group_size: int, allow_bf16: bool = False) -> None:
    ok_dtype = isinstance(x, torch.Tensor) and (x.dtype == torch.float16 or (allow_bf16 and x.dtype == torch.bfloat16))
    if not isinstance(x, torch.Tensor) or not x.is_cuda or not ok_dtype or x.dim() != 2:
        raise TypeError("x must be a 2-D fp16 CUDA tensor [M, K]" + (" (or bf16)" if allow_bf16 else ""))
    if not x.is_contiguous():
        raise ValueError("x must be contiguous")
    if packed.dtype != torch.int32 or scales.dtype != torch.float16:
        raise TypeError("packed must be int32 and scales fp16 (see kernelforge.quantize)")
    k = x.shape[1]
    if k % group_size != 0:
        raise ValueError(f"K={k} is not a multiple of group_size={group_size}")
    if packed.shape[1] * 8 != k:
        raise ValueError(f"packed has K/8={packed.shape[1]} columns but x has K={k}")


def _check_int4_storage(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, group_size: int) -> None:
    # what the reference re-checks in C++ (csrc/gemm/dequant_gemv.cu:5-19)
    if group_size not in INT4_GROUP_SIZES:
        raise ValueError(f"group_size must be one of {INT4_GROUP_SIZES}, got {group_size}")
    if packed.device != x.device or scales.device != x.device:
        raise ValueError("x, packed and scales must be on the same CUDA device")
    if packed.dim() != 2 or not packed.is_contiguous() or not scales.is_contiguous():
        raise ValueError("packed must be a contiguous [N, K/8] tensor and scales contiguous")
    if tuple(scales.shape) != (packed.shape[0], x.shape[1] // group_size):
        raise ValueError(f"scales must be [N, K/group_size] = {(packed.shape[0], x.shape[1] // group_size)}, "
                         f"got {tuple(scales.shape)}")


def _gemv_launch(x, packed, scales, group_size: int, flags: int = 0, small_batch: bool = False) -> torch.Tensor:
    m, k = x.shape
    n = packed.shape[0]
    y = torch.empty(m, n, dtype=torch.float16, device=x.device)
    if n == 0:
        return y
    entry = _capi.lib().kfb_int4_small_batch if small_batch else _capi.lib().kfb_int4_gemv
    with _capi.on_device(x.device):
        _capi.check(entry(x.data_ptr(), packed.data_ptr(), scales.data_ptr(), y.data_ptr(),
                          m, n, k, group_size, flags, _capi.stream_ptr(x.device)))
    return y


def _gemm_launch(x, packed, scales, group_size: int) -> torch.Tensor:
    m, k = x.shape
    n = packed.shape[0]
    y = torch.empty(m, n, dtype=x.dtype, device=x.device)
    if n == 0 or m == 0:
        return y
    lib = _capi.lib()
    ws_bytes = lib.kfb_int4_gemm_ws_bytes(m, n, k, group_size)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=x.device)
    entry = lib.kfb_int4_gemm_bf16 if x.dtype == torch.bfloat16 else lib.kfb_int4_gemm
    with _capi.on_device(x.device):
        _capi.check(entry(x.data_ptr(), packed.data_ptr(), scales.data_ptr(), y.data_ptr(), m, n, k,
                                      group_size, ws.data_ptr(), ws_bytes, _capi.stream_ptr(x.device)))
    return y


def int4_gemv(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, group_size: int = 128) -> torch.Tensor:
    """Fused INT4 dequant GEMV for M in [1, 8]: x [M, K] fp16 @ W_hat^T -> [M, N] fp16."""
    _check_int4(x, packed, scales, group_size)
    if not 1 <= x.shape[0] <= 8:
        raise ValueError(f"int4_gemv handles M in [1, 8], got M={x.shape[0]}")
    _check_int4_storage(x, packed, scales, group_size)
    return _gemv_launch(x, packed, scales, int(group_size))


FUSED_GEMV_MAX_M = 2
XFORM_NONE, XFORM_RMSNORM, XFORM_SILU_MUL = 0, 1, 2


def int4_gemv_fused(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, group_size: int = 128, xform: int = XFORM_NONE,
                    norm_weight: torch.Tensor | None = None, eps: float = 0.0, bias: torch.Tensor | None = None,
                    residual: torch.Tensor | None = None) -> torch.Tensor:
    """INT4 GEMV for M <= 2 with a decode step's element-wise neighbours fused in (see kfb_int4_gemv_fused):
    xform = XFORM_RMSNORM applies RMSNorm(x) * norm_weight first, XFORM_SILU_MUL takes x = [M, 2K] (gate | up) and
    multiplies silu(gate) * up first; bias [N] and residual [M, N] are added to the fp16 result."""
    m = x.shape[0]
    k = x.shape[1] // 2 if xform == XFORM_SILU_MUL else x.shape[1]
    n = packed.shape[0]
    if m > FUSED_GEMV_MAX_M:
        raise ValueError(f"int4_gemv_fused handles M in [1, {FUSED_GEMV_MAX_M}], got M={m}")
    if packed.shape[1] * 8 != k:
        raise ValueError(f"packed has K/8={packed.shape[1]} columns but the activations have K={k}")
    y = torch.empty(m, n, dtype=torch.float16, device=x.device)
    with _capi.on_device(x.device):
        _capi.check(_capi.lib().kfb_int4_gemv_fused(
            x.data_ptr(), packed.data_ptr(), scales.data_ptr(), y.data_ptr(), m, n, k, int(group_size), int(xform),
            norm_weight.data_ptr() if norm_weight is not None else None, float(eps),
            bias.data_ptr() if bias is not None else None, residual.data_ptr() if residual is not None else None,
            0, _capi.stream_ptr(x.device)))
    return y


# ----------------------------------------------------------------------------------------------------------------
# private prepacked weight cache (the reference's stated next step, docs/phase4-notes.md:59): a copy of the packed words
# in MMA-fragment order, keyed on the public tensor, which stays the format callers exchange
# ----------------------------------------------------------------------------------------------------------------
PREPACKED_GEMV_MAX_M = 32   # measured against the dispatcher's kernels on the public format: faster at every M <= 32
_PREPACKED: dict[int, tuple[int, torch.Tensor]] = {}


def prepack_supported(packed: torch.Tensor) -> bool:
    """Shapes the fragment-order GEMV runs: N % 16 == 0, K % 64 == 0, K <= 12288 (a warp holds its share of K in registers)."""
    k = packed.shape[1] * 8 if packed.dim() == 2 else 0
    return packed.dim() == 2 and packed.shape[0] % 16 == 0 and packed.shape[0] >= 16 and k % 64 == 0 and 64 <= k <= 12288


def prepack_int4(packed: torch.Tensor) -> torch.Tensor:
    """The fragment-order copy of a packed weight (kfb_int4_prepack): uint8 [N * K / 2], same size as `packed`."""
    if packed.dtype != torch.int32 or not packed.is_cuda or not packed.is_contiguous() or not prepack_supported(packed):
        raise ValueError("prepack_int4 takes a contiguous int32 CUDA tensor [N, K/8] with N % 16 == 0, K % 64 == 0 and K <= 12288")
    n, k = packed.shape[0], packed.shape[1] * 8
    out = torch.empty(n * k // 2, dtype=torch.uint8, device=packed.device)
    with _capi.on_device(packed.device):
        _capi.check(_capi.lib().kfb_int4_prepack(packed.data_ptr(), n, k, out.data_ptr(), _capi.stream_ptr(packed.device)))
    return out


def prepack_weight_(packed: torch.Tensor) -> torch.Tensor:
    """Builds (once) and caches the private fragment-order copy of `packed`; afterwards int4_linear / int4_matmul run
    batches of up to PREPACKED_GEMV_MAX_M rows on it (M = 1: only where it measured faster, see _prepacked_wins).  The cache entry is keyed on the public tensor (identity and
    version counter: an in-place change of the weight rebuilds the copy) and dies with it.  Costs as much memory again
    as the packed weight."""
    import weakref
    key = id(packed)
    hit = _PREPACKED.get(key)
    if hit is not None and hit[0] == packed._version and hit[1].device == packed.device:
        return hit[1]
    copy = prepack_int4(packed)
    if hit is None:
        weakref.finalize(packed, _PREPACKED.pop, key, None)
    _PREPACKED[key] = (packed._version, copy)
    return copy


def _prepacked_wins(m: int, n: int, k: int) -> bool:
    """Measured (B200, graph of L2-cold calls): the fragment-order GEMV is flat in M and wins from M = 2 on at every
    shape tried; at M = 1 it loses where N is small and K long (1536 x 8960: 8.2 against 5.3 us -- 96 CTAs of 18 K
    blocks per warp) and is within 0.3 us elsewhere."""
    return m >= 2 or n * 8 >= k * 5


def _prepacked_for(packed: torch.Tensor):
    hit = _PREPACKED.get(id(packed))
    if hit is None:
        return None
    if hit[0] != packed._version:   # the public weight was modified in place: rebuild
        return prepack_weight_(packed)
    return hit[1]


def _check_prepacked(x: torch.Tensor, prepacked: torch.Tensor, scales: torch.Tensor, group_size: int) -> tuple[int, int, int]:
    if x.dtype != torch.float16 or not x.is_cuda or not x.is_contiguous() or x.dim() != 2:
        raise TypeError("x must be a contiguous 2-D fp16 CUDA tensor [M, K]")
    m, k = x.shape
    n = scales.shape[0]
    if prepacked.numel() * prepacked.element_size() != n * k // 2 or tuple(scales.shape) != (n, k // group_size):
        raise ValueError("prepacked / scales do not match x: expected N * K / 2 bytes and scales [N, K / group_size]")
    return m, n, k


def int4_gemv_prepacked(x: torch.Tensor, prepacked: torch.Tensor, scales: torch.Tensor, group_size: int = 128,
                        bias: torch.Tensor | None = None, residual: torch.Tensor | None = None) -> torch.Tensor:
    """y[M, N] = x W^T (+ bias, + residual, fp16 adds) for 1 <= M <= 32 on the fragment-order copy of the weight."""
    m, n, k = _check_prepacked(x, prepacked, scales, group_size)
    y = torch.empty(m, n, dtype=torch.float16, device=x.device)
    with _capi.on_device(x.device):
        _capi.check(_capi.lib().kfb_int4_gemv_prepacked(x.data_ptr(), prepacked.data_ptr(), scales.data_ptr(), y.data_ptr(), m, n, k,
                                                        int(group_size), None if bias is None else bias.data_ptr(),
                                                        None if residual is None else residual.data_ptr(),
                                                        _capi.stream_ptr(x.device)))
    return y


def int4_gemv_prepacked_silu_pair(x: torch.Tensor, prepacked: torch.Tensor, scales: torch.Tensor, group_size: int = 128) -> torch.Tensor:
    """int4_gemv_silu_pair on the fragment-order copy of the (gate/up-interleaved) weight, for M <= 8."""
    m, n, k = _check_prepacked(x, prepacked, scales, group_size)
    act = torch.empty(m, n // 2, dtype=torch.float16, device=x.device)
    with _capi.on_device(x.device):
        _capi.check(_capi.lib().kfb_int4_gemv_prepacked_silu_pair(x.data_ptr(), prepacked.data_ptr(), scales.data_ptr(), act.data_ptr(),
                                                                  m, n, k, int(group_size), _capi.stream_ptr(x.device)))
    return act


def int4_gemv_prepacked_rope_kv(x: torch.Tensor, prepacked: torch.Tensor, scales: torch.Tensor, group_size: int, cos: torch.Tensor,
                                sin: torch.Tensor, pos: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, heads: int) -> torch.Tensor:
    """int4_gemv_rope_kv on the fragment-order copy of the (RoPE-pair-ordered) fused qkv weight, for M <= 8."""
    b, n, k = _check_prepacked(x, prepacked, scales, group_size)
    hk, lmax, d = k_cache.shape[1], k_cache.shape[2], k_cache.shape[3]
    if not (k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.shape == v_cache.shape and k_cache.shape[0] == b):
        raise ValueError("k_cache / v_cache must be contiguous [B, Hk, Lmax, D] tensors of the same shape")
    if n != (heads + 2 * hk) * d:
        raise ValueError(f"the fused qkv weight has {n} rows, expected (H + 2 Hk) * D")
    q = torch.empty(b, heads, 1, d, dtype=torch.float16, device=x.device)
    with _capi.on_device(x.device):
        _capi.check(_capi.lib().kfb_int4_gemv_prepacked_rope_kv(x.data_ptr(), prepacked.data_ptr(), scales.data_ptr(), b, k, int(group_size),
                                                                cos.data_ptr(), sin.data_ptr(), pos.data_ptr(), q.data_ptr(),
                                                                k_cache.data_ptr(), v_cache.data_ptr(), heads, hk, d, lmax,
                                                                _capi.stream_ptr(x.device)))
    return q


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Rows (gate_0, up_0, gate_1, up_1, ...): the row order int4_gemv_silu_pair expects (quantise the result)."""
    return torch.stack([gate, up], dim=1).reshape(2 * gate.shape[0], gate.shape[1])


def interleave_qkv_for_rope(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, head_dim: int) -> torch.Tensor:
    """The row order int4_gemv_rope_kv expects: per q head, then per k head, rows (j, j + D/2) adjacent; v unchanged."""
    def pairs(w):
        heads = w.shape[0] // head_dim
        w4 = w.reshape(heads, 2, head_dim // 2, w.shape[1])          # [head, lo / hi half, j, K]
        return w4.transpose(1, 2).reshape(w.shape[0], w.shape[1])    # [head, j, lo / hi, K]
    return torch.cat([pairs(q), pairs(k), v], dim=0)


def int4_gemv_silu_pair(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, group_size: int = 128,
                        norm_weight: torch.Tensor | None = None, eps: float = 0.0) -> torch.Tensor:
    """act[M, N/2] = silu(gate . x) * (up . x) for a weight whose rows were interleaved with interleave_gate_up (M <= 2).
    With `norm_weight`, x is RMS-normalised in the kernel's prologue first."""
    _check_int4(x, packed, scales, group_size)
    m, k = x.shape
    n = packed.shape[0]
    act = torch.empty(m, n // 2, dtype=torch.float16, device=x.device)
    with _capi.on_device(x.device):
        _capi.check(_capi.lib().kfb_int4_gemv_silu_pair(x.data_ptr(), packed.data_ptr(), scales.data_ptr(), act.data_ptr(), m, n, k,
                                                        int(group_size), XFORM_NONE if norm_weight is None else XFORM_RMSNORM,
                                                        None if norm_weight is None else norm_weight.data_ptr(), float(eps), 0,
                                                        _capi.stream_ptr(x.device)))
    return act


def int4_gemv_rope_kv(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, group_size: int, cos: torch.Tensor,
                      sin: torch.Tensor, pos: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, heads: int,
                      norm_weight: torch.Tensor | None = None, eps: float = 0.0) -> torch.Tensor:
    """The fused q/k/v projection of one decode position with RoPE and the KV-cache write in its epilogue (weight rows in
    the order of interleave_qkv_for_rope, M <= 2).  Returns the rotated q [B, H, 1, D]; row `pos` of the caches is written.
    With `norm_weight`, x is RMS-normalised in the kernel's prologue first."""
    _check_int4(x, packed, scales, group_size)
    b, k = x.shape
    if not (k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.shape == v_cache.shape and k_cache.shape[0] == b):
        raise ValueError("k_cache / v_cache must be contiguous [B, Hk, Lmax, D] tensors of the same shape")
    if packed.shape[0] != (heads + 2 * k_cache.shape[1]) * k_cache.shape[3]:
        raise ValueError(f"the fused qkv weight has {packed.shape[0]} rows, expected (H + 2 Hk) * D")
    hk, lmax, d = k_cache.shape[1], k_cache.shape[2], k_cache.shape[3]
    q = torch.empty(b, heads, 1, d, dtype=torch.float16, device=x.device)
    with _capi.on_device(x.device):
        _capi.check(_capi.lib().kfb_int4_gemv_rope_kv(x.data_ptr(), packed.data_ptr(), scales.data_ptr(), b, k, int(group_size),
                                                      XFORM_NONE if norm_weight is None else XFORM_RMSNORM,
                                                      None if norm_weight is None else norm_weight.data_ptr(), float(eps),
                                                      cos.data_ptr(), sin.data_ptr(), pos.data_ptr(),
                                                      q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), heads, hk, d, lmax, 0,
                                                      _capi.stream_ptr(x.device)))
    return q


def int4_small_batch(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, group_size: int = 128) -> torch.Tensor:
    """The GEMV's weight-streaming kernel for M in [1, SMALL_BATCH_MAX_M]: every block of 8 batch rows is one more
    MMA on the already unpacked weight fragment.  Not in the reference (its GEMV stops at M = 8)."""
    _check_int4(x, packed, scales, group_size)
    if not 1 <= x.shape[0] <= SMALL_BATCH_MAX_M:
        raise ValueError(f"int4_small_batch handles M in [1, {SMALL_BATCH_MAX_M}], got M={x.shape[0]}")
    _check_int4_storage(x, packed, scales, group_size)
    return _gemv_launch(x, packed, scales, int(group_size), small_batch=True)


SMALL_BATCH_MAX_M = 32

# Largest M served by the GEMV entry point.  The reference measured 7 on its GPU (kernelforge/ops.py:193,
# bench/sweep_int4_dispatch.py:47-57).  On B200 (CUDA graph, L2-cold weights, us, GEMV / GEMM):
#   5632x2048  M=4 6.3/11.8  M=8 7.7/12.1    2048x2048  3.8/8.1  4.4/8.2    8960x1536  6.0/12.2  7.0/12.6
#   1536x8960  8.6/12.1  11.8/12.2           11264x2048  10.5/18.0  12.3/17.9   32000x2048  15.2/24.3  18.3/24.3
# so the GEMV keeps all of its range.
GEMV_MAX_M = 8


def _small_batch_wins(m: int, n: int, k: int) -> bool:
    """Where int4_small_batch measured faster than the tcgen05 GEMM for 8 < M <= 16 (same method as above, us):
    M = 12: 5632x2048 10.1/12.3, 2048x2048 5.9/8.3, 8960x1536 9.1/13.1, 11264x2048 16.6/18.0, 128256x4096 128/153, but
    1536x8960 16.1/12.3, 2048x5632 12.1/11.4 and 32000x2048 26.8/24.4;  M = 16: 5632x2048 11.3/12.6, 2048x2048 6.5/8.3,
    8960x1536 9.6/13.3, 11264x2048 18.3/18.0, 128256x4096 133/153.  From M = 24 on the GEMM wins everywhere."""
    if n >= 75776:                       # the persistent streaming kernel
        return m <= 16
    return m <= 16 and k <= 2048 and n <= 16384


def int4_gemm(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, group_size: int = 128) -> torch.Tensor:
    """Fused INT4 dequant GEMM on the tcgen05 tensor cores, any M, N a multiple of 64."""
    _check_int4(x, packed, scales, group_size)
    if packed.shape[0] % 64 != 0:
        raise ValueError(f"int4_gemm needs N to be a multiple of 64, got N={packed.shape[0]}")
    _check_int4_storage(x, packed, scales, group_size)
    return _gemm_launch(x, packed, scales, int(group_size))


def int4_gemm_ragged(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, group_size: int = 128) -> torch.Tensor:
    """The same GEMM without the N % 64 rule of the reference wrapper: output-feature shards
    (N/8 = 32, 192, 1120 rows) are not multiples of 64 and the kernel handles them."""
    _check_int4(x, packed, scales, group_size)
    _check_int4_storage(x, packed, scales, group_size)
    return _gemm_launch(x, packed, scales, int(group_size))


def int4_matmul(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, group_size: int = 128) -> torch.Tensor:
    """y = x @ W_hat^T for INT4 weights from kernelforge.quantize, choosing the kernel by M.

    M <= GEMV_MAX_M: the bandwidth-bound GEMV (FP32 accumulation); a little above it, where measured faster, the same
    kernel with more batch columns (int4_small_batch).  Larger M: the tcgen05 GEMM.  bf16 activations (not in the
    reference, README.md:103) take the GEMM at every M.
    """
    if x.dtype == torch.bfloat16:
        _check_int4(x, packed, scales, group_size, allow_bf16=True)
        _check_int4_storage(x, packed, scales, group_size)
        return _gemm_launch(x, packed, scales, int(group_size))
    if x.shape[0] <= PREPACKED_GEMV_MAX_M and x.dtype == torch.float16:
        private = _prepacked_for(packed)          # set by prepack_weight_(packed)
        if private is not None and _prepacked_wins(x.shape[0], packed.shape[0], x.shape[1]):
            _check_int4(x, packed, scales, group_size)
            _check_int4_storage(x, packed, scales, group_size)
            return int4_gemv_prepacked(x, private, scales, group_size)
    if x.shape[0] <= GEMV_MAX_M:
        return int4_gemv(x, packed, scales, group_size)
    if x.shape[0] <= 16 and _small_batch_wins(x.shape[0], packed.shape[0], x.shape[1]):
        return int4_small_batch(x, packed, scales, group_size)
    # the GEMM kernel takes any N; only the public int4_gemm wrapper keeps the reference's N % 64 rule,
    # so an nn.Linear with an odd N that worked below the reference's crossover (M <= 7) keeps working
    return int4_gemm_ragged(x, packed, scales, group_size)


# ---------------------------------------------------------------------------
# Attention
# ---------------------------------------------------------------------------

def _check_attn(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool, strided_kv: bool = False) -> None:
    for name, t in (("q", q), ("k", k), ("v", v)):
        if not isinstance(t, torch.Tensor) or not t.is_cuda:
            raise ValueError(f"{name} must be a CUDA tensor")
        if t.dim() != 4:
            raise ValueError(f"{name} must be 4-D [B, heads, N, D], got shape {tuple(t.shape)}")
        if t.dtype not in TC_ATTN_DTYPES:
            raise TypeError(f"{name} must be fp16 or bf16, got {t.dtype}")
        if not t.is_contiguous() and not (strided_kv and name != "q"):
            raise ValueError(f"{name} must be contiguous (call .contiguous() first)")
    if not (q.dtype == k.dtype == v.dtype):
        raise TypeError(f"q, k, v must share a dtype, got {q.dtype}, {k.dtype}, {v.dtype}")
    if k.shape != v.shape:
        raise ValueError(f"k and v must have the same shape, got {tuple(k.shape)} and {tuple(v.shape)}")
    (b, h, nq, d), (bk, hk, nk, dk) = q.shape, k.shape
    if b != bk or d != dk:
        raise ValueError(f"q {tuple(q.shape)} and k {tuple(k.shape)} must match in batch and head dim")
    if d not in ATTN_HEAD_DIMS:
        raise ValueError(f"head dim must be one of {ATTN_HEAD_DIMS}, got {d}")
    if h % hk != 0:
        raise ValueError(f"query heads ({h}) must be a multiple of key/value heads ({hk})")
    if causal and nq > nk:
        raise ValueError(f"causal attention needs Nq <= Nk (queries are the last Nq positions), got {nq} > {nk}")


def _attn_launch(q, k, v, causal: bool, scale: float, kv_strides=None) -> torch.Tensor:
    b, h, nq, d = q.shape
    hk, nk = k.shape[1], k.shape[2]
    o = torch.empty_like(q)
    if q.numel() == 0:
        return o
    if nk == 0:
        raise ValueError("attention needs at least one key (Nk >= 1)")
    lib = _capi.lib()
    ws_bytes = lib.kfb_flash_attn_ws_bytes(b, h, hk, nq, nk, d)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device) if ws_bytes else None
    strides = None
    if kv_strides is not None:
        strides = (ctypes.c_int64 * 3)(*kv_strides)
    with _capi.on_device(q.device):
        _capi.check(lib.kfb_flash_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                                           _capi.dtype_code(q.dtype), b, h, hk, nq, nk, d, int(causal), scale, strides,
                                           ws.data_ptr() if ws is not None else None, ws_bytes,
                                           _capi.stream_ptr(q.device)))
    return o


@torch.library.custom_op("kernelforge::flash_attn", mutates_args=())
def _flash_attn_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool, scale: float) -> torch.Tensor:
    return _attn_launch(q, k, v, causal, scale)


@_flash_attn_op.register_fake
def _(q, k, v, causal, scale):
    return torch.empty_like(q)


def flash_attn(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = False,
               scale: float | None = None) -> torch.Tensor:
    """Fused attention forward, the stable entry point.

    q: [B, H, Nq, D], k and v: [B, Hk, Nk, D], fp16 or bf16, contiguous, D in {64, 128}.
    H must be a multiple of Hk (grouped-query attention, no K/V copies). Nq may be smaller
    than Nk (decode or chunked prefill against a KV cache): with causal=True, query i is
    treated as position Nk - Nq + i and sees keys 0 .. Nk - Nq + i.
    Returns [B, H, Nq, D] in the input dtype. Inference only (no backward).
    """
    _check_attn(q, k, v, causal)
    if _plain_eager(q):
        return _attn_launch(q, k, v, bool(causal), _resolve_scale(scale, q.shape[-1]))
    return _flash_attn_op(q, k, v, bool(causal), _resolve_scale(scale, q.shape[-1]))


def _plain_eager(t: torch.Tensor) -> bool:
    """True for an ordinary tensor outside torch.compile / export tracing.  The torch.library op costs ~15 us of
    dispatcher time per call, which is as long as a small kernel; it is only needed when the call is being
    traced (fake tensors, dynamo), so plain eager calls -- CUDA-graph capture included -- go straight to the library."""
    return type(t) is torch.Tensor and not torch.compiler.is_compiling()


def flash_attn_kv_view(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = False,
                       scale: float | None = None) -> torch.Tensor:
    """flash_attn for K/V that are strided views of a cache, e.g. `cache[:, :, :L]` of a
    [B, Hk, Lmax, D] buffer: the kernel reads the view in place (the reference copies it with
    .contiguous(), kernelforge/modules.py:95).  Views whose D axis is not dense, whose strides
    differ between k and v, or are not multiples of 8 elements, are copied first."""
    _check_attn(q, k, v, causal, strided_kv=True)
    if k.is_contiguous() and v.is_contiguous():
        if _plain_eager(q):
            return _attn_launch(q, k, v, bool(causal), _resolve_scale(scale, q.shape[-1]))
        return _flash_attn_op(q, k, v, bool(causal), _resolve_scale(scale, q.shape[-1]))
    if k.stride() != v.stride() or k.stride(3) != 1 or any(s % 8 for s in k.stride()[:3]):
        return _flash_attn_op(q, k.contiguous(), v.contiguous(), bool(causal), _resolve_scale(scale, q.shape[-1]))
    return _attn_launch(q, k, v, bool(causal), _resolve_scale(scale, q.shape[-1]), kv_strides=k.stride()[:3])


def flash_attn_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, kv_len: torch.Tensor,
                      scale: float | None = None) -> torch.Tensor:
    """One decode step against a static KV cache.

    q: [B, H, 1, D]; k_cache, v_cache: [B, Hk, Lmax, D] (contiguous or a strided view with a dense D axis);
    kv_len: int32 CUDA tensor [B], the number of valid cache rows per sequence (the new token's K/V already
    written).  The length is read on the device, so the call can be captured once in a CUDA graph and
    replayed while the cache fills (the reference's graph-mode decode has to use SDPA instead,
    bench/e2e_model.py:91-92).  Returns [B, H, 1, D]."""
    _check_attn(q, k_cache, v_cache, False, strided_kv=True)
    if q.shape[2] != 1:
        raise ValueError(f"flash_attn_decode takes one query position per sequence, got Nq={q.shape[2]}")
    if kv_len.dtype != torch.int32 or not kv_len.is_cuda or kv_len.numel() != q.shape[0]:
        raise TypeError("kv_len must be an int32 CUDA tensor with one entry per batch item")
    if k_cache.stride() != v_cache.stride() or k_cache.stride(3) != 1 or any(s % 8 for s in k_cache.stride()[:3]):
        raise ValueError("k_cache and v_cache must share strides, with a dense D axis and strides that are multiples of 8")
    b, h, _, d = q.shape
    hk, nk = k_cache.shape[1], k_cache.shape[2]
    o = torch.empty_like(q)
    lib = _capi.lib()
    ws_bytes = lib.kfb_flash_attn_ws_bytes(b, h, hk, 1, nk, d)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=q.device)
    strides = (ctypes.c_int64 * 3)(*k_cache.stride()[:3])
    with _capi.on_device(q.device):
        _capi.check(lib.kfb_flash_attn_decode_kvlen(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), o.data_ptr(),
                                                    _capi.dtype_code(q.dtype), b, h, hk, nk, d,
                                                    _resolve_scale(scale, d), strides, kv_len.data_ptr(),
                                                    ws.data_ptr(), ws_bytes, _capi.stream_ptr(q.device)))
    return o


def flash_attn_decode_partial(q: torch.Tensor, k_shard: torch.Tensor, v_shard: torch.Tensor,
                              kv_len: torch.Tensor | None = None, scale: float | None = None) -> torch.Tensor:
    """Softmax partials of one decode step over ONE SHARD of the keys (see kfb_flash_attn_decode_partial): a flat fp32
    buffer holding, per (batch, kv-head slot, key split), the unnormalised output, the running maximum and the sum.
    q: [B, H, 1, D]; k_shard, v_shard: [B, Hk, Nk_shard, D]; kv_len: optional int32 [B], valid rows of this shard."""
    _check_attn(q, k_shard, v_shard, False, strided_kv=True)
    b, h, _, d = q.shape
    hk, nk = k_shard.shape[1], k_shard.shape[2]
    lib = _capi.lib()
    nbytes = lib.kfb_flash_attn_decode_partial_bytes(b, h, hk, nk, d, None)
    partial = torch.empty(nbytes // 4, dtype=torch.float32, device=q.device)
    strides = (ctypes.c_int64 * 3)(*k_shard.stride()[:3])
    with _capi.on_device(q.device):
        _capi.check(lib.kfb_flash_attn_decode_partial(q.data_ptr(), k_shard.data_ptr(), v_shard.data_ptr(), _capi.dtype_code(q.dtype),
                                                      b, h, hk, nk, d, _resolve_scale(scale, d), strides,
                                                      kv_len.data_ptr() if kv_len is not None else None, partial.data_ptr(),
                                                      nbytes, _capi.stream_ptr(q.device)))
    return partial


def flash_attn_merge_partials(partials: torch.Tensor, like_q: torch.Tensor, hk: int, nk_per_shard: int) -> torch.Tensor:
    """Merges the partial buffers of several shards ([n_shards, floats_per_shard] fp32, same shard shape each, in shard
    order) into the attention output [B, H, 1, D]."""
    b, h, _, d = like_q.shape
    o = torch.empty_like(like_q)
    n_sets = partials.shape[0] if partials.dim() == 2 else 1
    stride = partials.stride(0) * 4 if partials.dim() == 2 else 0
    with _capi.on_device(like_q.device):
        _capi.check(_capi.lib().kfb_flash_attn_merge_partials(partials.data_ptr(), n_sets, stride, o.data_ptr(),
                                                              _capi.dtype_code(like_q.dtype), b, h, hk, nk_per_shard, d,
                                                              _capi.stream_ptr(like_q.device)))
    return o


# ---------------------------------------------------------------------------
# int4_linear: the nn.Linear-shaped entry point
# ---------------------------------------------------------------------------

@torch.library.custom_op("kernelforge::int4_matmul", mutates_args=())
def _int4_matmul_op(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, group_size: int) -> torch.Tensor:
    return int4_matmul(x, packed, scales, group_size)


@_int4_matmul_op.register_fake
def _(x, packed, scales, group_size):
    return x.new_empty(x.shape[0], packed.shape[0])   # fp16 in -> fp16 out, bf16 in -> bf16 out


def int4_linear(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, group_size: int = 128,
                bias: torch.Tensor | None = None) -> torch.Tensor:
    """y = x @ W_hat^T (+ bias) for INT4 weights from kernelforge.quantize. x: [..., K] fp16.

    Leading dimensions are flattened into M, so [B, T, K] works like nn.Linear. The kernel is
    chosen by M (int4_matmul). Inference only (no backward).
    """
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    _check_int4(x2, packed, scales, group_size, allow_bf16=True)
    if _plain_eager(x2):
        if bias is not None and x2.shape[0] <= FUSED_GEMV_MAX_M and bias.dtype == torch.float16 and bias.is_contiguous():
            # decode-sized call: the bias goes into the GEMV epilogue (same two roundings as `y + bias`)
            _check_int4_storage(x2, packed, scales, group_size)
            return int4_gemv_fused(x2, packed, scales, int(group_size), bias=bias).reshape(*lead, packed.shape[0])
        y = int4_matmul(x2, packed, scales, int(group_size))
    else:
        y = _int4_matmul_op(x2, packed, scales, int(group_size))
    if bias is not None:
        y = y + bias
    return y.reshape(*lead, packed.shape[0])


# ---------------------------------------------------------------------------
# Fused element-wise steps of a decode step (not part of the reference's operator surface, which leaves
# them to torch; used by kernelforge.llama_decode)
# ---------------------------------------------------------------------------

def add_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: torch.Tensor | None = None):
    """(y, s): s = x + residual (x itself when residual is None), y = RMSNorm(s) * weight.  fp16 [rows, hidden]."""
    rows, hidden = x.shape
    y = torch.empty_like(x)
    s = torch.empty_like(x) if residual is not None else x
    with _capi.on_device(x.device):
        _capi.check(_capi.lib().kfb_add_rmsnorm(x.data_ptr(), residual.data_ptr() if residual is not None else None,
                                                weight.data_ptr(), y.data_ptr(),
                                                s.data_ptr() if residual is not None else None, rows, hidden, eps,
                                                _capi.stream_ptr(x.device)))
    return y, s


def rope_kv_write(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos: torch.Tensor, k_cache: torch.Tensor,
                  v_cache: torch.Tensor, heads: int) -> torch.Tensor:
    """Rotates q and k of one decode position, writes k and v into row `pos` of the caches, returns q [B, H, 1, D]."""
    b = qkv.shape[0]
    hk, lmax, d = k_cache.shape[1], k_cache.shape[2], k_cache.shape[3]
    q = torch.empty(b, heads, 1, d, dtype=torch.float16, device=qkv.device)
    with _capi.on_device(qkv.device):
        _capi.check(_capi.lib().kfb_rope_kv_write(qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), pos.data_ptr(), q.data_ptr(),
                                                  k_cache.data_ptr(), v_cache.data_ptr(), b, heads, hk, d, lmax,
                                                  _capi.stream_ptr(qkv.device)))
    return q


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up for gate_up = [rows, 2 * inter] (gate | up)."""
    rows, two = gate_up.shape
    out = torch.empty(rows, two // 2, dtype=torch.float16, device=gate_up.device)
    with _capi.on_device(gate_up.device):
        _capi.check(_capi.lib().kfb_silu_mul(gate_up.data_ptr(), out.data_ptr(), rows, two // 2, _capi.stream_ptr(gate_up.device)))
    return out


def lm_head_argmax(h: torch.Tensor, lm_head: torch.Tensor, logits: torch.Tensor | None = None,
                   best: torch.Tensor | None = None) -> torch.Tensor:
    """logits[M, V] = h[M, K] @ lm_head[V, K]^T (fp16, FP32 accumulation) for M <= 32 with the weight streamed once.
    `best` (int64 CUDA tensor [M], zero before the call) receives the greedy-argmax keys, see kfb_fp16_gemv_argmax;
    `decode_finalize` turns them into token ids."""
    m, k = h.shape
    v = lm_head.shape[0]
    if logits is None:
        logits = torch.empty(m, v, dtype=torch.float16, device=h.device)
    with _capi.on_device(h.device):
        _capi.check(_capi.lib().kfb_fp16_gemv_argmax(h.data_ptr(), lm_head.data_ptr(), logits.data_ptr(),
                                                     best.data_ptr() if best is not None else None, m, v, k,
                                                     _capi.stream_ptr(h.device)))
    return logits


def decode_finalize(best: torch.Tensor, tok: torch.Tensor, pos: torch.Tensor, kv_len: torch.Tensor) -> None:
    """tok <- argmax indices held in `best`, best <- 0, kv_len += 1, pos += 1 (one launch)."""
    with _capi.on_device(tok.device):
        _capi.check(_capi.lib().kfb_decode_finalize(best.data_ptr(), tok.data_ptr(), pos.data_ptr(), kv_len.data_ptr(),
                                                    tok.numel(), _capi.stream_ptr(tok.device)))


def embed_rmsnorm(tok: torch.Tensor, embed: torch.Tensor, weight: torch.Tensor, eps: float):
    """(y, x): x = embed[tok] (tok int64 [rows]), y = RMSNorm(x) * weight, in one pass."""
    rows, (vocab, hidden) = tok.numel(), embed.shape
    y = torch.empty(rows, hidden, dtype=torch.float16, device=embed.device)
    x = torch.empty_like(y)
    with _capi.on_device(embed.device):
        _capi.check(_capi.lib().kfb_embed_rmsnorm(tok.data_ptr(), embed.data_ptr(), weight.data_ptr(), y.data_ptr(), x.data_ptr(),
                                                  rows, hidden, vocab, eps, _capi.stream_ptr(embed.device)))
    return y, x
