"""Symmetric group-wise INT4 weight quantisation in KernelForge's packed layout.

Same public surface and the same bits as the reference module (kernelforge/quantize.py:38-126):

    scale[n, g] = fp16(max(max|W[n, gG:(g+1)G]| / 7, 2^-14)),   1 for an all-zero group
    q[n, k]     = clamp(rint(W[n, k] / scale), -8, 7)           IEEE fp32, ties to even
    packed      = int32 [N, K/8]; nibble position i of word j holds q[n, 8j + (0,2,4,6,1,3,5,7)[i]] + 8
    scales      = fp16  [N, K/G]

so that `(word >> 4i) & 0x000F000F` holds the pair (k = 2i, k = 2i+1) in its two 16-bit halves.

CUDA tensors are processed by the library's kernels (kfb_quantize_pack, kfb_pack_int4,
kfb_unpack_int4, kfb_dequantize).  The reference module is device-agnostic torch code and its
tests call it on CPU tensors too (tests/test_quantize.py:9); CPU tensors are therefore handled
with torch ops here as well -- a CUDA tensor never takes that route.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _capi

DEFAULT_GROUP_SIZE = 128
SUPPORTED_GROUP_SIZES = (64, 128)
_NIBBLE_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)  # k offset stored at nibble position i
_SHIFT_OF_K = tuple(4 * _NIBBLE_ORDER.index(k) for k in range(8))  # bit offset of k offset k


@dataclass
class QuantizedWeight:
    packed: torch.Tensor  # int32 [N, K // 8]
    scales: torch.Tensor  # fp16 [N, K // group_size]
    group_size: int
    shape: tuple[int, int]  # (N, K) of the original weight

    @property
    def nbytes(self) -> int:
        return self.packed.numel() * 4 + self.scales.numel() * 2


def _check_shape(weight: torch.Tensor, group_size: int) -> tuple[int, int]:
    if weight.dim() != 2:
        raise ValueError(f"weight must be 2-D [N, K], got shape {tuple(weight.shape)}")
    if group_size not in SUPPORTED_GROUP_SIZES:
        raise ValueError(f"group_size must be one of {SUPPORTED_GROUP_SIZES}, got {group_size}")
    n, k = weight.shape
    if k % group_size != 0:
        raise ValueError(f"K={k} is not a multiple of group_size={group_size}. Pad K or pick another group size.")
    return n, k


def _kernel_input(weight: torch.Tensor) -> torch.Tensor:
    w = weight.detach()
    if w.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        w = w.float()
    return w.contiguous()


def _cuda_quantize_pack(weight: torch.Tensor, group_size: int) -> tuple[torch.Tensor, torch.Tensor]:
    n, k = weight.shape
    w = _kernel_input(weight)
    packed = torch.empty(n, k // 8, dtype=torch.int32, device=w.device)
    scales = torch.empty(n, k // group_size, dtype=torch.float16, device=w.device)
    if n:
        with _capi.on_device(w.device):
            _capi.check(_capi.lib().kfb_quantize_pack(w.data_ptr(), _capi.dtype_code(w.dtype), n, k, group_size,
                                                      packed.data_ptr(), scales.data_ptr(), _capi.stream_ptr(w.device)))
    return packed, scales


def quantize_int4(weight: torch.Tensor, group_size: int = DEFAULT_GROUP_SIZE) -> tuple[torch.Tensor, torch.Tensor]:
    """Returns (q, scales): q int8 [N, K] in [-8, 7], scales fp16 [N, K / group_size]."""
    n, k = _check_shape(weight, group_size)
    if weight.is_cuda:
        packed, scales = _cuda_quantize_pack(weight, group_size)
        return unpack_int4(packed), scales
    groups = weight.detach().float().reshape(n, k // group_size, group_size)
    peak = groups.abs().amax(dim=-1, keepdim=True)
    tiny = torch.finfo(torch.float16).tiny
    scale16 = torch.clamp(peak / 7.0, min=tiny).to(torch.float16)
    scale16 = torch.where(peak == 0, torch.ones_like(scale16), scale16)
    q = (groups / scale16.float()).round_().clamp_(-8, 7).to(torch.int8)
    return q.reshape(n, k), scale16.reshape(n, k // group_size)


def pack_int4(q: torch.Tensor) -> torch.Tensor:
    """int8 [N, K] in [-8, 7] -> int32 [N, K / 8] in the kernel layout (see module docstring)."""
    if q.dim() != 2 or q.shape[1] % 8 != 0:
        raise ValueError(f"q must be [N, K] with K a multiple of 8, got {tuple(q.shape)}")
    if q.numel() and (q.min() < -8 or q.max() > 7):
        raise ValueError("q values must lie in [-8, 7]")
    n, k = q.shape
    if q.is_cuda:
        q8 = q.to(torch.int8).contiguous()
        packed = torch.empty(n, k // 8, dtype=torch.int32, device=q.device)
        if n:
            with _capi.on_device(q.device):
                _capi.check(_capi.lib().kfb_pack_int4(q8.data_ptr(), n, k, packed.data_ptr(), _capi.stream_ptr(q.device)))
        return packed
    nibbles = (q.to(torch.int64) + 8).reshape(n, k // 8, 8)
    word = (nibbles << torch.tensor(_SHIFT_OF_K, dtype=torch.int64)).sum(dim=-1)
    return (((word + 2**31) % 2**32) - 2**31).to(torch.int32)  # reinterpret the low 32 bits as signed


def unpack_int4(packed: torch.Tensor) -> torch.Tensor:
    """Inverse of pack_int4: int32 [N, K / 8] -> int8 [N, K] in [-8, 7]."""
    n, kw = packed.shape
    if packed.is_cuda:
        p = packed.contiguous()
        q = torch.empty(n, kw * 8, dtype=torch.int8, device=p.device)
        if n:
            with _capi.on_device(p.device):
                _capi.check(_capi.lib().kfb_unpack_int4(p.data_ptr(), n, kw * 8, q.data_ptr(), _capi.stream_ptr(p.device)))
        return q
    bits = packed.to(torch.int64).unsqueeze(-1) >> torch.tensor(_SHIFT_OF_K, dtype=torch.int64)
    return ((bits & 0xF) - 8).to(torch.int8).reshape(n, kw * 8)


def quantize_weight(weight: torch.Tensor, group_size: int = DEFAULT_GROUP_SIZE) -> QuantizedWeight:
    """Quantize and pack an nn.Linear weight [N, K] for the INT4 kernels."""
    n, k = _check_shape(weight, group_size)
    if weight.is_cuda:
        packed, scales = _cuda_quantize_pack(weight, group_size)
    else:
        q, scales = quantize_int4(weight, group_size)
        packed, scales = pack_int4(q).contiguous(), scales.contiguous()
    return QuantizedWeight(packed=packed, scales=scales, group_size=group_size, shape=(n, k))


def dequantize(qw: QuantizedWeight, dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """W_hat = q * scale, [N, K].  fp16: one fp16 multiply; otherwise the exact FP32 product cast to `dtype`."""
    n, k = qw.shape
    if qw.packed.is_cuda:
        kernel_dtype = torch.float16 if dtype == torch.float16 else torch.float32
        out = torch.empty(n, k, dtype=kernel_dtype, device=qw.packed.device)
        if n:
            p, s = qw.packed.contiguous(), qw.scales.contiguous()
            with _capi.on_device(p.device):
                _capi.check(_capi.lib().kfb_dequantize(p.data_ptr(), s.data_ptr(), n, k, qw.group_size, out.data_ptr(),
                                                       _capi.dtype_code(kernel_dtype), _capi.stream_ptr(p.device)))
        return out if dtype == kernel_dtype else out.to(dtype)
    q = unpack_int4(qw.packed).reshape(n, k // qw.group_size, qw.group_size)
    s = qw.scales.unsqueeze(-1)
    if dtype == torch.float16:
        return (q.to(torch.float16) * s).reshape(n, k)
    return (q.float() * s.float()).reshape(n, k).to(dtype)


def quantization_error(weight: torch.Tensor, qw: QuantizedWeight) -> dict:
    """Error of the INT4 approximation vs the original weights (independent of any kernel)."""
    w = weight.float()
    diff = dequantize(qw, torch.float32) - w
    return {
        "max_abs_err": diff.abs().max().item(),
        "rmse": diff.pow(2).mean().sqrt().item(),
        "rel_fro_err": (diff.norm() / w.norm().clamp_min(1e-30)).item(),
        "bits_per_weight": 8.0 * qw.nbytes / w.numel(),
    }
