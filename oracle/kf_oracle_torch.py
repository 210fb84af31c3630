"""Torch-on-CPU restatement of the reference's FP32 oracles, used as the TIMED CPU baseline.

Test infrastructure, not product code: only tests/, __graft_entry__.smoke() and the cpu_baseline / --impl reference
legs of bench.py may import this module; nothing under kernel-forge_b200/ does.

The reference's own FP32 CPU path is plain torch (its test oracles run unchanged on CPU tensors), so the baseline
that is timed beside every GPU result uses the same library calls on the host cores:
  attention     reference_general, tests/test_attention.py:217-226 (K/V heads repeated, bottom-right causal mask,
                softmax in FP32)
  int4 linear   x.float() @ dequantize(qw, torch.float32).T, tests/test_gemm.py:32, kernelforge/quantize.py:108-114
                (unpack: quantize.py:88-97)
The numpy module kf_oracle.py stays the parity checker; tests/test_oracle_golden.py pins both to the same fixtures.
"""

from __future__ import annotations

import math

import torch

_SHIFTS = torch.tensor([0, 16, 4, 20, 8, 24, 12, 28], dtype=torch.int32)  # nibble of element e sits at bit _SHIFTS[e]


def unpack_int4(packed: torch.Tensor) -> torch.Tensor:
    """int32 [N, K/8] -> int8 [N, K] in [-8, 7] (kernelforge/quantize.py:88-97: element 8j + e is nibble
    (0, 4, 1, 5, 2, 6, 3, 7)[e] of word j)."""
    n, kw = packed.shape
    u = (packed.unsqueeze(-1) >> _SHIFTS) & 0xF
    return (u - 8).to(torch.int8).reshape(n, kw * 8)


def dequantize(packed: torch.Tensor, scales: torch.Tensor, group: int, dtype=torch.float32) -> torch.Tensor:
    q = unpack_int4(packed).to(torch.float32)
    n, k = q.shape
    return (q.view(n, k // group, group) * scales.to(torch.float32).unsqueeze(-1)).view(n, k).to(dtype)


def int4_linear(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, group: int = 128) -> torch.Tensor:
    return x.float() @ dequantize(packed, scales, group, torch.float32).T


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool, scale: float | None = None) -> torch.Tensor:
    h, hk = q.shape[1], k.shape[1]
    kf = k.float().repeat_interleave(h // hk, dim=1)
    vf = v.float().repeat_interleave(h // hk, dim=1)
    s = (q.float() @ kf.transpose(-1, -2)) * (scale if scale is not None else 1.0 / math.sqrt(q.shape[-1]))
    if causal:
        nq, nk = q.shape[2], k.shape[2]
        rows = torch.arange(nq)[:, None] + (nk - nq)
        s = s.masked_fill(torch.arange(nk)[None, :] > rows, float("-inf"))
    return torch.softmax(s, dim=-1) @ vf
