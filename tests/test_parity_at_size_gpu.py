"""Parity at the sizes the benchmark runs, against the FP32 oracle.

The oracle needs an [Nq, Nk] FP32 score matrix per (batch, head), so at N = 4096 / 8192 it is evaluated on blocks
of query rows of a few (batch, head) slices: rows are independent, and under the bottom-right causal mask the rows
[a, b) of a square problem see exactly keys [0, b), which is the oracle's own convention for Nq = b - a, Nk = b.
Every case prints its worst absolute error, the rounding floor of the same reference values in the output type
(max |round(ref) - ref|) and the bound (the reference's criterion, tests/test_attention.py:17,69-70 /
tests/test_gemm.py:17,40-42); run with `-rP` to see the lines.
"""

import math

import numpy as np
import pytest
import torch

from helpers import ATTN_ATOL, assert_int4_close, attn_oracle, int4_case, qkv_case
from kernelforge import ops

pytestmark = pytest.mark.gpu


def _floor(ref: np.ndarray, dtype) -> float:
    r = torch.from_numpy(ref)
    return float((r.to(dtype).float() - r).abs().max())


def _check_rows(out, q, k, v, causal, slices, row_blocks, what):
    worst, floor = 0.0, 0.0
    for (b, h) in slices:
        hk = h // (q.shape[1] // k.shape[1])
        for (a, e) in row_blocks:
            qq = q[b:b + 1, h:h + 1, a:e]
            kk, vv = k[b:b + 1, hk:hk + 1], v[b:b + 1, hk:hk + 1]
            if causal:
                kk, vv = kk[:, :, :e], vv[:, :, :e]   # rows [a, e) see keys [0, e): bottom-right aligned in the oracle
            ref = attn_oracle(qq, kk, vv, causal)
            got = out[b:b + 1, h:h + 1, a:e].float().cpu().numpy()
            worst = max(worst, float(np.abs(got - ref).max()))
            floor = max(floor, _floor(ref, q.dtype))
    s_max = 6.0 * math.sqrt(q.shape[-1]) / math.sqrt(q.shape[-1])   # |s| stays below ~6 sigma on unit-normal inputs
    bound = ATTN_ATOL[q.dtype] + 8 * 2.0**-24 * s_max * 6.0
    print(f"PARITY {what}: max_abs_err {worst:.3e}  rounding_floor {floor:.3e}  bound {bound:.3e}")
    assert worst <= bound, f"{what}: max abs err {worst:.3e} > {bound:.3e}"


@pytest.mark.parametrize("causal", [False, True], ids=["full", "causal"])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("n", [4096, 8192])
def test_attention_sweep_sizes(n, d, causal):
    """B = 2, H = 16, N in {4096, 8192}, D in {64, 128}: the sizes of the attention sweep."""
    q, k, v = qkv_case(2, 16, 16, n, n, d, torch.float16, seed=n + d)
    out = ops.flash_attn(q.cuda(), k.cuda(), v.cuda(), causal=causal)
    assert torch.isfinite(out).all()
    blocks = [(0, 200), (n // 2 - 77, n // 2 + 180), (n - 300, n)]   # start, a tile boundary, the end
    _check_rows(out, q, k, v, causal, [(0, 0), (1, 9), (1, 15)], blocks, f"attn fp16 B2 H16 N{n} D{d} {'causal' if causal else 'full'}")


def test_attention_sweep_bf16_8192():
    q, k, v = qkv_case(1, 4, 4, 8192, 8192, 64, torch.bfloat16, seed=5)
    out = ops.flash_attn(q.cuda(), k.cuda(), v.cuda(), causal=True)
    _check_rows(out, q, k, v, True, [(0, 1), (0, 3)], [(0, 130), (5000, 5300), (8000, 8192)], "attn bf16 B1 H4 N8192 D64 causal")


def test_gqa_causal_prefill_2048():
    """GQA prefill at size: B = 1, Hq = 32, Hkv = 4, N = 2048, D = 64, causal."""
    q, k, v = qkv_case(1, 32, 4, 2048, 2048, 64, torch.float16, seed=11)
    out = ops.flash_attn(q.cuda(), k.cuda(), v.cuda(), causal=True)
    assert torch.isfinite(out).all()
    _check_rows(out, q, k, v, True, [(0, 0), (0, 7), (0, 8), (0, 21), (0, 31)], [(0, 2048)], "attn fp16 GQA B1 Hq32 Hkv4 N2048 D64 causal")


@pytest.mark.parametrize("b,nk", [(64, 4096), (8, 16384), (32, 4096)])
def test_gqa_decode_at_size(b, nk):
    """KV-cache decode (q_len 1) at the benchmarked batch sizes, every (batch, head) against the oracle."""
    q, k, v = qkv_case(b, 32, 4, 1, nk, 64, torch.float16, seed=b + nk)
    out = ops.flash_attn(q.cuda(), k.cuda(), v.cuda(), causal=True)
    ref = attn_oracle(q, k, v, True)
    err = float(np.abs(out.float().cpu().numpy() - ref).max())
    print(f"PARITY decode fp16 B{b} Hq32 Hkv4 Nk{nk} D64: max_abs_err {err:.3e}  rounding_floor {_floor(ref, torch.float16):.3e}  bound {ATTN_ATOL[torch.float16]:.3e}")
    assert err <= ATTN_ATOL[torch.float16]


@pytest.mark.parametrize("n,k", [(1536, 1536), (256, 1536), (8960, 1536), (1536, 8960)], ids=["qo", "kv", "gate_up", "down"])
@pytest.mark.parametrize("m", [1, 16, 128, 1024])
def test_int4_linear_qwen_shapes(m, n, k):
    """The decoder-linear shapes of a Qwen2.5-1.5B layer at M in {1, 16, 128, 1024} through the dispatcher."""
    _, x, packed, scales, ref = int4_case(m, n, k, 128, seed=m + n + k)
    out = ops.int4_linear(torch.from_numpy(x).cuda(), torch.from_numpy(packed).cuda(), torch.from_numpy(scales).cuda(), 128)
    err, peak, rms, floor = assert_int4_close(out, ref, f"qwen m{m} n{n} k{k}")
    print(f"PARITY int4_linear M{m} N{n} K{k} g128: max_abs_err {err:.3e}  rounding_floor {floor:.3e}  "
          f"bound(2e-3*max|ref|) {2e-3 * peak:.3e}  err/rms {err / rms:.2e}")


def test_int4_linear_baseline_config():
    """M = 1, K = 2048, N = 5632, group 128: the stated INT4 configuration."""
    _, x, packed, scales, ref = int4_case(1, 5632, 2048, 128, seed=1)
    out = ops.int4_linear(torch.from_numpy(x).cuda(), torch.from_numpy(packed).cuda(), torch.from_numpy(scales).cuda(), 128)
    err, peak, rms, floor = assert_int4_close(out, ref, "C1")
    print(f"PARITY int4_linear M1 N5632 K2048 g128: max_abs_err {err:.3e}  rounding_floor {floor:.3e}  "
          f"bound(2e-3*max|ref|) {2e-3 * peak:.3e}  err/rms {err / rms:.2e}")
