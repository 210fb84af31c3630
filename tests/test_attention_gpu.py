"""Fused attention forward against the FP32 oracle (reference contract: tests/test_attention.py:86-130 for the
square grid and edge cases, :229-257 for GQA / KV-cache shapes, :167-214 for validation messages).

Tolerances are the reference's: max-abs 2e-3 (fp16), 1.6e-2 (bf16) on unit-normal inputs, plus
8 * 2^-24 * max|s| * max|v| for large scores (tests/test_attention.py:17, :69-70)."""

import glob
import math

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from helpers import ATTN_ATOL, attn_oracle, qkv_case
from kernelforge import _capi, ops

pytestmark = pytest.mark.gpu

SEQ_LENS = [1, 7, 16, 31, 63, 64, 65, 127, 128, 129, 257, 1000]


def run(q, k, v, causal, scale=None, atol=None):
    out = ops.flash_attn(q.cuda(), k.cuda(), v.cuda(), causal=causal, scale=scale)
    assert out.shape == q.shape and out.dtype == q.dtype
    assert torch.isfinite(out).all(), "non-finite values in output"
    ref = attn_oracle(q, k, v, causal, scale)
    err = float(np.abs(out.float().cpu().numpy() - ref).max())
    sc = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    s_max = float((q.float() @ k.float().repeat_interleave(q.shape[1] // k.shape[1], dim=1).transpose(-1, -2)).abs().max()) * sc
    bound = (atol if atol is not None else ATTN_ATOL[q.dtype]) + 8 * 2.0**-24 * s_max * float(v.float().abs().max())
    assert err <= bound, f"max abs err {err:.3e} > {bound:.3e}"
    return err


@pytest.mark.parametrize("causal", [False, True], ids=["full", "causal"])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("n", SEQ_LENS)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["float16", "bfloat16"])
def test_random_grid(dtype, n, d, causal):
    q, k, v = qkv_case(2, 3, 3, n, n, d, dtype, seed=n * 1000 + d)
    run(q, k, v, causal)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["float16", "bfloat16"])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("causal", [False, True], ids=["full", "causal"])
@pytest.mark.parametrize("heads", [(8, 8), (8, 2), (32, 4)], ids=["mha", "gqa4", "gqa8"])
@pytest.mark.parametrize("nq,nk", [(1, 1), (1, 37), (1, 300), (7, 64), (64, 64), (65, 300), (130, 131)])
def test_gqa_and_kv_cache(dtype, d, causal, heads, nq, nk):
    h, hk = heads
    q, k, v = qkv_case(2, h, hk, nq, nk, d, dtype, seed=nq * 31 + nk + h + d)
    run(q, k, v, causal)


@pytest.mark.parametrize("causal", [False, True], ids=["full", "causal"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["float16", "bfloat16"])
def test_all_equal_scores(dtype, causal):
    q, k, v = qkv_case(2, 3, 3, 129, 129, 64, dtype, seed=1)
    run(torch.zeros_like(q), k, v, causal)


@pytest.mark.parametrize("causal", [False, True], ids=["full", "causal"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["float16", "bfloat16"])
def test_large_magnitude(dtype, causal):
    q, k, v = qkv_case(2, 3, 3, 200, 200, 64, dtype, seed=2, scale_q=20.0, scale_k=20.0)
    run(q, k, v, causal)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["float16", "bfloat16"])
def test_large_constant_offset(dtype):
    q = torch.full((2, 3, 96, 64), 8.0).to(dtype)
    k = torch.full((2, 3, 96, 64), 8.0).to(dtype)
    v = torch.randn(2, 3, 96, 64, generator=torch.Generator().manual_seed(4)).to(dtype)
    run(q, k, v, False)


def test_custom_scale():
    q, k, v = qkv_case(2, 3, 3, 100, 100, 64, torch.float16, seed=3)
    run(q, k, v, False, scale=0.05)


@pytest.mark.parametrize("path", sorted(glob.glob(str(GOLDEN / "attn_*.npz"))), ids=lambda p: p.split("/")[-1])
def test_golden(path):
    z = np.load(path)
    scale = float(z["scale"]) if "scale" in z.files else None
    q, k, v = (torch.from_numpy(z[n]).cuda() for n in ("q", "k", "v"))
    out = ops.flash_attn(q, k, v, causal=bool(z["causal"]), scale=scale)
    assert np.abs(out.float().cpu().numpy() - z["ref"]).max() <= ATTN_ATOL[torch.float16]


@pytest.mark.parametrize("b,nk", [(1, 4096), (4, 4096), (1, 16384), (16, 1024)])
def test_decode_gqa_long_cache(b, nk):
    """The decode configuration: Hq = 32, Hkv = 4, D = 64, q_len 1 against a long cache (split-KV path)."""
    q, k, v = qkv_case(b, 32, 4, 1, nk, 64, torch.float16, seed=nk + b)
    run(q, k, v, True)


def test_prefill_benchmark_shape_properties():
    """B=2 H=16 N=2048 D=64: too large for the oracle in seconds on every row, so check a sample of heads
    against the oracle plus two size-independent properties (row-stochastic mixing, permutation of keys)."""
    q, k, v = qkv_case(2, 16, 16, 2048, 2048, 64, torch.float16, seed=7)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    for causal in (False, True):
        out = ops.flash_attn(qc, kc, vc, causal=causal)
        ref = attn_oracle(q[:1, 3:5], k[:1, 3:5], v[:1, 3:5], causal)
        assert np.abs(out[:1, 3:5].float().cpu().numpy() - ref).max() <= ATTN_ATOL[torch.float16]
        # V = const  =>  O = const (softmax rows sum to 1)
        ones = torch.ones_like(vc)
        assert (ops.flash_attn(qc, kc, ones, causal=causal).float() - 1).abs().max().item() <= 2e-3
    # non-causal attention is invariant under a permutation of the keys
    perm = torch.randperm(2048, generator=torch.Generator().manual_seed(0)).cuda()
    a = ops.flash_attn(qc, kc, vc).float()
    bperm = ops.flash_attn(qc, kc[:, :, perm].contiguous(), vc[:, :, perm].contiguous()).float()
    assert (a - bperm).abs().max().item() <= 2e-3


def test_kv_cache_view_is_read_in_place():
    q, k, v = qkv_case(2, 8, 2, 1, 300, 64, torch.float16, seed=9)
    cache_k = torch.zeros(2, 2, 512, 64, dtype=torch.float16).cuda()
    cache_v = torch.zeros_like(cache_k)
    cache_k[:, :, :300], cache_v[:, :, :300] = k.cuda(), v.cuda()
    out = ops.flash_attn_kv_view(q.cuda(), cache_k[:, :, :300], cache_v[:, :, :300], causal=True)
    ref = attn_oracle(q, k, v, True)
    assert np.abs(out.float().cpu().numpy() - ref).max() <= ATTN_ATOL[torch.float16]
    q2, k2, v2 = qkv_case(2, 8, 2, 70, 300, 64, torch.float16, seed=10)
    cache_k[:, :, :300], cache_v[:, :, :300] = k2.cuda(), v2.cuda()
    out = ops.flash_attn_kv_view(q2.cuda(), cache_k[:, :, :300], cache_v[:, :, :300], causal=True)
    assert np.abs(out.float().cpu().numpy() - attn_oracle(q2, k2, v2, True)).max() <= ATTN_ATOL[torch.float16]


@pytest.mark.parametrize("b,h,hk,cap,d", [(2, 32, 4, 512, 64), (1, 8, 8, 256, 128), (3, 16, 2, 4096, 64)])
def test_decode_with_device_side_length(b, h, hk, cap, d):
    """Static cache of capacity `cap`; only kv_len[b] rows are valid, the rest holds garbage that must be ignored."""
    q, k, v = qkv_case(b, h, hk, 1, cap, d, torch.float16, seed=cap + d)
    lens = [cap, max(1, cap // 3), 1][:b] + [cap // 2] * max(0, b - 3)
    kc, vc = k.clone(), v.clone()
    for i, n in enumerate(lens):
        kc[i, :, n:] = 1000.0       # poison what lies beyond the valid length
        vc[i, :, n:] = float("nan")
    out = ops.flash_attn_decode(q.cuda(), kc.cuda(), vc.cuda(), torch.tensor(lens, dtype=torch.int32).cuda())
    assert torch.isfinite(out).all()
    for i, n in enumerate(lens):
        ref = attn_oracle(q[i:i + 1], k[i:i + 1, :, :n], v[i:i + 1, :, :n], True)
        assert np.abs(out[i:i + 1].float().cpu().numpy() - ref).max() <= ATTN_ATOL[torch.float16]


@pytest.mark.parametrize("nk,d", [(512, 64), (4096, 64), (256, 128)])
def test_decode_with_zero_length_row_gives_zeros(nk, d):
    """A sequence with no valid key (kv_len = 0, e.g. a decode step captured before any prefill) yields zeros, not
    0 / 0, in the unsplit and in the split-KV path; the other rows of the batch are unaffected."""
    q, k, v = qkv_case(3, 8, 2, 1, nk, d, torch.float16, seed=nk + d)
    lens = [0, nk, 5]
    out = ops.flash_attn_decode(q.cuda(), k.cuda(), v.cuda(), torch.tensor(lens, dtype=torch.int32).cuda())
    assert torch.isfinite(out).all()
    assert bool((out[0] == 0).all())
    for i in (1, 2):
        ref = attn_oracle(q[i:i + 1], k[i:i + 1, :, :lens[i]], v[i:i + 1, :, :lens[i]], True)
        assert np.abs(out[i:i + 1].float().cpu().numpy() - ref).max() <= ATTN_ATOL[torch.float16]


def test_decode_length_is_read_at_replay_time():
    """One captured launch, replayed while the device-side length grows: the result follows the length."""
    q, k, v = qkv_case(1, 8, 2, 1, 256, 64, torch.float16, seed=77)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    n = torch.tensor([10], dtype=torch.int32).cuda()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        ops.flash_attn_decode(qc, kc, vc, n)
        side.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            out = ops.flash_attn_decode(qc, kc, vc, n)
    for length in (10, 11, 200, 256):
        n.fill_(length)
        g.replay()
        torch.cuda.synchronize()
        ref = attn_oracle(q, k[:, :, :length], v[:, :, :length], True)
        assert np.abs(out.float().cpu().numpy() - ref).max() <= ATTN_ATOL[torch.float16]


def test_determinism_and_status_word():
    q, k, v = qkv_case(1, 32, 4, 1, 4096, 64, torch.float16, seed=5)
    a = ops.flash_attn(q.cuda(), k.cuda(), v.cuda(), causal=True)
    b = ops.flash_attn(q.cuda(), k.cuda(), v.cuda(), causal=True)
    assert torch.equal(a, b)
    q, k, v = qkv_case(2, 4, 4, 300, 300, 64, torch.float16, seed=6)
    a = ops.flash_attn(q.cuda(), k.cuda(), v.cuda(), causal=True)
    b = ops.flash_attn(q.cuda(), k.cuda(), v.cuda(), causal=True)
    assert torch.equal(a, b)
    assert _capi.device_status(torch.device("cuda", 0)) == 0  # no bounded wait has expired


class TestValidation:
    def test_shape_mismatch(self):
        q = torch.randn(1, 2, 8, 64, device="cuda", dtype=torch.float16)
        k = torch.randn(1, 2, 9, 64, device="cuda", dtype=torch.float16)
        v = torch.randn(1, 2, 8, 64, device="cuda", dtype=torch.float16)
        with pytest.raises(ValueError, match="same shape"):
            ops.flash_attn(q, k, v)

    def test_cpu_tensor(self):
        q = torch.randn(1, 2, 8, 64, dtype=torch.float16)
        with pytest.raises(ValueError, match="CUDA"):
            ops.flash_attn(q, q, q)

    def test_bad_rank(self):
        q = torch.randn(2, 8, 64, device="cuda", dtype=torch.float16)
        with pytest.raises(ValueError, match=r"\[B, heads, N, D\]"):
            ops.flash_attn(q, q, q)

    def test_non_contiguous(self):
        q = torch.randn(1, 8, 2, 64, device="cuda", dtype=torch.float16).transpose(1, 2)
        with pytest.raises(ValueError, match="contiguous"):
            ops.flash_attn(q, q, q)

    def test_bad_dtype(self):
        q = torch.randn(1, 2, 8, 64, device="cuda", dtype=torch.float32)
        with pytest.raises(TypeError, match="fp16 or bf16"):
            ops.flash_attn(q, q, q)

    def test_mixed_dtype(self):
        q = torch.randn(1, 2, 8, 64, device="cuda", dtype=torch.float16)
        with pytest.raises(TypeError, match="share a dtype"):
            ops.flash_attn(q, q.to(torch.bfloat16), q)

    def test_bad_scale_and_head_dim(self):
        q = torch.randn(1, 2, 8, 64, device="cuda", dtype=torch.float16)
        with pytest.raises(ValueError, match="positive"):
            ops.flash_attn(q, q, q, scale=-1.0)
        q96 = torch.randn(1, 2, 8, 96, device="cuda", dtype=torch.float16)
        with pytest.raises(ValueError, match="head dim"):
            ops.flash_attn(q96, q96, q96)

    def test_bad_gqa_and_causal_shapes(self):
        q = torch.randn(1, 6, 8, 64, device="cuda", dtype=torch.float16)
        k = torch.randn(1, 4, 8, 64, device="cuda", dtype=torch.float16)
        with pytest.raises(ValueError, match="multiple of key/value heads"):
            ops.flash_attn(q, k, k)
        q2 = torch.randn(1, 4, 9, 64, device="cuda", dtype=torch.float16)
        with pytest.raises(ValueError, match="Nq <= Nk"):
            ops.flash_attn(q2, k, k, causal=True)


@pytest.mark.parametrize("b,h,hk,nk,d,shards", [(1, 32, 4, 16384, 64, 4), (2, 8, 8, 3000, 128, 3), (3, 16, 2, 1024, 64, 2)])
def test_decode_over_a_sequence_sharded_cache(b, h, hk, nk, d, shards):
    """The partial / merge pair that serves a KV cache split along the sequence (one shard per GPU): here every shard
    is processed on this GPU, one call each, the partial buffers are stacked as an all-gather would leave them, and
    the merge must reproduce attention over the whole cache -- including a ragged total length that leaves the last
    shards partly or wholly empty."""
    q, k, v = qkv_case(b, h, hk, 1, nk, d, torch.float16, seed=nk + shards)
    per = nk // shards
    qc = q.cuda()
    for total in (nk, per + 5, 1):
        parts = []
        for r in range(shards):
            ks, vs = k[:, :, r * per:(r + 1) * per].contiguous().cuda(), v[:, :, r * per:(r + 1) * per].contiguous().cuda()
            local = torch.full((b,), max(0, min(per, total - r * per)), dtype=torch.int32).cuda()
            parts.append(ops.flash_attn_decode_partial(qc, ks, vs, local))
        out = ops.flash_attn_merge_partials(torch.stack(parts), qc, hk, per)
        ref = attn_oracle(q, k[:, :, :total], v[:, :, :total], True)
        assert np.abs(out.float().cpu().numpy() - ref).max() <= ATTN_ATOL[torch.float16], f"total {total}"
