"""INT4 tensor-core GEMM against the FP32 oracle (reference grid: tests/test_gemm.py:82-99), ragged N for
output-feature shards, split-K determinism, and the M dispatcher."""

import glob

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from helpers import LAYER_SHAPES, assert_int4_close, int4_case
from kernelforge import _capi, ops

pytestmark = pytest.mark.gpu


def run_case(fn, m, n, k, group, what):
    _, x, packed, scales, ref = int4_case(m, n, k, group, seed=m * 7 + n + k)
    out = fn(torch.from_numpy(x).cuda(), torch.from_numpy(packed).cuda(), torch.from_numpy(scales).cuda(), group)
    assert out.shape == (m, n) and out.dtype == torch.float16
    return assert_int4_close(out, ref, what)


@pytest.mark.parametrize("group", [64, 128])
@pytest.mark.parametrize("m", [1, 8, 9, 16, 17, 32, 64, 65, 128])
@pytest.mark.parametrize("layer", list(LAYER_SHAPES))
def test_gemm_layer_shapes(layer, m, group):
    n, k = LAYER_SHAPES[layer]
    run_case(ops.int4_gemm, m, n, k, group, f"{layer} m{m} g{group}")


@pytest.mark.parametrize("m,n,k", [(129, 2048, 2048), (300, 1536, 1536), (1024, 5632, 2048), (1024, 1536, 8960)])
def test_gemm_large_m(m, n, k):
    run_case(ops.int4_gemm, m, n, k, 128, f"m{m} n{n} k{k}")


@pytest.mark.parametrize("n", [1, 7, 32, 100, 129, 192, 1120])
@pytest.mark.parametrize("m", [3, 16, 130])
def test_gemm_ragged_n(m, n):
    """N-sharding over 8 GPUs gives 32, 192 and 1120 rows; the reference wrapper refuses N % 64 != 0."""
    run_case(ops.int4_gemm_ragged, m, n, 512, 128, f"ragged m{m} n{n}")


def test_gemm_forces_split_k_and_is_deterministic():
    # N = 128, K = 4096: one tile, so K is split; two runs must agree bit for bit
    _, x, packed, scales, ref = int4_case(33, 128, 4096, 128, seed=17)
    xs, ps, ss = (torch.from_numpy(a).cuda() for a in (x, packed, scales))
    assert _capi.lib().kfb_int4_gemm_ws_bytes(33, 128, 4096, 128) > 0
    a = ops.int4_gemm(xs, ps, ss, 128)
    b = ops.int4_gemm(xs, ps, ss, 128)
    assert torch.equal(a, b)
    assert_int4_close(a, ref, "split-k")


@pytest.mark.parametrize("m", [1, 8, 9, 128])
def test_matmul_dispatcher(m):
    run_case(ops.int4_matmul, m, 2048, 2048, 128, "dispatch")


@pytest.mark.parametrize("path", sorted(glob.glob(str(GOLDEN / "int4_linear_*.npz"))), ids=lambda p: p.split("/")[-1])
def test_gemm_golden(path):
    z = np.load(path)
    out = ops.int4_gemm_ragged(torch.from_numpy(z["x"]).cuda(), torch.from_numpy(z["packed"]).cuda(),
                               torch.from_numpy(z["scales"]).cuda(), int(z["group"]))
    assert_int4_close(out, z["ref"], path)


def test_gemm_rejects_n_not_multiple_of_64():
    _, x, packed, scales, _ = int4_case(16, 100, 256, 128, seed=0)
    with pytest.raises(ValueError, match="multiple of 64"):
        ops.int4_gemm(torch.from_numpy(x).cuda(), torch.from_numpy(packed).cuda(), torch.from_numpy(scales).cuda(), 128)


def test_status_word_clean_after_gemm():
    assert _capi.device_status(torch.device("cuda", 0)) == 0


@pytest.mark.parametrize("m", [1, 5, 16, 130, 1024])
@pytest.mark.parametrize("n,k,group", [(2048, 2048, 128), (1536, 8960, 128), (200, 512, 64), (8960, 1536, 128)])
def test_bf16_activations(m, n, k, group):
    """bf16 activations (the reference is fp16 only): the tcgen05 GEMM with bf16(q * s) weights, against the FP32
    oracle on the same bf16 bits.  Bound: 8x the fp16 bound (bf16 carries 3 bits less), as for attention."""
    from oracle import kf_oracle as ko
    rng = np.random.default_rng(m + n + k)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
    packed, scales = ko.quantize_weight(w, group)
    x = torch.from_numpy(rng.standard_normal((m, k), dtype=np.float32)).bfloat16()
    ref = x.float().numpy() @ ko.dequantize(packed, scales, group, np.float32).T
    out = ops.int4_linear(x.cuda(), torch.from_numpy(packed).cuda(), torch.from_numpy(scales).cuda(), group)
    assert out.dtype == torch.bfloat16 and out.shape == (m, n)
    err = float(np.abs(out.float().cpu().numpy() - ref).max())
    assert err <= 1.6e-2 * float(np.abs(ref).max()), f"bf16 m{m} n{n} k{k}: max abs err {err:.3e}"
