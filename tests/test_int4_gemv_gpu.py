"""INT4 GEMV (M = 1..8) against the FP32 oracle `x.float() @ dequantize(qw, fp32).T`
(reference grid: tests/test_gemm.py:48-79; golden vectors made by the reference itself)."""

import glob

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from helpers import LAYER_SHAPES, assert_int4_close, int4_case
from kernelforge import ops
from kernelforge import quantize as kq

pytestmark = pytest.mark.gpu


def run_case(fn, m, n, k, group, what):
    _, x, packed, scales, ref = int4_case(m, n, k, group, seed=m * 7 + n + k)
    out = fn(torch.from_numpy(x).cuda(), torch.from_numpy(packed).cuda(), torch.from_numpy(scales).cuda(), group)
    assert out.shape == (m, n) and out.dtype == torch.float16
    return assert_int4_close(out, ref, what)


@pytest.mark.parametrize("group", [64, 128])
@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 6, 7, 8])
@pytest.mark.parametrize("layer", list(LAYER_SHAPES))
def test_gemv_layer_shapes(layer, m, group):
    n, k = LAYER_SHAPES[layer]
    run_case(ops.int4_gemv, m, n, k, group, f"{layer} m{m} g{group}")


@pytest.mark.parametrize("n", [1, 7, 9, 129])
def test_gemv_ragged_n(n):
    run_case(ops.int4_gemv, 3, n, 256, 128, f"ragged_n{n}")


@pytest.mark.parametrize("m,n,k,group", [
    (1, 80005, 256, 128),    # ragged last tile, warps with 2 and with 3 tiles (pairs + a single)
    (5, 94720, 128, 128),    # one chunk holding a single round
    (8, 76800, 192, 64),     # last chunk partly past K, scalar scale loads
    (2, 151552, 384, 128),   # even ranges everywhere
])
def test_gemv_large_n_streaming_path(m, n, k, group):
    """N beyond ~76k rows takes the persistent kernel (contiguous tile ranges per warp, ring running across tiles)."""
    run_case(ops.int4_gemv, m, n, k, group, f"large_n m{m} n{n} k{k} g{group}")


@pytest.mark.parametrize("group", [64, 128])
@pytest.mark.parametrize("m", [9, 12, 16, 17, 24, 32])
@pytest.mark.parametrize("layer", ["qwen_down", "tinyllama_gate_up", "ragged"])
def test_small_batch_shapes(layer, m, group):
    """M up to 32 on the weight-streaming kernel (2 and 4 column blocks), split-K shapes and a ragged N."""
    n, k = {"ragged": (1000, 1280)}.get(layer) or LAYER_SHAPES[layer]
    run_case(ops.int4_small_batch, m, n, k, group, f"small_batch {layer} m{m} g{group}")


@pytest.mark.parametrize("m,n,k,group", [(16, 80005, 256, 128), (32, 76800, 192, 64), (11, 94720, 128, 128)])
def test_small_batch_large_n_streaming_path(m, n, k, group):
    run_case(ops.int4_small_batch, m, n, k, group, f"small_batch large_n m{m} n{n}")


def test_small_batch_rejects_m33():
    _, x, packed, scales, _ = int4_case(33, 64, 256, 128, seed=0)
    xs, ps, ss = (torch.from_numpy(a).cuda() for a in (x, packed, scales))
    with pytest.raises(ValueError, match=r"M in \[1, 32\]"):
        ops.int4_small_batch(xs, ps, ss, 128)


def test_gemv_streaming_path_dependent_launch_and_graph():
    """The persistent kernel launched with programmatic dependent launch, back to back inside a CUDA graph, gives the
    same bits as a plain call (its weight prefetch may start before the previous kernel has finished, x and y may not)."""
    from kernelforge import _capi
    _, x, packed, scales, ref = int4_case(3, 80005, 256, 128, seed=21)
    xs, ps, ss = (torch.from_numpy(a).cuda() for a in (x, packed, scales))
    plain = ops.int4_gemv(xs, ps, ss, 128)
    ys = [torch.zeros(3, 80005, dtype=torch.float16, device="cuda") for _ in range(3)]
    lib = _capi.lib()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for y in ys:
                _capi.check(lib.kfb_int4_gemv(xs.data_ptr(), ps.data_ptr(), ss.data_ptr(), y.data_ptr(), 3, 80005, 256, 128, 1,
                                              side.cuda_stream))
    graph.replay()
    torch.cuda.synchronize()
    for y in ys:
        assert torch.equal(y, plain)
    assert_int4_close(plain, ref, "streaming path")
    assert _capi.device_status(xs.device) == 0


@pytest.mark.parametrize("impl", ["cuda_core"])
def test_gemv_cuda_core_kernel_still_matches(impl):
    """The tensor-core-free kernel stays reachable through flag bit 1; bit 0 (dependent launch) works with both."""
    from kernelforge import _capi
    _, x, packed, scales, ref = int4_case(2, 2048, 1024, 128, seed=4)
    xs, ps, ss = (torch.from_numpy(a).cuda() for a in (x, packed, scales))
    y = torch.empty(2, 2048, dtype=torch.float16, device="cuda")
    for flags in (2, 3, 1):
        y.zero_()
        _capi.check(_capi.lib().kfb_int4_gemv(xs.data_ptr(), ps.data_ptr(), ss.data_ptr(), y.data_ptr(), 2, 2048, 1024, 128, flags,
                                              torch.cuda.current_stream().cuda_stream))
        assert_int4_close(y, ref, f"{impl} flags={flags}")


@pytest.mark.parametrize("path", sorted(glob.glob(str(GOLDEN / "int4_linear_m[1-8]_*.npz"))), ids=lambda p: p.split("/")[-1])
def test_gemv_golden(path):
    z = np.load(path)
    out = ops.int4_gemv(torch.from_numpy(z["x"]).cuda(), torch.from_numpy(z["packed"]).cuda(),
                        torch.from_numpy(z["scales"]).cuda(), int(z["group"]))
    assert_int4_close(out, z["ref"], path)


def test_gemv_guard_band_and_determinism():
    """Rows past N must not be written and two runs must agree bit for bit."""
    _, x, packed, scales, ref = int4_case(3, 129, 256, 128, seed=5)
    xs, ps, ss = (torch.from_numpy(a).cuda() for a in (x, packed, scales))
    a = ops.int4_gemv(xs, ps, ss, 128)
    b = ops.int4_gemv(xs, ps, ss, 128)
    assert torch.equal(a, b)
    _, x, packed, scales, ref = int4_case(1, 5632, 2048, 128, seed=11)
    xs, ps, ss = (torch.from_numpy(a).cuda() for a in (x, packed, scales))
    assert torch.equal(ops.int4_gemv(xs, ps, ss, 128), ops.int4_gemv(xs, ps, ss, 128))


def test_gemv_linearity_full_size():
    """Size-independent property at the benchmark shape: y(x1 + x2) = y(x1) + y(x2) up to fp16 rounding."""
    g = torch.Generator().manual_seed(3)
    w = torch.randn(5632, 2048, generator=g) * 0.02
    qw = kq.quantize_weight(w.cuda(), 128)
    x1 = (torch.randn(1, 2048, generator=g) * 0.5).half().cuda()
    x2 = (torch.randn(1, 2048, generator=g) * 0.5).half().cuda()
    y12 = ops.int4_gemv(x1 + x2, qw.packed, qw.scales, 128).float()
    ysum = ops.int4_gemv(x1, qw.packed, qw.scales, 128).float() + ops.int4_gemv(x2, qw.packed, qw.scales, 128).float()
    # x1 + x2 is rounded to fp16 once (rel 2^-11 per element), outputs are rounded to fp16
    assert (y12 - ysum).abs().max().item() <= 4e-3 * ysum.abs().max().item()


def test_gemv_rejections():
    x = torch.randn(1, 200).half().cuda()
    with pytest.raises(ValueError, match="not a multiple of group_size"):
        ops.int4_gemv(x, torch.zeros(16, 25, dtype=torch.int32).cuda(), torch.ones(16, 2, dtype=torch.float16).cuda(), 128)
    _, x, packed, scales, _ = int4_case(9, 64, 256, 128, seed=0)
    xs, ps, ss = (torch.from_numpy(a).cuda() for a in (x, packed, scales))
    with pytest.raises(ValueError, match=r"M in \[1, 8\]"):
        ops.int4_gemv(xs, ps, ss, 128)
    with pytest.raises(ValueError, match="K/8"):
        ops.int4_gemv(xs[:1, :128].contiguous(), ps, ss, 128)
    with pytest.raises(TypeError, match="2-D fp16 CUDA tensor"):
        ops.int4_gemv(xs[:1].float(), ps, ss, 128)


def test_int4_linear_shapes_and_bias():
    _, x, packed, scales, ref = int4_case(6, 72, 512, 64, seed=2)
    xs, ps, ss = (torch.from_numpy(a).cuda() for a in (x, packed, scales))
    bias = torch.linspace(-1, 1, 72).half().cuda()
    y = ops.int4_linear(xs.reshape(2, 3, 512), ps, ss, 64, bias)
    assert y.shape == (2, 3, 72) and y.dtype == torch.float16
    want = torch.from_numpy(ref).cuda().half() + bias
    assert (y.reshape(6, 72).float() - want.float()).abs().max().item() <= 4e-3 * float(np.abs(ref).max() + 1)


@pytest.mark.parametrize("group", [64, 128])
@pytest.mark.parametrize("m", [1, 3, 8])
@pytest.mark.parametrize("kind", ["abs", "shifted"])
@pytest.mark.parametrize("n,k", [(2048, 2048), (94720, 256)], ids=["split_k", "stream"])
def test_gemv_one_signed_activations(n, k, kind, m, group):
    """Activations with a large mean (post-ReLU / GELU inputs): the mma formulation accumulates offset forms of the
    nibbles and subtracts class sums of x afterwards, so a one-signed x makes the cancelled magnitude largest.  Checked
    against the oracle with the usual bound, and the mean error must show no systematic bias."""
    rng = np.random.default_rng(n + k + m + group)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
    from oracle import kf_oracle as ko
    packed, scales = ko.quantize_weight(w, group)
    x = rng.standard_normal((m, k), dtype=np.float32)
    x = (np.abs(x) if kind == "abs" else x + 4.0).astype(np.float16)
    ref = x.astype(np.float32) @ ko.dequantize(packed, scales, group, np.float32).T
    for flags in (4, 2):   # the mma kernel, the CUDA-core kernel
        y = torch.empty(m, n, dtype=torch.float16, device="cuda")
        from kernelforge import _capi
        xs, ps, ss = torch.from_numpy(x).cuda(), torch.from_numpy(packed).cuda(), torch.from_numpy(scales).cuda()
        _capi.check(_capi.lib().kfb_int4_gemv(xs.data_ptr(), ps.data_ptr(), ss.data_ptr(), y.data_ptr(), m, n, k, group, flags,
                                              _capi.stream_ptr(torch.device("cuda", 0))))
        err, peak, rms, floor = assert_int4_close(y, ref, f"{kind} flags{flags}")
        bias = float((y.float().cpu().numpy() - ref).mean())
        assert abs(bias) <= 0.1 * floor + 1e-6, f"systematic bias {bias:.3e} (fp16 floor {floor:.3e}) with flags {flags}"


def test_prepack_layout_is_the_documented_permutation():
    """kfb_int4_prepack against the layout stated in the header: block (rb, kb) = 32 lanes x 16 bytes, lane 4g + t =
    words (row 16rb+g: 2), (row 16rb+g+8: 2) covering k in [64kb + 16t, +16).  Bit-exact."""
    rng = np.random.default_rng(5)
    n, k = 48, 192
    packed = rng.integers(-2**31, 2**31 - 1, size=(n, k // 8), dtype=np.int64).astype(np.int32)
    got = ops.prepack_int4(torch.from_numpy(packed).cuda()).cpu().numpy().view(np.int32)
    want = packed.reshape(n // 16, 2, 8, k // 64, 4, 2).transpose(0, 3, 2, 4, 1, 5).reshape(-1)   # [rb, kb, g, t, half, word]
    assert np.array_equal(got, want)


@pytest.mark.parametrize("group", [64, 128])
@pytest.mark.parametrize("m", [1, 2, 3, 5, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("n,k", [(5632, 2048), (2048, 5632), (1536, 8960), (8960, 1536), (256, 1536), (16, 64 * 2), (48, 128 * 3),
                                 (32000, 2048)])
def test_prepacked_gemv_against_the_oracle(n, k, m, group):
    """The M <= 32 GEMV on the fragment-order copy of the weight: same bound as the other GEMV kernels, against the FP32
    oracle, including one-signed activations (no systematic bias: the weights enter the MMA as exact integers)."""
    if k % group:
        pytest.skip("K is not a multiple of the group size")
    for kind in ("randn", "abs"):
        rng = np.random.default_rng(n + k + m + group)
        w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
        from oracle import kf_oracle as ko
        packed, scales = ko.quantize_weight(w, group)
        x = rng.standard_normal((m, k), dtype=np.float32)
        x = (np.abs(x) if kind == "abs" else x).astype(np.float16)
        ref = x.astype(np.float32) @ ko.dequantize(packed, scales, group, np.float32).T
        ps, ss, xs = torch.from_numpy(packed).cuda(), torch.from_numpy(scales).cuda(), torch.from_numpy(x).cuda()
        y = ops.int4_gemv_prepacked(xs, ops.prepack_int4(ps), ss, group)
        err, peak, rms, floor = assert_int4_close(y, ref, f"prepacked {kind} n{n} k{k} m{m} g{group}")
        if n * m >= 4096:   # (the mean of a handful of rounding errors says nothing)
            bias = float((y.float().cpu().numpy() - ref).mean())
            assert abs(bias) <= 0.1 * floor + 1e-6


def test_prepacked_cache_follows_the_public_tensor():
    """ops.prepack_weight_ keys the private copy on the public tensor: int4_linear then runs small batches on it, an
    in-place change of the weight rebuilds it, and the entry dies with the tensor."""
    from kernelforge import quantize as kq
    g = torch.Generator().manual_seed(2)
    qw = kq.quantize_weight((torch.randn(512, 256, generator=g) * 0.02).cuda(), 128)
    x = torch.randn(3, 256, generator=g).half().cuda()
    before = ops.int4_linear(x, qw.packed, qw.scales, 128)
    ops.prepack_weight_(qw.packed)
    assert id(qw.packed) in ops._PREPACKED
    after = ops.int4_linear(x, qw.packed, qw.scales, 128)
    assert (after.float() - before.float()).abs().max().item() <= 2e-3 * before.float().abs().max().item()
    other = kq.quantize_weight((torch.randn(512, 256, generator=g) * 0.02).cuda(), 128)
    qw.packed.copy_(other.packed)   # the version counter moves: the copy is rebuilt on the next call
    changed = ops.int4_linear(x, qw.packed, other.scales, 128)
    want = ops.int4_gemv(x, other.packed, other.scales, 128)
    assert (changed.float() - want.float()).abs().max().item() <= 2e-3 * want.float().abs().max().item()
    key = id(qw.packed)
    del qw
    import gc
    gc.collect()
    assert key not in ops._PREPACKED
