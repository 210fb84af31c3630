"""GPU quantise / pack / unpack / dequantise kernels: bit-exact against the reference-generated fixtures and
against the numpy oracle (reference contract: kernelforge/quantize.py:61-114, tests/test_quantize.py)."""

import glob

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from kernelforge import quantize as kq
from oracle import kf_oracle as ko

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("path", sorted(glob.glob(str(GOLDEN / "quant_*.npz"))), ids=lambda p: p.split("/")[-1])
def test_golden_bits(path):
    z = np.load(path)
    group = int(z["group"])
    w = torch.from_numpy(z["w"])
    w = w.half() if "_f16" in path else w.bfloat16() if "_bf16" in path else w
    qw = kq.quantize_weight(w.cuda(), group)
    assert qw.packed.dtype == torch.int32 and qw.scales.dtype == torch.float16
    assert np.array_equal(qw.packed.cpu().numpy(), z["packed"])
    assert np.array_equal(qw.scales.cpu().numpy().view(np.uint16), z["scales"].view(np.uint16))
    q, s = kq.quantize_int4(w.cuda(), group)
    assert np.array_equal(q.cpu().numpy(), z["q"]) and q.dtype == torch.int8
    assert np.array_equal(kq.pack_int4(q).cpu().numpy(), z["packed"])
    assert np.array_equal(kq.dequantize(qw, torch.float32).cpu().numpy(), z["deq32"])
    assert np.array_equal(kq.dequantize(qw, torch.float16).cpu().numpy().view(np.uint16), z["deq16"].view(np.uint16))


@pytest.mark.parametrize("n,k,group", [(5632, 2048, 128), (256, 1536, 64), (1536, 8960, 128), (7, 192, 64), (1, 128, 128)])
def test_random_weights_vs_oracle(n, k, group):
    rng = np.random.default_rng(n + k)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
    packed, scales = ko.quantize_weight(w, group)
    qw = kq.quantize_weight(torch.from_numpy(w).cuda(), group)
    assert np.array_equal(qw.packed.cpu().numpy(), packed)
    assert np.array_equal(qw.scales.cpu().numpy().view(np.uint16), scales.view(np.uint16))
    assert np.array_equal(kq.unpack_int4(qw.packed).cpu().numpy(), ko.unpack_int4(packed))
    assert np.array_equal(kq.dequantize(qw, torch.float32).cpu().numpy(), ko.dequantize(packed, scales, group))


def test_pack_unpack_roundtrip_is_exact():
    g = torch.Generator().manual_seed(0)
    q = torch.randint(-8, 8, (64, 256), generator=g, dtype=torch.int8).cuda()
    assert torch.equal(kq.unpack_int4(kq.pack_int4(q)), q)
    # idempotence at full size: quantising the dequantised weight reproduces the same bits
    w = torch.randn(2048, 5632, generator=g) * 0.02
    qw = kq.quantize_weight(w.cuda(), 128)
    qw2 = kq.quantize_weight(kq.dequantize(qw, torch.float32), 128)
    assert torch.equal(qw.packed, qw2.packed) and torch.equal(qw.scales, qw2.scales)


def test_absmax_and_zero_groups_and_rejections():
    w = torch.zeros(2, 128)
    w[0, 5], w[0, 9] = -3.5, 1.0
    q, s = kq.quantize_int4(w.cuda(), 128)
    assert q[0, 5].item() == -7 and s[0, 0].item() == pytest.approx(0.5, rel=1e-3)
    assert (q[1] == 0).all() and s[1, 0].item() == 1.0
    with pytest.raises(ValueError, match="not a multiple of group_size"):
        kq.quantize_weight(torch.randn(16, 200).cuda(), 128)
    with pytest.raises(ValueError, match=r"\[-8, 7\]"):
        kq.pack_int4(torch.full((1, 8), 9, dtype=torch.int8).cuda())
