"""The numpy oracle against fixtures produced by the reference's own code (tests/golden/make_golden.py)
and against the reference's known-answer nibble layout (reference tests/test_quantize.py:16-25)."""

import glob

import numpy as np
import pytest

from oracle import kf_oracle as ko
from conftest import GOLDEN


@pytest.mark.parametrize("path", sorted(glob.glob(str(GOLDEN / "quant_*.npz"))), ids=lambda p: p.split("/")[-1])
def test_quantizer_bit_exact(path):
    z = np.load(path)
    group = int(z["group"])
    q, s = ko.quantize_int4(z["w"], group)
    assert np.array_equal(q, z["q"])
    assert np.array_equal(s.view(np.uint16), z["scales"].view(np.uint16))
    assert np.array_equal(ko.pack_int4(q), z["packed"])
    assert np.array_equal(ko.unpack_int4(z["packed"]), z["q"])
    assert np.array_equal(ko.dequantize(z["packed"], z["scales"], group, np.float32), z["deq32"])
    assert np.array_equal(ko.dequantize(z["packed"], z["scales"], group, np.float16).view(np.uint16),
                          z["deq16"].view(np.uint16))


def test_known_answer_nibble_layout():
    q = np.arange(8, dtype=np.int8).reshape(1, 8)
    word = int(ko.pack_int4(q).view(np.uint32)[0, 0])
    assert [(word >> (4 * i)) & 0xF for i in range(8)] == [8, 10, 12, 14, 9, 11, 13, 15]
    for i in range(4):
        pair = (word >> (4 * i)) & 0x000F000F
        assert (pair & 0xF, pair >> 16) == (2 * i + 8, 2 * i + 1 + 8)


def test_absmax_and_zero_group():
    w = np.zeros((2, 128), np.float32)
    w[0, 5], w[0, 9] = -3.5, 1.0
    q, s = ko.quantize_int4(w, 128)
    assert q[0, 5] == -7 and float(s[0, 0]) == pytest.approx(0.5, rel=1e-3)
    assert (q[1] == 0).all() and float(s[1, 0]) == 1.0


def test_roundtrip_all_nibbles():
    rng = np.random.default_rng(0)
    q = rng.integers(-8, 8, size=(64, 256)).astype(np.int8)
    assert np.array_equal(ko.unpack_int4(ko.pack_int4(q)), q)


@pytest.mark.parametrize("path", sorted(glob.glob(str(GOLDEN / "int4_linear_*.npz"))), ids=lambda p: p.split("/")[-1])
def test_int4_linear_matches_reference(path):
    z = np.load(path)
    y = ko.int4_linear(z["x"], z["packed"], z["scales"], int(z["group"]))
    # both are FP32 matmuls of identical operands; only the summation order differs
    assert np.abs(y - z["ref"]).max() <= 2e-5 * np.abs(z["ref"]).max()


@pytest.mark.parametrize("path", sorted(glob.glob(str(GOLDEN / "attn_*.npz"))), ids=lambda p: p.split("/")[-1])
def test_attention_matches_reference(path):
    z = np.load(path)
    scale = float(z["scale"]) if "scale" in z.files else None
    o = ko.attention(z["q"], z["k"], z["v"], bool(z["causal"]), scale)
    assert np.abs(o - z["ref"]).max() <= 2e-6


def test_rejections():
    with pytest.raises(ValueError, match="not a multiple of group_size"):
        ko.quantize_weight(np.zeros((16, 200), np.float32), 128)
    with pytest.raises(ValueError, match="group_size"):
        ko.quantize_weight(np.zeros((16, 256), np.float32), 32)
    with pytest.raises(ValueError, match=r"\[-8, 7\]"):
        ko.pack_int4(np.full((1, 8), 9, np.int8))


def test_torch_restatement_matches_the_same_fixtures():
    """oracle/kf_oracle_torch.py (the torch-on-CPU form that bench.py times as the CPU baseline) against the fixtures
    the reference's own code produced: unpack / dequantise bit-exact, linear and attention to FP32 summation order."""
    import torch
    from oracle import kf_oracle_torch as kt
    for path in sorted(glob.glob(str(GOLDEN / "*.npz"))):
        z = np.load(path)
        name = path.split("/")[-1]
        if name.startswith("quant_"):
            packed, scales = torch.from_numpy(z["packed"]), torch.from_numpy(z["scales"])
            assert np.array_equal(kt.unpack_int4(packed).numpy(), z["q"]), name
            assert np.array_equal(kt.dequantize(packed, scales, int(z["group"])).numpy(), z["deq32"]), name
        elif name.startswith("int4_linear_"):
            y = kt.int4_linear(torch.from_numpy(z["x"]), torch.from_numpy(z["packed"]), torch.from_numpy(z["scales"]),
                               int(z["group"])).numpy()
            assert np.abs(y - z["ref"]).max() <= 2e-5 * np.abs(z["ref"]).max(), name
        elif name.startswith("attn_"):
            scale = float(z["scale"]) if "scale" in z.files else None
            o = kt.attention(torch.from_numpy(z["q"]), torch.from_numpy(z["k"]), torch.from_numpy(z["v"]),
                             bool(z["causal"]), scale).numpy()
            assert np.abs(o - z["ref"]).max() <= 2e-6, name
