"""CPU-side checks of the boundary: the C-ABI library loads and exports everything the header declares,
and the package's host logic (CPU-tensor quantiser, validators, custom-op registration) behaves like the
reference's (kernelforge/quantize.py, kernelforge/ops.py:171-302).  No kernel is launched here."""

import ctypes
import re
import glob

import numpy as np
import pytest
import torch

from conftest import ROOT, GOLDEN
from kernelforge import _capi, ops
from kernelforge import quantize as kq


def _declared_functions():
    text = (ROOT / "include" / "kfb200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(kfb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = _declared_functions()
    assert len(names) >= 10
    handle = ctypes.CDLL(str(ROOT / "kernel-forge_b200" / "kernelforge" / "libkfb200.so"))
    for name in names:
        assert hasattr(handle, name), f"{name} is declared in include/kfb200.h but not exported"
    assert sorted(_capi.exported_symbols()) == names  # the ctypes table binds exactly the header
    assert _capi.lib().kfb_version() >= 100
    assert _capi.lib().kfb_last_error() is not None


@pytest.mark.parametrize("path", sorted(glob.glob(str(GOLDEN / "quant_*.npz"))), ids=lambda p: p.split("/")[-1])
def test_cpu_tensor_quantizer_matches_reference_bits(path):
    z = np.load(path)
    group = int(z["group"])
    w = torch.from_numpy(z["w"])
    if "_f16" in path:
        w = w.half()
    elif "_bf16" in path:
        w = w.bfloat16()
    qw = kq.quantize_weight(w, group)
    assert np.array_equal(qw.packed.numpy(), z["packed"])
    assert np.array_equal(qw.scales.numpy().view(np.uint16), z["scales"].view(np.uint16))
    assert np.array_equal(kq.unpack_int4(qw.packed).numpy(), z["q"])
    assert np.array_equal(kq.dequantize(qw, torch.float32).numpy(), z["deq32"])
    assert np.array_equal(kq.dequantize(qw, torch.float16).numpy().view(np.uint16), z["deq16"].view(np.uint16))
    assert qw.nbytes == z["packed"].size * 4 + z["scales"].size * 2 and qw.shape == tuple(z["w"].shape)


def test_bit_layout_known_answer():
    q = torch.arange(0, 8, dtype=torch.int8).reshape(1, 8)
    word = kq.pack_int4(q).item() & 0xFFFFFFFF
    assert [(word >> (4 * i)) & 0xF for i in range(8)] == [8, 10, 12, 14, 9, 11, 13, 15]


def test_quantization_error_stats():
    g = torch.Generator().manual_seed(1)
    w = torch.randn(256, 1024, generator=g) * 0.02
    for group in (64, 128):
        qw = kq.quantize_weight(w, group)
        step = qw.scales.float().repeat_interleave(group, dim=1)
        assert ((kq.dequantize(qw, torch.float32) - w).abs() <= 0.5 * step + 1e-8).all()
        stats = kq.quantization_error(w, qw)
        assert stats["rel_fro_err"] < 0.15 and stats["bits_per_weight"] == pytest.approx(4 + 16 / group)


def test_quantizer_rejections():
    with pytest.raises(ValueError, match="not a multiple of group_size"):
        kq.quantize_weight(torch.randn(16, 200), 128)
    with pytest.raises(ValueError, match="group_size"):
        kq.quantize_weight(torch.randn(16, 256), 32)
    with pytest.raises(ValueError, match="2-D"):
        kq.quantize_weight(torch.randn(4, 16, 256), 128)
    with pytest.raises(ValueError, match=r"\[-8, 7\]"):
        kq.pack_int4(torch.full((1, 8), 9, dtype=torch.int8))
    with pytest.raises(ValueError, match="multiple of 8"):
        kq.pack_int4(torch.zeros(2, 12, dtype=torch.int8))


def test_validators_reject_cpu_tensors_like_the_reference():
    q = torch.randn(1, 2, 8, 64, dtype=torch.float16)
    with pytest.raises(ValueError, match="CUDA"):
        ops.flash_attn(q, q, q)
    with pytest.raises(TypeError, match="2-D fp16 CUDA tensor"):
        ops.int4_linear(torch.randn(2, 256).half(), torch.zeros(8, 32, dtype=torch.int32),
                        torch.ones(8, 2, dtype=torch.float16))
    with pytest.raises(ValueError, match="positive"):
        ops._resolve_scale(-1.0, 64)
    assert ops._resolve_scale(None, 64) == pytest.approx(0.125)


def test_custom_ops_registered_with_fakes():
    assert hasattr(torch.ops.kernelforge, "flash_attn") and hasattr(torch.ops.kernelforge, "int4_matmul")
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        q = torch.empty(2, 8, 16, 64, dtype=torch.float16, device="cuda")
        k = torch.empty(2, 2, 48, 64, dtype=torch.float16, device="cuda")
        assert torch.ops.kernelforge.flash_attn(q, k, k, True, 0.125).shape == q.shape
        x = torch.empty(3, 256, dtype=torch.float16, device="cuda")
        p = torch.empty(40, 32, dtype=torch.int32, device="cuda")
        s = torch.empty(40, 2, dtype=torch.float16, device="cuda")
        assert torch.ops.kernelforge.int4_matmul(x, p, s, 128).shape == (3, 40)


def test_int4_matmul_routing_table():
    """Which kernel int4_matmul picks by shape (pure host logic): GEMV up to M = 8, the same kernel with more batch columns
    for 8 < M <= 16 where it measured faster, the tcgen05 GEMM otherwise."""
    from kernelforge import ops
    assert ops.GEMV_MAX_M == 8 and ops.SMALL_BATCH_MAX_M == 32
    wins = ops._small_batch_wins
    assert wins(12, 5632, 2048) and wins(16, 2048, 2048) and wins(16, 8960, 1536)
    assert wins(16, 128256, 4096)                      # large N: the persistent streaming kernel
    assert not wins(12, 1536, 8960)                    # long K, few rows: the GEMM was faster
    assert not wins(12, 32000, 2048)                   # between the two regimes


def test_decoder_refuses_steps_that_do_not_fit_the_cache():
    """Host-side position check of the end-to-end decoder (the step graph reads the position on the device, so the
    host must make sure a replay is never asked to write past the KV cache).  Nothing is launched: built on CPU."""
    from kernelforge.llama_decode import LlamaInt4Decoder, LlamaShape
    shape = LlamaShape(hidden=128, layers=1, heads=2, kv_heads=1, head_dim=64, intermediate=128, vocab=64)
    dec = LlamaInt4Decoder.random_init(shape, "cpu", batch=1, max_len=8)
    with pytest.raises(ValueError, match="no room"):
        dec.prefill(torch.zeros(1, 8, dtype=torch.long))          # a prompt as long as the cache
    dec._host_pos = 6                                             # as after a 6-token prompt
    with pytest.raises(ValueError, match="do not fit"):
        dec.decode(3)
    dec._host_pos = 8
    with pytest.raises(ValueError, match="full"):
        dec.capture()


@pytest.mark.parametrize("n_rows,k,group", [(2560, 2048, 128), (2048, 2048, 128), (11264, 2048, 128), (2048, 5632, 128),
                                            (32000, 2048, 0), (512, 256, 128), (1024, 256, 64), (320, 256, 0)])
@pytest.mark.parametrize("n_ctas", [148, 132, 7])
def test_persistent_step_schedule_covers_every_row_once(n_rows, k, group, n_ctas):
    """kfb_decode_step_slice (host only): the row slices of the CTAs tile the matrix without gap or overlap, start on the
    16-byte boundaries the bulk copies need (weights and scales), and a ring slot's worth of rows fits its 44 KB."""
    import ctypes
    from kernelforge import _capi
    lib = _capi.lib()
    r0, rows, rpc = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    nxt = 0
    row_w = k // 2 if group else k * 2
    row_s = (k // group) * 2 if group else 0
    for cta in range(n_ctas):
        _capi.check(lib.kfb_decode_step_slice(n_rows, k, group, 0, cta, n_ctas, ctypes.byref(r0), ctypes.byref(rows), ctypes.byref(rpc)))
        assert r0.value == nxt and rows.value >= 0
        nxt += rows.value
        assert (r0.value * row_w) % 16 == 0 and (r0.value * row_s) % 16 == 0
        assert rpc.value >= 1 and rpc.value * (row_w + row_s) <= 45056
        if group:
            assert rows.value % 2 == 0 and rpc.value % 2 == 0      # pairs of rows stay together
            assert (rpc.value * row_s) % 16 == 0
    assert nxt == n_rows


def test_prepack_shape_rules_and_routing_rule():
    """Host-side rules of the private prepacked weight cache: which shapes get a fragment-order copy, and where the
    measured M = 1 exception applies (small N with long K stays on the public-format kernel)."""
    import torch
    from kernelforge import ops
    ok = lambda n, k: ops.prepack_supported(torch.empty(n, k // 8, dtype=torch.int32))
    assert ok(5632, 2048) and ok(16, 64) and ok(1536, 8960) and ok(32000, 2048)
    assert not ok(5630, 2048)        # N % 16
    assert not ok(64, 96)            # K % 64
    assert not ok(64, 12288 + 64)    # a warp's share of K must fit its registers
    assert not ops.prepack_supported(torch.empty(8, dtype=torch.int32))
    assert ops._prepacked_wins(2, 1536, 8960) and ops._prepacked_wins(32, 256, 1536)
    assert ops._prepacked_wins(1, 5632, 2048) and not ops._prepacked_wins(1, 1536, 8960)
    with pytest.raises(ValueError):
        ops.prepack_int4(torch.empty(64, 8, dtype=torch.int32))   # not on a CUDA device: no CPU fallback


def test_private_row_orders_are_permutations_prefill_can_undo():
    """ops.interleave_qkv_for_rope / interleave_gate_up only permute rows: the projection of the permuted matrix, read back
    the way LlamaInt4Decoder.prefill and _mlp read it, equals the projection of the natural matrix (pure torch, on CPU)."""
    import torch
    from kernelforge import ops
    g = torch.Generator().manual_seed(0)
    h, hk, d, k, inter, b, t = 4, 2, 64, 96, 40, 2, 3
    wq, wk, wv = (torch.randn(n, k, generator=g, dtype=torch.float64) for n in (h * d, hk * d, hk * d))
    x = torch.randn(b, t, k, generator=g, dtype=torch.float64)
    nat = x @ torch.cat([wq, wk, wv], 0).T
    qkv = x @ ops.interleave_qkv_for_rope(wq, wk, wv, d).T
    nq, nkv = h * d, hk * d
    unpair = lambda z, heads: z.reshape(b, t, heads, d // 2, 2).transpose(-1, -2).reshape(b, t, heads * d)
    back = torch.cat([unpair(qkv[..., :nq], h), unpair(qkv[..., nq:nq + nkv], hk), qkv[..., nq + nkv:]], -1)
    assert torch.equal(back, nat)
    # the pair (2j, 2j + 1) of a q / k head holds features (j, j + D/2): what the rotate-half embedding mixes
    perm = ops.interleave_qkv_for_rope(torch.arange(h * d, dtype=torch.float64)[:, None], torch.zeros(hk * d, 1, dtype=torch.float64),
                                       torch.zeros(hk * d, 1, dtype=torch.float64), d)[:h * d, 0].reshape(h, d // 2, 2)
    assert torch.equal(perm[..., 1] - perm[..., 0], torch.full((h, d // 2), float(d // 2), dtype=torch.float64))
    gate, up = (torch.randn(inter, k, generator=g, dtype=torch.float64) for _ in range(2))
    gu = (x @ ops.interleave_gate_up(gate, up).T).view(b, t, inter, 2)
    assert torch.equal(gu[..., 0], x @ gate.T) and torch.equal(gu[..., 1], x @ up.T)
