"""The three fused element-wise kernels of the decode step against their torch formulations (fp16 models)."""

import pytest
import torch

from kernelforge import ops

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,hidden", [(1, 2048), (32, 2048), (3, 1536), (2, 8192), (5, 256)])
def test_add_rmsnorm(rows, hidden):
    g = torch.Generator().manual_seed(hidden + rows)
    x = torch.randn(rows, hidden, generator=g).half().cuda()
    r = torch.randn(rows, hidden, generator=g).half().cuda()
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).half().cuda()
    for res in (None, r):
        y, s = ops.add_rmsnorm(x, w, 1e-5, res)
        s_ref = x if res is None else x + res
        sf = s_ref.float()
        y_ref = (sf * torch.rsqrt(sf.pow(2).mean(-1, keepdim=True) + 1e-5)).half() * w
        assert torch.equal(s, s_ref)
        assert (y.float() - y_ref.float()).abs().max().item() <= 2e-3 * y_ref.float().abs().max().item()


@pytest.mark.parametrize("b,h,hk,d", [(1, 32, 4, 64), (3, 8, 2, 128)])
def test_rope_kv_write(b, h, hk, d):
    g = torch.Generator().manual_seed(b + d)
    lmax, pos = 40, 17
    qkv = torch.randn(b, (h + 2 * hk) * d, generator=g).half().cuda()
    inv = 1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    ang = torch.outer(torch.arange(lmax, dtype=torch.float32), inv)
    ang = torch.cat([ang, ang], -1)
    cos, sin = ang.cos().cuda(), ang.sin().cuda()
    kc = torch.zeros(b, hk, lmax, d, dtype=torch.float16).cuda()
    vc = torch.zeros_like(kc)
    q = ops.rope_kv_write(qkv, cos, sin, torch.tensor([pos]).cuda(), kc, vc, h)

    def rope(t):
        tf = t.float()
        rot = torch.cat([-tf[..., d // 2:], tf[..., :d // 2]], -1)
        return (tf * cos[pos] + rot * sin[pos]).half()

    qr = qkv[:, :h * d].view(b, h, d)
    kr = qkv[:, h * d:(h + hk) * d].view(b, hk, d)
    vr = qkv[:, (h + hk) * d:].view(b, hk, d)
    assert (q[:, :, 0].float() - rope(qr).float()).abs().max().item() <= 2e-3
    assert (kc[:, :, pos].float() - rope(kr).float()).abs().max().item() <= 2e-3
    assert torch.equal(vc[:, :, pos], vr)
    untouched = torch.ones(lmax, dtype=torch.bool)
    untouched[pos] = False
    assert kc[:, :, untouched].abs().max().item() == 0 and vc[:, :, untouched].abs().max().item() == 0


def test_rope_kv_write_stays_inside_the_cache():
    """The position is read on the device.  In range: the row after the last cache row of the last (batch, kv head)
    (a guard row of the same allocation) stays untouched.  Out of range: nothing is written at all and the device
    status word reports 0x701; after a reset the kernel works again."""
    from kernelforge import _capi
    b, h, hk, d, lmax = 2, 8, 2, 64, 16
    g = torch.Generator().manual_seed(1)
    qkv = torch.randn(b, (h + 2 * hk) * d, generator=g).half().cuda()
    ang = torch.outer(torch.arange(lmax, dtype=torch.float32), 1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d)))
    ang = torch.cat([ang, ang], -1)
    cos, sin = ang.cos().cuda(), ang.sin().cuda()
    # caches with one guard row behind them: [b * hk * lmax + 1, d], the kernel is given the first b * hk * lmax rows
    kbuf = torch.full((b * hk * lmax + 1, d), 3.0, dtype=torch.float16).cuda()
    vbuf = torch.full((b * hk * lmax + 1, d), 3.0, dtype=torch.float16).cuda()
    kc, vc = kbuf[:-1].view(b, hk, lmax, d), vbuf[:-1].view(b, hk, lmax, d)
    dev = torch.device("cuda", 0)
    ops.rope_kv_write(qkv, cos, sin, torch.tensor([lmax - 1]).cuda(), kc, vc, h)     # last legal position
    torch.cuda.synchronize()
    assert bool((kbuf[-1] == 3.0).all()) and bool((vbuf[-1] == 3.0).all())
    assert not bool((kc[:, :, lmax - 1] == 3.0).all())
    assert _capi.device_status(dev) == 0
    before_k, before_v = kbuf.clone(), vbuf.clone()
    try:
        for bad in (lmax, lmax + 5, -1):
            ops.rope_kv_write(qkv, cos, sin, torch.tensor([bad]).cuda(), kc, vc, h)
            torch.cuda.synchronize()
            assert torch.equal(kbuf, before_k) and torch.equal(vbuf, before_v), f"position {bad} wrote to the cache"
        assert _capi.device_status(dev) == 0x701
    finally:
        _capi.device_status_reset(dev)
        torch.cuda.synchronize()
    assert _capi.device_status(dev) == 0
    ops.rope_kv_write(qkv, cos, sin, torch.tensor([3]).cuda(), kc, vc, h)
    torch.cuda.synchronize()
    assert not bool((kc[:, :, 3] == 3.0).all())


@pytest.mark.parametrize("rows,inter", [(1, 5632), (32, 5632), (4, 8960)])
def test_silu_mul(rows, inter):
    gu = torch.randn(rows, 2 * inter, generator=torch.Generator().manual_seed(rows)).half().cuda()
    out = ops.silu_mul(gu)
    ref = torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]
    assert (out.float() - ref.float()).abs().max().item() <= 4e-3 * ref.float().abs().max().item()


@pytest.mark.parametrize("m", [1, 3, 8, 9, 32])
@pytest.mark.parametrize("v,k", [(32000, 2048), (1000, 256), (77, 64)])
def test_lm_head_gemv_with_fused_argmax(m, v, k):
    """fp16 lm_head GEMV against an FP32 matmul of the same bits; the fused argmax must equal torch.argmax of the
    logits the kernel itself produced (ties to the lowest index), and decode_finalize must publish it."""
    g = torch.Generator().manual_seed(m + v)
    h = torch.randn(m, k, generator=g).half()
    w = (torch.randn(v, k, generator=g) * 0.05).half()
    w[5] = w[3]                                        # two identical rows: equal logits, the tie goes to row 3
    ref = h.float() @ w.float().T
    best = torch.zeros(m, dtype=torch.int64, device="cuda")
    logits = ops.lm_head_argmax(h.cuda(), w.cuda(), None, best)
    err = (logits.float().cpu() - ref).abs().max().item()
    floor = (ref.half().float() - ref).abs().max().item()
    assert err <= 2e-3 * ref.abs().max().item() and err <= 4 * floor + 1e-6
    tok = torch.zeros(m, dtype=torch.int64, device="cuda")
    pos = torch.tensor([41], device="cuda")
    kv_len = torch.full((m,), 42, dtype=torch.int32, device="cuda")
    ops.decode_finalize(best, tok, pos, kv_len)
    assert torch.equal(tok.cpu(), logits.float().cpu().argmax(-1))
    assert int(pos.item()) == 42 and bool((kv_len == 43).all()) and bool((best == 0).all())


@pytest.mark.parametrize("rows,hidden,vocab", [(1, 2048, 32000), (32, 2048, 32000), (3, 256, 50)])
def test_embed_rmsnorm(rows, hidden, vocab):
    g = torch.Generator().manual_seed(rows + hidden)
    emb = torch.randn(vocab, hidden, generator=g).half().cuda()
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).half().cuda()
    tok = torch.randint(0, vocab, (rows,), generator=g).cuda()
    y, x = ops.embed_rmsnorm(tok, emb, w, 1e-5)
    assert torch.equal(x, emb[tok])
    y_ref, _ = ops.add_rmsnorm(emb[tok].contiguous(), w, 1e-5)
    assert torch.equal(y, y_ref)


@pytest.mark.parametrize("m", [1, 2])
@pytest.mark.parametrize("n,k", [(2560, 2048), (2048, 5632), (11264, 2048), (100, 256)])
def test_int4_gemv_fused_matches_the_separate_kernels(m, n, k):
    """ops.int4_gemv_fused against the sequence of separate kernels it replaces (same roundings): bias + residual
    epilogue and the SiLU * up prologue bit for bit; the RMSNorm prologue up to the summation order of mean(x^2)."""
    from kernelforge import quantize as kq
    g = torch.Generator().manual_seed(n + k + m)
    qw = kq.quantize_weight((torch.randn(n, k, generator=g) * 0.02).cuda(), 128)
    x = torch.randn(m, k, generator=g).half().cuda()
    bias = torch.randn(n, generator=g).half().cuda()
    res = torch.randn(m, n, generator=g).half().cuda()
    def cuda_core_gemv(xx):   # the same kernel family as the fused entry (flag bit 1), so results can be compared bit for bit
        from kernelforge import _capi
        y = torch.empty(xx.shape[0], n, dtype=torch.float16, device="cuda")
        _capi.check(_capi.lib().kfb_int4_gemv(xx.data_ptr(), qw.packed.data_ptr(), qw.scales.data_ptr(), y.data_ptr(),
                                              xx.shape[0], n, k, 128, 2, _capi.stream_ptr(torch.device("cuda", 0))))
        return y

    plain = cuda_core_gemv(x)
    fused = ops.int4_gemv_fused(x, qw.packed, qw.scales, 128, bias=bias, residual=res)
    assert torch.equal(fused, (plain + bias) + res)
    assert torch.equal(ops.int4_gemv_fused(x, qw.packed, qw.scales, 128), plain)
    # SiLU * up prologue
    gu = torch.randn(m, 2 * k, generator=g).half().cuda()
    want = cuda_core_gemv(ops.silu_mul(gu)) + res
    got = ops.int4_gemv_fused(gu, qw.packed, qw.scales, 128, ops.XFORM_SILU_MUL, residual=res)
    assert torch.equal(got, want)
    # RMSNorm prologue
    w = (1 + 0.1 * torch.randn(k, generator=g)).half().cuda()
    normed, _ = ops.add_rmsnorm(x, w, 1e-5)
    want = cuda_core_gemv(normed)
    got = ops.int4_gemv_fused(x, qw.packed, qw.scales, 128, ops.XFORM_RMSNORM, w, 1e-5)
    assert (got.float() - want.float()).abs().max().item() <= 2e-3 * want.float().abs().max().item()


def test_int4_linear_bias_goes_through_the_fused_epilogue():
    from kernelforge import quantize as kq
    g = torch.Generator().manual_seed(3)
    qw = kq.quantize_weight((torch.randn(1536, 1536, generator=g) * 0.02).cuda(), 128)
    bias = torch.randn(1536, generator=g).half().cuda()
    for m in (1, 2, 5):
        x = torch.randn(m, 1536, generator=g).half().cuda()
        got, want = ops.int4_linear(x, qw.packed, qw.scales, 128, bias), ops.int4_linear(x, qw.packed, qw.scales, 128) + bias
        if m == 2:   # without a bias M = 2 runs on the mma kernel: same sums, another order
            assert (got.float() - want.float()).abs().max().item() <= 2e-3 * want.float().abs().max().item()
        else:
            assert torch.equal(got, want)


def _cuda_core_gemv(x, qw, group=128):
    from kernelforge import _capi
    n, k = qw.packed.shape[0], x.shape[1]
    y = torch.empty(x.shape[0], n, dtype=torch.float16, device="cuda")
    _capi.check(_capi.lib().kfb_int4_gemv(x.data_ptr(), qw.packed.data_ptr(), qw.scales.data_ptr(), y.data_ptr(),
                                          x.shape[0], n, k, group, 2, _capi.stream_ptr(torch.device("cuda", 0))))
    return y


@pytest.mark.parametrize("m", [1, 2])
@pytest.mark.parametrize("inter,k,group", [(5632, 2048, 128), (8960, 1536, 128), (50, 256, 64)])
def test_silu_pair_epilogue_matches_gemv_then_silu_mul(m, inter, k, group):
    """The gate_up GEMV with SiLU * up in its epilogue (rows interleaved gate_p, up_p) against the plain GEMV on the
    concatenated matrix followed by the separate kernel: bit for bit."""
    from kernelforge import quantize as kq
    g = torch.Generator().manual_seed(inter + k + m)
    gate, up = (torch.randn(inter, k, generator=g) * 0.05).half().cuda(), (torch.randn(inter, k, generator=g) * 0.05).half().cuda()
    x = torch.randn(m, k, generator=g).half().cuda()
    natural = kq.quantize_weight(torch.cat([gate, up], 0), group)
    paired = kq.quantize_weight(ops.interleave_gate_up(gate, up), group)
    want = ops.silu_mul(_cuda_core_gemv(x, natural, group))
    got = ops.int4_gemv_silu_pair(x, paired.packed, paired.scales, group)
    assert got.shape == (m, inter) and torch.equal(got, want)
    # with the RMSNorm prologue: equal up to the summation order of mean(x^2)
    w = (1 + 0.1 * torch.randn(k, generator=g)).half().cuda()
    normed, _ = ops.add_rmsnorm(x, w, 1e-5)
    want = ops.silu_mul(_cuda_core_gemv(normed, natural, group)).float()
    got = ops.int4_gemv_silu_pair(x, paired.packed, paired.scales, group, w, 1e-5).float()
    assert (got - want).abs().max().item() <= 4e-3 * want.abs().max().item()


@pytest.mark.parametrize("b", [1, 2])
@pytest.mark.parametrize("h,hk,d,k", [(32, 4, 64, 2048), (12, 2, 128, 1536), (2, 1, 64, 256)])
def test_rope_kv_epilogue_matches_gemv_then_rope_kv_write(b, h, hk, d, k):
    """The fused q/k/v GEMV with RoPE + cache write in its epilogue against the plain GEMV followed by
    ops.rope_kv_write: q, the written cache row and the untouched rest of the caches, bit for bit."""
    from kernelforge import quantize as kq
    g = torch.Generator().manual_seed(h + d + b)
    lmax, pos = 24, 9
    wq, wk, wv = ((torch.randn(n, k, generator=g) * 0.05).half().cuda() for n in (h * d, hk * d, hk * d))
    x = torch.randn(b, k, generator=g).half().cuda()
    ang = torch.outer(torch.arange(lmax, dtype=torch.float32), 1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d)))
    ang = torch.cat([ang, ang], -1)
    cos, sin = ang.cos().cuda(), ang.sin().cuda()
    pos_dev = torch.tensor([pos], dtype=torch.long, device="cuda")
    natural = kq.quantize_weight(torch.cat([wq, wk, wv], 0), 128)
    paired = kq.quantize_weight(ops.interleave_qkv_for_rope(wq, wk, wv, d), 128)
    base = torch.randn(b, hk, lmax, d, generator=g).half().cuda()
    kc0, vc0, kc1, vc1 = base.clone(), base.clone() * 2, base.clone(), base.clone() * 2
    q_want = ops.rope_kv_write(_cuda_core_gemv(x, natural), cos, sin, pos_dev, kc0, vc0, h)
    q_got = ops.int4_gemv_rope_kv(x, paired.packed, paired.scales, 128, cos, sin, pos_dev, kc1, vc1, h)
    assert torch.equal(q_got, q_want) and torch.equal(kc1, kc0) and torch.equal(vc1, vc0)
    assert not torch.equal(kc1[:, :, pos], base[:, :, pos])


def test_rope_kv_epilogue_stays_inside_the_cache():
    """A position outside the cache: nothing is written, code 0x701 in the status word (then reset)."""
    from kernelforge import _capi, quantize as kq
    h, hk, d, k, lmax = 2, 1, 64, 256, 8
    g = torch.Generator().manual_seed(1)
    w = kq.quantize_weight((torch.randn((h + 2 * hk) * d, k, generator=g) * 0.05).half().cuda(), 128)
    x = torch.randn(1, k, generator=g).half().cuda()
    cos = torch.ones(lmax, d, device="cuda"); sin = torch.zeros(lmax, d, device="cuda")
    kc = torch.zeros(1, hk, lmax, d, dtype=torch.float16, device="cuda"); vc = torch.zeros_like(kc)
    dev = torch.device("cuda", 0)
    for bad in (lmax, -1):
        ops.int4_gemv_rope_kv(x, w.packed, w.scales, 128, cos, sin, torch.tensor([bad], dtype=torch.long, device="cuda"), kc, vc, h)
        torch.cuda.synchronize()
        assert _capi.device_status(dev) == 0x701
        assert not kc.any() and not vc.any()
        _capi.device_status_reset(dev)
        assert _capi.device_status(dev) == 0


@pytest.mark.parametrize("m", [1, 2, 5, 8])
def test_prepacked_gemv_epilogues_match_the_separate_kernels(m):
    """The fragment-order GEMV with bias / residual, SiLU-pair and RoPE + cache-write epilogues (M <= 8) against the
    plain GEMV followed by the separate kernels; the projections differ only in summation order, so the comparison
    carries the GEMV tolerance."""
    from kernelforge import quantize as kq
    g = torch.Generator().manual_seed(40 + m)
    k, inter, h, hk, d, lmax, pos = 512, 704, 8, 2, 64, 24, 5
    def close(a, b, what):
        assert (a.float() - b.float()).abs().max().item() <= 4e-3 * b.float().abs().max().item(), what
    x = torch.randn(m, k, generator=g).half().cuda()
    # bias + residual
    w = kq.quantize_weight((torch.randn(1024, k, generator=g) * 0.05).cuda(), 128)
    bias, res = torch.randn(1024, generator=g).half().cuda(), torch.randn(m, 1024, generator=g).half().cuda()
    pre = ops.prepack_int4(w.packed)
    close(ops.int4_gemv_prepacked(x, pre, w.scales, 128, bias, res), (_cuda_core_gemv(x, w) + bias) + res, "bias + residual")
    # SiLU pair
    gate, up = ((torch.randn(inter, k, generator=g) * 0.05).half().cuda() for _ in range(2))
    natural = kq.quantize_weight(torch.cat([gate, up], 0), 128)
    paired = kq.quantize_weight(ops.interleave_gate_up(gate, up), 128)
    close(ops.int4_gemv_prepacked_silu_pair(x, ops.prepack_int4(paired.packed), paired.scales, 128),
          ops.silu_mul(_cuda_core_gemv(x, natural)), "silu pair")
    # RoPE + cache write
    wq, wk, wv = ((torch.randn(n, k, generator=g) * 0.05).half().cuda() for n in (h * d, hk * d, hk * d))
    ang = torch.outer(torch.arange(lmax, dtype=torch.float32), 1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d)))
    ang = torch.cat([ang, ang], -1)
    cos, sin = ang.cos().cuda(), ang.sin().cuda()
    pos_dev = torch.tensor([pos], dtype=torch.long, device="cuda")
    natural = kq.quantize_weight(torch.cat([wq, wk, wv], 0), 128)
    paired = kq.quantize_weight(ops.interleave_qkv_for_rope(wq, wk, wv, d), 128)
    base = torch.randn(m, hk, lmax, d, generator=g).half().cuda()
    kc0, vc0, kc1, vc1 = base.clone(), base.clone() * 2, base.clone(), base.clone() * 2
    q_want = ops.rope_kv_write(_cuda_core_gemv(x, natural), cos, sin, pos_dev, kc0, vc0, h)
    q_got = ops.int4_gemv_prepacked_rope_kv(x, ops.prepack_int4(paired.packed), paired.scales, 128, cos, sin, pos_dev, kc1, vc1, h)
    close(q_got, q_want, "rope q"); close(kc1, kc0, "k cache"); close(vc1, vc0, "v cache")
    untouched = [i for i in range(lmax) if i != pos]
    assert torch.equal(kc1[:, :, untouched], base[:, :, untouched]) and torch.equal(vc1[:, :, untouched], (base * 2)[:, :, untouched])
