"""End-to-end greedy decode (prefill + CUDA-graph decode steps) of a small random-init Llama-architecture model
on the INT4 + fused-attention kernels, against an FP32 Hugging Face model that holds the dequantised weights and is
teacher-forced on the same tokens (greedy tokens of a random-init model are numerically fragile; logits are not).
Also the reference's own end-to-end criterion: graph tokens == eager tokens, exactly (bench/e2e_model.py:207)."""

import copy

import pytest
import torch

transformers = pytest.importorskip("transformers")
from transformers import LlamaConfig, LlamaForCausalLM  # noqa: E402

from kernelforge import modules as km  # noqa: E402
from kernelforge import quantize as kq  # noqa: E402
from kernelforge.llama_decode import LlamaInt4Decoder  # noqa: E402

pytestmark = pytest.mark.gpu


def assert_same_decode(ta, la, tb, lb, tol):
    """Two greedy decodes of the same model from the same state.  Step i's logits come from identical inputs as long as
    the tokens fed so far agree, so they must agree within `tol` (relative to the logit scale) up to the first step at which
    the two paths choose different tokens -- which may only happen at a genuine near-tie of the two best logits."""
    scale = lb.float().abs().max().item()
    steps = ta.shape[1]
    same = (ta == tb).all(dim=0)                      # ta[:, i] is the token FED at step i
    first_diff = steps if bool(same.all()) else int((~same).nonzero()[0])
    upto = min(steps, first_diff)                     # logits of steps < first_diff were computed from equal inputs
    err = (la[:, :upto].float() - lb[:, :upto].float()).abs().max().item() if upto else 0.0
    assert err <= tol * scale, f"logits differ by {err:.3e} (scale {scale:.3f}) before any token differs"
    if first_diff < steps:                            # the token fed at step first_diff was chosen at step first_diff - 1
        assert first_diff >= 1
        top2 = lb[:, first_diff - 1].float().topk(2, dim=-1).values
        gap = (top2[:, 0] - top2[:, 1]).min().item()
        assert gap <= 2 * tol * scale, f"paths chose different tokens at a gap of {gap:.3e} (scale {scale:.3f})"
    return err, scale


def build(layers=3, hidden=256, heads=4, kv_heads=2, inter=512, vocab=320):
    cfg = LlamaConfig(hidden_size=hidden, num_hidden_layers=layers, num_attention_heads=heads, num_key_value_heads=kv_heads,
                      intermediate_size=inter, vocab_size=vocab, head_dim=64, max_position_embeddings=512, rms_norm_eps=1e-5)
    torch.manual_seed(0)
    base = LlamaForCausalLM(cfg).eval()
    ref = copy.deepcopy(base).float()
    with torch.no_grad():
        for p in ref.parameters():
            p.copy_(p.half().float())
        for name, mod in ref.named_modules():
            if name.split(".")[-1] in km.DECODER_LINEARS and isinstance(mod, torch.nn.Linear):
                mod.weight.copy_(kq.dequantize(kq.quantize_weight(mod.weight.detach().half(), 128), torch.float32))
    return base, ref


@pytest.mark.parametrize("batch", [1, 2])
def test_prefill_and_graph_decode_logits_match_fp32_model(batch):
    base, ref = build()
    prompt_len, steps = 24, 12
    ids = torch.randint(0, 320, (batch, prompt_len), generator=torch.Generator().manual_seed(3))
    dec = LlamaInt4Decoder.from_hf(base, "cuda", batch, max_len=64)
    pre = dec.prefill(ids).float().cpu()
    toks, logs = dec.decode(steps, keep_logits=True)
    torch.cuda.synchronize()
    full = torch.cat([ids, toks.cpu()], dim=1)
    with torch.no_grad():
        want = ref(full).logits
    scale = want.abs().max().item()
    assert (pre - want[:, :prompt_len]).abs().max().item() <= 2e-2 * scale
    got = logs.float().cpu()                       # logits after feeding generated token i (position prompt_len + i)
    assert (got - want[:, prompt_len:]).abs().max().item() <= 2e-2 * scale
    assert torch.equal(toks[:, 0].cpu(), pre[:, -1].argmax(-1))


@pytest.mark.parametrize("batch", [1, 2])
@pytest.mark.parametrize("prompt_len", [1, 24, 200])
def test_persistent_step_matches_the_step_of_separate_kernels(batch, prompt_len):
    """The one-kernel decode step against the step of separate kernels on the same weights and cache: same arithmetic up
    to summation order (and FP32 instead of fp16 attention probabilities), so the logits agree far inside the bound
    against the FP32 model, and both choose the same tokens."""
    base, _ = build()
    steps = 10
    ids = torch.randint(0, 320, (batch, prompt_len), generator=torch.Generator().manual_seed(5 + prompt_len))
    a = LlamaInt4Decoder.from_hf(base, "cuda", batch, max_len=prompt_len + steps + 3)
    assert a.persistent_ok
    a.persistent = True
    b = LlamaInt4Decoder.from_hf(base, "cuda", batch, max_len=prompt_len + steps + 3)
    assert not b.persistent
    a.prefill(ids); b.prefill(ids)
    ta, la = a.decode(steps, keep_logits=True)
    tb, lb = b.decode(steps, keep_logits=True)
    assert_same_decode(ta, la, tb, lb, 4e-3)
    assert torch.equal(a.pos, b.pos) and torch.equal(a.kv_len, b.kv_len)
    if torch.equal(ta, tb):
        # the cache rows written by the two paths agree to fp16 rounding of the same projections
        assert (a.k_cache.float() - b.k_cache.float()).abs().max().item() <= 4e-3 * b.k_cache.float().abs().max().item()
        assert (a.v_cache.float() - b.v_cache.float()).abs().max().item() <= 4e-3 * b.v_cache.float().abs().max().item()


def test_graph_tokens_equal_eager_tokens():
    base, _ = build(layers=2)
    ids = torch.randint(0, 320, (2, 16), generator=torch.Generator().manual_seed(4))
    a = LlamaInt4Decoder.from_hf(base, "cuda", 2, max_len=48)
    a.prefill(ids)
    graph_toks, _ = a.decode(10)
    b = LlamaInt4Decoder.from_hf(base, "cuda", 2, max_len=48)
    b.prefill(ids)
    eager = []
    for _ in range(10):
        eager.append(b.tok.clone())
        b._step()
    assert torch.equal(graph_toks, torch.stack(eager, 1))


def test_decode_past_the_cache_raises_and_writes_nothing():
    base, _ = build(layers=1)
    ids = torch.randint(0, 320, (1, 10), generator=torch.Generator().manual_seed(5))
    dec = LlamaInt4Decoder.from_hf(base, "cuda", 1, max_len=16)
    dec.prefill(ids)
    dec.decode(6)                       # positions 10..15: the cache is now full
    with pytest.raises(ValueError, match="do not fit"):
        dec.decode(1)
    from kernelforge import _capi
    assert _capi.device_status(torch.device("cuda", 0)) == 0


def test_tinyllama_architecture_logits_at_size():
    """The end-to-end configuration at full size: 22 layers, hidden 2048, 32 heads / 4 KV heads of dim 64, SiLU MLP
    5632, vocab 32000, random init (std 0.02), INT4 g128 decoder linears, prompt 512 + 256 generated tokens under a
    CUDA graph.  Logits of the prefill and of every decode step are compared with an FP32 model holding the
    dequantised weights, teacher-forced on the same 768 tokens (the reference's FP32 model run; here the FP32 model
    runs on the GPU in true FP32 -- TF32 is off -- to keep the test short)."""
    cfg = LlamaConfig(hidden_size=2048, num_hidden_layers=22, num_attention_heads=32, num_key_value_heads=4,
                      intermediate_size=5632, vocab_size=32000, head_dim=64, max_position_embeddings=2048,
                      rms_norm_eps=1e-5)
    torch.manual_seed(0)
    base = LlamaForCausalLM(cfg).eval()
    prompt_len, steps = 512, 256
    ids = torch.randint(0, 32000, (1, prompt_len), generator=torch.Generator().manual_seed(0))
    dec = LlamaInt4Decoder.from_hf(base, "cuda", 1, max_len=prompt_len + steps + 8)
    pre = dec.prefill(ids).float().cpu()
    toks, logs = dec.decode(steps, keep_logits=True)
    torch.cuda.synchronize()
    got = torch.cat([pre, logs.float().cpu()], dim=1)            # [1, 768, vocab]
    full = torch.cat([ids, toks.cpu()], dim=1)[:, :prompt_len + steps]
    del dec
    torch.cuda.empty_cache()
    ref = base.float().cuda()
    with torch.no_grad():
        for p in ref.parameters():
            p.copy_(p.half().float())
        for name, mod in ref.named_modules():
            if name.split(".")[-1] in km.DECODER_LINEARS and isinstance(mod, torch.nn.Linear):
                mod.weight.copy_(kq.dequantize(kq.quantize_weight(mod.weight.detach().half(), 128), torch.float32))
        want = ref(full.cuda()).logits.float().cpu()
    scale = want.abs().max().item()
    err_pre = (got[:, :prompt_len] - want[:, :prompt_len]).abs().max().item()
    err_dec = (got[:, prompt_len:] - want[:, prompt_len:]).abs().max().item()
    agree = (got.argmax(-1) == want.argmax(-1)).float().mean().item()
    print(f"PARITY tinyllama-arch 22 layers, 768 tokens: logit scale {scale:.3f}  max_abs_err prefill {err_pre:.3e} "
          f"decode {err_dec:.3e}  bound {2e-2 * scale:.3e}  greedy-token agreement {agree:.4f}")
    assert err_pre <= 2e-2 * scale and err_dec <= 2e-2 * scale


def test_persistent_step_at_tinyllama_size():
    """The persistent step on the TinyLlama-1.1B shape (22 layers, 148 CTAs with 2-chunk gate_up slices, 32 key splits)
    against the step of separate kernels: logits within 4e-3 of the logit scale, same tokens, over 12 steps from a
    300-token prompt."""
    from kernelforge.llama_decode import TINYLLAMA_1B
    ids = torch.randint(0, 32000, (1, 300), generator=torch.Generator().manual_seed(11))
    outs = []
    for persistent in (True, False):
        dec = LlamaInt4Decoder.random_init(TINYLLAMA_1B, "cuda", 1, 320, seed=1)
        dec.persistent = persistent
        dec.prefill(ids)
        outs.append(dec.decode(12, keep_logits=True))
        dec.release()
        del dec
        torch.cuda.empty_cache()
    (ta, la), (tb, lb) = outs
    err, scale = assert_same_decode(ta, la, tb, lb, 4e-3)
    print(f"PARITY persistent step vs separate kernels, tinyllama-arch: max_abs_diff {err:.3e} logit scale {scale:.3f}")
