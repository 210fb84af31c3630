"""kernelforge.modules drop-ins (reference: kernelforge/modules.py:19-115).  CPU part: registration, fallback
counting, module swap and state-dict names.  GPU part: a small random-init Llama runs through the fused attention
kernel and the INT4 linears and matches an FP32 model that holds the dequantised weights."""

import copy

import pytest
import torch

transformers = pytest.importorskip("transformers")
from transformers import LlamaConfig, LlamaForCausalLM  # noqa: E402

from kernelforge import modules as km  # noqa: E402
from kernelforge import quantize as kq  # noqa: E402


def tiny_llama(layers=2, hidden=256, heads=4, kv_heads=2, inter=512, vocab=320, head_dim=64):
    cfg = LlamaConfig(hidden_size=hidden, num_hidden_layers=layers, num_attention_heads=heads,
                      num_key_value_heads=kv_heads, intermediate_size=inter, vocab_size=vocab, head_dim=head_dim,
                      max_position_embeddings=512, rms_norm_eps=1e-5)
    torch.manual_seed(0)
    return LlamaForCausalLM(cfg).eval()


def test_registration_and_cpu_fallback_is_counted():
    model = km.enable_kf_attention(tiny_llama())
    assert model.config._attn_implementation == km.KF_ATTN_NAME
    before = dict(km.ATTN_STATS)
    ids = torch.randint(0, 320, (1, 12))
    with torch.no_grad():
        out = model(ids).logits
    assert out.shape == (1, 12, 320) and torch.isfinite(out).all()
    assert km.ATTN_STATS["sdpa_fallback_calls"] == before["sdpa_fallback_calls"] + 2  # fp32 on CPU: both layers fall back
    assert km.ATTN_STATS["kernelforge_calls"] == before["kernelforge_calls"]


def test_quantize_linears_swaps_decoder_linears_only():
    model = tiny_llama()
    n = km.quantize_linears_(model, 128)
    assert n == 2 * 7
    assert isinstance(model.lm_head, torch.nn.Linear)
    lin = model.model.layers[0].mlp.down_proj
    assert isinstance(lin, km.KFLinearInt4) and (lin.in_features, lin.out_features) == (512, 256)
    sd = lin.state_dict()
    assert set(sd) == {"packed", "scales"} and sd["packed"].dtype == torch.int32 and sd["scales"].dtype == torch.float16
    assert "int4" in repr(lin)
    with pytest.raises(TypeError, match="fp16 activations"):
        lin(torch.randn(1, 512))


@pytest.mark.gpu
def test_llama_forward_matches_fp32_model_with_dequantised_weights():
    base = tiny_llama(layers=2)
    # FP32 reference model whose decoder linears hold W_hat = dequantize(quantize(W)) of the fp16 weights
    ref = copy.deepcopy(base).float()
    with torch.no_grad():
        for name, mod in ref.named_modules():
            if name.split(".")[-1] in km.DECODER_LINEARS and isinstance(mod, torch.nn.Linear):
                w16 = mod.weight.detach().half()
                mod.weight.copy_(kq.dequantize(kq.quantize_weight(w16, 128), torch.float32))
        for p in ref.parameters():           # everything else rounded to fp16 like the model under test
            p.copy_(p.half().float())
    model = base.half().cuda()
    assert km.quantize_linears_(model, 128) == 14
    km.enable_kf_attention(model)
    before = dict(km.ATTN_STATS)
    ids = torch.randint(0, 320, (2, 70), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        got = model(ids.cuda()).logits.float().cpu()
        want = ref(ids).logits
    assert km.ATTN_STATS["kernelforge_calls"] == before["kernelforge_calls"] + 2
    assert km.ATTN_STATS["sdpa_fallback_calls"] == before["sdpa_fallback_calls"]
    # fp16 activations through 2 layers vs FP32: compare against the logit scale
    err = (got - want).abs().max().item()
    assert err <= 2e-2 * want.abs().max().item(), f"logit err {err} vs scale {want.abs().max().item()}"


@pytest.mark.gpu
def test_decode_with_dynamic_cache_uses_the_kernel():
    model = tiny_llama(layers=1).half().cuda()
    km.quantize_linears_(model, 128)
    km.enable_kf_attention(model)
    ids = torch.randint(0, 320, (1, 40), generator=torch.Generator().manual_seed(2)).cuda()
    before = dict(km.ATTN_STATS)
    with torch.no_grad():
        full = model(ids).logits[:, -1]
        out = model(ids[:, :-1], use_cache=True)
        step = model(ids[:, -1:], past_key_values=out.past_key_values, use_cache=True).logits[:, -1]
    assert km.ATTN_STATS["sdpa_fallback_calls"] == before["sdpa_fallback_calls"]
    assert km.ATTN_STATS["kernelforge_calls"] == before["kernelforge_calls"] + 3
    assert (full.float() - step.float()).abs().max().item() <= 3e-2 * full.float().abs().max().item()


@pytest.mark.gpu
def test_prepacked_linears_give_the_same_decode_logits():
    """modules.prepack_linears_: every INT4 linear gets its private fragment-order copy (keyed on the `packed` buffer);
    small-batch calls then run on it and the logits agree with the public-format kernels; state dicts are unchanged."""
    from kernelforge import ops
    model = tiny_llama(layers=2).half().cuda()
    km.quantize_linears_(model, 128)
    km.enable_kf_attention(model)
    ids = torch.randint(0, 320, (3, 1), generator=torch.Generator().manual_seed(5)).cuda()   # 3 rows: a small-batch call
    with torch.no_grad():
        before = model(ids).logits.float()
    keys = set(model.state_dict().keys())
    assert km.prepack_linears_(model) == 14
    lin = model.model.layers[0].mlp.down_proj
    assert id(lin.packed) in ops._PREPACKED
    with torch.no_grad():
        after = model(ids).logits.float()
    assert set(model.state_dict().keys()) == keys
    assert (after - before).abs().max().item() <= 5e-3 * before.abs().max().item()
