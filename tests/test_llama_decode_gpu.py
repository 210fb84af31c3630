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
