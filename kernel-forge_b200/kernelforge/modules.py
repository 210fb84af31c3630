"""Drop-in modules that put the B200 kernels inside Hugging Face models.

Same surface as the reference (kernelforge/modules.py:19-115), and the body follows the reference's file
function by function, in places line by line: this is glue between Hugging Face classes and the operator
surface, and buffer names, the attention-interface registration, the reuse of the flash_attention_2 mask
builder and the ATTN_STATS keys are all part of the contract.

- KFLinearInt4: nn.Linear replacement holding group-wise INT4 weights, forward via ops.int4_linear.
- quantize_linears_: swap a model's decoder linears (q, k, v, o, gate, up, down) for KFLinearInt4.
- enable_kf_attention / register_kf_attention: register ops.flash_attn with transformers'
  attention interface under the name "kernelforge" and switch a model to it.

Differences that stay behind the same API: weights are quantised on the GPU when the linear
lives there (bit-identical to the torch quantiser), and strided KV-cache views are handed to the
kernel in place instead of being copied with .contiguous() (reference: modules.py:95).
Inference only.
"""

from __future__ import annotations

import torch
from torch import nn

from . import ops
from . import quantize as kq

DECODER_LINEARS = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")


class KFLinearInt4(nn.Module):
    """INT4 weight-only nn.Linear: y = x W_hat^T + b, W_hat dequantised inside the kernel.

    Buffers keep the reference's names (`packed` int32 [N, K/8], `scales` fp16 [N, K/G], `bias` fp16 or
    None), so state dicts are interchangeable.  4 + 16/G bits per weight.  Activations: fp16 (every kernel) or bf16
    (the tcgen05 GEMM at every M; the reference is fp16 only).
    """

    def __init__(self, qw: kq.QuantizedWeight, bias: torch.Tensor | None):
        super().__init__()
        self.out_features, self.in_features = qw.shape
        self.group_size = qw.group_size
        self.register_buffer("packed", qw.packed)
        self.register_buffer("scales", qw.scales)
        self.register_buffer("bias", None if bias is None else bias.detach().half())

    @classmethod
    def from_linear(cls, linear: nn.Linear, group_size: int = kq.DEFAULT_GROUP_SIZE) -> "KFLinearInt4":
        return cls(kq.quantize_weight(linear.weight.detach(), group_size), linear.bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.dtype not in ops.INT4_ACT_DTYPES:
            raise TypeError(f"KFLinearInt4 takes fp16 activations (or bf16), got {x.dtype}")
        bias = self.bias if self.bias is None or x.dtype == torch.float16 else self.bias.to(x.dtype)
        return ops.int4_linear(x, self.packed, self.scales, self.group_size, bias)

    def prepack_(self) -> "KFLinearInt4":
        """Builds the private fragment-order copy of the weight (ops.prepack_weight_, keyed on the `packed` buffer; the
        reference's stated next step, docs/phase4-notes.md:59): batches of up to 8 rows then run on it.  Costs as much
        memory again as `packed`; state dicts are unaffected.  A no-op for shapes the copy does not support."""
        if self.packed.is_cuda and ops.prepack_supported(self.packed) and self.in_features <= 12288:
            ops.prepack_weight_(self.packed)
        return self

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, "
                f"group_size={self.group_size}, int4")


def prepack_linears_(model: nn.Module) -> int:
    """Calls KFLinearInt4.prepack_() on every INT4 linear of `model` (after the model is on its CUDA device: the private
    copies are keyed on the buffers' identity).  Returns the number of layers that got a private copy."""
    done = 0
    for mod in model.modules():
        if isinstance(mod, KFLinearInt4) and mod.packed.is_cuda and ops.prepack_supported(mod.packed) and mod.in_features <= 12288:
            mod.prepack_()
            done += 1
    return done


@torch.no_grad()
def quantize_linears_(model: nn.Module, group_size: int = kq.DEFAULT_GROUP_SIZE,
                      names: tuple[str, ...] = DECODER_LINEARS, prepack: bool = False) -> int:
    """Replace, in place, every nn.Linear whose attribute name is in `names` by KFLinearInt4.

    Embeddings and lm_head keep their dtype.  Returns the number of layers replaced.  `prepack` (not in the reference):
    also build the private fragment-order copies (prepack_linears_) when the model already sits on a CUDA device.
    """
    todo = []
    for parent in model.modules():
        for name, child in parent.named_children():
            if name in names and isinstance(child, nn.Linear):
                todo.append((parent, name, child))
    for parent, name, child in todo:
        setattr(parent, name, KFLinearInt4.from_linear(child, group_size))
    replaced = len(todo)
    if prepack:
        prepack_linears_(model)
    del todo  # drop the last references to the fp16 weights before returning their memory
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
    return replaced


# ---------------------------------------------------------------------------
# Attention
# ---------------------------------------------------------------------------

KF_ATTN_NAME = "kernelforge"
ATTN_STATS = {"kernelforge_calls": 0, "sdpa_fallback_calls": 0}


def _kf_attention_forward(module, query, key, value, attention_mask, dropout=0.0, scaling=None,
                          is_causal=None, **kwargs):
    """transformers attention function: query [B, H, Nq, D], key/value [B, Hk, Nk, D] (KV heads not repeated).

    Runs ops.flash_attn when it applies (no padding mask, no dropout, head dim 64/128, fp16/bf16, CUDA); the
    causal mask is bottom-right aligned, i.e. the KV-cache convention, so one call serves prefill and decode.
    Anything else goes to transformers' SDPA path, and every such call is counted in ATTN_STATS.
    Returns ([B, Nq, H, D], None) like sdpa_attention_forward.
    """
    from transformers.integrations.sdpa_attention import sdpa_attention_forward

    causal = is_causal if is_causal is not None else getattr(module, "is_causal", True)
    usable = (attention_mask is None and dropout == 0.0 and query.is_cuda
              and query.shape[-1] in ops.ATTN_HEAD_DIMS and query.dtype in ops.TC_ATTN_DTYPES
              and not kwargs.get("output_attentions", False))
    if not usable:
        ATTN_STATS["sdpa_fallback_calls"] += 1
        return sdpa_attention_forward(module, query, key, value, attention_mask, dropout=dropout,
                                      scaling=scaling, is_causal=is_causal, **kwargs)
    ATTN_STATS["kernelforge_calls"] += 1
    out = ops.flash_attn_kv_view(query.contiguous(), key, value, causal=bool(causal), scale=scaling)
    return out.transpose(1, 2).contiguous(), None


def register_kf_attention() -> str:
    """Registers the "kernelforge" attention function and its mask builder with transformers."""
    from transformers import AttentionInterface
    from transformers.masking_utils import ALL_MASK_ATTENTION_FUNCTIONS

    AttentionInterface.register(KF_ATTN_NAME, _kf_attention_forward)
    # the flash-attention mask builder yields None when there is no padding, which is what lets the fused
    # kernel run; with padding it yields a 2-D mask and the call falls back (and is counted)
    ALL_MASK_ATTENTION_FUNCTIONS.register(KF_ATTN_NAME, ALL_MASK_ATTENTION_FUNCTIONS["flash_attention_2"])
    return KF_ATTN_NAME


def enable_kf_attention(model: nn.Module) -> nn.Module:
    """Switch a loaded transformers model to the fused attention kernel."""
    register_kf_attention()
    model.set_attn_implementation(KF_ATTN_NAME)
    return model
