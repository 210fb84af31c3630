"""Greedy decoding of a Llama-architecture model on the B200 kernels, one CUDA graph per decode step.

What the reference measures with `bench/e2e_model.py::graph_decode` (97-141): prefill on a static KV cache,
then one captured decode step replayed per token.  There the captured step has to use SDPA because the
reference's attention kernel takes the KV length from the tensor shape (docstring 91-92, README.md:101).
Here the step runs `ops.flash_attn_decode`, which reads the valid cache length from a device tensor, and
`ops.int4_linear` for the seven decoder linears of every layer; token ids, position and KV length all live
on the device, so a step is a pure graph replay with no host synchronisation.

Prefill uses torch for everything that is not one of the two hot paths (embedding, RMSNorm, RoPE, SiLU * up,
residual adds, lm_head), as the reference does.  The decode step is launch-bound at batch 1, so there those
element-wise steps run as three fused kernels (ops.add_rmsnorm, ops.rope_kv_write, ops.silu_mul) and q/k/v and
gate/up are stored as one quantised matrix each: 11 kernels per layer instead of ~48 (2.39 -> 0.85 ms per step
on the TinyLlama-1.1B architecture).  Embedding lookup, the fp16 lm_head and argmax stay torch.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import ops
from . import quantize as kq


@dataclass
class LlamaShape:
    hidden: int = 2048
    layers: int = 22
    heads: int = 32
    kv_heads: int = 4
    head_dim: int = 64
    intermediate: int = 5632
    vocab: int = 32000
    rope_theta: float = 10000.0
    rms_eps: float = 1e-5


TINYLLAMA_1B = LlamaShape()


class _Int4:
    __slots__ = ("packed", "scales", "group")

    def __init__(self, w: torch.Tensor, group: int):
        qw = kq.quantize_weight(w, group)
        self.packed, self.scales, self.group = qw.packed, qw.scales, group

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return ops.int4_linear(x, self.packed, self.scales, self.group)


class LlamaInt4Decoder:
    """fp16 activations, INT4 g128 decoder linears, fused attention, static KV cache."""

    def __init__(self, shape: LlamaShape, weights: dict, device, batch: int, max_len: int, group: int = 128):
        self.s, self.dev, self.b, self.max_len = shape, torch.device(device), batch, max_len
        s = shape
        f16 = lambda t: t.to(self.dev, torch.float16).contiguous()
        self.embed = f16(weights["embed"])
        self.lm_head = f16(weights["lm_head"])
        self.final_norm = f16(weights["final_norm"])
        self.layers = []
        for lw in weights["layers"]:
            # q/k/v and gate/up share their input, so they are stored as ONE quantised matrix each (rows
            # concatenated: groups run along K, so this is bit-identical to quantising them separately)
            self.layers.append({
                "in_norm": f16(lw["in_norm"]), "post_norm": f16(lw["post_norm"]),
                "qkv": _Int4(torch.cat([f16(lw["q"]), f16(lw["k"]), f16(lw["v"])], 0), group),
                "o": _Int4(f16(lw["o"]), group),
                "gate_up": _Int4(torch.cat([f16(lw["gate"]), f16(lw["up"])], 0), group),
                "down": _Int4(f16(lw["down"]), group),
            })
        self.k_cache = torch.zeros(s.layers, batch, s.kv_heads, max_len, s.head_dim, dtype=torch.float16, device=self.dev)
        self.v_cache = torch.zeros_like(self.k_cache)
        inv = 1.0 / (s.rope_theta ** (torch.arange(0, s.head_dim, 2, dtype=torch.float32) / s.head_dim))
        ang = torch.outer(torch.arange(max_len, dtype=torch.float32), inv)
        ang = torch.cat([ang, ang], dim=-1)
        self.cos, self.sin = ang.cos().to(self.dev), ang.sin().to(self.dev)  # [max_len, D] fp32
        # device-side decode state
        self.tok = torch.zeros(batch, dtype=torch.long, device=self.dev)
        self.pos = torch.zeros(1, dtype=torch.long, device=self.dev)        # position of the token being fed
        self.kv_len = torch.zeros(batch, dtype=torch.int32, device=self.dev)
        self.step_logits = torch.zeros(batch, s.vocab, dtype=torch.float16, device=self.dev)
        self.graph = None

    # ------------------------------------------------------------------ construction helpers
    @classmethod
    def random_init(cls, shape: LlamaShape, device, batch: int, max_len: int, seed: int = 0, std: float = 0.02):
        """Weights ~ N(0, std), norms = 1: the initialisation of a fresh Hugging Face Llama."""
        g = torch.Generator().manual_seed(seed)
        s = shape
        rn = lambda *sz: torch.randn(*sz, generator=g) * std
        qd, kd = s.heads * s.head_dim, s.kv_heads * s.head_dim
        layers = [{"in_norm": torch.ones(s.hidden), "post_norm": torch.ones(s.hidden), "q": rn(qd, s.hidden),
                   "k": rn(kd, s.hidden), "v": rn(kd, s.hidden), "o": rn(s.hidden, qd), "gate": rn(s.intermediate, s.hidden),
                   "up": rn(s.intermediate, s.hidden), "down": rn(s.hidden, s.intermediate)} for _ in range(s.layers)]
        weights = {"embed": rn(s.vocab, s.hidden), "lm_head": rn(s.vocab, s.hidden), "final_norm": torch.ones(s.hidden),
                   "layers": layers}
        return cls(shape, weights, device, batch, max_len)

    @classmethod
    def from_hf(cls, model, device, batch: int, max_len: int):
        """From a transformers LlamaForCausalLM (any dtype; weights are rounded to fp16, then quantised)."""
        c = model.config
        theta = getattr(c, "rope_theta", None) or (getattr(c, "rope_parameters", None) or {}).get("rope_theta", 10000.0)
        shape = LlamaShape(c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads,
                           getattr(c, "head_dim", None) or c.hidden_size // c.num_attention_heads, c.intermediate_size,
                           c.vocab_size, float(theta), c.rms_norm_eps)
        sd = model.state_dict()
        layers = []
        for i in range(shape.layers):
            p = f"model.layers.{i}."
            layers.append({"in_norm": sd[p + "input_layernorm.weight"], "post_norm": sd[p + "post_attention_layernorm.weight"],
                           "q": sd[p + "self_attn.q_proj.weight"], "k": sd[p + "self_attn.k_proj.weight"],
                           "v": sd[p + "self_attn.v_proj.weight"], "o": sd[p + "self_attn.o_proj.weight"],
                           "gate": sd[p + "mlp.gate_proj.weight"], "up": sd[p + "mlp.up_proj.weight"],
                           "down": sd[p + "mlp.down_proj.weight"]})
        weights = {"embed": sd["model.embed_tokens.weight"], "lm_head": sd["lm_head.weight"],
                   "final_norm": sd["model.norm.weight"], "layers": layers}
        return cls(shape, weights, device, batch, max_len)

    # ------------------------------------------------------------------ building blocks (torch)
    def _rms(self, x, w):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.s.rms_eps)).to(torch.float16) * w

    @staticmethod
    def _rope(t, cos, sin):  # t [B, heads, T, D]; cos/sin broadcastable [T, D]
        tf = t.float()
        half = tf.shape[-1] // 2
        rot = torch.cat([-tf[..., half:], tf[..., :half]], dim=-1)
        return (tf * cos + rot * sin).to(torch.float16)

    def _mlp(self, L, x):
        h = self._rms(x, L["post_norm"])
        gu = L["gate_up"](h)
        inter = self.s.intermediate
        return x + L["down"](torch.nn.functional.silu(gu[..., :inter]) * gu[..., inter:])

    # ------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prefill(self, ids: torch.Tensor) -> torch.Tensor:
        """ids [B, T] -> logits [B, T, vocab] (fp16); fills the cache and arms the decode state with the
        greedy next token."""
        s, (b, t) = self.s, ids.shape
        ids = ids.to(self.dev)
        x = self.embed[ids]
        cos, sin = self.cos[:t], self.sin[:t]
        for li, L in enumerate(self.layers):
            h = self._rms(x, L["in_norm"])
            qkv = L["qkv"](h)
            nq, nkv = s.heads * s.head_dim, s.kv_heads * s.head_dim
            q = qkv[..., :nq].reshape(b, t, s.heads, s.head_dim).transpose(1, 2)
            k = qkv[..., nq:nq + nkv].reshape(b, t, s.kv_heads, s.head_dim).transpose(1, 2)
            v = qkv[..., nq + nkv:].reshape(b, t, s.kv_heads, s.head_dim).transpose(1, 2)
            q, k = self._rope(q, cos, sin), self._rope(k, cos, sin)
            self.k_cache[li, :, :, :t] = k
            self.v_cache[li, :, :, :t] = v
            a = ops.flash_attn_kv_view(q.contiguous(), self.k_cache[li, :, :, :t], self.v_cache[li, :, :, :t], causal=True)
            x = x + L["o"](a.transpose(1, 2).reshape(b, t, s.heads * s.head_dim))
            x = self._mlp(L, x)
        logits = self._rms(x, self.final_norm) @ self.lm_head.T
        self.tok.copy_(logits[:, -1].float().argmax(-1))
        self.pos.fill_(t)
        self.kv_len.fill_(t + 1)
        return logits

    # ------------------------------------------------------------------ one decode step (graph body)
    @torch.no_grad()
    def _step(self):
        """One decode step: 11 kernels per layer (norm, qkv, rope + cache write, attention x2, o, add + norm,
        gate_up, silu * up, down; the last residual add is fused into the next layer's norm)."""
        s, b = self.s, self.b
        x = self.embed[self.tok]                                   # [B, hidden]
        res = None                                                 # pending residual branch output
        for li, L in enumerate(self.layers):
            h, x = ops.add_rmsnorm(x, L["in_norm"], s.rms_eps, res)
            qkv = L["qkv"](h)
            q = ops.rope_kv_write(qkv, self.cos, self.sin, self.pos, self.k_cache[li], self.v_cache[li], s.heads)
            a = ops.flash_attn_decode(q, self.k_cache[li], self.v_cache[li], self.kv_len)
            o = L["o"](a.view(b, s.heads * s.head_dim))
            h, x = ops.add_rmsnorm(x, L["post_norm"], s.rms_eps, o)
            res = L["down"](ops.silu_mul(L["gate_up"](h)))
        h, x = ops.add_rmsnorm(x, self.final_norm, s.rms_eps, res)
        logits = h @ self.lm_head.T
        self.step_logits.copy_(logits)
        self.tok.copy_(logits.float().argmax(-1))
        self.pos.add_(1)
        self.kv_len.add_(1)

    def capture(self):
        """Captures one decode step.  State is saved and restored around the warm-up / capture runs."""
        saved = (self.tok.clone(), self.pos.clone(), self.kv_len.clone())
        side = torch.cuda.Stream(self.dev)
        with torch.cuda.stream(side):
            self._step()
            side.synchronize()
            self.tok.copy_(saved[0]); self.pos.copy_(saved[1]); self.kv_len.copy_(saved[2])
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=side):
                self._step()
            self.tok.copy_(saved[0]); self.pos.copy_(saved[1]); self.kv_len.copy_(saved[2])
            side.synchronize()
        return self

    @torch.no_grad()
    def decode(self, steps: int, keep_logits: bool = False):
        """Runs `steps` greedy steps from the armed state.  Returns (tokens [B, steps] fed to the model,
        logits [B, steps, vocab] or None)."""
        if self.graph is None:
            self.capture()
        toks, logs = [], []
        for _ in range(steps):
            toks.append(self.tok.clone())
            self.graph.replay()
            if keep_logits:
                logs.append(self.step_logits.clone())
        return torch.stack(toks, 1), (torch.stack(logs, 1) if keep_logits else None)
