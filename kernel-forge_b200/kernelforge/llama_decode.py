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
on the TinyLlama-1.1B architecture).  The embedding lookup is fused into the first norm (ops.embed_rmsnorm), the fp16
lm_head is this library's streaming GEMV with the greedy argmax fused (ops.lm_head_argmax: the lm_head is the largest
single read of a step), and one kernel publishes the token and advances the device-side counters
(ops.decode_finalize).

Tensor parallelism (one process per GPU, `group` given): every decoder linear is sharded over its OUTPUT features, so
no reduction is ever needed.  Rank r owns a block of query heads with their KV heads (a KV head is replicated when
there are more ranks than KV heads), the matching rows of the fused qkv matrix, 1/W of the rows of o_proj and
down_proj, and the gate and up rows of 1/W of the intermediate features (SiLU * up stays local).  Four all-gathers
per layer rebuild the activations: attention output, o_proj output, activation, down_proj output.  Norms, residual
stream, embedding and lm_head are replicated, so every rank holds the same logits and picks the same token.  At batch
1 a gather costs more than the kernels it connects; the numbers are reported as they are.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import ops
from . import quantize as kq


def tp_plan(shape: "LlamaShape", rank: int, world: int) -> dict:
    """Which query heads, KV heads, hidden rows and intermediate features rank `rank` of `world` owns.

    KV heads are split over the ranks when there are enough of them; otherwise the query heads of one KV head are
    split over world / kv_heads ranks and that KV head is replicated.  All ranges are contiguous and in rank order, so
    concatenating the ranks' outputs restores the natural feature order."""
    from .parallel import row_bounds
    h, hk = shape.heads, shape.kv_heads
    g = h // hk
    if hk % world == 0:
        per = hk // world
        kv = (rank * per, (rank + 1) * per)
        q = (rank * per * g, (rank + 1) * per * g)
    elif world % hk == 0 and g % (world // hk) == 0:
        split = world // hk
        gq = g // split
        kv = (rank // split, rank // split + 1)
        q = (kv[0] * g + (rank % split) * gq, kv[0] * g + (rank % split + 1) * gq)
    else:
        raise ValueError(f"cannot split heads={h}, kv_heads={hk} over {world} ranks without breaking a KV group")
    return {"q_heads": q, "kv_heads": kv, "hidden_rows": row_bounds(shape.hidden, world)[rank],
            "inter": row_bounds(shape.intermediate, world)[rank],
            "attn_bounds": [(r * (q[1] - q[0]) * shape.head_dim, (r + 1) * (q[1] - q[0]) * shape.head_dim) for r in range(world)],
            "hidden_bounds": row_bounds(shape.hidden, world), "inter_bounds": row_bounds(shape.intermediate, world)}


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
    __slots__ = ("packed", "scales", "group", "pre")

    def __init__(self, w: torch.Tensor, group: int, prepack: bool = False):
        qw = kq.quantize_weight(w, group)
        self.packed, self.scales, self.group = qw.packed, qw.scales, group
        # the private fragment-order copy the small-batch GEMV of a decode step runs on (ops.prepack_int4)
        self.pre = ops.prepack_int4(self.packed) if prepack else None

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return ops.int4_linear(x, self.packed, self.scales, self.group)


class LlamaInt4Decoder:
    """fp16 activations, INT4 g128 decoder linears, fused attention, static KV cache."""

    def __init__(self, shape: LlamaShape, weights: dict, device, batch: int, max_len: int, group: int = 128, tp_group=None,
                 programmatic_launch: bool = True, peer_gather: bool = True, prepack: bool = True):
        self.s, self.dev, self.b, self.max_len = shape, torch.device(device), batch, max_len
        # decode steps are launched with programmatic dependent launch (every kernel of the step waits for its
        # predecessor before touching activations); with tensor parallelism only when the gathers are this library's
        # peer-memory kernels too (NCCL kernels in between know nothing of the protocol)
        self.pdl = programmatic_launch and (tp_group is None or peer_gather)
        # The 5-kernels-per-layer step (_step_fused, batch <= 2: RMSNorm in the prologue of the consuming GEMV, residual adds
        # and pair epilogues in the producing ones) is available but not the default: a fused prologue (norm over the whole
        # row, two block barriers) sits on every GEMV's critical path and costs what the two launches it removes would have.
        # Measured, ms per step on the TinyLlama-1.1B shape with programmatic dependent launch: batch 1 0.624 fused against
        # 0.620 separate, batch 2 0.80 against 0.64 (the separate step runs on the prepacked GEMV there).
        self.fused = False
        s = shape
        self.tp_group = tp_group
        self.world = 1
        if tp_group is not None:
            import torch.distributed as dist
            self.world, self.rank = dist.get_world_size(tp_group), dist.get_rank(tp_group)
        self.plan = tp_plan(s, self.rank, self.world) if self.world > 1 else None
        self._xchg = None
        if self.plan is not None and peer_gather:
            from .parallel import PeerExchange
            widest = max(s.hidden, s.intermediate, s.heads * s.head_dim)
            self._xchg = PeerExchange(batch, widest, tp_group, self.dev)   # 4 gathers per layer: an even number per step
        # local sizes (the whole model when not tensor-parallel)
        self.h_loc = s.heads if self.plan is None else self.plan["q_heads"][1] - self.plan["q_heads"][0]
        self.hk_loc = s.kv_heads if self.plan is None else self.plan["kv_heads"][1] - self.plan["kv_heads"][0]
        self.inter_loc = s.intermediate if self.plan is None else self.plan["inter"][1] - self.plan["inter"][0]
        # Batch <= 2 on one GPU: the rows of the fused qkv and gate_up matrices are stored in the order the pair
        # epilogues of the GEMV want (ops.interleave_qkv_for_rope / interleave_gate_up), so RoPE + cache write and
        # SiLU * up happen in the epilogue of the projection (8 kernels per layer instead of 10).  Rows are quantised
        # independently, so this is exact; prefill reads the same matrices and undoes the order with a view.
        # Batch 2..8 on one GPU: the decode-step GEMVs run on private fragment-order copies of the weights
        # (ops.prepack_int4; as much memory again as the packed weights), with the same pair epilogues.  Measured,
        # ms per step on the TinyLlama-1.1B shape, dispatcher kernels -> prepacked: batch 1 0.675 -> 0.681 (a tie: the
        # CUDA-core GEMV stays, and the memory is saved), batch 2 0.80 -> 0.70, batch 8 1.01 -> 0.75.
        # With tensor parallelism the same holds for the rank's own rows (local heads, local share of the hidden and
        # intermediate features); only the four gathers per layer are added.
        hidden_loc = s.hidden if self.plan is None else self.plan["hidden_rows"][1] - self.plan["hidden_rows"][0]
        kdims = (s.hidden, s.heads * s.head_dim, s.intermediate)
        ndims = ((self.h_loc + 2 * self.hk_loc) * s.head_dim, hidden_loc, 2 * self.inter_loc)
        groups = s.hidden // group     # (the pair epilogues above 8 batch rows exist for K split 8 ways, <= 12 blocks of 64 per warp)
        wide_ok = batch <= 8 or (groups >= 8 and -(-groups // 8) * (group // 64) <= 12)
        self.prepacked = (prepack and 2 <= batch <= ops.PREPACKED_GEMV_MAX_M and wide_ok
                          and all(k % 64 == 0 and k % group == 0 and k <= 12288 for k in kdims) and all(n % 16 == 0 for n in ndims))
        self.pair_rows = batch <= ops.FUSED_GEMV_MAX_M or self.prepacked
        f16 = lambda t: t.to(self.dev, torch.float16).contiguous()
        self.embed = f16(weights["embed"])
        self.lm_head = f16(weights["lm_head"])
        self.final_norm = f16(weights["final_norm"])
        self.layers = []
        d = s.head_dim
        for lw in weights["layers"]:
            q, k, v, o, gate, up, down = (lw[n] for n in ("q", "k", "v", "o", "gate", "up", "down"))
            if self.plan is not None:   # rows of this rank (output features); groups run along K: no requantisation issue
                (q0, q1), (k0, k1) = self.plan["q_heads"], self.plan["kv_heads"]
                (r0, r1), (i0, i1) = self.plan["hidden_rows"], self.plan["inter"]
                q, k, v = q[q0 * d:q1 * d], k[k0 * d:k1 * d], v[k0 * d:k1 * d]
                o, down, gate, up = o[r0:r1], down[r0:r1], gate[i0:i1], up[i0:i1]
            # q/k/v and gate/up share their input, so they are stored as ONE quantised matrix each (rows
            # concatenated: groups run along K, so this is bit-identical to quantising them separately)
            if self.pair_rows:
                qkv_rows, gate_up_rows = ops.interleave_qkv_for_rope(f16(q), f16(k), f16(v), d), ops.interleave_gate_up(f16(gate), f16(up))
            else:
                qkv_rows, gate_up_rows = torch.cat([f16(q), f16(k), f16(v)], 0), torch.cat([f16(gate), f16(up)], 0)
            self.layers.append({
                "in_norm": f16(lw["in_norm"]), "post_norm": f16(lw["post_norm"]),
                "qkv": _Int4(qkv_rows, group, self.prepacked),
                "o": _Int4(f16(o), group, self.prepacked),
                "gate_up": _Int4(gate_up_rows, group, self.prepacked),
                "down": _Int4(f16(down), group, self.prepacked),
            })
        self.k_cache = torch.zeros(s.layers, batch, self.hk_loc, max_len, s.head_dim, dtype=torch.float16, device=self.dev)
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
        self.best = torch.zeros(batch, dtype=torch.int64, device=self.dev)   # argmax keys of the step, see ops.lm_head_argmax
        # Batch <= 2, head dim 64, one GPU: the whole step can run as ONE persistent cooperative kernel
        # (kfb_decode_step_persistent) plus the finalize kernel: set `persistent = True` before capture().  Not the default:
        # measured on the TinyLlama-1.1B shape it takes 0.98 ms per step at batch 1 against 0.68 ms for the step of
        # separate kernels chained by programmatic dependent launch -- five grid-wide barriers per layer at ~2 us each
        # plus the L2 round trip that re-reads the activations after each of them cost more than the launches they replace.
        self.persistent_ok = self.pair_rows and self.plan is None and batch <= 2 and s.head_dim == 64
        self.persistent = False
        self._step_desc = self._persistent_descriptor() if self.persistent_ok else None
        self.graph = None
        # Host mirror of `pos`: the number of cache rows in use.  The step graph reads the position on the device,
        # so the host checks here that a replay can never be asked to write past the cache.
        self._host_pos = 0

    # ------------------------------------------------------------------ construction helpers
    def _persistent_descriptor(self):
        """The argument block of kfb_decode_step_persistent: a device table of 12 pointers per layer, the workspace."""
        from . import _capi
        s = self.s
        rows = [[L["qkv"].packed.data_ptr(), L["qkv"].scales.data_ptr(), L["o"].packed.data_ptr(), L["o"].scales.data_ptr(),
                 L["gate_up"].packed.data_ptr(), L["gate_up"].scales.data_ptr(), L["down"].packed.data_ptr(),
                 L["down"].scales.data_ptr(), L["in_norm"].data_ptr(), L["post_norm"].data_ptr(),
                 self.k_cache[li].data_ptr(), self.v_cache[li].data_ptr()] for li, L in enumerate(self.layers)]
        self._layer_table = torch.tensor(rows, dtype=torch.int64).to(self.dev)
        nbytes = _capi.lib().kfb_decode_step_ws_bytes(self.b, s.hidden, s.heads, s.kv_heads, s.head_dim, s.intermediate)
        self._step_ws = torch.empty(nbytes, dtype=torch.uint8, device=self.dev)
        d = _capi.DecodeStep()
        d.layer_table = self._layer_table.data_ptr()
        d.layers, d.batch, d.hidden, d.heads, d.kv_heads = s.layers, self.b, s.hidden, s.heads, s.kv_heads
        d.head_dim, d.intermediate, d.vocab, d.max_len, d.group = s.head_dim, s.intermediate, s.vocab, self.max_len, self.layers[0]["qkv"].group
        d.rms_eps = s.rms_eps
        d.embed, d.final_norm, d.lm_head = self.embed.data_ptr(), self.final_norm.data_ptr(), self.lm_head.data_ptr()
        d.cos_table, d.sin_table = self.cos.data_ptr(), self.sin.data_ptr()
        d.tok, d.pos, d.kv_len = self.tok.data_ptr(), self.pos.data_ptr(), self.kv_len.data_ptr()
        d.logits, d.best = self.step_logits.data_ptr(), self.best.data_ptr()
        d.workspace, d.workspace_bytes = self._step_ws.data_ptr(), nbytes
        return d

    def _step_persistent(self):
        """The whole step as one persistent cooperative kernel, then the kernel that publishes token / position / length."""
        import ctypes
        from . import _capi
        with _capi.on_device(self.dev):
            _capi.check(_capi.lib().kfb_decode_step_persistent(ctypes.byref(self._step_desc), _capi.stream_ptr(self.dev)))
        ops.decode_finalize(self.best, self.tok, self.pos, self.kv_len)

    def _gather(self, y_local: torch.Tensor, bounds_key: str) -> torch.Tensor:
        """All-gather of the ranks' column blocks ([rows, n_local] -> [rows, n]); the identity without tensor parallelism.
        Decode-sized blocks go over peer memory (parallel.PeerExchange: one launch of this library's kernel per gather,
        no NCCL kernel in the step graph); larger ones (prefill) through NCCL."""
        if self.plan is None:
            return y_local
        rows = y_local.shape[0]
        if self._xchg is not None and rows <= self.b:
            return self._xchg.allgather_columns(y_local, self.plan[bounds_key])
        from .parallel import gather_columns
        return gather_columns(y_local, self.plan[bounds_key], self.tp_group)

    @classmethod
    def random_init(cls, shape: LlamaShape, device, batch: int, max_len: int, seed: int = 0, std: float = 0.02, tp_group=None):
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
        return cls(shape, weights, device, batch, max_len, tp_group=tp_group)

    @classmethod
    def from_hf(cls, model, device, batch: int, max_len: int, tp_group=None):
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
        return cls(shape, weights, device, batch, max_len, tp_group=tp_group)

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
        inter = self.inter_loc
        if self.pair_rows:
            gu = gu.view(*gu.shape[:-1], inter, 2)
            act = torch.nn.functional.silu(gu[..., 0]) * gu[..., 1]
        else:
            act = torch.nn.functional.silu(gu[..., :inter]) * gu[..., inter:]
        lead = act.shape[:-1]
        act = self._gather(act.reshape(-1, inter), "inter_bounds").reshape(*lead, self.s.intermediate)
        down = L["down"](act)
        return x + self._gather(down.reshape(-1, down.shape[-1]), "hidden_bounds").reshape(*lead, self.s.hidden)

    # ------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prefill(self, ids: torch.Tensor) -> torch.Tensor:
        """ids [B, T] -> logits [B, T, vocab] (fp16); fills the cache and arms the decode state with the
        greedy next token."""
        s, (b, t) = self.s, ids.shape
        if t >= self.max_len:
            raise ValueError(f"prompt of {t} tokens leaves no room in a cache of {self.max_len} rows for a decode step")
        ids = ids.to(self.dev)
        x = self.embed[ids]
        cos, sin = self.cos[:t], self.sin[:t]
        for li, L in enumerate(self.layers):
            h = self._rms(x, L["in_norm"])
            qkv = L["qkv"](h)
            nq, nkv = self.h_loc * s.head_dim, self.hk_loc * s.head_dim
            if self.pair_rows:   # features (j, j + D/2) sit side by side: back to the natural order
                unpair = lambda z, heads: z.reshape(b, t, heads, s.head_dim // 2, 2).transpose(-1, -2).reshape(b, t, heads, s.head_dim)
                q = unpair(qkv[..., :nq], self.h_loc).transpose(1, 2)
                k = unpair(qkv[..., nq:nq + nkv], self.hk_loc).transpose(1, 2)
            else:
                q = qkv[..., :nq].reshape(b, t, self.h_loc, s.head_dim).transpose(1, 2)
                k = qkv[..., nq:nq + nkv].reshape(b, t, self.hk_loc, s.head_dim).transpose(1, 2)
            v = qkv[..., nq + nkv:].reshape(b, t, self.hk_loc, s.head_dim).transpose(1, 2)
            q, k = self._rope(q, cos, sin), self._rope(k, cos, sin)
            self.k_cache[li, :, :, :t] = k
            self.v_cache[li, :, :, :t] = v
            a = ops.flash_attn_kv_view(q.contiguous(), self.k_cache[li, :, :, :t], self.v_cache[li, :, :, :t], causal=True)
            a = self._gather(a.transpose(1, 2).reshape(b * t, nq), "attn_bounds")
            o = self._gather(L["o"](a), "hidden_bounds")
            x = x + o.reshape(b, t, s.hidden)
            x = self._mlp(L, x)
        logits = self._rms(x, self.final_norm) @ self.lm_head.T
        self.tok.copy_(logits[:, -1].float().argmax(-1))
        self.pos.fill_(t)
        self.kv_len.fill_(t + 1)
        self._host_pos = t
        return logits

    # ------------------------------------------------------------------ one decode step (graph body)
    @torch.no_grad()
    def _step_fused(self):
        """The step for batch <= 2 on one GPU with everything fused: 5 kernels per layer.  Both RMSNorms run in the
        prologue of the GEMV that consumes them, RoPE + cache write and SiLU * up in the epilogue of the GEMV that
        produces their input, both residual adds in the epilogues of o_proj and down_proj; only the attention itself
        stays a kernel of its own."""
        s, b = self.s, self.b
        _, x = ops.embed_rmsnorm(self.tok, self.embed, self.layers[0]["in_norm"], s.rms_eps)   # x: the residual stream
        for li, L in enumerate(self.layers):
            q = ops.int4_gemv_rope_kv(x, L["qkv"].packed, L["qkv"].scales, L["qkv"].group, self.cos, self.sin, self.pos,
                                      self.k_cache[li], self.v_cache[li], self.h_loc, L["in_norm"], s.rms_eps)
            a = ops.flash_attn_decode(q, self.k_cache[li], self.v_cache[li], self.kv_len).view(b, self.h_loc * s.head_dim)
            x = ops.int4_gemv_fused(a, L["o"].packed, L["o"].scales, L["o"].group, residual=x)
            act = ops.int4_gemv_silu_pair(x, L["gate_up"].packed, L["gate_up"].scales, L["gate_up"].group, L["post_norm"], s.rms_eps)
            x = ops.int4_gemv_fused(act, L["down"].packed, L["down"].scales, L["down"].group, residual=x)
        h, _ = ops.add_rmsnorm(x, self.final_norm, s.rms_eps)
        ops.lm_head_argmax(h, self.lm_head, self.step_logits, self.best)
        ops.decode_finalize(self.best, self.tok, self.pos, self.kv_len)

    @torch.no_grad()
    def _step(self):
        """One decode step: 9 or 10 kernels per layer (add + norm, qkv, rope + cache write, attention (+ merge when the
        keys are split), o, add + norm, gate_up, silu * up, down; the last residual add is fused into the next layer's
        norm; the embedding gather is fused into the first norm) -- 7 or 8 at batch <= 2 on one GPU, where rope +
        cache write and silu * up run in the epilogues of the qkv and gate_up GEMVs -- then final norm, lm_head with fused argmax, and
        one kernel that publishes the token and advances position and KV length.  Every kernel of the step is one
        of this library's: no torch or cuBLAS kernel is left in the graph."""
        if self.persistent:
            return self._step_persistent()
        if self.plan is None and self.b <= ops.FUSED_GEMV_MAX_M and self.fused:
            return self._step_fused()
        s, b = self.s, self.b
        res = None                                                 # pending residual branch output
        for li, L in enumerate(self.layers):
            if li == 0:
                h, x = ops.embed_rmsnorm(self.tok, self.embed, L["in_norm"], s.rms_eps)   # [B, hidden] each
            else:
                h, x = ops.add_rmsnorm(x, L["in_norm"], s.rms_eps, res)
            if self.prepacked:
                q = ops.int4_gemv_prepacked_rope_kv(h, L["qkv"].pre, L["qkv"].scales, L["qkv"].group, self.cos, self.sin, self.pos,
                                                    self.k_cache[li], self.v_cache[li], self.h_loc)
            elif self.pair_rows:
                q = ops.int4_gemv_rope_kv(h, L["qkv"].packed, L["qkv"].scales, L["qkv"].group, self.cos, self.sin, self.pos,
                                          self.k_cache[li], self.v_cache[li], self.h_loc)
            else:
                qkv = L["qkv"](h)
                q = ops.rope_kv_write(qkv, self.cos, self.sin, self.pos, self.k_cache[li], self.v_cache[li], self.h_loc)
            a = ops.flash_attn_decode(q, self.k_cache[li], self.v_cache[li], self.kv_len)
            a = self._gather(a.view(b, self.h_loc * s.head_dim), "attn_bounds")
            o = ops.int4_gemv_prepacked(a, L["o"].pre, L["o"].scales, L["o"].group) if self.prepacked else L["o"](a)
            o = self._gather(o, "hidden_bounds")
            h, x = ops.add_rmsnorm(x, L["post_norm"], s.rms_eps, o)
            if self.prepacked:
                act = ops.int4_gemv_prepacked_silu_pair(h, L["gate_up"].pre, L["gate_up"].scales, L["gate_up"].group)
            elif self.pair_rows:
                act = ops.int4_gemv_silu_pair(h, L["gate_up"].packed, L["gate_up"].scales, L["gate_up"].group)
            else:
                act = ops.silu_mul(L["gate_up"](h))
            act = self._gather(act, "inter_bounds")
            res = ops.int4_gemv_prepacked(act, L["down"].pre, L["down"].scales, L["down"].group) if self.prepacked else L["down"](act)
            res = self._gather(res, "hidden_bounds")
        h, x = ops.add_rmsnorm(x, self.final_norm, s.rms_eps, res)
        ops.lm_head_argmax(h, self.lm_head, self.step_logits, self.best)
        ops.decode_finalize(self.best, self.tok, self.pos, self.kv_len)

    def capture(self):
        """Captures one decode step.  State is saved and restored around the warm-up / capture runs (the warm-up
        step writes cache row `pos`, which the first real step rewrites with the same values)."""
        if self._host_pos >= self.max_len:
            raise ValueError(f"the KV cache ({self.max_len} rows) is full: no room for the warm-up step")
        from . import _capi
        saved = (self.tok.clone(), self.pos.clone(), self.kv_len.clone())
        side = torch.cuda.Stream(self.dev)
        with torch.cuda.stream(side), _capi.programmatic_launch(self.pdl):
            self._step()
            side.synchronize()
            self.tok.copy_(saved[0]); self.pos.copy_(saved[1]); self.kv_len.copy_(saved[2])
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=side):
                self._step()
            self.tok.copy_(saved[0]); self.pos.copy_(saved[1]); self.kv_len.copy_(saved[2])
            side.synchronize()
        return self

    def release(self):
        """Drops the captured graph.  With tensor parallelism this must happen before the process group is destroyed:
        a live CUDA graph that holds captured NCCL all-gathers makes destroy_process_group() wait forever."""
        self.graph = None
        import gc
        gc.collect()
        torch.cuda.synchronize(self.dev)

    @torch.no_grad()
    def decode(self, steps: int, keep_logits: bool = False, check_status: bool = True):
        """Runs `steps` greedy steps from the armed state.  Returns (tokens [B, steps] fed to the model,
        logits [B, steps, vocab] or None).  Raises ValueError when the steps do not fit in the KV cache (every
        step writes one cache row; nothing is launched then).  With `check_status` the device status word is read
        after the last step (one 4-byte copy, synchronising) and a kernel that gave up raises DeviceStatusError."""
        if steps < 0 or self._host_pos + steps > self.max_len:
            raise ValueError(f"{steps} decode steps from position {self._host_pos} do not fit in a KV cache of "
                             f"{self.max_len} rows")
        if self.graph is None:
            self.capture()
        toks, logs = [], []
        for _ in range(steps):
            toks.append(self.tok.clone())
            self.graph.replay()
            if keep_logits:
                logs.append(self.step_logits.clone())
        self._host_pos += steps
        if check_status:
            from . import _capi
            _capi.raise_on_device_status(self.dev)
        return torch.stack(toks, 1), (torch.stack(logs, 1) if keep_logits else None)
