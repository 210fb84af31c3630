"""Multi-GPU use of the two hot paths, one process per GPU over torch.distributed.

The reference is single-GPU (no distributed code at all).  The paths shard naturally:

* attention is independent per (batch, head): `shard_attention_heads` gives each rank a block of
  query heads together with the KV heads they read; no communication at all.
* int4_linear shards over output features N: rank r keeps rows [lo_r, hi_r) of `packed` / `scales`,
  computes y[:, lo_r:hi_r] with the same kernels (the GEMM takes any N: 8960/8 = 1120, 1536/8 = 192 and
  256/8 = 32 rows are not multiples of 64) and ONE all-gather over NCCL / NVLink rebuilds y [M, N].

Nothing here launches a kernel itself; the compute goes through `kernelforge.ops`.
"""

from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist

from . import ops
from . import quantize as kq


def row_bounds(n: int, world: int) -> list[tuple[int, int]]:
    """Contiguous, near-equal split of n rows over `world` ranks (the first n % world ranks get one more)."""
    base, extra = divmod(n, world)
    out, lo = [], 0
    for r in range(world):
        hi = lo + base + (1 if r < extra else 0)
        out.append((lo, hi))
        lo = hi
    return out


def shard_quantized_weight(qw: kq.QuantizedWeight, rank: int, world: int) -> kq.QuantizedWeight:
    """Rows [lo, hi) of a quantised weight.  Groups run along K, so a row shard needs no requantisation."""
    lo, hi = row_bounds(qw.shape[0], world)[rank]
    return kq.QuantizedWeight(packed=qw.packed[lo:hi].contiguous(), scales=qw.scales[lo:hi].contiguous(),
                              group_size=qw.group_size, shape=(hi - lo, qw.shape[1]))


def shard_attention_heads(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, rank: int, world: int):
    """This rank's (q, k, v) for head-parallel attention.

    KV heads are split over ranks when Hk >= world (each rank takes its KV heads and their H/Hk query heads);
    when world > Hk (e.g. 8 GPUs, 4 KV heads) the query heads of one KV head are split over world/Hk ranks and
    that KV head is replicated.  Outputs concatenate along the head axis in rank order.
    """
    h, hk = q.shape[1], k.shape[1]
    g = h // hk
    if hk % world == 0:
        per = hk // world
        ks = slice(rank * per, (rank + 1) * per)
        qs = slice(rank * per * g, (rank + 1) * per * g)
    elif world % hk == 0 and g % (world // hk) == 0:
        split = world // hk
        kv = rank // split
        gq = g // split
        ks = slice(kv, kv + 1)
        qs = slice(kv * g + (rank % split) * gq, kv * g + (rank % split + 1) * gq)
    else:
        raise ValueError(f"cannot split H={h}, Hk={hk} over {world} ranks without breaking a KV group")
    return q[:, qs].contiguous(), k[:, ks].contiguous(), v[:, ks].contiguous()


def sequence_sharded_decode_attention(q: torch.Tensor, k_shard: torch.Tensor, v_shard: torch.Tensor, total_len: torch.Tensor | int,
                                      group: dist.ProcessGroup | None = None) -> torch.Tensor:
    """One decode step of a sequence whose KV cache is split along the sequence over the ranks of `group` (cross-GPU
    split-KV for a single long context): rank r holds rows [r * Nk_shard, (r + 1) * Nk_shard) of the cache.

    Each rank runs the split-KV decode kernel on its shard (ops.flash_attn_decode_partial), the FP32 partials --
    (O, m, l) per head, a few KB -- are all-gathered, and every rank merges them in rank order (deterministic), so all
    ranks hold the same output.  q: [B, H, 1, D] (replicated); total_len: int or int32 tensor [B], the valid length of
    the whole cache."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    b = q.shape[0]
    nk = k_shard.shape[2]
    if not torch.is_tensor(total_len):
        total_len = torch.full((b,), int(total_len), dtype=torch.int32, device=q.device)
    local_len = (total_len.to(torch.int32) - rank * nk).clamp_(0, nk)
    part = ops.flash_attn_decode_partial(q, k_shard, v_shard, local_len)
    gathered = torch.empty(world, part.numel(), dtype=torch.float32, device=q.device)
    dist.all_gather_into_tensor(gathered, part, group=group)
    return ops.flash_attn_merge_partials(gathered, q, k_shard.shape[1], nk)


class ShardedInt4Linear(torch.nn.Module):
    """Output-feature-parallel INT4 linear: local shard compute + one all-gather.

    `matmul` is the local compute (default: the kernels, any N); tests on CPU ranks pass a stand-in so
    the sharding and gather logic can run under gloo without a GPU.
    """

    def __init__(self, qw_full_shape: tuple[int, int], local: kq.QuantizedWeight, bias: torch.Tensor | None = None,
                 group: dist.ProcessGroup | None = None,
                 matmul: Callable[[torch.Tensor, torch.Tensor, torch.Tensor, int], torch.Tensor] | None = None):
        super().__init__()
        self.out_features, self.in_features = qw_full_shape
        self.group_size = local.group_size
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.bounds = row_bounds(self.out_features, self.world)
        assert local.shape[0] == self.bounds[self.rank][1] - self.bounds[self.rank][0]
        self.register_buffer("packed", local.packed)
        self.register_buffer("scales", local.scales)
        self.register_buffer("bias", None if bias is None else bias.detach().half())
        self._matmul = matmul or _local_int4_matmul

    @classmethod
    def from_full(cls, qw: kq.QuantizedWeight, bias=None, group=None, matmul=None) -> "ShardedInt4Linear":
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        return cls(qw.shape, shard_quantized_weight(qw, rank, world), bias, group, matmul)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        y_local = self._matmul(x2, self.packed, self.scales, self.group_size)  # [M, n_local]
        y = gather_columns(y_local, self.bounds, self.group)
        if self.bias is not None:
            y = y + self.bias
        return y.reshape(*lead, self.out_features)


def _local_int4_matmul(x, packed, scales, group_size):
    if x.shape[0] <= ops.GEMV_MAX_M:
        return ops.int4_gemv(x, packed, scales, group_size)
    return ops.int4_gemm_ragged(x, packed, scales, group_size)


def gather_columns(y_local: torch.Tensor, bounds: list[tuple[int, int]], group=None) -> torch.Tensor:
    """All-gather of column blocks: rank r contributes y[:, lo_r:hi_r]; returns the full [M, N] on every rank.

    Equal blocks use one all_gather_into_tensor (a single NCCL collective); ragged blocks are padded to the
    widest block first."""
    world = len(bounds)
    m = y_local.shape[0]
    widths = [hi - lo for lo, hi in bounds]
    wmax = max(widths)
    send = y_local if y_local.shape[1] == wmax else torch.nn.functional.pad(y_local, (0, wmax - y_local.shape[1]))
    flat = torch.empty(world * m, wmax, dtype=y_local.dtype, device=y_local.device)  # rank-major concatenation
    dist.all_gather_into_tensor(flat, send.contiguous(), group=group)
    recv = flat.view(world, m, wmax)
    if all(w == wmax for w in widths):
        return recv.permute(1, 0, 2).reshape(m, world * wmax)
    return torch.cat([recv[r, :, :w] for r, w in enumerate(widths)], dim=1)


def expected_arrivals(world: int, ctas_per_rank: int = 1) -> int:
    """Arrivals one rank receives per device-side rendezvous: every rank signals once per signalling CTA."""
    return world * ctas_per_rank


class PeerExchange:
    """Symmetric-memory buffers and arrival counters for device-side exchanges between the ranks of a group
    (kfb_peer_signal_wait / kfb_peer_allgather: plain peer stores and system-scope atomic adds over NVLink, a bounded
    wait, no NCCL kernel and no host synchronisation, so the calls can sit inside a captured CUDA graph).

    Two result buffers alternate.  A rank that runs ahead cannot overwrite a result a slower peer is still reading:
    before it may store into a buffer again it must have passed the rendezvous of the call in between, which needs that
    peer's arrival, which the peer sends only after -- in its own stream order -- the consumers of its earlier result
    were enqueued ahead of its next call.  A graph that is replayed must therefore hold an EVEN number of calls.
    """

    def __init__(self, rows: int, cols: int, group: dist.ProcessGroup | None = None, device=None, timeout_s: float = 2.0):
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.rows, self.cols = rows, cols
        self.timeout_ns = int(timeout_s * 1e9)
        dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.dev = dev
        data_elems = 2 * rows * cols
        pad = (-data_elems) % 8
        # one symmetric allocation: two fp16 result buffers, then two uint64 arrival counters (as four fp16 each)
        self._mem = symm.empty(data_elems + pad + 8, dtype=torch.float16, device=dev)
        self._mem.zero_()
        hdl = symm.rendezvous(self._mem, self.group.group_name)
        base = [int(p) for p in hdl.buffer_ptrs]
        self._data_ptrs = [[b + t * rows * cols * 2 for b in base] for t in range(2)]
        self._counter_ptrs = [[b + (data_elems + pad) * 2 + t * 8 for b in base] for t in range(2)]
        self._targets = torch.zeros(2, dtype=torch.int64, device=dev)   # advanced by the kernels
        self._turn = 0
        self.calls = 0
        torch.cuda.synchronize(dev)
        dist.barrier(group=self.group)   # every rank has zeroed its counters before anyone signals

    def buffer(self, turn: int, m: int, n: int) -> torch.Tensor:
        """The local result buffer of `turn` viewed as [m, n] (a view of the symmetric allocation)."""
        return self._mem[turn * self.rows * self.cols: turn * self.rows * self.cols + m * n].view(m, n)

    def next_turn(self) -> int:
        turn = self._turn
        self._turn ^= 1
        self.calls += 1
        return turn

    def _ptr_array(self, ptrs):
        import ctypes
        return (ctypes.c_void_p * self.world)(*ptrs)

    def signal_wait(self, turn: int) -> None:
        """Rendezvous on the current stream: everything this stream stored into the peers is visible to a rank once it
        has seen the arrival; returns (on the stream) when every rank has arrived."""
        from . import _capi
        with _capi.on_device(self.dev):
            _capi.check(_capi.lib().kfb_peer_signal_wait(self._ptr_array(self._counter_ptrs[turn]), self.world,
                                                         self._counter_ptrs[turn][self.rank], self._targets[turn:].data_ptr(),
                                                         self.timeout_ns, _capi.stream_ptr(self.dev)))

    def allgather_columns(self, y_local: torch.Tensor, bounds: list[tuple[int, int]]) -> torch.Tensor:
        """All-gather of column blocks: returns the full [M, N] as a view of this rank's buffer (valid until the call after
        the next one)."""
        from . import _capi
        m, w = y_local.shape
        n = bounds[-1][1]
        lo, hi = bounds[self.rank]
        if hi - lo != w or m * n > self.rows * self.cols:
            raise ValueError(f"block {tuple(y_local.shape)} does not match columns [{lo}, {hi}) or exceeds the buffer")
        if y_local.dtype != torch.float16 or not y_local.is_contiguous():
            y_local = y_local.to(torch.float16).contiguous()
        turn = self.next_turn()
        with _capi.on_device(self.dev):
            _capi.check(_capi.lib().kfb_peer_allgather(y_local.data_ptr(), self._ptr_array(self._data_ptrs[turn]),
                                                       self._ptr_array(self._counter_ptrs[turn]), self.world, m, w, n, lo,
                                                       self._counter_ptrs[turn][self.rank], self._targets[turn:].data_ptr(),
                                                       self.timeout_ns, _capi.stream_ptr(self.dev)))
        return self.buffer(turn, m, n)


class FusedShardedInt4Linear(torch.nn.Module):
    """Output-feature-parallel INT4 linear whose all-gather is fused into the GEMM epilogue.

    Every rank owns two result buffers [max_m, N] in symmetric memory (torch.distributed._symmetric_memory: each
    buffer is mapped into every process of the group).  `kfb_int4_gemm_allgather` stores this rank's column block into
    the current buffer of EVERY rank with plain peer stores over NVLink while the tiles are still being produced; a
    device-side rendezvous on the stream (PeerExchange.signal_wait: arrival counters in peer memory, bounded wait)
    then orders the ranks -- when it has passed, every rank's kernel, and with it every store into this rank's buffer,
    has completed.  No NCCL kernel and no host synchronisation are involved, so the call can be captured in a CUDA
    graph.  Only stores and atomic adds cross the link, never loads.

    Lifetime of the result: by default forward() returns a private copy.  With `alias=True` it returns a view of
    the symmetric buffer itself (no copy): that view is valid only until the next-but-one forward() of this
    module -- the peers then store the new result into the same memory -- and every consumer of it must be
    enqueued on the calling stream before that call.  Do not keep an aliased result in a list, across two calls,
    or read it from another stream.
    """

    def __init__(self, qw_full_shape: tuple[int, int], local: kq.QuantizedWeight, max_m: int,
                 bias: torch.Tensor | None = None, group: dist.ProcessGroup | None = None, alias: bool = False):
        super().__init__()
        self.alias = alias
        self.out_features, self.in_features = qw_full_shape
        self.group_size = local.group_size
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.bounds = row_bounds(self.out_features, self.world)
        self.max_m = max_m
        self.register_buffer("packed", local.packed)
        self.register_buffer("scales", local.scales)
        self.register_buffer("bias", None if bias is None else bias.detach().half())
        dev = local.packed.device
        self._xchg = PeerExchange(max_m, self.out_features, self.group, dev)
        from . import _capi
        lo, hi = self.bounds[self.rank]
        # split-K workspace for the largest call, allocated once
        ws_bytes = max(_capi.lib().kfb_int4_gemm_ws_bytes(m, hi - lo, self.in_features, self.group_size)
                       for m in {1, 16, 32, 64, 128, 256, max_m} if m <= max_m)
        self._ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)

    @classmethod
    def from_full(cls, qw: kq.QuantizedWeight, max_m: int, bias=None, group=None, alias: bool = False) -> "FusedShardedInt4Linear":
        g = group if group is not None else dist.group.WORLD
        return cls(qw.shape, shard_quantized_weight(qw, dist.get_rank(g), dist.get_world_size(g)), max_m, bias, g, alias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        import ctypes
        from . import _capi
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        m, k = x2.shape
        if m > self.max_m:
            raise ValueError(f"M={m} exceeds the symmetric buffers (max_m={self.max_m})")
        ops._check_int4(x2, self.packed, self.scales, self.group_size)
        lo, hi = self.bounds[self.rank]
        turn = self._xchg.next_turn()
        lib = _capi.lib()
        ws_bytes = lib.kfb_int4_gemm_ws_bytes(m, hi - lo, k, self.group_size)
        if ws_bytes > self._ws.numel():
            self._ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x2.device)
        ptrs = (ctypes.c_void_p * self.world)(*self._xchg._data_ptrs[turn])
        with _capi.on_device(x2.device):
            _capi.check(lib.kfb_int4_gemm_allgather(x2.data_ptr(), self.packed.data_ptr(), self.scales.data_ptr(), ptrs,
                                                    self.world, m, hi - lo, k, self.group_size, self.out_features, lo,
                                                    self._ws.data_ptr(), ws_bytes, _capi.stream_ptr(x2.device)))
        self._xchg.signal_wait(turn)   # device-side rendezvous: every rank's stores have landed
        y = self._xchg.buffer(turn, m, self.out_features)
        if self.bias is not None:
            y = y + self.bias          # a new tensor already
        elif not self.alias:
            y = y.clone()
        return y.reshape(*lead, self.out_features)
