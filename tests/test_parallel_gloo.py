"""The N > 1 path on CPU: two gloo ranks run the sharding / gather logic of kernelforge.parallel.  The local
compute is replaced by the oracle (CPU ranks cannot launch the kernels); what is tested is the host side: row
bounds, shard slicing, the all-gather reassembly (equal and ragged blocks) and head-parallel attention shards."""

import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _oracle_matmul(x, packed, scales, group):
    from oracle import kf_oracle as ko
    y = ko.int4_linear(x.numpy(), packed.numpy(), scales.numpy(), group)
    return torch.from_numpy(y.astype(np.float16))


def _worker(rank, world, port, n):
    for p in (str(ROOT), str(ROOT / "kernel-forge_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from kernelforge import parallel as kp
        from kernelforge import quantize as kq
        from oracle import kf_oracle as ko
        g = torch.Generator().manual_seed(0)
        w = torch.randn(n, 256, generator=g) * 0.02
        x = torch.randn(3, 256, generator=g).half()
        qw = kq.quantize_weight(w, 128)
        lin = kp.ShardedInt4Linear.from_full(qw, bias=torch.arange(n).float() / n, matmul=_oracle_matmul)
        lo, hi = kp.row_bounds(n, world)[rank]
        assert lin.packed.shape[0] == hi - lo and torch.equal(lin.packed, qw.packed[lo:hi])
        y = lin(x.reshape(1, 3, 256))
        ref = ko.int4_linear(x.numpy(), qw.packed.numpy(), qw.scales.numpy(), 128).astype(np.float16)
        want = torch.from_numpy(ref) + (torch.arange(n).float() / n).half()
        assert y.shape == (1, 3, n)
        assert torch.equal(y.reshape(3, n), want), "gathered result differs from the unsharded computation"
        # head-parallel attention shards: concatenating per-rank oracle outputs reproduces the full result
        q = torch.randn(1, 8, 5, 64, generator=g).half()
        k = torch.randn(1, 2, 9, 64, generator=g).half()
        v = torch.randn(1, 2, 9, 64, generator=g).half()
        ql, kl, vl = kp.shard_attention_heads(q, k, v, rank, world)
        o_local = torch.from_numpy(ko.attention(ql.numpy(), kl.numpy(), vl.numpy(), True))
        parts = [torch.empty_like(o_local) for _ in range(world)]
        dist.all_gather(parts, o_local)
        full = torch.from_numpy(ko.attention(q.numpy(), k.numpy(), v.numpy(), True))
        assert torch.allclose(torch.cat(parts, dim=1), full, atol=1e-6)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n", [64, 129])  # equal blocks / ragged blocks
def test_two_gloo_ranks(n):
    port = 29500 + (os.getpid() % 2000) + n
    mp.spawn(_worker, args=(2, port, n), nprocs=2, join=True)


def test_row_bounds_and_head_shards():
    from kernelforge import parallel as kp
    assert kp.row_bounds(8960, 8) == [(i * 1120, (i + 1) * 1120) for i in range(8)]
    assert kp.row_bounds(10, 4) == [(0, 3), (3, 6), (6, 8), (8, 10)]
    q = torch.zeros(1, 32, 1, 64); k = torch.zeros(1, 4, 7, 64)
    for world in (2, 4, 8):
        heads = [kp.shard_attention_heads(q, k, k, r, world) for r in range(world)]
        assert sum(t[0].shape[1] for t in heads) == 32
        assert all(t[0].shape[1] % t[1].shape[1] == 0 for t in heads)
    with pytest.raises(ValueError, match="KV group"):
        kp.shard_attention_heads(q, k, k, 0, 3)


def test_tensor_parallel_plan_partitions_heads_rows_and_features():
    """Ownership ranges of the tensor-parallel decoder: contiguous, in rank order, covering everything once; a KV head
    is replicated only when there are more ranks than KV heads."""
    from kernelforge.llama_decode import TINYLLAMA_1B, LlamaShape, tp_plan
    for shape in (TINYLLAMA_1B, LlamaShape(hidden=1536, heads=12, kv_heads=2, head_dim=128, intermediate=8960)):
        for world in (1, 2, 4, 8):
            if shape.heads % world or (shape.kv_heads % world and world % shape.kv_heads):
                continue
            plans = [tp_plan(shape, r, world) for r in range(world)]
            for key, total in (("q_heads", shape.heads), ("hidden_rows", shape.hidden), ("inter", shape.intermediate)):
                assert plans[0][key][0] == 0 and plans[-1][key][1] == total
                assert all(plans[r][key][1] == plans[r + 1][key][0] for r in range(world - 1))
            g = shape.heads // shape.kv_heads
            for p in plans:   # every query head of a rank reads one of the rank's KV heads
                assert p["kv_heads"][0] * g <= p["q_heads"][0] and p["q_heads"][1] <= p["kv_heads"][1] * g
            width = (plans[0]["q_heads"][1] - plans[0]["q_heads"][0]) * shape.head_dim
            assert plans[0]["attn_bounds"] == [(r * width, (r + 1) * width) for r in range(world)]
    import pytest
    with pytest.raises(ValueError, match="cannot split"):
        tp_plan(LlamaShape(heads=12, kv_heads=4), 0, 8)


class _HostPeerModel:
    """Host-side model of the device rendezvous protocol (kfb_peer_signal_wait / kfb_peer_allgather): per turn one arrival
    counter per rank and one target per rank; a rank signals every peer (gloo all-reduce of its increments stands in
    for the atomic adds over NVLink), then polls its own counter with a time limit.  Mirrors parallel.PeerExchange:
    alternating turns, target += expected_arrivals(world, ctas)."""

    def __init__(self, world, rank, ctas=1):
        from kernelforge import parallel as kp
        self.world, self.rank, self.inc = world, rank, kp.expected_arrivals(world, ctas)
        self.ctas = ctas
        self.counter = [0, 0]
        self.target = [0, 0]
        self.turn = 0
        self.status = 0

    def call(self, drop_signal_from=None):
        turn, self.turn = self.turn, self.turn ^ 1
        sent = torch.zeros(self.world, dtype=torch.int64)            # arrivals this rank adds to each peer's counter
        if drop_signal_from != self.rank:
            sent += self.ctas
        dist.all_reduce(sent)                                        # sent[r] = what rank r receives in total
        self.counter[turn] += int(sent[self.rank])
        self.target[turn] += self.inc
        if self.counter[turn] < self.target[turn]:                   # the bounded wait ran out
            self.status = self.status or 0x801
            return False
        return True


def _peer_protocol_worker(rank, world, port):
    for p in (str(ROOT), str(ROOT / "kernel-forge_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        for ctas in (1, 8):
            m = _HostPeerModel(world, rank, ctas)
            for _ in range(6):                                       # both buffers, several rounds: targets stay in step
                assert m.call()
            assert m.counter == m.target == [3 * world * ctas, 3 * world * ctas] and m.status == 0
            # a rank that never signals: every rank's wait for that call gives up and the status code is recorded,
            # nothing waits forever; the shortfall is permanent for that turn (the host must reset), the other turn is fine
            assert not m.call(drop_signal_from=1)
            assert m.status == 0x801
            assert m.call()            # the other turn's counter is unaffected
            assert not m.call()        # the turn that lost an arrival stays short
    finally:
        dist.destroy_process_group()


def test_peer_rendezvous_protocol_on_gloo_ranks():
    port = 31500 + (os.getpid() % 2000)
    mp.spawn(_peer_protocol_worker, args=(2, port), nprocs=2, join=True)
