"""Two-GPU checks of the sharded INT4 linear: NCCL all-gather version and the version whose gather is fused into the
GEMM epilogue (peer stores into symmetric memory).  Skipped with fewer than two GPUs."""

import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT

pytestmark = pytest.mark.gpu


def _worker(rank, world, port):
    for p in (str(ROOT), str(ROOT / "kernel-forge_b200"), str(ROOT / "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from kernelforge import parallel as kp
        from kernelforge import quantize as kq
        from oracle import kf_oracle as ko
        dev = torch.device("cuda", rank)
        g = torch.Generator().manual_seed(0)
        for (n, k, ms) in ((1536, 1536, (128, 3)), (8960, 1536, (300,)), (200, 512, (16,))):
            w = torch.randn(n, k, generator=g) * 0.02
            qw_cpu = kq.quantize_weight(w, 128)
            qw = kq.QuantizedWeight(qw_cpu.packed.to(dev), qw_cpu.scales.to(dev), 128, qw_cpu.shape)
            plain = kp.ShardedInt4Linear.from_full(qw)
            fused = kp.FusedShardedInt4Linear.from_full(qw, max_m=max(ms))
            for m in ms:
                for rep in range(3):  # alternating buffers, repeated calls
                    x = torch.randn(m, k, generator=g).half()
                    ref = ko.int4_linear(x.numpy(), qw_cpu.packed.numpy(), qw_cpu.scales.numpy(), 128)
                    y_f = fused(x.to(dev)).float().cpu().numpy()
                    y_p = plain(x.to(dev)).float().cpu().numpy()
                    tol = 2e-3 * float(np.abs(ref).max())
                    assert np.abs(y_f - ref).max() <= tol, f"fused n{n} m{m} rep{rep}"
                    assert np.abs(y_p - ref).max() <= tol, f"nccl n{n} m{m} rep{rep}"
                    if m > 4:  # both paths then run the same GEMM kernel on the same shard
                        assert np.array_equal(y_f, y_p)
        # lifetime of the result: by default forward() returns a private copy, so a result kept across later calls (which
        # overwrite both symmetric buffers) does not change; with alias=True it is a view that the next-but-one call replaces
        keep = fused(torch.randn(16, 512, generator=g).half().to(dev))
        saved = keep.clone()
        for _ in range(3):
            fused(torch.randn(16, 512, generator=g).half().to(dev))
        torch.cuda.synchronize()
        assert torch.equal(keep, saved)
        # the peer-memory all-gather on its own (ragged column blocks), eagerly and replayed from a CUDA graph holding an
        # even number of calls (the two result buffers alternate)
        xchg = kp.PeerExchange(4, 1000, device=dev)
        bounds = kp.row_bounds(1000, world)          # 500 / 500
        rag = [(0, 333), (333, 1000)]                # ragged: not multiples of 8
        for bnd in (bounds, rag):
            lo, hi = bnd[rank]
            full_ref = torch.arange(4 * 1000, dtype=torch.float32).reshape(4, 1000).half()
            mine = full_ref[:, lo:hi].contiguous().to(dev)
            for _ in range(3):
                got = xchg.allgather_columns(mine, bnd)
                torch.cuda.synchronize()
                assert torch.equal(got.cpu(), full_ref)
        if xchg.calls % 2:
            xchg.allgather_columns(mine, rag)
        src = torch.zeros(4, 500, dtype=torch.float16, device=dev)
        side = torch.cuda.Stream(dev)
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                a = xchg.allgather_columns(src, bounds)
                a_copy = a.clone()
                b = xchg.allgather_columns(src + 1, bounds)
                b_copy = b.clone()
        for it in range(4):
            src.fill_(float(10 * it + rank))
            graph.replay()
            torch.cuda.synchronize()
            want = torch.cat([torch.full((4, 500), float(10 * it + r)) for r in range(world)], 1).half()
            assert torch.equal(a_copy.cpu(), want) and torch.equal(b_copy.cpu(), want + 1)
        # cross-GPU split-KV: a single sequence whose cache is split along the sequence over the two GPUs
        from helpers import attn_oracle, qkv_case
        q, k, v = qkv_case(1, 32, 4, 1, 8192, 64, torch.float16, seed=21)   # same seed on both ranks
        per = 8192 // world
        ks, vs = k[:, :, rank * per:(rank + 1) * per].contiguous().to(dev), v[:, :, rank * per:(rank + 1) * per].contiguous().to(dev)
        for total in (8192, per + 77, 100):
            out = kp.sequence_sharded_decode_attention(q.to(dev), ks, vs, total)
            ref = attn_oracle(q, k[:, :, :total], v[:, :, :total], True)
            assert np.abs(out.float().cpu().numpy() - ref).max() <= 2e-3, f"sequence-sharded decode, total {total}"
        from kernelforge import _capi
        assert _capi.device_status(dev) == 0
        torch.cuda.synchronize()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_linear_two_gpus():
    mp.spawn(_worker, args=(2, 29600 + os.getpid() % 1000), nprocs=2, join=True)


def _tp_decode_worker(rank, world, port):
    for p in (str(ROOT), str(ROOT / "kernel-forge_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=90))   # a failing rank must not keep the other waiting 10 minutes
    tp = None
    try:
        from test_llama_decode_gpu import build
        from kernelforge.llama_decode import LlamaInt4Decoder
        base, ref = build()                      # same seed on every rank: identical weights
        dev = torch.device("cuda", rank)
        batch, prompt_len, steps = 2, 24, 10
        ids = torch.randint(0, 320, (batch, prompt_len), generator=torch.Generator().manual_seed(3))
        tp = LlamaInt4Decoder.from_hf(base, dev, batch, max_len=64, tp_group=dist.group.WORLD)
        assert tp.h_loc == 2 and tp.hk_loc == 1 and tp.inter_loc == 256
        assert tp.pair_rows and tp.prepacked       # the rank's rows in pair order, on the fragment-order GEMV
        pre = tp.prefill(ids).float().cpu()
        toks, logs = tp.decode(steps, keep_logits=True)      # CUDA graph with the four all-gathers per layer captured
        torch.cuda.synchronize()
        full = torch.cat([ids, toks.cpu()], dim=1)
        with torch.no_grad():
            want = ref(full).logits
        scale = want.abs().max().item()
        assert (pre - want[:, :prompt_len]).abs().max().item() <= 2e-2 * scale
        assert (logs.float().cpu() - want[:, prompt_len:]).abs().max().item() <= 2e-2 * scale
        # every rank holds the same logits and therefore the same tokens
        mine = toks.to(dev).contiguous()
        both = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(both, mine)
        assert all(torch.equal(both[0], t) for t in both)
        # and they agree with the single-GPU decoder on the same weights (different kernel shapes: close, not bit-equal)
        single = LlamaInt4Decoder.from_hf(base, dev, batch, max_len=64)
        pre1 = single.prefill(ids).float().cpu()
        assert (pre1 - pre).abs().max().item() <= 5e-3 * scale
    finally:
        if tp is not None:
            tp.release()   # a live graph with captured all-gathers would make the teardown below wait forever
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tensor_parallel_decode_two_gpus():
    pytest.importorskip("transformers")
    mp.spawn(_tp_decode_worker, args=(2, 29700 + os.getpid() % 1000), nprocs=2, join=True)
