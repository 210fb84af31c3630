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
    for p in (str(ROOT), str(ROOT / "kernel-forge_b200")):
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
        torch.cuda.synchronize()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_linear_two_gpus():
    mp.spawn(_worker, args=(2, 29600 + os.getpid() % 1000), nprocs=2, join=True)
