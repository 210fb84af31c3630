"""The device status word: a bounded wait that runs out is reported, later launches return at once without writing,
and kfb_device_status_reset restores normal operation.  The wait that runs out is the library's own self-test (one
warp, an mbarrier nothing arrives on, a limit of 2 ms): the kernel returns normally, nothing faults or spins forever."""

import ctypes

import numpy as np
import pytest
import torch

from helpers import ATTN_ATOL, attn_oracle, qkv_case
from kernelforge import _capi, ops

pytestmark = pytest.mark.gpu


def test_expired_wait_is_reported_and_cleared():
    dev = torch.device("cuda", 0)
    lib = _capi.lib()
    assert _capi.device_status(dev) == 0
    outcome = torch.zeros(1, dtype=torch.int32, device=dev)
    try:
        with _capi.on_device(dev):
            _capi.check(lib.kfb_selftest_wait_expiry(2_000_000, outcome.data_ptr(), _capi.stream_ptr(dev)))
        torch.cuda.synchronize()
        assert int(outcome.item()) == 2, "the wait must give up, not complete"
        assert _capi.device_status(dev) == 0x601
        with pytest.raises(_capi.DeviceStatusError):
            _capi.raise_on_device_status(dev)
        # while the word is set, kernels with bounded waits return at once and leave their output alone
        q, k, v = qkv_case(1, 4, 4, 300, 300, 64, torch.float16, seed=3)
        qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
        o = torch.full_like(qc, 7.0)
        _capi.check(lib.kfb_flash_attn_fwd(qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), o.data_ptr(), 0, 1, 4, 4, 300, 300, 64,
                                           0, 0.125, None, None, 0, _capi.stream_ptr(dev)))
        torch.cuda.synchronize()
        assert bool((o == 7.0).all()), "a launch on a device with a non-zero status word must not write"
        assert _capi.device_status(dev) == 0x601   # the first code stays
    finally:
        _capi.device_status_reset(dev)
        torch.cuda.synchronize()
    assert _capi.device_status(dev) == 0
    out = ops.flash_attn(qc, kc, vc, causal=True)
    assert np.abs(out.float().cpu().numpy() - attn_oracle(q, k, v, True)).max() <= ATTN_ATOL[torch.float16]
    assert _capi.device_status(dev) == 0


def test_selftest_rejects_limits_out_of_range():
    dev = torch.device("cuda", 0)
    outcome = torch.zeros(1, dtype=torch.int32, device=dev)
    with pytest.raises(ValueError):
        _capi.check(_capi.lib().kfb_selftest_wait_expiry(10, outcome.data_ptr(), None))
    with pytest.raises(ValueError):
        _capi.check(_capi.lib().kfb_selftest_wait_expiry(10**10, outcome.data_ptr(), None))


def test_peer_wait_gives_up_when_an_arrival_never_comes():
    """kfb_peer_signal_wait on one GPU with its own counter as the only 'peer': one arrival comes (its own); with the
    target set ahead as if another rank were expected, the wait runs out after its limit (2 ms), records 0x801 and the
    kernel returns.  With the right target the same call passes at once."""
    dev = torch.device("cuda", 0)
    lib = _capi.lib()
    counter = torch.zeros(1, dtype=torch.int64, device=dev)
    target = torch.zeros(1, dtype=torch.int64, device=dev)
    ptrs = (ctypes.c_void_p * 1)(counter.data_ptr())
    with _capi.on_device(dev):
        _capi.check(lib.kfb_peer_signal_wait(ptrs, 1, counter.data_ptr(), target.data_ptr(), 2_000_000, _capi.stream_ptr(dev)))
    torch.cuda.synchronize()
    assert int(counter.item()) == 1 and int(target.item()) == 1 and _capi.device_status(dev) == 0
    target.fill_(5)   # as if four more arrivals were owed
    try:
        with _capi.on_device(dev):
            _capi.check(lib.kfb_peer_signal_wait(ptrs, 1, counter.data_ptr(), target.data_ptr(), 2_000_000, _capi.stream_ptr(dev)))
        torch.cuda.synchronize()
        assert _capi.device_status(dev) == 0x801
    finally:
        _capi.device_status_reset(dev)
        torch.cuda.synchronize()
    assert _capi.device_status(dev) == 0


def test_grid_barrier_of_the_persistent_step_gives_up():
    """The grid-wide barrier of the persistent decode step, through the library's self-test: 4 CTAs run one barrier that
    expects 5 arrivals, every wait runs out after its limit (2 ms), each CTA reports that it gave up, the status word
    holds 0x901, and after a reset the persistent step itself runs normally."""
    dev = torch.device("cuda", 0)
    lib = _capi.lib()
    assert _capi.device_status(dev) == 0
    outcome = torch.zeros(4, dtype=torch.int32, device=dev)
    scratch = torch.empty(1024, dtype=torch.uint8, device=dev)
    try:
        with _capi.on_device(dev):
            _capi.check(lib.kfb_selftest_grid_barrier_expiry(2_000_000, outcome.data_ptr(), scratch.data_ptr(), 1024, _capi.stream_ptr(dev)))
        torch.cuda.synchronize()
        assert outcome.tolist() == [2, 2, 2, 2], "every CTA must give the barrier up, none may pass it"
        assert _capi.device_status(dev) == 0x901
    finally:
        _capi.device_status_reset(dev)
        torch.cuda.synchronize()
    assert _capi.device_status(dev) == 0
