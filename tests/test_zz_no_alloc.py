"""kfb_flash_attn_decode_noalloc: decode attention for callers that cannot allocate device memory
(a server whose pool owns the GPU, code inside a stream capture, a runtime with no device allocator).

The split-KV scratch of this entry point is an array inside the library instead of a caller
workspace.  It must give the same output as kfb_flash_attn_fwd on the same inputs -- the kernels are
the same and the merge order is fixed, so the comparison is bit for bit, which is inside the 2e-3
tolerance the attention tests use -- on two calls in a row (the array keeps the first call's
contents), and refuse sizes beyond the array.  Collected last on purpose (file name)."""

import ctypes

import pytest
import torch

from helpers import ATTN_ATOL, attn_oracle, qkv_case
from kernelforge import _capi

pytestmark = pytest.mark.gpu


def _existing_entry(q, k, v, scale):
    lib = _capi.lib()
    b, h, _, d = q.shape
    hk, nk = k.shape[1], k.shape[2]
    o = torch.empty_like(q)
    ws_bytes = lib.kfb_flash_attn_ws_bytes(b, h, hk, 1, nk, d)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=q.device)
    _capi.check(lib.kfb_flash_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), _capi.dtype_code(q.dtype),
                                       b, h, hk, 1, nk, d, 1, scale, None, ws.data_ptr(), ws_bytes,
                                       _capi.stream_ptr(q.device)))
    return o, ws_bytes


def _noalloc_entry(q, k, v, scale):
    lib = _capi.lib()
    b, h, _, d = q.shape
    hk, nk = k.shape[1], k.shape[2]
    o = torch.full_like(q, float("nan"))
    _capi.check(lib.kfb_flash_attn_decode_noalloc(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                                                  _capi.dtype_code(q.dtype), b, h, hk, nk, d, scale, None,
                                                  _capi.stream_ptr(q.device)))
    return o


@pytest.mark.parametrize("b,h,hk,nk,d", [(1, 32, 4, 4096, 64), (2, 8, 2, 1000, 128)])
def test_noalloc_matches_workspace_entry_twice(b, h, hk, nk, d):
    scale = d ** -0.5
    first = None
    for call in range(2):  # second call runs on the array as the first one left it
        q, k, v = qkv_case(b, h, hk, 1, nk, d, torch.float16, seed=100 + call)
        qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
        want, ws_bytes = _existing_entry(qc, kc, vc, scale)
        assert ws_bytes > 0, "the case must exercise the split-KV scratch"
        got = _noalloc_entry(qc, kc, vc, scale)
        torch.cuda.synchronize()
        assert torch.isfinite(got).all()
        assert (got.float() - want.float()).abs().max().item() <= ATTN_ATOL[torch.float16]
        assert torch.equal(got, want)
        if call == 0:
            first = got.clone()
            ref = attn_oracle(q, k, v, True)
            assert abs(got.float().cpu().numpy() - ref).max() <= ATTN_ATOL[torch.float16]
    assert not torch.equal(first, got)  # the two calls really had different inputs


def test_noalloc_rejects_sizes_beyond_the_array():
    # 128 (batch, kv head) groups split 10 ways at D = 64: 1280 partials of 4224 bytes = 5.4 MB > the 4 MiB
    # array.  The refusal must come before any launch.
    lib = _capi.lib()
    b, h, hk, nk, d = 32, 32, 4, 16384, 64
    need = lib.kfb_flash_attn_ws_bytes(b, h, hk, 1, nk, d)
    if need <= (4 << 20):
        pytest.skip(f"plan needs only {need} bytes on this device")
    dummy = torch.zeros(16, dtype=torch.float16, device="cuda")
    rc = lib.kfb_flash_attn_decode_noalloc(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), 0,
                                           b, h, hk, nk, d, 0.1, None, None)
    assert rc == -4 and b"built-in array" in lib.kfb_last_error()
