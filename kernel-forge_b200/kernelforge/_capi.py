"""ctypes binding of libkfb200.so, the C-ABI library declared in include/kfb200.h.

Takes the place of the reference's pybind11 module `kernelforge._C` (csrc/bindings.cpp:12-28).
There is no fallback: if the library has not been built, the first kernel call raises
ImportError, exactly as the reference does for a missing `_C` (kernelforge/ops.py:23-28).
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p

import torch

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libkfb200.so")
_lib = None
_load_error: Exception | None = None

KFB_F16, KFB_BF16, KFB_F32 = 0, 1, 2
_DTYPE_CODE = {torch.float16: KFB_F16, torch.bfloat16: KFB_BF16, torch.float32: KFB_F32}



class DecodeStep(ctypes.Structure):
    """kfb_decode_step_t of include/kfb200.h."""
    _fields_ = [("layer_table", c_void_p),
                ("layers", c_int), ("batch", c_int), ("hidden", c_int), ("heads", c_int), ("kv_heads", c_int),
                ("head_dim", c_int), ("intermediate", c_int), ("vocab", c_int), ("max_len", c_int), ("group", c_int),
                ("rms_eps", c_float),
                ("embed", c_void_p), ("final_norm", c_void_p), ("lm_head", c_void_p), ("cos_table", c_void_p),
                ("sin_table", c_void_p), ("tok", c_void_p), ("pos", c_void_p), ("kv_len", c_void_p),
                ("logits", c_void_p), ("best", c_void_p), ("workspace", c_void_p), ("workspace_bytes", c_size_t)]


_SIGNATURES = {
    "kfb_version": (c_int, []),
    "kfb_last_error": (c_char_p, []),
    "kfb_device_status": (c_int, [ctypes.POINTER(ctypes.c_uint)]),
    "kfb_device_status_reset": (c_int, [c_void_p]),
    "kfb_set_programmatic_launch": (c_int, [c_int]),
    "kfb_selftest_wait_expiry": (c_int, [ctypes.c_ulonglong, c_void_p, c_void_p]),
    "kfb_quantize_pack": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "kfb_unpack_int4": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "kfb_pack_int4": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "kfb_dequantize": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p]),
    "kfb_int4_gemv": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "kfb_int4_gemv_fused": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float,
                                    c_void_p, c_void_p, c_int, c_void_p]),
    "kfb_int4_gemv_silu_pair": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float,
                                        c_int, c_void_p]),
    "kfb_int4_gemv_rope_kv": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "kfb_int4_prepack_bytes": (c_size_t, [c_int, c_int]),
    "kfb_int4_prepack": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "kfb_int4_gemv_prepacked": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                        c_void_p]),
    "kfb_int4_gemv_prepacked_silu_pair": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "kfb_int4_gemv_prepacked_rope_kv": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                                c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "kfb_int4_small_batch": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "kfb_int4_gemm_ws_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "kfb_int4_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_size_t,
                              c_void_p]),
    "kfb_int4_gemm_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_size_t,
                                   c_void_p]),
    "kfb_int4_gemm_allgather": (c_int, [c_void_p, c_void_p, c_void_p, ctypes.POINTER(c_void_p), c_int, c_int, c_int, c_int, c_int,
                                        c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "kfb_peer_signal_wait": (c_int, [ctypes.POINTER(c_void_p), c_int, c_void_p, c_void_p, ctypes.c_ulonglong, c_void_p]),
    "kfb_peer_allgather": (c_int, [c_void_p, ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p), c_int, c_int, c_int, c_int, c_int,
                                   c_void_p, c_void_p, ctypes.c_ulonglong, c_void_p]),
    "kfb_flash_attn_ws_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int, c_int]),
    "kfb_flash_attn_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                   c_int, c_int, c_float, ctypes.POINTER(c_int64), c_void_p, c_size_t, c_void_p]),
    "kfb_add_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p]),
    "kfb_rope_kv_write": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                  c_int, c_int, c_void_p]),
    "kfb_silu_mul": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "kfb_fp16_gemv_argmax": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "kfb_decode_finalize": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "kfb_embed_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p]),
    "kfb_selftest_grid_barrier_expiry": (c_int, [ctypes.c_ulonglong, c_void_p, c_void_p, c_size_t, c_void_p]),
    "kfb_decode_step_slice": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, ctypes.POINTER(c_int), ctypes.POINTER(c_int),
                                      ctypes.POINTER(c_int)]),
    "kfb_decode_step_ws_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int, c_int]),
    "kfb_decode_step_persistent": (c_int, [ctypes.POINTER(DecodeStep), c_void_p]),
    "kfb_flash_attn_decode_kvlen": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                            c_float, ctypes.POINTER(c_int64), c_void_p, c_void_p, c_size_t, c_void_p]),
    "kfb_flash_attn_decode_partial_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int, ctypes.POINTER(c_int)]),
    "kfb_flash_attn_decode_partial": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                              ctypes.POINTER(c_int64), c_void_p, c_void_p, c_size_t, c_void_p]),
    "kfb_flash_attn_merge_partials": (c_int, [c_void_p, c_int, c_size_t, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "kfb_flash_attn_decode_noalloc": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                              c_int, c_float, ctypes.POINTER(c_int64), c_void_p]),
}


def exported_symbols() -> tuple[str, ...]:
    """Every function include/kfb200.h declares."""
    return tuple(_SIGNATURES)


def lib() -> ctypes.CDLL:
    """Loads libkfb200.so on first use.  Raises ImportError when it is not built."""
    global _lib, _load_error
    if _lib is None:
        try:
            handle = ctypes.CDLL(_LIB_PATH)
            for name, (res, args) in _SIGNATURES.items():
                fn = getattr(handle, name)
                fn.restype, fn.argtypes = res, args
            _lib = handle
        except (OSError, AttributeError) as exc:
            _load_error = exc
            raise ImportError(
                f"libkfb200.so is not built or incomplete ({exc}). Run `python kernel-forge_b200/build.py`."
            ) from exc
    return _lib


def check(rc: int) -> None:
    """Turns a kfb_status into the exception type the reference raises for that class of error."""
    if rc == 0:
        return
    msg = lib().kfb_last_error().decode("utf-8", "replace")
    if rc in (-1, -2):  # invalid argument / alignment: std::invalid_argument -> ValueError in the reference
        raise ValueError(msg)
    raise RuntimeError(f"kfb200 error {rc}: {msg}")


def device_status(device: torch.device) -> int:
    """The device status word: 0 unless a bounded wait inside a kernel has expired (synchronises)."""
    out = ctypes.c_uint(0)
    with on_device(device):
        check(lib().kfb_device_status(ctypes.byref(out)))
    return int(out.value)


def device_status_reset(device: torch.device) -> None:
    """Clears the device status word (enqueued on the current stream of `device`)."""
    with on_device(device):
        check(lib().kfb_device_status_reset(stream_ptr(device)))


class DeviceStatusError(RuntimeError):
    """A bounded wait inside a kernel expired (or a kernel refused a device-side argument): every launch since
    then returned without writing its output."""


def raise_on_device_status(device: torch.device) -> None:
    """Synchronising check for host code at a natural sync point: raises DeviceStatusError when the status word of
    `device` is non-zero.  The word is left as it is; clear it with device_status_reset once the cause is known."""
    code = device_status(device)
    if code:
        raise DeviceStatusError(
            f"kfb200 device status 0x{code:x} on {device}: a kernel gave up a bounded wait or rejected a device-side "
            "argument; results enqueued since then are not valid (see kfb_device_status_reset in include/kfb200.h)")


class programmatic_launch:
    """Context manager: the kernels launched inside carry the programmatic-dependent-launch attribute
    (kfb_set_programmatic_launch).  Process-wide; restores the previous setting on exit."""

    def __init__(self, enable: bool = True):
        self.enable, self.prev = enable, 0

    def __enter__(self):
        self.prev = lib().kfb_set_programmatic_launch(1 if self.enable else 0)
        return self

    def __exit__(self, *exc):
        lib().kfb_set_programmatic_launch(self.prev)
        return False


def dtype_code(dtype: torch.dtype) -> int:
    return _DTYPE_CODE[dtype]


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


class on_device:
    """Makes `device` current for the duration of a library call (the C ABI launches on the current device)."""

    __slots__ = ("idx", "prev")

    def __init__(self, device: torch.device):
        self.idx = device.index if device.index is not None else torch.cuda.current_device()
        self.prev = -1

    def __enter__(self):
        cur = torch.cuda.current_device()
        if cur != self.idx:
            self.prev = cur
            torch.cuda.set_device(self.idx)
        return self

    def __exit__(self, *exc):
        if self.prev >= 0:
            torch.cuda.set_device(self.prev)
        return False
