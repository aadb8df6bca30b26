"""ctypes binding of libfat_b200.so (the C ABI declared in include/fat_b200.h).

The library is the only implementation: if it is missing or fails to load, every op raises.
There is no CPU or PyTorch fallback.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libfat_b200.so")

F32, BF16, F16, F64 = 0, 1, 2, 3
PATH_AUTO, PATH_SIMT, PATH_TENSOR, PATH_TENSOR_DETERMINISTIC = 0, 1, 2, 3
DTYPE_TAG = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16, torch.float64: F64}

_lock = threading.Lock()
_lib = None

_i64, _int, _dbl, _ptr, _sz = C.c_int64, C.c_int, C.c_double, C.c_void_p, C.c_size_t
_p64 = C.POINTER(C.c_int64)

# name -> (restype, argtypes); must list every symbol include/fat_b200.h declares
PROTOTYPES = {
    "fat_version": (_int, []),
    "fat_error_string": (C.c_char_p, [_int]),
    "fat_last_error": (C.c_char_p, []),
    "fat_launch_count": (C.c_ulonglong, []),
    "fat_swiglu_fwd": (_int, [_ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _int, _ptr]),
    "fat_swiglu_bwd": (_int, [_ptr] * 5 + [_i64] * 7 + [_int, _ptr]),
    "fat_norm_fwd": (_int, [_ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _dbl, _int, _ptr]),
    "fat_norm_bwd_workspace_bytes": (_sz, [_i64, _i64, _int]),
    "fat_norm_bwd": (_int, [_ptr] * 7 + [_sz] + [_i64] * 5 + [_dbl, _int, _ptr]),
    "fat_add_norm_fwd": (_int, [_ptr] * 6 + [_i64] * 6 + [_dbl, _int, _ptr]),
    "fat_add_norm_bwd": (_int, [_ptr] * 8 + [_sz] + [_i64] * 6 + [_dbl, _int, _ptr]),
    "fat_norm_bwd_static_capacity": (_sz, []),
    "fat_norm_bwd_static": (_int, [_ptr] * 6 + [_i64] * 5 + [_dbl, _int, _ptr]),
    "fat_shifted_ce_fwd": (_int, [_ptr] * 5 + [_int] * 3 + [_i64] * 5 + [_int, _ptr]),
    "fat_scale_unless_one": (_int, [_ptr, _i64, _ptr, _int, _ptr]),
    "fat_softmax_fwd": (_int, [_ptr, _ptr, _i64, _i64, _i64, _i64, _dbl, _int, _ptr]),
    "fat_softmax_bwd": (_int, [_ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _dbl, _int, _ptr]),
    "fat_attn_fwd": (_int, [_ptr] * 7 + [_int] * 4 + [_p64] * 4 + [_dbl, _dbl, _int, _int, _int, _ptr, _ptr]),
    "fat_attn_bwd_workspace_bytes": (_sz, [_int] * 6),
    "fat_attn_bwd": (_int, [_ptr] * 12 + [_sz] + [_int] * 4 + [_p64] * 8 + [_dbl, _dbl, _int, _int, _int, _ptr, _ptr]),
    "fat_attn_select_path": (_int, [_int] * 6),
    "fat_key_mask_words": (_int, [_int]),
    "fat_pack_key_mask": (_int, [_ptr, _ptr, _int, _int, _i64, _i64, _ptr]),
    "fat_attn_fwd_masked": (_int, [_ptr] * 8 + [_int] * 4 + [_p64] * 4 + [_dbl, _dbl, _int, _int, _int, _ptr, _ptr]),
    "fat_attn_bwd_masked": (_int, [_ptr] * 13 + [_sz] + [_int] * 4 + [_p64] * 8 + [_dbl, _dbl, _int, _int, _int, _ptr, _ptr]),
    "fat_attn_decode": (_int, [_ptr] * 8 + [_int] * 4 + [_p64] * 6 + [_dbl, _dbl, _int, _ptr, _ptr]),
}


def lib() -> C.CDLL:
    """The loaded library.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise RuntimeError(
                        f"{LIB_PATH} is missing: build it with `python -m fastalgebraictransformer_b200.build` "
                        "(nvcc, sm_100a).  This package has no fallback implementation.")
                handle = C.CDLL(LIB_PATH)
                for name, (res, args) in PROTOTYPES.items():
                    fn = getattr(handle, name)
                    fn.restype, fn.argtypes = res, args
                _lib = handle
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        l = lib()
        raise RuntimeError(f"libfat_b200: {l.fat_error_string(rc).decode()} — {l.fat_last_error().decode()}")


def dtype_tag(t: torch.Tensor) -> int:
    try:
        return DTYPE_TAG[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}") from None


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def strides3(t: torch.Tensor):
    """(batch, head, token) element strides of a [B,H,T,D] tensor as a C array."""
    return (C.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))


def device_status(device: torch.device) -> torch.Tensor:
    """The int32 status word the attention kernels of this device write (a bounded wait that ran out, an operand outside
    float16's range); owned by the operator library."""
    from . import ops  # noqa: F401  (loads the operator library on first use)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    return torch.ops.algebraic.device_status(idx)


def check_device_status(device=None) -> None:
    """Synchronise and raise if a kernel reported something on `device` (default: the current device) since the last check."""
    dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    word = device_status(torch.device("cuda", idx))
    v = int(word.item())
    if v:
        word.zero_()
        if v & 0x40000000:
            raise RuntimeError(f"libfat_b200: device {idx} status word 0x{v:08x}: the fused attention backward found its "
                               "dynamic shared memory not 1024-byte aligned and did nothing; request path 3 "
                               "(PATH_TENSOR_DETERMINISTIC) on this platform")
        if v & 0x20000000:
            raise RuntimeError(f"libfat_b200: device {idx} status word 0x{v:08x}: the tensor-core attention kernels met a magnitude "
                               "of 65536 or more in a bfloat16 tensor (v in the forward, q or k in the backward); they work on float16 "
                               "copies of those operands, which were clamped to 65504, so the results of this call are wrong; request "
                               "path 1 (PATH_SIMT) for tensors of that magnitude")
        if v & 0x10000000:
            raise RuntimeError(f"libfat_b200: device {idx} status word 0x{v:08x}: a decode step found a key/value cache without room "
                               "for the new row (or a negative length); nothing was appended and that sequence's output is zero")
        raise RuntimeError(f"libfat_b200: device {idx} status word 0x{v:08x} "
                           f"(code {(v >> 24) & 0xf}: a bounded wait inside a kernel ran out, detail {v & 0xffffff})")


class device_guard:
    """Make ``device`` current for the duration of a launch (no-op when it already is)."""

    def __init__(self, device: torch.device):
        self.idx = device.index
        self.prev = None

    def __enter__(self):
        if self.idx is not None and self.idx != torch.cuda.current_device():
            self.prev = torch.cuda.current_device()
            torch.cuda.set_device(self.idx)

    def __exit__(self, *exc):
        if self.prev is not None:
            torch.cuda.set_device(self.prev)
        return False
