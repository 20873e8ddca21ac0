"""ctypes binding of ``libnvfp4_b200.so`` (the C ABI declared in ``include/nvfp4_b200.h``)."""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int64, c_size_t, c_uint32, c_void_p

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libnvfp4_b200.so")

DT_BF16, DT_FP16, DT_FP32 = 0, 1, 2
_DTYPES = {torch.bfloat16: DT_BF16, torch.float16: DT_FP16, torch.float32: DT_FP32}

_lib = None

# name -> (restype, argtypes); the exported surface of include/nvfp4_b200.h
SIGNATURES = {
    "nvfp4_abi_version": (c_int, []),
    "nvfp4_last_error": (c_char_p, []),
    "nvfp4_pack": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                           c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p]),
    "nvfp4_pack_dual": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int, c_int64, c_int64, c_int64,
                                c_void_p, c_int, c_uint32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "nvfp4_vproj_pack": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int,
                                 c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                 c_void_p, c_void_p]),
    "nvfp4_pack_mx8_t": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int, c_int64, c_int64, c_int64, c_void_p,
                                 c_void_p, c_void_p, c_void_p]),
    "nvfp4_pack_qkv": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64,
                               c_int64, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                               c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "nvfp4_kv_append": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int64, c_int, c_int64,
                                c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64,
                                c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int64,
                                c_void_p]),
    "nvfp4_decode_plan": (c_int, [c_int64, c_int64, c_int, c_int, POINTER(c_int), POINTER(c_int64),
                                  POINTER(c_size_t)]),
    "nvfp4_decode": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                             c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int64,
                             c_int, c_int, c_int64, c_float, c_void_p, c_void_p, c_void_p, c_size_t,
                             c_int, c_int64, c_void_p, c_void_p]),
    "nvfp4_decode_hybrid": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                                    c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                    c_int, c_int, c_int64, c_float, c_void_p, c_void_p, c_void_p, c_size_t,
                                    c_int, c_int64, c_int, c_void_p, c_void_p]),
    "nvfp4_window_partials": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_int64,
                                      c_int, c_int, c_int64, c_int64, c_int64, c_float, c_int, c_void_p,
                                      c_int64, c_int64, c_void_p]),
    "nvfp4_decode_static_capacity": (c_size_t, []),
    "nvfp4_decode_static": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_int64, c_void_p,
                                    c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64,
                                    c_int64, c_int64, c_int, c_int, c_int64, c_float, c_void_p,
                                    c_void_p, c_int, c_int64, c_void_p, c_void_p]),
    "nvfp4_lse_merge": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64,
                                c_int, c_void_p]),
    "nvfp4_window_attention": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p,
                                       c_int64, c_int64, c_int, c_int, c_int64, c_int64, c_int64,
                                       c_float, c_void_p, c_void_p, c_void_p]),
    "nvfp4_rope_pack": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int, c_int64, c_int64, c_void_p, c_void_p,
                                c_void_p, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64,
                                c_void_p]),
    "nvfp4_bwd_prep": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p,
                               c_int64, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p,
                               c_void_p]),
    "nvfp4_bwd_hp": (c_int, [c_void_p] * 16 + [c_int, c_int64, c_int64, c_int64, c_int64, c_int64,
                             c_int, c_float, c_int, c_void_p, c_void_p]),
    "nvfp4_peak_probe": (c_int, [c_int, c_int, POINTER(ctypes.c_double), c_void_p, c_void_p, c_void_p]),
    "nvfp4_selftest_wait_timeout": (c_int, [c_int, ctypes.c_uint, c_void_p, c_void_p]),
    "nvfp4_bwd_fp4": (c_int, [c_void_p] * 23 + [c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                              c_int64, c_int, c_float, c_int, c_uint32, c_void_p, c_void_p]),
    "nvfp4_fwd": (c_int, [c_void_p] * 10 + [c_int, c_int64, c_int64, c_int64, c_void_p, c_int64,
                          c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_float, c_int,
                          c_void_p, c_void_p]),
}


def lib() -> ctypes.CDLL:
    """Load the CUDA library once; there is no fallback when it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m sageattention_b200.build` "
                "(needs nvcc with sm_100a support). There is no CPU or Triton fallback.")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name, None)
            if fn is None:
                raise RuntimeError(f"{LIB_PATH} does not export {name}; rebuild it with "
                                   "`python -m sageattention_b200.build -f`")
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(rc: int, what: str = "nvfp4") -> None:
    if rc != 0:
        msg = lib().nvfp4_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{what} failed (code {rc}): {msg}")


_entries: dict = {}


def call(name: str, device, *args) -> None:
    """Run the C entry ``name`` with ``device`` current and raise on a non-zero return.

    The C entries launch on the calling thread's current device (tensor maps, SM counts and the
    static scratch address are all per device), so every launch goes through this guard: a tensor
    on ``cuda:1`` is served correctly while ``cuda:0`` is current.  With ``NVFP4_CHECK_STATUS=1`` in
    the environment the device status word is read back (a synchronising read) after the call and
    an expired in-kernel wait raises instead of returning undefined tensors.
    """
    dev = device if isinstance(device, torch.device) else torch.device(device)
    if dev.type != "cuda":
        raise RuntimeError(f"{name}: operands must live on a CUDA device (got {dev})")
    fn = _entries.get(name)
    if fn is None:
        fn = _entries[name] = getattr(lib(), name)
    if dev.index is None or dev.index == torch.cuda.current_device():
        rc = fn(*args)                       # already current: skip the (slow) context manager
    else:
        with torch.cuda.device(dev):
            rc = fn(*args)
    check(rc, name)
    if os.environ.get("NVFP4_CHECK_STATUS", "0") == "1":
        st = read_status(dev)
        if st:
            raise RuntimeError(f"{name}: a bounded in-kernel wait expired (status 0x{st:x}: "
                               f"site {st & 0xFF}); outputs of this call are undefined")


def same_device(*tensors) -> torch.device:
    """The one CUDA device all given tensors (None entries skipped) live on."""
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(
                f"operands must be CUDA tensors: sageattention_b200 has no CPU path (got device {t.device})")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"operands live on different devices: {dev} and {t.device}")
    if dev is None:
        raise RuntimeError("no tensor operand")
    return dev


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPES[dt]
    except KeyError:
        raise TypeError(f"unsupported dtype {dt}; expected bfloat16, float16 or float32") from None


def require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(
            f"{name} must be a CUDA tensor: sageattention_b200 has no CPU path (got device {t.device})")


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


_status_words: dict = {}


def status_word(device) -> torch.Tensor:
    """Per-device int32 the kernels write when one of their bounded waits expires."""
    key = torch.device(device).index
    w = _status_words.get(key)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[key] = w
    return w


def read_status(device) -> int:
    """Synchronising read-and-clear of the device status word (for tests and debugging)."""
    w = status_word(device)
    v = int(w.item())
    if v:
        w.zero_()
    return v
