"""ctypes binding of ``liboal_b200.so`` (the C ABI declared in include/oal_b200.h).

There is no CPU fallback and no alternative backend: if the CUDA library is
missing, importing the symbols raises, and so does every operator call.
"""

from __future__ import annotations

import ctypes
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "liboal_b200.so"

HEAD_DIM = 64
MAX_GROUPS = 16
E_PAD = 80

DTYPE_CODES = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
PRECISION_CODES = {"fp32_ieee": 0, "bf16_tensorcore": 1}

GRAD_Q, GRAD_K, GRAD_V, GRAD_COEF, GRAD_REUSE_STATE_STAGE = 1, 2, 4, 8, 16
STATE_ROWS = 2432
FLAG_OUT_TOKEN_MAJOR = 1
STATUS_NONFINITE, STATUS_DENOMINATOR, STATUS_WAIT_TIMEOUT, STATUS_BAD_LAYOUT = 1, 2, 4, 8

# every symbol include/oal_b200.h declares
EXPORTED_SYMBOLS = (
    "oal_workspace_bytes",
    "oal_forward",
    "oal_backward",
    "oal_last_error_string",
    "oal_version_string",
    "oal_selftest_umma",
    "oal_selftest_wait_timeout",
    "oal_launch_count",
    "oal_profile_enable",
    "oal_profile_report",
    "oal_set_overlap",
    "oal_status_defer",
    "oal_status_poll",
    "oal_expand_factor",
    "oal_expand_factor_grad",
    "oal_forward_static_scratch",
    "oal_forward_local_state",
    "oal_backward_local_state",
    "oal_rope_pack",
    "oal_rope_unpack_grad",
)


class OalProblem(ctypes.Structure):
    _fields_ = [
        ("batch", ctypes.c_int32),
        ("q_heads", ctypes.c_int32),
        ("kv_heads", ctypes.c_int32),
        ("seq_len", ctypes.c_int32),
        ("head_dim", ctypes.c_int32),
        ("value_dim", ctypes.c_int32),
        ("groups", ctypes.c_int32),
        ("chunk", ctypes.c_int32),
        ("io_dtype", ctypes.c_int32),
        ("out_dtype", ctypes.c_int32),
        ("precision", ctypes.c_int32),
        ("grad_mask", ctypes.c_int32),
        ("scale", ctypes.c_float),
        ("floor", ctypes.c_float),
        ("flags", ctypes.c_int32),
    ]


_lib = None


def load() -> ctypes.CDLL:
    """Load the CUDA library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m oal_b200.build` "
            "(oal_b200 has no CPU or library fallback)")
    lib = ctypes.CDLL(str(LIB_PATH))
    vp, i32p, f32p = ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p
    pp = ctypes.POINTER(OalProblem)
    lib.oal_workspace_bytes.argtypes = [pp, ctypes.c_int]
    lib.oal_workspace_bytes.restype = ctypes.c_int64
    lib.oal_forward.argtypes = [pp, vp, vp, vp, i32p, i32p, f32p, f32p, f32p, vp, f32p, f32p, vp, f32p,
                                vp, ctypes.c_size_t, i32p, vp]
    lib.oal_forward.restype = ctypes.c_int
    lib.oal_forward_static_scratch.argtypes = [pp, vp, vp, vp, i32p, i32p, f32p, f32p, f32p, vp, f32p, f32p, vp,
                                               i32p, vp]
    lib.oal_forward_static_scratch.restype = ctypes.c_int
    lib.oal_forward_local_state.argtypes = [pp, vp, vp, f32p, vp, ctypes.c_size_t, i32p, vp]
    lib.oal_forward_local_state.restype = ctypes.c_int
    lib.oal_backward_local_state.argtypes = [pp, vp, i32p, i32p, f32p, f32p, f32p, f32p, f32p, vp, vp, f32p, f32p,
                                             f32p, vp, ctypes.c_size_t, i32p, vp]
    lib.oal_backward_local_state.restype = ctypes.c_int
    lib.oal_backward.argtypes = [pp, vp, vp, vp, i32p, i32p, f32p, f32p, f32p, f32p, f32p, vp, vp, f32p,
                                 f32p, vp, vp, vp, f32p, f32p, f32p, f32p, vp, ctypes.c_size_t, i32p, vp]
    lib.oal_backward.restype = ctypes.c_int
    ci = ctypes.c_int
    lib.oal_rope_pack.argtypes = [vp, vp, vp, f32p, f32p, vp, vp, vp, ci, ci, ci, ci, vp]
    lib.oal_rope_pack.restype = ctypes.c_int
    lib.oal_rope_unpack_grad.argtypes = [vp, vp, vp, f32p, f32p, vp, vp, vp, ci, ci, ci, ci, vp]
    lib.oal_rope_unpack_grad.restype = ctypes.c_int
    lib.oal_selftest_umma.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, vp, vp, f32p, i32p, vp]
    lib.oal_selftest_umma.restype = ctypes.c_int
    lib.oal_selftest_wait_timeout.argtypes = [ctypes.c_int64, i32p, vp]
    lib.oal_selftest_wait_timeout.restype = ctypes.c_int
    lib.oal_launch_count.restype = ctypes.c_int64
    lib.oal_profile_enable.argtypes = [ctypes.c_int]
    lib.oal_profile_enable.restype = None
    lib.oal_set_overlap.argtypes = [ctypes.c_int]
    lib.oal_set_overlap.restype = None
    lib.oal_status_defer.argtypes = [i32p, vp, ctypes.POINTER(ctypes.c_int64)]
    lib.oal_status_defer.restype = ctypes.c_int
    lib.oal_status_poll.argtypes = [ctypes.c_int64, ctypes.c_int, ctypes.POINTER(ctypes.c_int32)]
    lib.oal_status_poll.restype = ctypes.c_int
    lib.oal_expand_factor.argtypes = [f32p, ci, ci, ci, ctypes.c_float, f32p, f32p, f32p, vp]
    lib.oal_expand_factor.restype = ctypes.c_int
    lib.oal_expand_factor_grad.argtypes = [f32p, ci, ci, ci, f32p, f32p, f32p, f32p, vp]
    lib.oal_expand_factor_grad.restype = ctypes.c_int
    lib.oal_profile_report.argtypes = [ctypes.c_char_p, ctypes.c_size_t]
    lib.oal_profile_report.restype = ctypes.c_int
    lib.oal_last_error_string.restype = ctypes.c_char_p
    lib.oal_version_string.restype = ctypes.c_char_p
    _lib = lib
    return lib


def ptr(t: torch.Tensor | None):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def device_guard(t: torch.Tensor):
    """Context manager that makes ``t``'s CUDA device current for the duration of a library call.

    The kernels launch on the calling thread's current device while the stream that is passed in
    belongs to the tensors' device; the reference is plain torch code and follows the tensors, so
    every entry into the library goes through this guard."""
    return torch.cuda.device(t.device)


def check(rc: int) -> None:
    """Map a negative return code to the exception type the reference raises."""
    if rc >= 0:
        return
    msg = load().oal_last_error_string().decode()
    if rc == -2:
        raise TypeError(msg)
    if rc in (-1, -3):
        raise ValueError(msg)
    raise RuntimeError(msg)


def workspace_bytes(problem: OalProblem, phase: int) -> int:
    n = load().oal_workspace_bytes(ctypes.byref(problem), phase)
    check(n)
    return int(n)


def launch_count() -> int:
    """Kernels launched by the library in this process so far."""
    return int(load().oal_launch_count())


def profile_enable(on: bool) -> None:
    """Per-kernel event timing; while it is on, the library's side streams are off so that every kernel
    runs alone and its time means something."""
    load().oal_set_overlap(0 if on else 1)
    load().oal_profile_enable(1 if on else 0)


def profile_report() -> dict:
    """{"kernel name": [launches, total milliseconds]} since the last report (synchronises)."""
    import json

    buf = ctypes.create_string_buffer(8192)
    check(load().oal_profile_report(buf, len(buf)))
    return json.loads(buf.value.decode())
