"""ctypes binding of libomni_moe_b200.so (the C ABI declared in include/omni_moe_b200.h).

There is no fallback: if the library has not been built, or a call is rejected, an exception is
raised.  Build with ``python -m omni_moe_b200.build``.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libomni_moe_b200.so")

OMNI_F32, OMNI_BF16, OMNI_F16 = 0, 1, 2
ST_BAD_EXPERT_INDEX, ST_WAIT_TIMEOUT, ST_BAD_TOKEN_INDEX = 1, 2, 4

_DTYPE_CODE = {torch.float32: OMNI_F32, torch.bfloat16: OMNI_BF16, torch.float16: OMNI_F16}

# name -> (restype, argtypes); must list every symbol of the header
SIGNATURES = {
    "omni_version": (c_int, []),
    "omni_last_error": (c_char_p, []),
    "omni_router_topk": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_void_p, c_void_p, c_int,
                                 c_void_p, c_void_p]),
    "omni_router_logits_topk": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p,
                                        c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "omni_router_gate": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "omni_schedule_workspace_bytes": (c_size_t, [c_int64, c_int64]),
    "omni_schedule": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int64, c_int, c_int64, c_void_p, c_void_p, c_void_p,
                              c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "omni_schedule_static_max_pairs": (c_int64, []),
    "omni_schedule_static": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int64, c_int, c_int64, c_void_p, c_void_p,
                                     c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "omni_expert_coef": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int64,
                                 c_void_p, c_void_p, c_void_p]),
    "omni_expert_coef_hot_workspace": (c_int64, [c_int64, c_int]),
    "omni_expert_coef_hot": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int64,
                                     c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "omni_expert_combine": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int64, c_void_p, c_void_p,
                                    c_int, c_void_p, c_void_p]),
    "omni_expert_dots": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int64, c_void_p, c_void_p,
                                 c_void_p]),
    "omni_partition_keys": (c_int, [c_void_p, c_int64, c_int, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "omni_partition_records": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int64, c_int, c_int, c_int64,
                                       c_void_p, c_void_p]),
    "omni_expert_coef_pairs": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int,
                                       c_int64, c_void_p, c_void_p, c_void_p]),
    "omni_expert_combine_segments": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int64, c_void_p,
                                             c_void_p, c_int, c_void_p, c_void_p]),
    "omni_expert_fused": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int64,
                                  c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "omni_router_bwd": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "omni_expert_bwd_dots": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int,
                                     c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "omni_expert_bwd_dots_fuses_dx": (c_int, [c_int]),
    "omni_expert_bwd_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_int64, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_size_t,
                                     c_void_p, c_void_p]),
    "omni_expert_bwd_rows_scratch_bytes": (c_size_t, [c_int64, c_int]),
    "omni_gemm_bf16_nt": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_void_p]),
    "omni_transpose_bf16": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p]),
    "omni_swiglu_bwd": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "omni_mlp_gate_up_save": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "omni_gemm_bf16": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_void_p, c_int64,
                               c_void_p, c_void_p]),
    "omni_gemm_bf16_stacked_b": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64,
                                         c_void_p, c_int64, c_void_p, c_void_p]),
    "omni_mlp_gate_up_limit": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p,
                                       c_void_p]),
    "omni_swiglu_bwd_limit": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_float, c_void_p, c_void_p, c_void_p, c_int64, c_void_p,
                                      c_void_p]),
    "omni_router_bn_train_scratch_bytes": (c_size_t, [c_int64, c_int]),
    "omni_router_bn_train": (c_int, [c_void_p, c_int64, c_int64, c_int, c_float, c_float, c_float, c_float, c_void_p, c_void_p,
                                     c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t,
                                     c_void_p]),
    "omni_router_norm_bwd_scratch_bytes": (c_size_t, [c_int64, c_int]),
    "omni_router_norm_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int, c_int,
                                     c_int, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    "omni_selftest_wait_timeout": (c_int, [c_void_p, c_int, c_void_p]),
    "omni_expert_fused_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int64,
                                      c_void_p, c_void_p, c_void_p, c_void_p]),
    "omni_route_expert_fused": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                        c_int, c_int, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_void_p]),
    "omni_mlp_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p,
                             c_void_p, c_void_p, c_void_p]),
    "omni_mlp_gate_up": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "omni_mlp_gate_up_router": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int,
                                        c_void_p, c_void_p, c_void_p, c_void_p]),
    "omni_mlp_down": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library (once).  Raises if it is missing: there is no other code path."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} not found: the CUDA library has not been built "
                "(run `python -m omni_moe_b200.build`); omni_moe_b200 has no fallback path")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        msg = load().omni_last_error().decode()
        raise RuntimeError(f"libomni_moe_b200 rejected the call (code {rc}): {msg}")


def ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dt]
    except KeyError:
        raise TypeError(f"unsupported dtype {dt}") from None


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("omni_moe_b200 runs on CUDA tensors only (sm_100a); got a tensor on " + str(t.device))


def status_message(word: int) -> str:
    parts = []
    if word & ST_BAD_EXPERT_INDEX:
        parts.append("an expert index was outside [0, num_experts)")
    if word & ST_WAIT_TIMEOUT:
        parts.append("a bounded wait inside a kernel ran out (results are invalid)")
    if word & ST_BAD_TOKEN_INDEX:
        parts.append("a scheduled pair pointed outside the token range")
    return "; ".join(parts) or "ok"


def check_status(status: torch.Tensor) -> None:
    """Synchronises and raises if a kernel reported a device-side fault in ``status``."""
    word = int(status.item())
    if word:
        raise RuntimeError("omni_moe_b200 kernel status: " + status_message(word))


_DEVICE_STATUS: dict = {}


def device_status(device) -> torch.Tensor:
    """The int32 status word of ``device`` that the operator wrappers hand to every kernel they launch when the
    caller passes none: kernels OR fault bits into it (bad expert index, a bounded wait that ran out) and
    never clear it, so one word per device collects everything since the last :func:`check_device_status`.
    Allocated once per device (no fill kernel per call)."""
    dev = torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    st = _DEVICE_STATUS.get(key)
    if st is None:
        st = torch.zeros(1, device=torch.device("cuda", key), dtype=torch.int32)
        _DEVICE_STATUS[key] = st
    return st


def check_device_status(device=None) -> None:
    """Synchronises and raises if any kernel launched through the operator wrappers on ``device`` (default:
    every device used so far) reported a fault; the word is cleared afterwards."""
    keys = list(_DEVICE_STATUS) if device is None else [torch.device(device).index or 0]
    for key in keys:
        st = _DEVICE_STATUS.get(key)
        if st is None:
            continue
        word = int(st.item())
        if word:
            st.zero_()
            raise RuntimeError("omni_moe_b200 kernel status: " + status_message(word))
