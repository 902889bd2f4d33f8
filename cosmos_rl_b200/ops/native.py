"""ctypes bridge to ``libb200rl.so`` (the sm_100a kernel library built from ``csrc/``).

The library exposes a plain C ABI (``csrc/api.h``): raw device pointers plus a stream. This module loads
it, declares the argument types, and offers small helpers to pass ``torch.Tensor`` arguments. On a machine
with a GPU a missing library is an error, never a silent fallback: :func:`lib` raises.
"""
from __future__ import annotations

import ctypes
import functools
import os
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parent / "libb200rl.so"

ST_NAMES = {
    0: "ok",
    1: "timeout waiting for a TMA stage (full barrier)",
    2: "timeout waiting for a free shared-memory stage (empty barrier)",
    3: "timeout waiting for a finished accumulator (tmem full)",
    4: "timeout waiting for a drained accumulator (tmem empty)",
    5: "timeout waiting for a peer flag",
    6: "bad argument",
}


class NativeError(RuntimeError):
    pass


class CopyDesc(ctypes.Structure):
    """Mirror of ``B200CopyDesc`` in ``csrc/api.h``."""

    _fields_ = [
        ("src", c_void_p),
        ("dst", c_void_p),
        ("dst_scale", c_void_p),
        ("src_ld", c_longlong),
        ("dst_ld", c_longlong),
        ("rows", c_int),
        ("cols", c_int),
        ("ld_scale", c_int),
        ("quant", c_int),
    ]


_SIGS = {
    "b200_gemm_bf16_nt": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong,
                          c_int, c_int, c_void_p, c_int, c_void_p],
    "b200_gemm_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong,
                       c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p],
    "b200_gemm_bf16_ex": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong,
                          c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p],
    "b200_gemm_skinny_splits": [c_int, c_int, c_int, c_int, c_int],
    "b200_gemm_skinny": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong,
                         c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p],
    "b200_splitk_reduce": [c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_longlong, c_void_p],
    "b200_splitk_reduce_residual_rmsnorm": [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p,
                                            c_void_p, c_void_p],
    "b200_splitk_reduce_qkv_rope_append": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p,
                                           c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "b200_lmhead_logprob_partial": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong,
                                    c_longlong, c_float, c_int, c_void_p, c_int, c_void_p],
    "b200_logprob_combine": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "b200_lmhead_dlogits": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                            c_int, c_int, c_longlong, c_longlong, c_int, c_int, c_longlong, c_float, c_void_p, c_int,
                            c_void_p],
    "b200_rmsnorm_fwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
    "b200_rmsnorm_bwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                         c_void_p],
    "b200_rmsnorm_bwd2": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int,
                          c_void_p],
    "b200_colsum_f32": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "b200_rope_inplace": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_float,
                          c_int, c_void_p],
    "b200_swiglu_fwd": [c_void_p, c_void_p, c_longlong, c_int, c_void_p],
    "b200_swiglu_bwd": [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_void_p],
    "b200_adamw": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_float, c_float, c_float,
                   c_float, c_float, c_float, c_float, c_void_p, c_void_p],
    "b200_sumsq": [c_void_p, c_int, c_longlong, c_void_p, c_void_p],
    "b200_clip_coef": [c_void_p, c_float, c_void_p, c_void_p, c_void_p],
    "b200_tp_gemm": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong,
                     c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_int, c_ulonglong,
                     c_void_p, c_int, c_void_p],
    "b200_flash_fwd": [c_void_p] * 7 + [c_int] * 6 + [c_longlong] * 4 + [c_int, c_int, c_float, c_void_p, c_void_p],
    "b200_flash_bwd": [c_void_p] * 12 + [c_int] * 6 + [c_longlong] * 7 + [c_int, c_int, c_float, c_void_p, c_void_p],
    "b200_gemm_fp8_block": [c_void_p] * 5 + [c_int] * 3 + [c_longlong] * 3 + [c_int, c_int, c_void_p, c_int, c_void_p],
    "b200_ag_gemm": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_void_p,
                     c_void_p, c_void_p, c_int, c_int, c_longlong, c_int, c_ulonglong, c_void_p, c_int, c_void_p],
    "b200_grpo_loss": [c_void_p] * 6 + [c_int, c_float, c_float, c_float, c_int, c_float, c_int, c_int, c_float,
                       c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "b200_sample": [c_void_p, c_int, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_ulonglong,
                    c_ulonglong, c_void_p, c_void_p, c_void_p, c_void_p],
    "b200_kv_append": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_int,
                       c_void_p],
    "b200_paged_decode": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                          c_int, c_int, c_int, c_float, c_void_p],
    "b200_kv_append_vt": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_int,
                          c_void_p],
    "b200_paged_decode_tc": [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                             c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_int, c_void_p],
    "b200_paged_decode_prefix_tc": [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                    c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_int, c_int,
                                    c_void_p, c_int, c_void_p],
    "b200_moe_route_topk": [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    "b200_moe_offsets": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "b200_moe_permute": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "b200_moe_scatter_scaled": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "b200_moe_combine": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "b200_moe_combine_dprob": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "b200_grouped_gemm": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_void_p,
                          c_void_p, c_int, c_int, c_void_p, c_int, c_void_p],
    "b200_grouped_wgrad": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong,
                           c_void_p, c_int, c_int, c_void_p, c_int, c_void_p],
    "b200_quant_mxfp4": [c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "b200_dequant_mxfp4": [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p],
    "b200_quant_fp8_block": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_void_p],
    "b200_reshard_pull": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p],
}


def available() -> bool:
    return _LIB_PATH.exists()


@functools.lru_cache(maxsize=1)
def lib() -> ctypes.CDLL:
    if not _LIB_PATH.exists():
        raise NativeError(
            f"{_LIB_PATH} is missing: build it with `python -m cosmos_rl_b200.ops.build` "
            "(CUDA tensors are never routed to a PyTorch fallback)")
    handle = ctypes.CDLL(str(_LIB_PATH), mode=ctypes.RTLD_GLOBAL)
    for name, args in _SIGS.items():
        if hasattr(handle, name):
            fn = getattr(handle, name)
            fn.argtypes = args
            fn.restype = c_int
    return handle


def ptr(t):
    """Device (or host) address of a tensor, ``None`` -> NULL."""
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


LAUNCHES = [0]  # launcher calls into libb200rl since import (CUDA-graph replays add their captured count)


def add_launches(n: int) -> None:
    LAUNCHES[0] += n


def check(rc: int, what: str) -> None:
    LAUNCHES[0] += 1
    if rc != 0:
        names = {-1: "bad argument", -2: "tensor map encode failed", -3: "kernel launch failed",
                 -4: "size beyond the supported maximum", -5: "CUDA runtime error"}
        detail = ""
        if rc == -2:
            try:
                e = lib().b200_last_tmap_error()
                detail = f" (reason {e >> 24}, site {(e >> 16) & 0xff}, CUresult {e & 0xffff})"
            except Exception:
                pass
        raise NativeError(f"{what}: {names.get(rc, rc)}{detail}")


@functools.lru_cache(maxsize=8)
def num_sms(device_index: int) -> int:
    return torch.cuda.get_device_properties(device_index).multi_processor_count


_status_words: dict = {}


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device uint32 status word that tensor-core kernels write on a bounded-wait timeout."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    w = _status_words.get(key)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[key] = w
    return w


def read_status(device: torch.device, reset: bool = True) -> int:
    """Synchronising read of the status word; raises if a kernel reported a timeout."""
    w = status_word(device)
    v = int(w.item())
    if v != 0:
        if reset:
            w.zero_()
        raise NativeError(f"kernel status {v}: {ST_NAMES.get(v, 'unknown')}")
    return v
