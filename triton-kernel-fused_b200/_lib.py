"""ctypes binding of libb200moe.so (the C ABI declared in include/b200moe.h).

The shared library is built in-tree by `build()` (make + nvcc, sm_100a only).  There is no
fallback: if the library is missing or a call fails, a Python exception is raised.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_HERE, "csrc")
LIB_PATH = os.path.join(_HERE, "libb200moe.so")

_lock = threading.Lock()
_lib = None

c_void_p, c_int, c_int64, c_float, c_size_t = (ctypes.c_void_p, ctypes.c_int, ctypes.c_int64,
                                              ctypes.c_float, ctypes.c_size_t)

# name -> (restype, argtypes); mirrors include/b200moe.h one to one
_SIGNATURES = {
    "b200moe_version": (ctypes.c_char_p, []),
    "b200moe_last_error_string": (ctypes.c_char_p, []),
    "b200moe_status_string": (ctypes.c_char_p, [c_int]),
    "b200moe_padded_rows_cap": (c_int64, [c_int64, c_int]),
    "b200moe_set_reserved_sms": (c_int, [c_int]),
    "b200moe_set_exchange_sms": (c_int, [c_int]),
    "b200moe_selftest_bounded_wait": (c_int, [c_void_p, c_int64, c_void_p]),
    "b200moe_router_topk_fwd": (c_int, [c_void_p, c_int, c_void_p, c_int64, c_int, c_int, c_int, c_float,
                                        c_void_p, c_void_p, c_void_p, c_void_p]),
    "b200moe_router_topk_bwd": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int, c_int, c_int,
                                        c_float, c_void_p, c_void_p]),
    "b200moe_router_bias_update": (c_int, [c_void_p, c_void_p, c_int, c_float, c_void_p]),
    "b200moe_conv_unfold": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "b200moe_conv_fold": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "b200moe_conv_gemm_fwd": (c_int, [c_void_p] * 3 + [c_int64] * 4 + [c_int, c_void_p, c_void_p]),
    "b200moe_conv_gemm_dx": (c_int, [c_void_p] * 3 + [c_int64] * 4 + [c_int, c_void_p, c_void_p]),
    "b200moe_conv_gemm_dw_splitk": (c_int, [c_void_p] * 3 + [c_int64] * 4 + [c_int, c_int64, c_void_p, c_void_p]),
    "b200moe_gemm_nt": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p]),
    "b200moe_gemm_nn": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p]),
    "b200moe_gemm_tn_splitk": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                       c_void_p, c_void_p]),
    "b200moe_splitk_reduce": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "b200moe_permute_ws_bytes": (c_size_t, [c_int64, c_int]),
    "b200moe_permute_build": (c_int, [c_void_p, c_int64, c_int, c_int] + [c_void_p] * 8 +
                              [c_void_p, c_size_t, c_void_p, c_void_p]),
    "b200moe_permute_build_static": (c_int, [c_void_p, c_int64, c_int, c_int] + [c_void_p] * 8 + [c_void_p, c_void_p]),
    "b200moe_gather_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p]),
    "b200moe_expert_gate_up_swiglu": (c_int, [c_void_p] * 4 + [c_int64, c_int, c_int64, c_int64] + [c_void_p] * 4),
    "b200moe_expert_gate_up_act": (c_int, [c_void_p] * 5 + [c_int64] * 3 + [c_int, c_int64, c_int64] + [c_void_p] * 4),
    "b200moe_expert_down_dgrad_act": (c_int, [c_void_p] * 6 + [c_int64] * 3 + [c_int, c_int64, c_int64] + [c_void_p] * 3),
    "b200moe_expert_linear": (c_int, [c_void_p] * 4 + [c_int64, c_int, c_int64, c_int64] + [c_void_p] * 3),
    "b200moe_expert_linear_t": (c_int, [c_void_p] * 4 + [c_int64, c_int, c_int64, c_int64] + [c_void_p] * 3),
    "b200moe_glu_fwd_rows": (c_int, [c_void_p] * 5 + [c_int64, c_int64, c_void_p, c_void_p]),
    "b200moe_glu_bwd_rows": (c_int, [c_void_p] * 6 + [c_int64, c_int64] + [c_void_p] * 4),
    "b200moe_expert_row_sums": (c_int, [c_void_p] * 3 + [c_int, c_void_p, c_void_p]),
    "b200moe_special_rows": (c_int, [c_void_p] * 4 + [c_int, c_int, c_int64, c_int64, c_void_p, c_void_p]),
    "b200moe_expert_down": (c_int, [c_void_p] * 4 + [c_int64, c_int, c_int64, c_int64] + [c_void_p] * 3),
    "b200moe_expert_down_dgrad_glu": (c_int, [c_void_p] * 5 + [c_int64, c_int, c_int64, c_int64] + [c_void_p] * 3),
    "b200moe_expert_gate_up_dgrad": (c_int, [c_void_p] * 4 + [c_int64, c_int, c_int64, c_int64] + [c_void_p] * 3),
    "b200moe_expert_wgrad": (c_int, [c_void_p] * 4 + [c_int64, c_int, c_int64, c_int64] + [c_void_p] * 3),
    "b200moe_mxfp8_sf_bytes": (c_size_t, [c_int64, c_int64]),
    "b200moe_mxfp8_quant_rows": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p]),
    "b200moe_mxfp8_quant_transpose": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p]),
    "b200moe_mxfp8_quant_both": (c_int, [c_void_p] + [c_int64] * 4 + [c_void_p] * 5),
    "b200moe_mxfp8_gemm_nt": (c_int, [c_void_p] * 5 + [c_int64] * 3 + [c_void_p, c_void_p]),
    "b200moe_mxfp8_expert_gemm": (c_int, [c_int] + [c_void_p] * 6 + [c_int64, c_int, c_int64, c_int64, c_int64] +
                                  [c_void_p] * 6),
    "b200moe_mxfp8_gather_quant_both": (c_int, [c_void_p] * 3 + [c_int, c_int64, c_int64] + [c_void_p] * 5),
    "b200moe_mxfp8_gather_quant": (c_int, [c_void_p] * 3 + [c_int, c_int64, c_int64] + [c_void_p] * 4),
    "b200moe_mxfp8_expert_wgrad": (c_int, [c_void_p] * 6 + [c_int64, c_int, c_int64, c_int64] + [c_void_p] * 3),
    "b200moe_ep_plan": (c_int, [c_void_p, c_int, c_int, c_int] + [c_void_p] * 5 + [c_int64, c_void_p, c_void_p]),
    "b200moe_ep_local_rows": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "b200moe_ep_publish": (c_int, [c_void_p] * 4 + [c_int64, c_int, c_int, c_int, c_int64, c_int] + [c_void_p] * 5),
    "b200moe_ep_barrier": (c_int, [c_void_p, c_int, c_int, ctypes.c_uint32, c_int64, c_void_p, c_void_p]),
    "b200moe_ep_gather_pull": (c_int, [c_void_p] * 7 + [c_int] * 6 + [c_int64, c_int, c_int64] + [c_void_p] * 4),
    "b200moe_slot_dots": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int64, c_void_p, c_void_p]),
    "b200moe_expert_linear_push": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int, c_int64, c_int64] +
                                   [c_void_p] * 5),
    "b200moe_ep_combine_pull": (c_int, [c_void_p] * 6 + [c_int, c_int, c_int64, c_int, c_int64] + [c_void_p] * 5),
    "b200moe_ep_combine_bwd_pull": (c_int, [c_void_p] * 9 + [c_int] * 6 + [c_int64, c_int, c_int64] + [c_void_p] * 3),
    "b200moe_combine": (c_int, [c_void_p] * 3 + [c_int64, c_int, c_int64, c_void_p, c_void_p]),
    "b200moe_combine_bwd": (c_int, [c_void_p] * 5 + [c_int, c_int64, c_int64, c_void_p, c_void_p, c_void_p]),
    "b200moe_muon_momentum": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_float, c_int, c_void_p]),
    "b200moe_muon_row_sumsq": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "b200moe_muon_prescale_rows": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_float, c_float, c_void_p, c_void_p,
                                           c_void_p]),
    "b200moe_muon_scale_rows": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p]),
    "b200moe_muon_update_rows": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_float, c_float, c_void_p, c_int, c_void_p]),
    "b200moe_muon_normalise_pack": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int, c_float,
                                            c_void_p, c_void_p, c_void_p]),
    "b200moe_expert_linear_axpby": (c_int, [c_void_p] * 3 + [c_float] * 3 + [c_int] + [c_void_p] * 2 +
                                    [c_int64, c_int, c_int64, c_int64] + [c_void_p] * 3),
    "b200moe_expert_gram": (c_int, [c_void_p] * 3 + [c_int64, c_int, c_int64, c_int] + [c_void_p] * 3),
    "b200moe_mirror_upper": (c_int, [c_void_p, c_int, c_int64, c_void_p]),
    "b200moe_axpby_bf16": (c_int, [c_void_p, c_float, c_void_p, c_float, c_float, c_int64, c_void_p, c_int64, c_void_p]),
    "b200moe_muon_apply": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int, c_float, c_float, c_float,
                                   c_void_p, c_int, c_void_p]),
}

EXPORTED = tuple(_SIGNATURES)

_ERRORS = {-1: ValueError, -2: ValueError, -3: ValueError, -4: ValueError, -5: RuntimeError, -6: ValueError}


def build(verbose: bool = False) -> str:
    """Compile libb200moe.so for sm_100a with nvcc (works without a GPU) and return its path."""
    cmd = ["make", "-C", _CSRC, "-j", str(min(8, os.cpu_count() or 1))]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        print(res.stdout[-4000:])
        print(res.stderr[-4000:])
    if res.returncode != 0 or not os.path.exists(LIB_PATH):
        raise RuntimeError("building libb200moe.so failed (see output above)")
    return LIB_PATH


def lib():
    """The loaded library; raises RuntimeError when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise RuntimeError(
                    f"{LIB_PATH} is missing: build it with `make -C {_CSRC}` (or __graft_entry__.build()); "
                    "this package has no fallback path")
            handle = ctypes.CDLL(LIB_PATH)
            for name, (res, args) in _SIGNATURES.items():
                fn = getattr(handle, name)
                fn.restype = res
                fn.argtypes = args
            _lib = handle
    return _lib


def check(rc: int) -> None:
    """Map a negative return code of the C ABI to ValueError / RuntimeError."""
    if rc == 0:
        return
    msg = lib().b200moe_last_error_string().decode()
    raise _ERRORS.get(rc, RuntimeError)(f"b200moe error {rc}: {msg}")


def ptr(t):
    return None if t is None else t.data_ptr()


def ptr_table(addresses):
    """Host array of device pointers (one per rank) for the `*_peers` arguments of the C ABI."""
    return (ctypes.c_void_p * len(addresses))(*[int(a) for a in addresses])


def stream_of(t: torch.Tensor):
    return torch.cuda.current_stream(t.device).cuda_stream


_status = {}


def status_word(device) -> torch.Tensor:
    """The per-device int32 word that kernels raise when a bounded wait ran out or an index was bad."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    t = _status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
        _status[key] = t
    return t


def check_status(device=None) -> None:
    """Synchronising read of the status word; raises RuntimeError (and clears it) when non-zero."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    w = status_word(dev)
    v = int(w.item())
    if v != 0:
        w.zero_()
    raise_for_status(v)


def raise_for_status(v: int) -> None:
    """RuntimeError for a non-zero value read from a status word (a bounded wait that ran out: a stalled GEMM
    pipeline, a peer rank missing at a barrier; an expert index out of range), with the library's text for it."""
    if v != 0:
        raise RuntimeError(f"b200moe kernel status {v}: {lib().b200moe_status_string(v).decode()}")


def padded_rows_cap(M: int, E: int) -> int:
    return int(lib().b200moe_padded_rows_cap(M, E))


def require(cond: bool, msg: str) -> None:
    if not cond:
        raise ValueError(msg)


def require_cuda_bf16(name: str, t: torch.Tensor) -> None:
    require(t.is_cuda, f"{name} must be a CUDA tensor (this package has no CPU path)")
    require(t.dtype == torch.bfloat16, f"{name} must be bfloat16, got {t.dtype}")
