"""ctypes binding of libkda_b200.so (the C ABI declared in include/kda_b200.h).

There is no fallback: if the library is missing or a call returns an error code, the caller
gets an exception.  Tensors cross the boundary as raw device pointers plus sizes; the stream
is torch's current CUDA stream.
"""

from __future__ import annotations

import contextlib
import ctypes
import os
from ctypes import c_float, c_int, c_int64, c_void_p

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libkda_b200.so")

KDA_F32, KDA_BF16, KDA_F16 = 0, 1, 2
_DTYPES = {torch.float32: KDA_F32, torch.bfloat16: KDA_BF16, torch.float16: KDA_F16}
_ERRORS = {-1: "invalid argument", -2: "unsupported shape", -3: "CUDA launch failed",
           -4: "problem exceeds the built-in scratch array"}

# kernels launched through this module since import (bench.py reports it as gpu_launches)
launch_count = 0

_SIGNATURES = {
    "kda_b200_version": (c_int, []),
    "kda_device_error_word": (c_int, []),
    "kda_selftest_bounded_wait": (c_int, [c_int, c_void_p]),
    "kda_stage_count": (c_int, []),
    "kda_stage_name": (ctypes.c_char_p, [c_int]),
    "kda_stage_timing_enable": (c_int, [c_int]),
    "kda_stage_timing_read": (c_int, [c_void_p, c_void_p, c_int]),
    "kda_prepare_chunk_offsets": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "kda_recurrent_fwd": (c_int, [c_void_p] * 5 + [c_int] * 5 + [c_void_p, c_void_p, c_void_p, c_int,
                                  c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int,
                                  c_int, c_float, c_void_p]),
    "kda_gate_cumsum_fwd": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int64,
                                    c_void_p]),
    "kda_gate_bwd_reduce": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "kda_gate_bwd_partial_rows": (c_int64, [c_int64]),
    "kda_gate_cumsum_bwd": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                    c_int, c_float, c_int64, c_void_p]),
    "kda_l2norm_fwd": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int, c_float, c_void_p]),
    "kda_l2norm_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int, c_void_p]),
    "kda_output_gate_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int, c_float, c_void_p]),
    "kda_output_gate_bwd_partial_rows": (c_int64, [c_int64]),
    "kda_output_gate_bwd": (c_int, [c_void_p] * 4 + [c_int] + [c_void_p] * 3 + [c_int64, c_int, c_float, c_void_p]),
    "kda_chunk_fwd_workspace_bytes": (c_int64, [c_int64, c_int]),
    "kda_chunk_fwd": (c_int, [c_void_p] * 12 + [c_int, c_int64, c_int, c_int, c_int, c_int, c_void_p,
                              c_int64, c_void_p]),
    "kda_chunk_fwd_save": (c_int, [c_void_p] * 12 + [c_int, c_int64, c_int, c_int, c_int, c_int,
                                   c_void_p, c_int64, c_void_p]),
    "kda_chunk_fwd_qknorm": (c_int, [c_void_p] * 12 + [c_float, c_void_p, c_void_p, c_int, c_int64, c_int,
                                     c_int, c_int, c_int, c_void_p, c_int64, c_int, c_void_p]),
    "kda_chunk_bwd_qknorm_saved": (c_int, [c_void_p] * 18 + [c_int, c_int64, c_int, c_int, c_int, c_int,
                                           c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "kda_chunk_fwd_noalloc": (c_int, [c_void_p] * 12 + [c_int, c_int64, c_int, c_int, c_int, c_int,
                                      c_void_p]),
    "kda_chunk_fwd_dense_workspace_bytes": (c_int64, [c_int, c_int64, c_int, c_int]),
    "kda_chunk_fwd_dense": (c_int, [c_void_p] * 10 + [c_int, c_int64, c_int, c_int, c_int, c_void_p,
                                    c_int64, c_void_p]),
    "kda_chunk_fwd_dense_save": (c_int, [c_void_p] * 10 + [c_int, c_int64, c_int, c_int, c_int,
                                         c_void_p, c_int64, c_void_p]),
    "kda_set_row_segments": (c_int, [c_int]),
    "kda_chunk_bwd_workspace_bytes": (c_int64, [c_int64, c_int, c_int64]),
    "kda_chunk_bwd": (c_int, [c_void_p] * 18 + [c_int, c_int64, c_int, c_int, c_int, c_int, c_void_p,
                              c_int64, c_void_p]),
    "kda_chunk_bwd_saved": (c_int, [c_void_p] * 18 + [c_int, c_int64, c_int, c_int, c_int, c_int,
                                    c_void_p, c_int64, c_void_p]),
    "kda_chunk_bwd_state_saved": (c_int, [c_void_p] * 7 + [c_int, c_int64, c_int, c_int, c_int, c_int,
                                          c_void_p, c_int64, c_void_p]),
    "kda_chunk_fwd_prepare": (c_int, [c_void_p] * 9 + [c_int, c_int64, c_int, c_int, c_void_p,
                                      c_int64, c_void_p]),
    "kda_chunk_fwd_state": (c_int, [c_void_p] * 7 + [c_int, c_int64, c_int, c_void_p, c_int,
                                    c_void_p, c_void_p]),
    "kda_chunk_slice_map": (c_int, [c_void_p] * 8 + [c_int, c_int64, c_int, c_void_p, c_void_p]),
    "kda_set_state_value_split": (c_int, [c_int]),
    "kda_state_affine": (c_int, [c_void_p] * 4 + [c_int, c_int, c_int, c_void_p]),
    "kda_conv1d_fwd": (c_int, [c_void_p] * 4 + [c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                               c_int, c_void_p]),
    "kda_conv1d_bwd_blocks": (c_int64, [c_int, c_int, c_int]),
    "kda_conv1d_bwd": (c_int, [c_void_p] * 8 + [c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                               c_int, c_void_p]),
    "kda_conv1d_dw_reduce": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int, c_void_p]),
    "kda_decode_prep": (c_int, [c_void_p] * 5 + [c_int] + [c_void_p] * 6 + [c_int] * 7 + [c_float, c_float,
                                                                                      c_void_p]),
    "kda_conv1d_decode": (c_int, [c_void_p] * 5 + [c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
}

_lib = None


def lib() -> ctypes.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m kda_b200.build` "
                "(there is no CPU or PyTorch fallback for the fused path)"
            )
        handle = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def exported_symbols():
    return list(_SIGNATURES)


def dt(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}") from None


def ptr(t):
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def profiler_range(name: str):
    """A named range in torch profiler traces, free when no profiler is active (the reference's
    mechanism, attn_gym/linear/kda/utils.py:269-273)."""
    if torch.autograd.profiler._is_profiler_enabled:
        return torch.profiler.record_function(name)
    return contextlib.nullcontext()


def call(name: str, launches: int, *args):
    """Invoke an entry point that returns a status code; raise on failure.  Under an active torch
    profiler the call is a range named after the entry point; inside it, every kernel launch is an
    NVTX range named after the reference stages it fuses (kda_cabi.cu)."""
    global launch_count
    with profiler_range("kda_b200/" + name):
        rc = getattr(lib(), name)(*args)
    if rc != 0:
        raise RuntimeError(f"{name} failed: {_ERRORS.get(rc, rc)}")
    launch_count += launches


def stage_timing(enable: bool) -> None:
    """Switch the library's per-kernel CUDA-event timing on or off."""
    lib().kda_stage_timing_enable(int(enable))


def read_stage_timing(reset: bool = True) -> dict:
    """{stage name: (launches, total milliseconds)} of the kernels timed since the last reset."""
    n = lib().kda_stage_count()
    launches = (c_int64 * n)()
    total = (c_float * n)()
    lib().kda_stage_timing_read(ctypes.cast(launches, c_void_p), ctypes.cast(total, c_void_p),
                                int(reset))
    return {lib().kda_stage_name(i).decode(): (int(launches[i]), float(total[i]))
            for i in range(n) if launches[i]}
