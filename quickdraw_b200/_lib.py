"""ctypes binding of ``libquickdraw_b200.so`` (declarations: ``include/quickdraw_b200.h``).

The library is the only execution path of this package: if it cannot be loaded the
import of any operator raises, there is no PyTorch or CPU fallback.
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_longlong, c_void_p
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "libquickdraw_b200.so"

P, I, F, L = c_void_p, c_int, c_float, c_longlong

SIGNATURES = {
    "qd_version": [],
    "qd_rms_norm": [P, P, P, I, I, F, I, P],
    "qd_add_rms_norm": [P, P, P, P, P, I, F, P],
    "qd_nvfp4_gemv": [P, P, P, P, P, P, I, I, I, I, P],
    "qd_nvfp4_expert_gemv": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, P],
    "qd_nvfp4_gate_up": [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, P],
    "qd_nvfp4_dequantize": [P, P, F, P, L, I, I, I, P],
    "qd_bf16_gemv": [P, P, P, I, I, P],
    "qd_fp8_gemv": [P, P, P, P, P, I, I, I, P],
    "qd_fp8_matmul": [P, P, P, P, P, I, I, I, P, I, P],
    "qd_route_topk": [P, I, I, I, P, P, P],
    "qd_moe_combine": [P, P, P, P, P, I, I, P],
    "qd_swiglu": [P, P, P, I, P],
    "qd_gdn_conv": [P, P, P, P, I, I, P],
    "qd_gdn_recurrence": [P, P, P, P, P, P, P, I, I, I, I, I, P],
    "qd_gdn_gated_norm": [P, P, P, P, I, I, F, P],
    "qd_attn_scratch_floats": [I, I, I, I],
    "qd_attn_decode": [P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, F, F, I, I, P],
    "qd_attn_decode_static": [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, F, F, I, P],
    "qd_moe_down_combine": [P, P, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, P],
    "qd_moe_finish": [P, P, P, I, I, P],
    "qd_model_create": [P, P],
    "qd_model_destroy": [P],
    "qd_model_set_layer": [P, I, P],
    "qd_decode_workspace_bytes": [P],
    "qd_decode_step": [P, P, P, P, I, P, P, P, I, P],
    "qd_program_bytes": [P],
    "qd_program_build": [P, P, P, L],
    "qd_decode_step_persistent": [P, P, P, P, I, P, P, P, P, P, I, P, P],
    "qd_exchange_bytes": [P],
    "qd_set_wait_limit_us": [ctypes.c_uint],
    "qd_set_chained_launches": [I],
    "qd_nvfp4_gemv_bank": [P, P, P, P, P, I, I, I, I, P],
    "qd_nvfp4_matmul": [P, P, P, P, P, I, I, I, I, P, P],
    "qd_nvfp4_matmul_rows_scratch_bytes": [I],
    "qd_nvfp4_matmul_rows": [P, P, P, P, P, P, I, I, I, I, P, I, P],
    "qd_nvfp4_matmul_rows3": [P, P, I, I, I, P, I, I, P, P, P, P, I, P, P, P, P, I, P, P, P, P, I, P],
    "qd_nvfp4_quantize_act": [P, I, I, P, P, P, P, P],
    "qd_nvfp4_matmul_w4a4": [P, P, P, P, P, P, P, I, I, I, I, P, P],
    "qd_nvfp4_grouped_matmul": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, P, P],
    "qd_nvfp4_expert_rows_scratch_bytes": [I, I],
    "qd_nvfp4_expert_rows2": [P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, P, I, P],
    "qd_nvfp4_expert_rows": [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, P, I, P],
    "qd_seq_add_rms_norm": [P, P, P, P, P, I, I, F, P],
    "qd_seq_bf16_matmul": [P, P, P, I, I, I, P],
    "qd_seq_bf16_matmul2": [P, P, P, I, P, P, I, I, I, P],
    "qd_seq_gdn_conv": [P, P, P, P, I, I, I, P],
    "qd_seq_gdn_recurrence": [P, P, P, P, P, P, P, I, I, I, I, I, P],
    "qd_seq_gdn_chunk_scratch_bytes": [I, I],
    "qd_seq_gdn_recurrence_chunked": [P, P, P, P, P, P, P, I, I, I, I, I, P, P],
    "qd_seq_attention": [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, F, P],
    "qd_seq_route_topk": [P, I, I, I, P, P, P],
    "qd_batch_gdn_conv": [P, P, P, L, P, I, I, I, P],
    "qd_batch_gdn_recurrence": [P, P, P, P, P, P, L, P, I, I, I, I, I, P],
    "qd_batch_attn_decode": [P, P, P, P, P, P, P, L, P, P, P, P, I, I, I, I, I, I, F, F, I, P],
    "qd_batch_attention": [P, P, P, P, P, P, P, L, P, P, P, P, P, I, I, I, I, I, I, F, F, I, P],
    "qd_seq_group_routes": [P, I, I, P, P, P],
    "qd_seq_moe_combine": [P, P, P, P, P, I, I, I, P],
    "qd_seq_moe_combine_norm": [P, P, P, P, P, P, P, P, I, I, I, F, P],
}

LONG_RESULTS = {"qd_decode_workspace_bytes", "qd_program_bytes", "qd_exchange_bytes",
                "qd_nvfp4_matmul_rows_scratch_bytes", "qd_seq_gdn_chunk_scratch_bytes",
                "qd_nvfp4_expert_rows_scratch_bytes"}

_lib = None


class LibraryMissing(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    """Load the CUDA library once; raise loudly if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise LibraryMissing(
                f"{LIB_PATH} not found: build it with `python -m quickdraw_b200.build` "
                "(this package has no fallback path)")
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, argtypes in SIGNATURES.items():
            fn = getattr(handle, name, None)
            if fn is None:
                continue
            fn.argtypes = argtypes
            fn.restype = c_longlong if name in LONG_RESULTS else c_int
        handle.qd_error_string.argtypes = [c_int]
        handle.qd_error_string.restype = c_char_p
        _lib = handle
    return _lib


def exported_symbols() -> list[str]:
    return sorted(SIGNATURES) + ["qd_error_string"]


def ptr(t: torch.Tensor | None):
    """Device address of a tensor (or NULL)."""
    return None if t is None else c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_of(t: torch.Tensor):
    """The current CUDA stream of the tensor's device as a C handle.  A prompt chunk is some 1 300
    launches: the raw-handle query (a fraction of a microsecond) instead of building a
    ``torch.cuda.Stream`` object per launch (several microseconds) is 3 ms of host time per chunk."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(t.device.index if t.device.index is not None else torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def check(code: int, name: str) -> None:
    if code != 0:
        raise RuntimeError(f"{name} failed: {lib().qd_error_string(code).decode()} (code {code})")


def call(name: str, *args) -> None:
    check(getattr(lib(), name)(*args), name)
