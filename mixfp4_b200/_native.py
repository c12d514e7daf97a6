"""ctypes binding of the C-ABI library (include/mixfp4_b200.h).

There is no fallback: if the shared library cannot be loaded every operation of
the package raises.  Tensors cross the boundary as raw device pointers plus
sizes; the stream is torch's current CUDA stream.
"""

from __future__ import annotations

import ctypes
import os

import torch

from . import build as _build

OK = 0
E_NULL, E_SHAPE, E_ALIGN, E_DTYPE, E_MODE, E_CUDA, E_WORKSPACE = -1, -2, -3, -4, -5, -6, -7
E_UNSUPPORTED, E_DEVICE_WAIT, E_TOO_LARGE = -8, -9, -10
BF16, F16, F32 = 0, 1, 2
MODE_ORACLE16, MODE_ALL_E2M1, MODE_ALL_E0M3, MODE_GIVEN = 0, 1, 2, 3
LAYOUT_CANONICAL, LAYOUT_KERNEL, LAYOUT_STREAM = 0, 1, 2
FLAG_OVERLAP_PREVIOUS = 1
FLAG_WIDE_TABLE = 2
WIDE_TABLE_BYTES = 4096 + 32768


def gemv_flags(overlap_previous: bool, *luts) -> int:
    """Flags of a decode call: programmatic dependent launch, and whether every table is a wide one."""
    wide = bool(luts) and all(t is not None and t.numel() >= WIDE_TABLE_BYTES for t in luts)
    return (FLAG_OVERLAP_PREVIOUS if overlap_previous else 0) | (FLAG_WIDE_TABLE if wide else 0)

DTYPE_CODE = {torch.bfloat16: BF16, torch.float16: F16, torch.float32: F32}

_lib = None


class MixFP4Error(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, fn: str, status: int, detail: str = ""):
        self.status = status
        text = f"{fn} failed with status {status} ({lib().mixfp4_status_string(status).decode()})"
        if detail:
            text += ": " + detail
        super().__init__(text)


class GemvSegment(ctypes.Structure):
    """struct mixfp4_gemv_segment of include/mixfp4_b200.h."""
    _fields_ = [("codes", ctypes.c_void_p), ("scales", ctypes.c_void_p), ("global_scale", ctypes.c_void_p),
                ("lut", ctypes.c_void_p), ("y", ctypes.c_void_p), ("ldy", ctypes.c_int64), ("n", ctypes.c_int64)]


def _declare(h: ctypes.CDLL) -> None:
    p, i64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    pp = ctypes.POINTER(ctypes.c_void_p)
    h.mixfp4_abi_version.restype = i32
    h.mixfp4_abi_version.argtypes = []
    h.mixfp4_status_string.restype = ctypes.c_char_p
    h.mixfp4_status_string.argtypes = [i32]
    h.mixfp4_last_cuda_error.restype = ctypes.c_char_p
    h.mixfp4_last_cuda_error.argtypes = []
    h.mixfp4_padded_k.restype = i64
    h.mixfp4_padded_k.argtypes = [i64]
    h.mixfp4_amax.restype = i32
    h.mixfp4_amax.argtypes = [p, i32, i64, i64, i64, p, p]
    h.mixfp4_quantize.restype = i32
    h.mixfp4_quantize.argtypes = [p, i32, i64, i64, i64, i32, p, p, p, p, p, p, p, p, p, p, i64, p]
    h.mixfp4_fake_quantize.restype = i32
    h.mixfp4_fake_quantize.argtypes = [p, i32, i64, i64, i64, i32, p, p, i64, p]
    h.mixfp4_select_regions.restype = i32
    h.mixfp4_select_regions.argtypes = [p, p, i64, i64, i32, i32, p, p]
    h.mixfp4_select_layer.restype = i32
    h.mixfp4_select_layer.argtypes = [p, p, i64, i64, p, p, p]
    h.mixfp4_selftest_division.restype = i32
    h.mixfp4_selftest_division.argtypes = [p, p]
    h.mixfp4_e0_four_over_six.restype = i32
    h.mixfp4_e0_four_over_six.argtypes = [p, i64, p, p, p, p, p, p, p]
    h.mixfp4_round_codebook.restype = i32
    h.mixfp4_round_codebook.argtypes = [p, p, i64, i32, p]
    h.mixfp4_dequant.restype = i32
    h.mixfp4_dequant.argtypes = [p, p, p, p, i64, i64, i32, p, i32, i64, p]
    h.mixfp4_repack.restype = i32
    h.mixfp4_repack.argtypes = [p, p, p, i64, i64, i32, p, p, p, p]
    h.mixfp4_decode_table_wide.restype = i32
    h.mixfp4_decode_table_wide.argtypes = [p, p, p]
    h.mixfp4_decode_table.restype = i32
    h.mixfp4_decode_table.argtypes = [p, p, p]
    h.mixfp4_fwht.restype = i32
    h.mixfp4_fwht.argtypes = [p, p, i32, i64, i64, i64, i64, i32, p, i32, p]
    h.mixfp4_gemv.restype = i32
    h.mixfp4_gemv.argtypes = [p, i64, i64, p, p, p, p, i64, i64, i32, p, p, i32, i64, i32, p]
    h.mixfp4_gemv_grouped.restype = i32
    h.mixfp4_gemv_grouped.argtypes = [p, i64, i64, i64, ctypes.POINTER(GemvSegment), i32, i32, i32, i32, p]
    h.mixfp4_gemv_x_fits.restype = i32
    h.mixfp4_gemv_x_fits.argtypes = [i64, i64, i32]
    h.mixfp4_stream_bytes.restype = i64
    h.mixfp4_stream_bytes.argtypes = [i64, i64]
    h.mixfp4_repack_stream.restype = i32
    h.mixfp4_repack_stream.argtypes = [p, p, p, i64, i64, p, p]
    h.mixfp4_repack_from_stream.restype = i32
    h.mixfp4_repack_from_stream.argtypes = [p, i64, i64, p, p, p, p]
    h.mixfp4_set_wait_limit_ns.restype = i32
    h.mixfp4_set_wait_limit_ns.argtypes = [ctypes.c_uint64]
    h.mixfp4_check_status.restype = i32
    h.mixfp4_check_status.argtypes = [p, ctypes.POINTER(ctypes.c_int), p]
    h.mixfp4_comm_buffer_bytes.restype = i64
    h.mixfp4_comm_buffer_bytes.argtypes = [i32, i64]
    h.mixfp4_comm_buffer.restype = i32
    h.mixfp4_comm_buffer.argtypes = [p, pp]
    h.mixfp4_comm_open_local.restype = i32
    h.mixfp4_comm_open_local.argtypes = [p, ctypes.POINTER(ctypes.c_void_p)]
    h.mixfp4_comm_create.restype = i32
    h.mixfp4_comm_create.argtypes = [i32, i32, i64, pp]
    h.mixfp4_comm_handle_bytes.restype = i32
    h.mixfp4_comm_handle_bytes.argtypes = []
    h.mixfp4_comm_handle.restype = i32
    h.mixfp4_comm_handle.argtypes = [p, p]
    h.mixfp4_comm_open.restype = i32
    h.mixfp4_comm_open.argtypes = [p, p]
    h.mixfp4_comm_destroy.restype = i32
    h.mixfp4_comm_destroy.argtypes = [p]
    h.mixfp4_gemv_allreduce.restype = i32
    h.mixfp4_gemv_allreduce.argtypes = [p, p, i64, i64, p, p, p, p, i64, i64, i32, p, i32, i64, p, i32, p]
    h.mixfp4_gemm_workspace_bytes.restype = i64
    h.mixfp4_gemm_workspace_bytes.argtypes = [i64, i64, i64]
    h.mixfp4_gemm.restype = i32
    h.mixfp4_gemm.argtypes = [p, i64, i64, p, p, p, p, i64, i64, i32, p, i32, p, i32, i64, p, i64, p, i32, p]
    h.mixfp4_gemm_a4.restype = i32
    h.mixfp4_gemm_a4.argtypes = [p, i64, i64, p, p, p, p, i64, i64, i32, p, i32, i32, p, i32, i64, p, i64, p, i32, p]
    h.mixfp4_gemm_h128_static_max_bytes.restype = i64
    h.mixfp4_gemm_h128_static_max_bytes.argtypes = []
    h.mixfp4_gemm_h128_static.restype = i32
    h.mixfp4_gemm_h128_static.argtypes = [p, i64, i64, p, p, p, p, i64, i64, i32, p, p, i32, i64, p, p]


# every symbol include/mixfp4_b200.h declares
EXPORTED = (
    "mixfp4_abi_version", "mixfp4_status_string", "mixfp4_last_cuda_error", "mixfp4_padded_k",
    "mixfp4_amax", "mixfp4_quantize", "mixfp4_fake_quantize", "mixfp4_select_regions", "mixfp4_select_layer", "mixfp4_selftest_division", "mixfp4_round_codebook", "mixfp4_e0_four_over_six", "mixfp4_dequant", "mixfp4_repack", "mixfp4_decode_table", "mixfp4_decode_table_wide", "mixfp4_fwht",
    "mixfp4_stream_bytes", "mixfp4_repack_stream", "mixfp4_repack_from_stream",
    "mixfp4_gemv", "mixfp4_gemv_x_fits", "mixfp4_gemv_grouped",
    "mixfp4_comm_create", "mixfp4_comm_handle_bytes", "mixfp4_comm_handle", "mixfp4_comm_open",
    "mixfp4_comm_buffer_bytes", "mixfp4_comm_buffer", "mixfp4_comm_open_local", "mixfp4_comm_destroy",
    "mixfp4_gemv_allreduce", "mixfp4_set_wait_limit_ns", "mixfp4_check_status",
    "mixfp4_gemm_workspace_bytes", "mixfp4_gemm", "mixfp4_gemm_a4", "mixfp4_gemm_h128_static_max_bytes", "mixfp4_gemm_h128_static",
)


def lib() -> ctypes.CDLL:
    """The loaded library; raises if it is missing (build it with ``python -m mixfp4_b200.build``)."""
    global _lib
    if _lib is None:
        path = _build.LIB_PATH
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} is missing: the CUDA library has not been built "
                "(run `python -m mixfp4_b200.build`); mixfp4_b200 has no fallback path")
        handle = ctypes.CDLL(path)
        _declare(handle)
        if handle.mixfp4_abi_version() != 3:
            raise RuntimeError("libmixfp4_b200.so ABI version mismatch; rebuild it")
        _lib = handle
    return _lib


def check(fn: str, status: int) -> None:
    if status != OK:
        detail = lib().mixfp4_last_cuda_error().decode() if status == -6 else ""
        raise MixFP4Error(fn, status, detail)


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what} must be a CUDA tensor (mixfp4_b200 has no CPU path)")
