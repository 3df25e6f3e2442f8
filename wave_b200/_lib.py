"""ctypes binding of libwave_b200.so (the C ABI declared in include/wave_b200.h).

There is no CPU fallback: when the shared library is missing or a call fails, an exception is
raised. Error classes follow the reference's launch path, which raises RuntimeError for device
errors (wave_lang/kernel/wave/runtime/runtime.cpp:96-109) and ValueError for bad arguments
(wave_lang/kernel/wave/utils/run_utils.py:110-121, wave_lang/kernel/wave/compile.py:1489-1500).
"""

from __future__ import annotations

import ctypes
import os
from pathlib import Path

WB200_OK = 0
WB200_ERR_INVALID_ARG = -1
WB200_ERR_ALIGNMENT = -2
WB200_ERR_WORKSPACE = -3
WB200_ERR_UNSUPPORTED = -4
WB200_ERR_DEVICE_TIMEOUT = -5
WB200_ERR_CUDA = -6

WB200_F32 = 0
WB200_BF16 = 1

PATH_AUTO = 0
PATH_TILE_1CTA = 1
PATH_TILE_2CTA = 2
PATH_SKINNY = 3
PATH_TILE_SPLITK = 4
PATH_MASK = 0xF
TILE_N128 = 0x10
TILE_N192 = 0x40
ACCUMULATE = 0x20
OVERLAP_PREVIOUS = 0x80
GROUP_N_MASK = 0xFF00
GROUP_N_ALL = 0xFF00


B_TILE_ROWS_MASK = 0x1F0000


def B_TILE_ROWS(h: int) -> int:
    """Flag bits saying that b's scales were packed per tile of h weight rows (include/wave_b200.h, WB200_B_TILE_ROWS)."""
    if h != 224 and (h % 8 or not 8 <= h <= 128):
        raise ValueError(f"{h} rows per tile: 8 .. 128 in steps of 8, or 224")
    return 0 if h == 128 else (h // 8) << 16


def GROUP_N(g: int) -> int:
    """Flag bits for a raster group of g N tiles (1..254); include/wave_b200.h, WB200_GROUP_N."""
    if not 1 <= int(g) <= 254:
        raise ValueError(f"raster group of {g} N tiles: 1..254 fit the flag bits")
    return int(g) << 8
E4M3 = 0
E5M2 = 1
B_FP4 = 0x10  # or into elem_format: b is packed E2M1 (include/wave_b200.h, WB200_B_FP4)

# Every symbol include/wave_b200.h declares; tests check that the built library exports them all.
EXPORTED_SYMBOLS = (
    "wb200_version",
    "wb200_last_error",
    "wb200_check_device_status",
    "wb200_selftest_wait_timeout",
    "wb200_debug_checks",
    "wb200_debug_checks_selftest",
    "wb200_packed_scale_bytes",
    "wb200_decode_tile_rows",
    "wb200_packed_scale_bytes_tiled",
    "wb200_repack_scales_tiled",
    "wb200_repack_scales",
    "wb200_repack_scales_broadcast",
    "wb200_repack_scales_grouped",
    "wb200_quantize_mxfp4",
    "wb200_mxfp4_dequant",
    "wb200_mxfp4_gemm_workspace_bytes",
    "wb200_workspace_init",
    "wb200_mxfp4_gemm",
    "wb200_mxfp4_gemm_repack_a",
    "wb200_mxfp8_gemm",
    "wb200_quantize_mxfp8",
    "wb200_mxfp4_gemm_skinny_noalloc",
    "wb200_mxfp4_grouped_gemm",
    "wb200_mxfp4_moe_gemm",
    "wb200_moe_align_block_size",
    "wb200_moe_gather_rows",
    "wb200_silu_and_mul",
    "wb200_moe_quantize_scatter",
    "wb200_moe_combine",
    "wb200_mxfp4_gemm_scatter_rows",
    "wb200_peer_buffer_create",
    "wb200_peer_buffer_open",
    "wb200_peer_buffer_close",
    "wb200_peer_buffer_destroy",
    "wb200_sum_slots",
    "wb200_copy_2d",
    "wb200_multi_gpu_create",
    "wb200_multi_gpu_destroy",
    "wb200_multi_gpu_num_devices",
    "wb200_multi_gpu_shard_bounds",
    "wb200_multi_gpu_wait_for",
    "wb200_multi_gpu_broadcast_a",
    "wb200_multi_gpu_gemm",
    "wb200_multi_gpu_gather_c",
    "wb200_multi_gpu_join",
    "wb200_multi_gpu_synchronize",
    "wb200_multi_gpu_time_begin",
    "wb200_multi_gpu_time_end",
)


class DeviceTimeoutError(RuntimeError):
    """A bounded device-side wait gave up; the outputs of the affected launches are invalid."""


def library_path() -> Path:
    env = os.environ.get("WAVE_B200_LIB")
    if env:
        return Path(env)
    return Path(__file__).resolve().parent / "libwave_b200.so"


_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library once. Raises RuntimeError when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not path.exists():
        raise RuntimeError(
            f"{path} not found: build it with `python -m wave_b200.build` (needs nvcc for sm_100a). "
            "wave_b200 has no CPU or PyTorch fallback."
        )
    lib = ctypes.CDLL(str(path))
    c_void_p, c_int, c_size_t, c_ll, c_uint = (
        ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_longlong, ctypes.c_uint)
    lib.wb200_version.restype = c_int
    lib.wb200_version.argtypes = []
    lib.wb200_last_error.restype = ctypes.c_char_p
    lib.wb200_last_error.argtypes = []
    lib.wb200_check_device_status.restype = c_int
    lib.wb200_check_device_status.argtypes = [c_void_p, ctypes.POINTER(c_int)]
    lib.wb200_selftest_wait_timeout.restype = c_int
    lib.wb200_selftest_wait_timeout.argtypes = [c_ll, c_void_p]
    lib.wb200_debug_checks.restype = c_int
    lib.wb200_debug_checks.argtypes = [ctypes.POINTER(ctypes.c_ulonglong), c_int]
    lib.wb200_debug_checks_selftest.restype = c_int
    lib.wb200_debug_checks_selftest.argtypes = [c_void_p]
    lib.wb200_packed_scale_bytes.restype = c_size_t
    lib.wb200_packed_scale_bytes.argtypes = [c_int, c_int]
    lib.wb200_decode_tile_rows.restype = c_int
    lib.wb200_decode_tile_rows.argtypes = [c_int]
    lib.wb200_packed_scale_bytes_tiled.restype = c_size_t
    lib.wb200_packed_scale_bytes_tiled.argtypes = [c_int, c_int, c_int]
    lib.wb200_repack_scales_tiled.restype = c_int
    lib.wb200_repack_scales_tiled.argtypes = [c_void_p, c_ll, c_int, c_int, c_int, c_void_p, c_void_p]
    lib.wb200_repack_scales.restype = c_int
    lib.wb200_repack_scales.argtypes = [c_void_p, c_ll, c_int, c_int, c_void_p, c_void_p]
    lib.wb200_repack_scales_broadcast.restype = c_int
    lib.wb200_repack_scales_broadcast.argtypes = [c_void_p, c_ll, c_int, c_int, c_void_p, c_void_p]
    lib.wb200_repack_scales_grouped.restype = c_int
    lib.wb200_repack_scales_grouped.argtypes = [c_void_p, c_ll, c_int, ctypes.POINTER(c_int), ctypes.POINTER(c_int), c_int,
                                                c_void_p, c_void_p]
    lib.wb200_quantize_mxfp4.restype = c_int
    lib.wb200_quantize_mxfp4.argtypes = [c_void_p, c_int, c_ll, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]
    lib.wb200_mxfp4_dequant.restype = c_int
    lib.wb200_mxfp4_dequant.argtypes = [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]
    lib.wb200_mxfp4_gemm_workspace_bytes.restype = c_size_t
    lib.wb200_mxfp4_gemm_workspace_bytes.argtypes = [c_int, c_int, c_int]
    lib.wb200_workspace_init.restype = c_int
    lib.wb200_workspace_init.argtypes = [c_void_p, c_size_t, c_void_p]
    lib.wb200_mxfp4_gemm.restype = c_int
    lib.wb200_mxfp4_gemm.argtypes = [c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_int, c_ll, c_void_p, c_size_t, c_uint, c_void_p]
    lib.wb200_mxfp4_gemm_repack_a.restype = c_int
    lib.wb200_mxfp4_gemm_repack_a.argtypes = [c_int, c_int, c_int, c_void_p, c_void_p, c_ll, c_void_p, c_void_p, c_void_p,
                                              c_void_p, c_int, c_ll, c_void_p, c_size_t, c_uint, c_void_p]
    lib.wb200_mxfp8_gemm.restype = c_int
    lib.wb200_mxfp8_gemm.argtypes = [c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_ll,
                                     c_int, c_void_p, c_size_t, c_uint, c_void_p]
    lib.wb200_quantize_mxfp8.restype = c_int
    lib.wb200_quantize_mxfp8.argtypes = [c_void_p, c_int, c_ll, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]
    lib.wb200_mxfp4_gemm_skinny_noalloc.restype = c_int
    lib.wb200_mxfp4_gemm_skinny_noalloc.argtypes = [c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                    c_int, c_ll, c_uint, c_void_p]
    lib.wb200_mxfp4_grouped_gemm.restype = c_int
    lib.wb200_mxfp4_grouped_gemm.argtypes = [c_int, ctypes.POINTER(c_int), ctypes.POINTER(c_int), c_int, c_int,
                                             c_void_p, c_void_p, ctypes.POINTER(c_void_p),
                                             ctypes.POINTER(c_void_p), c_void_p, c_int, c_ll, c_void_p]
    lib.wb200_mxfp4_moe_gemm.restype = c_int
    lib.wb200_mxfp4_moe_gemm.argtypes = [c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                         ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p), c_void_p, c_int, c_ll, c_void_p]
    lib.wb200_moe_align_block_size.restype = c_int
    lib.wb200_moe_align_block_size.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int,
                                               c_void_p, c_void_p, c_void_p]
    lib.wb200_moe_gather_rows.restype = c_int
    lib.wb200_moe_gather_rows.argtypes = [c_void_p, c_ll, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_ll, c_void_p]
    lib.wb200_silu_and_mul.restype = c_int
    lib.wb200_silu_and_mul.argtypes = [c_void_p, c_void_p, c_ll, c_ll, c_int, c_int, c_int, c_void_p, c_ll, c_void_p,
                                       c_void_p, c_void_p, c_void_p, c_void_p]
    lib.wb200_moe_quantize_scatter.restype = c_int
    lib.wb200_moe_quantize_scatter.argtypes = [c_void_p, c_int, c_ll, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                               c_void_p]
    lib.wb200_moe_combine.restype = c_int
    lib.wb200_moe_combine.argtypes = [c_void_p, c_ll, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_ll,
                                      c_void_p]
    lib.wb200_mxfp4_gemm_scatter_rows.restype = c_int
    lib.wb200_mxfp4_gemm_scatter_rows.argtypes = [c_int, ctypes.POINTER(c_int), c_int, c_int, c_void_p, c_void_p, c_void_p,
                                                  c_void_p, ctypes.POINTER(c_void_p), c_int, c_ll, c_uint, c_void_p]
    lib.wb200_peer_buffer_create.restype = c_int
    lib.wb200_peer_buffer_create.argtypes = [c_size_t, ctypes.POINTER(c_void_p), c_void_p]
    lib.wb200_peer_buffer_open.restype = c_int
    lib.wb200_peer_buffer_open.argtypes = [c_void_p, ctypes.POINTER(c_void_p)]
    lib.wb200_peer_buffer_close.restype = c_int
    lib.wb200_peer_buffer_close.argtypes = [c_void_p]
    lib.wb200_peer_buffer_destroy.restype = c_int
    lib.wb200_peer_buffer_destroy.argtypes = [c_void_p]
    lib.wb200_sum_slots.restype = c_int
    lib.wb200_sum_slots.argtypes = [c_void_p, c_int, c_ll, c_ll, c_void_p, c_int, c_void_p]
    lib.wb200_copy_2d.restype = c_int
    lib.wb200_copy_2d.argtypes = [c_void_p, c_size_t, c_void_p, c_size_t, c_size_t, c_size_t, c_void_p]

    class DeviceOperands(ctypes.Structure):
        """wb200_device_operands of include/wave_b200.h."""
        _fields_ = [("a", c_void_p), ("a_scale", c_void_p), ("a_scale_packed", c_void_p), ("b", c_void_p),
                    ("b_scale_packed", c_void_p), ("c", c_void_p), ("ldc", c_ll), ("workspace", c_void_p),
                    ("workspace_bytes", c_size_t)]

    lib.DeviceOperands = DeviceOperands
    p_int = ctypes.POINTER(c_int)
    p_ops = ctypes.POINTER(DeviceOperands)
    lib.wb200_multi_gpu_create.restype = c_int
    lib.wb200_multi_gpu_create.argtypes = [c_int, p_int, ctypes.POINTER(c_void_p)]
    lib.wb200_multi_gpu_destroy.restype = c_int
    lib.wb200_multi_gpu_destroy.argtypes = [c_void_p]
    lib.wb200_multi_gpu_num_devices.restype = c_int
    lib.wb200_multi_gpu_num_devices.argtypes = [c_void_p]
    lib.wb200_multi_gpu_shard_bounds.restype = c_int
    lib.wb200_multi_gpu_shard_bounds.argtypes = [c_int, c_int, c_int, c_int, p_int, p_int]
    lib.wb200_multi_gpu_wait_for.restype = c_int
    lib.wb200_multi_gpu_wait_for.argtypes = [c_void_p, c_int, c_void_p]
    lib.wb200_multi_gpu_broadcast_a.restype = c_int
    lib.wb200_multi_gpu_broadcast_a.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, p_ops]
    lib.wb200_multi_gpu_gemm.restype = c_int
    lib.wb200_multi_gpu_gemm.argtypes = [c_void_p, c_int, c_int, p_int, p_ops, c_int, c_uint]
    lib.wb200_multi_gpu_gather_c.restype = c_int
    lib.wb200_multi_gpu_gather_c.argtypes = [c_void_p, c_int, p_int, p_ops, c_int, c_int, ctypes.POINTER(c_void_p), p_int, c_ll]
    lib.wb200_multi_gpu_join.restype = c_int
    lib.wb200_multi_gpu_join.argtypes = [c_void_p, c_int, c_void_p]
    lib.wb200_multi_gpu_synchronize.restype = c_int
    lib.wb200_multi_gpu_synchronize.argtypes = [c_void_p]
    lib.wb200_multi_gpu_time_begin.restype = c_int
    lib.wb200_multi_gpu_time_begin.argtypes = [c_void_p]
    lib.wb200_multi_gpu_time_end.restype = c_int
    lib.wb200_multi_gpu_time_end.argtypes = [c_void_p, ctypes.POINTER(ctypes.c_float)]
    _lib = lib
    return lib


def check(rc: int) -> None:
    """Turn a status code of the C ABI into the exception class the reference would raise."""
    if rc == WB200_OK:
        return
    msg = load().wb200_last_error().decode("utf-8", "replace")
    if rc in (WB200_ERR_INVALID_ARG, WB200_ERR_ALIGNMENT, WB200_ERR_WORKSPACE):
        raise ValueError(f"wave_b200: {msg}")
    if rc == WB200_ERR_DEVICE_TIMEOUT:
        raise DeviceTimeoutError(f"wave_b200: {msg}")
    raise RuntimeError(f"wave_b200: {msg} (status {rc})")
