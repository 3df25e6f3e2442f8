"""Torch-tensor front ends of the C ABI: scale repack, dequantisation aid, and the GEMM launch.

PyTorch is used for device memory and streams only; every computation happens in
libwave_b200.so. Launches go to `torch.cuda.current_stream()` and return without synchronising,
as the reference's launch shim does (wave_lang/kernel/wave/utils/run_utils.py:87,134).
"""

from __future__ import annotations

import ctypes
import weakref
from collections import OrderedDict

import torch

from . import _lib

SCALE_GROUP_SIZE = 32


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _as_u8(t: torch.Tensor, what: str) -> torch.Tensor:
    if t.dtype not in (torch.uint8, torch.int8):
        raise ValueError(f"{what} must be uint8 or int8 (packed bytes), got {t.dtype}")
    if not t.is_cuda:
        raise ValueError(f"{what} must be a CUDA tensor; wave_b200 has no CPU path")
    return t


class PackedScales:
    """E8M0 scales of a [rows, K/32] matrix in the tcgen05 scale-factor layout (flat uint8). `tile_rows`: rows per
    512-byte atom row, 128 for the layout every kernel reads; a smaller value marks a WEIGHT packing made for the
    decode kernel's tile height (`repack_scales(..., tile_rows=decode_tile_rows(N))`), which only the M <= 128
    path reads."""

    __slots__ = ("data", "rows", "K", "tile_rows")

    def __init__(self, data: torch.Tensor, rows: int, K: int, tile_rows: int = 128):
        self.data, self.rows, self.K, self.tile_rows = data, rows, K, tile_rows

    @property
    def device(self):
        return self.data.device


def packed_scale_bytes(rows: int, K: int) -> int:
    return int(_lib.load().wb200_packed_scale_bytes(rows, K))


def decode_tile_rows(N: int, device=None) -> int:
    """Tile height of the M <= 128 kernel for which every SM of `device` gets the same number of weight tiles (a multiple
    of 8, at most 128; 128 when the usual packing is as good). Pack a weight's scales with it to use it."""
    lib = _lib.load()
    if device is None:
        return int(lib.wb200_decode_tile_rows(int(N)))
    with torch.cuda.device(device):
        return int(lib.wb200_decode_tile_rows(int(N)))


def repack_scales(scale: torch.Tensor, out: torch.Tensor | None = None, tile_rows: int = 128) -> PackedScales:
    """Row-major [rows, K/32] E8M0 scales -> PackedScales, on the current stream. tile_rows < 128: the weight packing
    of the decode kernel (one atom row per tile of that many rows, see `decode_tile_rows`)."""
    lib = _lib.load()
    _as_u8(scale, "scale")
    if scale.dim() != 2:
        raise ValueError(f"scale must be 2-D [rows, K/32], got shape {tuple(scale.shape)}")
    if scale.stride(1) != 1:
        scale = scale.contiguous()
    rows, kb = scale.shape
    K = kb * SCALE_GROUP_SIZE
    row_stride = scale.stride(0) if rows > 1 else kb  # the stride of a size-1 dimension is arbitrary
    tiled = tile_rows != 128
    nbytes = int(lib.wb200_packed_scale_bytes_tiled(rows, K, tile_rows)) if tiled else packed_scale_bytes(rows, K)
    if tiled and nbytes == 0:
        raise ValueError(f"repack_scales: {tile_rows} rows per tile (8 .. 128 in steps of 8)")
    if out is None:
        out = torch.empty(nbytes, dtype=torch.uint8, device=scale.device)
    elif out.numel() < nbytes or out.dtype != torch.uint8 or not out.is_contiguous():
        raise ValueError("repack_scales: `out` must be a contiguous uint8 tensor of at least packed_scale_bytes(rows, K)")

    def run():
        if tiled:
            return lib.wb200_repack_scales_tiled(scale.data_ptr(), row_stride, rows, K, tile_rows, out.data_ptr(), _stream())
        return lib.wb200_repack_scales(scale.data_ptr(), row_stride, rows, K, out.data_ptr(), _stream())

    dev_index = scale.device.index
    if dev_index is None or dev_index == torch.cuda.current_device():
        rc = run()
    else:
        with torch.cuda.device(scale.device):
            rc = run()
    if rc:
        _lib.check(rc)
    return PackedScales(out, rows, K, tile_rows)


def repack_scales_broadcast(scale: torch.Tensor, K: int, out: torch.Tensor | None = None) -> PackedScales:
    """One E8M0 scale per row ([rows] uint8), used for every K block of the row -> PackedScales.
    The a_scale argument of the reference's broadcast-scale kernel
    (wave_lang/kernel/wave/templates/test_kernels.py:98-116)."""
    lib = _lib.load()
    _as_u8(scale, "scale")
    if scale.dim() != 1:
        raise ValueError(f"scale must be 1-D [rows], got shape {tuple(scale.shape)}")
    rows = scale.shape[0]
    nbytes = packed_scale_bytes(rows, K)
    if out is None:
        out = torch.empty(nbytes, dtype=torch.uint8, device=scale.device)
    elif out.numel() < nbytes or out.dtype != torch.uint8 or not out.is_contiguous():
        raise ValueError("repack_scales_broadcast: `out` must be a contiguous uint8 tensor of at least packed_scale_bytes(rows, K)")
    stride = scale.stride(0) if rows > 1 else 1
    with torch.cuda.device(scale.device):
        _lib.check(lib.wb200_repack_scales_broadcast(scale.data_ptr(), stride, rows, K, out.data_ptr(), _stream()))
    return PackedScales(out, rows, K)


def dequant_mxfp4(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """[R, K/2] codes, [R, K/32] scales -> [R, K] f32 on the GPU (test aid)."""
    lib = _lib.load()
    q = _as_u8(q, "q").contiguous()
    scale = _as_u8(scale, "scale").contiguous()
    rows, K = q.shape[0], q.shape[1] * 2
    if tuple(scale.shape) != (rows, K // SCALE_GROUP_SIZE):
        raise ValueError(f"scale shape {tuple(scale.shape)} does not match q {tuple(q.shape)}")
    out = torch.empty(rows, K, dtype=torch.float32, device=q.device)
    with torch.cuda.device(q.device):
        _lib.check(lib.wb200_mxfp4_dequant(q.data_ptr(), scale.data_ptr(), rows, K, out.data_ptr(), _stream()))
    return out


class WorkspacePool:
    """Workspaces of the skinny (M <= 128) and split-K paths, one per (device, stream, kind).

    A workspace holds counters and partial tiles that a running GEMM owns, so two GEMMs that may overlap on
    the GPU (different streams) must not share one; and the skinny path expects its partial-tile region in the
    state `wb200_workspace_init` leaves it in (which it restores after every launch), so it does not share
    with the split-K path, which leaves partial products there. Each kernel object has its own pool, and the
    functional entry points share a module-level one.

    Workspaces are created and initialised eagerly. While a stream is being captured into a CUDA graph nothing
    is allocated: the call uses the workspace an earlier eager call (the warm-up) made for that device and kind.
    """

    def __init__(self):
        self._by_key: dict = {}

    def get(self, device: torch.device, nbytes: int, kind: str) -> torch.Tensor:
        idx = device.index if device.index is not None else torch.cuda.current_device()
        capturing = torch.cuda.is_current_stream_capturing()
        key = (idx, torch.cuda.current_stream(idx).cuda_stream, kind)
        ws = self._by_key.get(key)
        if ws is not None and ws.numel() >= nbytes:
            return ws
        if capturing:
            for (d, _, k), w in self._by_key.items():
                if d == idx and k == kind and w.numel() >= nbytes:
                    return w
            raise RuntimeError("this GEMM needs a workspace, which cannot be created while a CUDA graph is being captured: "
                               "call it once eagerly (with the same shapes) before the capture")
        ws = torch.empty(nbytes, dtype=torch.uint8, device=torch.device("cuda", idx))
        with torch.cuda.device(idx):
            _lib.check(_lib.load().wb200_workspace_init(ws.data_ptr(), nbytes, _stream()))
        self._by_key[key] = ws
        return ws

    def clear(self) -> None:
        self._by_key.clear()


_pool = WorkspacePool()


def _workspace(device: torch.device, nbytes: int, kind: str = "skinny", pool: WorkspacePool | None = None) -> torch.Tensor:
    return (pool or _pool).get(device, nbytes, kind)


_DTYPE_CODE = {torch.float32: _lib.WB200_F32, torch.bfloat16: _lib.WB200_BF16}


def split_k_pays() -> bool:
    """The split-K tile path halves the GPU time of small long-K shapes but its launch costs ~15 us more on the
    host (a 20 KB kernel parameter block plus a second kernel). From Python that only pays where the host cost
    is not in the loop: while the call is being captured into a CUDA graph. Eager calls pass no workspace for
    M > 128 and so stay on the plain tile path; C callers decide for themselves by passing one or not."""
    return torch.cuda.is_current_stream_capturing()


def scaled_gemm_packed(a: torch.Tensor, a_sf: PackedScales, b: torch.Tensor, b_sf: PackedScales, c: torch.Tensor,
                       flags: int = _lib.PATH_AUTO) -> None:
    """c[M, N] = dequant(a) @ dequant(b).T with both scale sets already packed. c may be a column
    block of a wider matrix (row stride >= N)."""
    lib = _lib.load()
    M, N, K = a.shape[0], b.shape[0], a.shape[1] * 2
    if c.dtype not in _DTYPE_CODE:
        raise ValueError(f"c must be float32 or bfloat16, got {c.dtype}")
    if c.dim() != 2 or tuple(c.shape) != (M, N) or c.stride(1) != 1:
        raise ValueError(f"c must be [M, N] = [{M}, {N}] with unit column stride, got {tuple(c.shape)} strides {c.stride()}")
    if b.shape[1] * 2 != K:
        raise ValueError(f"a and b disagree on K: {K} vs {b.shape[1] * 2}")
    if (a_sf.rows, a_sf.K) != (M, K) or (b_sf.rows, b_sf.K) != (N, K):
        raise ValueError("packed scales do not match the operand shapes")
    if a_sf.tile_rows != 128:
        raise ValueError("a's scales must be in the usual packing (tile_rows = 128)")
    if b_sf.tile_rows != 128:
        if (M > 128) != (b_sf.tile_rows == 224):
            raise ValueError(f"b's scales are packed per {b_sf.tile_rows}-row tile: 224 is read by the M > 128 tile kernel, "
                             f"smaller heights by the M <= 128 kernel (M = {M})")
        flags |= _lib.B_TILE_ROWS(b_sf.tile_rows)
    ldc = c.stride(0) if M > 1 else N  # the stride of a size-1 dimension is arbitrary
    ws_ptr = ws_bytes = 0
    if M <= 128 or (flags & _lib.PATH_MASK) == _lib.PATH_TILE_SPLITK or split_k_pays():
        ws_bytes = int(lib.wb200_mxfp4_gemm_workspace_bytes(M, N, K))  # skinny shapes and split-K shapes use one
        if ws_bytes:
            ws_ptr = _workspace(a.device, ws_bytes, "skinny" if M <= 128 else "splitk").data_ptr()
    dev_index = a.device.index
    if dev_index is None or dev_index == torch.cuda.current_device():
        rc = lib.wb200_mxfp4_gemm(M, N, K, a.data_ptr(), a_sf.data.data_ptr(), b.data_ptr(), b_sf.data.data_ptr(),
                                  c.data_ptr(), _DTYPE_CODE[c.dtype], ldc, ws_ptr, ws_bytes, flags, _stream())
    else:
        with torch.cuda.device(a.device):
            rc = lib.wb200_mxfp4_gemm(M, N, K, a.data_ptr(), a_sf.data.data_ptr(), b.data_ptr(), b_sf.data.data_ptr(),
                                      c.data_ptr(), _DTYPE_CODE[c.dtype], ldc, ws_ptr, ws_bytes, flags, _stream())
    if rc:
        _lib.check(rc)


_FP8_FORMATS = {torch.float8_e5m2: _lib.E5M2, torch.float8_e4m3fn: _lib.E4M3}


def quantize_mxfp8(x: torch.Tensor, dtype: torch.dtype = torch.float8_e5m2, want_rowmajor: bool = True, want_packed: bool = True):
    """f32 or bf16 [rows, K] -> (f8 [rows, K] of `dtype`, scales [rows, K/32] uint8 or None, PackedScales or None)."""
    lib = _lib.load()
    if not x.is_cuda or x.dtype not in _DTYPE_CODE or x.dim() != 2:
        raise ValueError(f"x must be a 2-D float32 or bfloat16 CUDA tensor, got {x.dtype} {tuple(x.shape)}")
    if dtype not in _FP8_FORMATS:
        raise ValueError(f"dtype must be torch.float8_e5m2 or torch.float8_e4m3fn, got {dtype}")
    if x.stride(1) != 1:
        x = x.contiguous()
    rows, K = x.shape
    if K % SCALE_GROUP_SIZE or not (want_rowmajor or want_packed):
        raise ValueError("K must be a multiple of 32 and at least one scale layout asked for")
    q = torch.empty(rows, K, dtype=torch.uint8, device=x.device)
    s_rm = torch.empty(rows, K // SCALE_GROUP_SIZE, dtype=torch.uint8, device=x.device) if want_rowmajor else None
    s_pk = torch.empty(packed_scale_bytes(rows, K), dtype=torch.uint8, device=x.device) if want_packed else None
    with torch.cuda.device(x.device):
        _lib.check(lib.wb200_quantize_mxfp8(x.data_ptr(), _DTYPE_CODE[x.dtype], x.stride(0) if rows > 1 else K, rows, K,
                                            _FP8_FORMATS[dtype], q.data_ptr(), s_rm.data_ptr() if want_rowmajor else None,
                                            s_pk.data_ptr() if want_packed else None, _stream()))
    return q.view(dtype), s_rm, (PackedScales(s_pk, rows, K) if want_packed else None)


def scaled_gemm_mxfp8_packed(a: torch.Tensor, a_sf: PackedScales, b: torch.Tensor, b_sf: PackedScales, c: torch.Tensor,
                             elem_format: int | None = None, flags: int = 0, b_fp4: bool = False) -> None:
    """c [M, N] = dequant(a) @ dequant(b)^T for 8-bit operands a [M, K], b [N, K] (torch float8 tensors, or
    int8 / uint8 bytes with `elem_format` given) and packed E8M0 scales, on the current stream.
    b_fp4: the mixed pair — b is packed E2M1, [N, K/2] uint8 as for the MXFP4 GEMM, a stays 8-bit (K % 128 == 0)."""
    lib = _lib.load()
    if elem_format is None:
        if a.dtype not in _FP8_FORMATS:
            raise ValueError(f"give elem_format for operands of type {a.dtype}")
        elem_format = _FP8_FORMATS[a.dtype]
    for name, t in (("a", a), ("b", b)):
        if t.element_size() != 1 or t.dim() != 2 or not t.is_cuda or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous 2-D CUDA tensor of 8-bit elements")
    M, K = a.shape
    N = b.shape[0]
    if a_sf.tile_rows != 128 or b_sf.tile_rows > 128 or (b_sf.tile_rows != 128 and M > 128):
        raise ValueError("the 8-bit GEMM reads per-tile weight scales (tile_rows < 128) on its M <= 128 path only")
    if b_sf.tile_rows != 128:
        flags |= _lib.B_TILE_ROWS(b_sf.tile_rows)
    if b_fp4:
        if b.dtype not in (torch.uint8, torch.int8) or K % 128:
            raise ValueError("4-bit weights: b must be uint8 [N, K/2] (packed E2M1) and K a multiple of 128")
        elem_format |= _lib.B_FP4
    if b.shape[1] * (2 if b_fp4 else 1) != K or (a_sf.rows, a_sf.K) != (M, K) or (b_sf.rows, b_sf.K) != (N, K):
        raise ValueError("operand and scale shapes do not agree")
    if c.dtype not in _DTYPE_CODE or tuple(c.shape) != (M, N) or c.stride(1) != 1:
        raise ValueError(f"c must be f32 or bf16 [{M}, {N}] with unit column stride")
    ws_ptr = ws_bytes = 0
    if M <= 128:  # the skinny stream-K path needs its workspace
        ws_bytes = int(lib.wb200_mxfp4_gemm_workspace_bytes(M, N, K))
        ws_ptr = _workspace(a.device, ws_bytes, "skinny").data_ptr()
    with torch.cuda.device(a.device):
        _lib.check(lib.wb200_mxfp8_gemm(M, N, K, a.data_ptr(), a_sf.data.data_ptr(), b.data_ptr(), b_sf.data.data_ptr(),
                                        c.data_ptr(), _DTYPE_CODE[c.dtype], c.stride(0) if M > 1 else N, elem_format, ws_ptr,
                                        ws_bytes, flags, _stream()))


class WeightScaleCache:
    """Packed copies of weight scales, so that a weight's scales are repacked once and reused by later calls.

    An entry belongs to one tensor OBJECT at one version: it is found by address, shape, strides and version counter,
    and used only while a weak reference shows that the very tensor it was made from is still alive. A new tensor
    that the allocator places at a freed tensor's address therefore never meets the old packing, and an in-place
    write (which bumps the version of every view) makes the next call repack. What the cache cannot see is a write
    through a raw pointer (a C extension, a CUDA graph replay that rewrites the scales): call `clear()` — or
    `ScaledGemmKernel.drop_cached_weights()` — after such a write."""

    def __init__(self, capacity: int = 64):
        self.capacity = capacity
        self._entries: OrderedDict = OrderedDict()

    def get(self, scale: torch.Tensor, tile_rows: int = 128) -> PackedScales:
        key = (scale.data_ptr(), tuple(scale.shape), scale.stride(), scale.device.index, scale._version, tile_rows)
        hit = self._entries.get(key)
        if hit is not None:
            owner, packed = hit
            if owner() is scale:
                self._entries.move_to_end(key)
                return packed
            del self._entries[key]  # same address, another (or a dead) tensor: the packing is not this tensor's
        packed = repack_scales(scale, tile_rows=tile_rows)
        self._entries[key] = (weakref.ref(scale), packed)
        while len(self._entries) > self.capacity:
            self._entries.popitem(last=False)
        return packed

    def drop(self, scale: torch.Tensor) -> None:
        """Forget every packing made from this tensor's memory (any version)."""
        for key in [k for k in self._entries if k[0] == scale.data_ptr() and k[3] == scale.device.index]:
            del self._entries[key]

    def clear(self) -> None:
        self._entries.clear()


def check_device_status() -> None:
    """Synchronise the current stream and raise DeviceTimeoutError if a kernel's bounded wait gave up."""
    detail = ctypes.c_int(0)
    _lib.check(_lib.load().wb200_check_device_status(_stream(), ctypes.byref(detail)))


def quantize_mxfp4(x: torch.Tensor, want_rowmajor: bool = True, want_packed: bool = True):
    """f32 or bf16 [rows, K] -> (codes [rows, K/2] uint8, scales [rows, K/32] uint8 or None, PackedScales or None),
    one pass on the current stream. The packed scales feed the GEMM directly, without a repack."""
    lib = _lib.load()
    if not x.is_cuda:
        raise ValueError("x must be a CUDA tensor; wave_b200 has no CPU path")
    if x.dtype not in _DTYPE_CODE or x.dim() != 2:
        raise ValueError(f"x must be a 2-D float32 or bfloat16 tensor, got {x.dtype} {tuple(x.shape)}")
    if x.stride(1) != 1:
        x = x.contiguous()
    rows, K = x.shape
    if K % SCALE_GROUP_SIZE:
        raise ValueError(f"K = {K} is not a multiple of {SCALE_GROUP_SIZE}")
    if not (want_rowmajor or want_packed):
        raise ValueError("ask for at least one scale layout")
    q = torch.empty(rows, K // 2, dtype=torch.uint8, device=x.device)
    s_rm = torch.empty(rows, K // SCALE_GROUP_SIZE, dtype=torch.uint8, device=x.device) if want_rowmajor else None
    s_pk = torch.empty(packed_scale_bytes(rows, K), dtype=torch.uint8, device=x.device) if want_packed else None
    with torch.cuda.device(x.device):
        _lib.check(lib.wb200_quantize_mxfp4(x.data_ptr(), _DTYPE_CODE[x.dtype], x.stride(0) if rows > 1 else K, rows, K, q.data_ptr(),
                                            s_rm.data_ptr() if want_rowmajor else None,
                                            s_pk.data_ptr() if want_packed else None, _stream()))
    return q, s_rm, (PackedScales(s_pk, rows, K) if want_packed else None)
