"""One call, several GPUs, one process: the form of the reference's multi-device launch.

In the reference, `wave_compile` with `options.num_devices > 1` (set by the kernel's `DeviceConstraint`s,
wave_lang/kernel/wave/compile.py:1141-1142) returns a kernel whose call takes tensors that live in one place,
slices them per device, dispatches one kernel per device and merges the output slices
(wave_lang/kernel/compiler/host_utils.py:158-376), all from one process through `MultiDeviceLaunchable`
(wave_lang/runtime/multi_device_launch.py:38-273; test: tests/kernel/dist_gemm_test.py:60-101).

Here the same call, `gemm(a, a_scale, b, b_scale, c)` with tensors on one GPU or in host memory, is served by the
native launcher of libwave_b200.so (`wb200_multi_gpu_*`): b is split by rows over the GPUs once and kept there
(a weight is sharded when it is first seen, not on every call), a is copied to every GPU over NVLink, every GPU
computes its column block of C on its own stream, and the blocks are copied side by side into c. PyTorch provides
the per-device memory; the copies between GPUs and the launches are the library's.
"""

from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from . import _lib, ops
from .lang import as_output_dtype


def shard_bounds(N: int, num_devices: int, index: int, granule: int = 128) -> tuple[int, int]:
    """Rows of b owned by device `index` (the library's rule: multiples of `granule`, dealt as evenly as possible)."""
    n0, n1 = ctypes.c_int(), ctypes.c_int()
    _lib.check(_lib.load().wb200_multi_gpu_shard_bounds(N, num_devices, index, granule, ctypes.byref(n0), ctypes.byref(n1)))
    return n0.value, n1.value


class MultiDeviceScaledGemm:
    """`gemm(a, a_scale, b, b_scale, c)` over `devices` (default: the first `num_devices` GPUs).

    a [M, K/2], a_scale [M, K/32], b [N, K/2], b_scale [N, K/32] are uint8 tensors on one GPU or in host memory
    (pinned host memory makes the copies asynchronous); c [M, N] (f32 or bf16 as the template says) likewise.
    The call is ordered after the current stream of the tensors' device and returns without waiting; that stream
    (or, for a host c, `synchronize()`) then waits for the result.
    """

    def __init__(self, template, options, devices: Optional[Sequence[int]] = None):
        self.template = template
        self.options = options
        self.out = as_output_dtype(template.output_dtype)
        n = options.num_devices
        self.devices = list(devices) if devices is not None else list(range(n))
        if len(self.devices) != n:
            raise ValueError(f"num_devices = {n} but {len(self.devices)} device ids were given")
        if torch.cuda.device_count() < n:
            raise RuntimeError(f"num_devices = {n} but this process sees {torch.cuda.device_count()} GPU(s); wave_b200 has no CPU path")
        self._lib = _lib.load()
        ids = (ctypes.c_int * n)(*self.devices)
        h = ctypes.c_void_p()
        _lib.check(self._lib.wb200_multi_gpu_create(n, ids, ctypes.byref(h)))
        self._h = h
        self._weights = None   # (key, bounds, per-device (b shard, packed scales))
        self._buffers = {}     # (M, K, N) -> per-device activation / output / workspace tensors
        self.last_gemm_ms: Optional[float] = None     # set by invoke(..., timed=True): longest device time of the GEMM step
        self.last_gather_ms: Optional[float] = None   # and of the copies that merge the column blocks into c

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                self._lib.wb200_multi_gpu_destroy(h)
            except Exception:
                pass

    # ---- weights: sharded once ----------------------------------------------------------------------------------
    def _shard_weights(self, b: torch.Tensor, b_scale: torch.Tensor):
        key = (b.data_ptr(), b_scale.data_ptr(), tuple(b.shape), b._version, b_scale._version, str(b.device))
        if self._weights is not None and self._weights[0] == key:
            return self._weights[1], self._weights[2]
        N = b.shape[0]
        G = len(self.devices)
        bounds = [shard_bounds(N, G, g)[0] for g in range(G)] + [N]
        shards = []
        for g, dev in enumerate(self.devices):
            n0, n1 = bounds[g], bounds[g + 1]
            if n1 == n0:
                shards.append((None, None))
                continue
            d = torch.device("cuda", dev)
            bg = b[n0:n1].to(d, non_blocking=True).contiguous()
            sg = b_scale[n0:n1].to(d, non_blocking=True).contiguous()
            with torch.cuda.device(d):
                shards.append((bg, ops.repack_scales(sg)))
        for dev in self.devices:
            torch.cuda.synchronize(dev)  # once per weight: the shards are resident before the first launch uses them
        self._weights = (key, bounds, shards)
        return bounds, shards

    def drop_cached_weights(self) -> None:
        """Forget the sharded copy of b (after b or b_scale was rewritten in a way torch does not see)."""
        self._weights = None

    def _device_buffers(self, M: int, K: int, bounds):
        key = (M, K, tuple(bounds))
        bufs = self._buffers.get(key)
        if bufs is not None:
            return bufs
        bufs = []
        u8 = torch.uint8
        for g, dev in enumerate(self.devices):
            d = torch.device("cuda", dev)
            n_g = bounds[g + 1] - bounds[g]
            ws_bytes = int(self._lib.wb200_mxfp4_gemm_workspace_bytes(M, max(n_g, 1), K)) if n_g else 0
            # eager callers stay on the plain tile path for M > 128 (see ops.split_k_pays); the skinny path needs its workspace
            if M > 128:
                ws_bytes = 0
            with torch.cuda.device(d):
                ws = torch.empty(max(ws_bytes, 1), dtype=u8, device=d)
                if ws_bytes:
                    _lib.check(self._lib.wb200_workspace_init(ws.data_ptr(), ws_bytes, torch.cuda.current_stream(d).cuda_stream))
                bufs.append(dict(a=torch.empty(M, K // 2, dtype=u8, device=d), a_scale=torch.empty(M, K // 32, dtype=u8, device=d),
                                 a_packed=torch.empty(ops.packed_scale_bytes(M, K), dtype=u8, device=d),
                                 c=torch.empty(M, max(n_g, 1), dtype=self.out.torch_dtype, device=d), ws=ws, ws_bytes=ws_bytes))
                torch.cuda.synchronize(d)
        self._buffers[key] = bufs
        return bufs

    # ---- the call ---------------------------------------------------------------------------------------------------
    def __call__(self, a, a_scale, b, b_scale, c) -> None:
        return self.invoke(a, a_scale, b, b_scale, c)

    def invoke(self, a, a_scale, b, b_scale, c, timed: bool = False) -> None:
        for name, t in (("a", a), ("a_scale", a_scale), ("b", b), ("b_scale", b_scale)):
            if t.dtype not in (torch.uint8, torch.int8) or t.dim() != 2:
                raise ValueError(f"{name} must be a 2-D uint8 / int8 tensor, got {t.dtype} {tuple(t.shape)}")
        M, K = a.shape[0], a.shape[1] * 2
        N = b.shape[0]
        if b.shape[1] * 2 != K or tuple(a_scale.shape) != (M, K // 32) or tuple(b_scale.shape) != (N, K // 32):
            raise ValueError("operand and scale shapes do not agree")
        if c.dtype != self.out.torch_dtype or tuple(c.shape) != (M, N) or c.stride(1) != 1:
            raise ValueError(f"c must be {self.out} [{M}, {N}] with unit column stride")
        a, a_scale = a.contiguous(), a_scale.contiguous()
        bounds, shards = self._shard_weights(b, b_scale)
        bufs = self._device_buffers(M, K, bounds)
        G = len(self.devices)
        Ops = self._lib.DeviceOperands
        arr = (Ops * G)()
        for g in range(G):
            bg, sg = shards[g]
            arr[g] = Ops(bufs[g]["a"].data_ptr(), bufs[g]["a_scale"].data_ptr(), bufs[g]["a_packed"].data_ptr(),
                         bg.data_ptr() if bg is not None else None, sg.data.data_ptr() if sg is not None else None,
                         bufs[g]["c"].data_ptr(), bufs[g]["c"].stride(0), bufs[g]["ws"].data_ptr() if bufs[g]["ws_bytes"] else None,
                         bufs[g]["ws_bytes"])
        nb = (ctypes.c_int * (G + 1))(*bounds)
        lib, h = self._lib, self._h
        src_dev = a.device.index if a.is_cuda else -1
        if a.is_cuda:  # the device streams start after whatever produced a on its device's current stream
            _lib.check(lib.wb200_multi_gpu_wait_for(h, src_dev, torch.cuda.current_stream(a.device).cuda_stream))
        if c.is_cuda and (not a.is_cuda or c.device != a.device):
            _lib.check(lib.wb200_multi_gpu_wait_for(h, c.device.index, torch.cuda.current_stream(c.device).cuda_stream))
        _lib.check(lib.wb200_multi_gpu_broadcast_a(h, M, K, a.data_ptr(), a_scale.data_ptr(), src_dev, arr))
        if timed:
            _lib.check(lib.wb200_multi_gpu_time_begin(h))
        flags = _lib.ACCUMULATE if getattr(self.template, "accumulate", False) else 0
        _lib.check(lib.wb200_multi_gpu_gemm(h, M, K, nb, arr, ops._DTYPE_CODE[self.out.torch_dtype], flags))
        if timed:
            ms = ctypes.c_float()
            _lib.check(lib.wb200_multi_gpu_time_end(h, ctypes.byref(ms)))
            self.last_gemm_ms = float(ms.value)
        dst = (ctypes.c_void_p * 1)(c.data_ptr())
        dst_dev = (ctypes.c_int * 1)(c.device.index if c.is_cuda else -1)
        if timed:
            _lib.check(lib.wb200_multi_gpu_time_begin(h))
        _lib.check(lib.wb200_multi_gpu_gather_c(h, M, nb, arr, ops._DTYPE_CODE[self.out.torch_dtype], 1, dst, dst_dev, c.stride(0)))
        if timed:
            ms = ctypes.c_float()
            _lib.check(lib.wb200_multi_gpu_time_end(h, ctypes.byref(ms)))
            self.last_gather_ms = float(ms.value)
        if c.is_cuda:
            _lib.check(lib.wb200_multi_gpu_join(h, c.device.index, torch.cuda.current_stream(c.device).cuda_stream))
        self._keep = (a, a_scale, arr)  # alive until the next call: the launches are asynchronous

    def synchronize(self) -> None:
        """Wait for every device stream (needed before reading a host-resident c) and raise if a device-side wait gave up."""
        _lib.check(self._lib.wb200_multi_gpu_synchronize(self._h))
