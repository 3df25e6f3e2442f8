"""Scaled GEMM on HOST buffers: copy in, compute, copy out, with the three stages of successive
calls overlapped on separate CUDA streams.

The reference's multi-device launcher takes host-resident tensors and moves slices to the devices
and back inside the call (wave_lang/kernel/compiler/host_utils.py:208-330). For a single GPU the
same job is a three-stage pipeline over PCIe: host-to-device copies of call i+1 and the
device-to-host copy of call i-1 run while the GEMM of call i computes. Inputs and outputs are
pinned host tensors; every call still moves all of its bytes.
"""

from __future__ import annotations

import torch

from .compile import wave_compile
from .templates import get_tagged_mxfp4_gemm


class HostScaledGemm:
    """submit(a, a_scale, b, b_scale, c_host) enqueues one GEMM on pinned host tensors and returns at
    once; drain() waits for everything submitted. `depth` device buffer sets are cycled, so a buffer
    is reused only after the call that used it has copied its result out."""

    def __init__(self, M: int, N: int, K: int, output_dtype, device=None, depth: int = 3):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        kernel, options = get_tagged_mxfp4_gemm((M, N, K), output_dtype=output_dtype)
        self.out_dtype = kernel.output_dtype.torch_dtype
        self.depth = depth
        self._gemms = [wave_compile(options, kernel) for _ in range(depth)]  # one activation-scale buffer each
        u8 = dict(dtype=torch.uint8, device=self.device)
        self._bufs = [(torch.empty(M, K // 2, **u8), torch.empty(M, K // 32, **u8), torch.empty(N, K // 2, **u8),
                       torch.empty(N, K // 32, **u8), torch.empty(M, N, dtype=self.out_dtype, device=self.device))
                      for _ in range(depth)]
        self._in, self._compute, self._out = (torch.cuda.Stream(self.device) for _ in range(3))
        self._copied_in = [torch.cuda.Event() for _ in range(depth)]
        self._computed = [torch.cuda.Event() for _ in range(depth)]
        self._copied_out = [torch.cuda.Event() for _ in range(depth)]
        self._count = 0

    def submit(self, a, a_scale, b, b_scale, c_host) -> None:
        for t in (a, a_scale, b, b_scale, c_host):
            if t.is_cuda or not t.is_pinned():
                raise ValueError("HostScaledGemm takes pinned host tensors")
        i = self._count % self.depth
        da, das, db, dbs, dc = self._bufs[i]
        with torch.cuda.stream(self._in):
            if self._count >= self.depth:
                self._in.wait_event(self._copied_out[i])  # the set's previous result has left the device
            for src, dst in ((a, da), (a_scale, das), (b, db), (b_scale, dbs)):
                dst.copy_(src, non_blocking=True)
            self._copied_in[i].record(self._in)
        with torch.cuda.stream(self._compute):
            self._compute.wait_event(self._copied_in[i])
            self._gemms[i](da, das, db, dbs, dc)
            self._computed[i].record(self._compute)
        with torch.cuda.stream(self._out):
            self._out.wait_event(self._computed[i])
            c_host.copy_(dc, non_blocking=True)
            self._copied_out[i].record(self._out)
        self._count += 1

    def drain(self) -> None:
        for s in (self._in, self._compute, self._out):
            s.synchronize()

    def join(self, stream=None) -> None:
        """Make `stream` (default: the current stream) wait, on the device, for every call submitted so
        far; the host does not block."""
        if self._count == 0:
            return
        s = torch.cuda.current_stream(self.device) if stream is None else stream
        s.wait_event(self._copied_out[(self._count - 1) % self.depth])  # copies out run in submission order
