"""CUDA-graph replay of a compiled scaled-GEMM call, for launch-bound shapes.

A decode-shaped GEMM (M <= 16) runs for ~25 microseconds; the Python call that launches it (argument
checks, ctypes marshalling, descriptor look-ups, two launches) costs about as much. The reference has
the same problem and only measures it (`profile_python_wrapper`, wave_lang/kernel/wave/compile.py:341-371).
Here the call is captured once into a CUDA graph over fixed buffers and replayed; new inputs are
copied into (or written directly to) those buffers by the caller.
"""

from __future__ import annotations

import torch


class GraphedScaledGemm:
    """Capture `gemm(a, a_scale, b, b_scale, c)` over the given tensors; `replay()` launches it again.

    The tensors are the graph's fixed buffers: update a, a_scale (and read c) in place between
    replays. The weights are taken as constant: b is read in place, but b_scale was packed once
    before the capture, so later changes to b_scale are not seen by the graph.
    The kernel is warmed up before capture, because the library's first call on a device does
    one-time set-up that must not run inside a capture.
    """

    def __init__(self, gemm, a, a_scale, b, b_scale, c, warmup: int = 2):
        self.tensors = (a, a_scale, b, b_scale, c)
        side = torch.cuda.Stream(a.device)
        side.wait_stream(torch.cuda.current_stream(a.device))
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):
                gemm(a, a_scale, b, b_scale, c)
        torch.cuda.current_stream(a.device).wait_stream(side)
        torch.cuda.synchronize(a.device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            gemm(a, a_scale, b, b_scale, c)

    def replay(self) -> None:
        self.graph.replay()
