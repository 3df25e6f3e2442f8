"""`wave_compile` and the callable it returns, for the MXFP4 scaled-GEMM templates.

The reference compiles a traced kernel with its JIT and returns a `WaveKernel` whose call launches
the generated binary (wave_lang/kernel/wave/compile.py:1021-1280 `wave_compile`, :140-339
`WaveKernel`). Here nothing is generated at run time: the templates are descriptors, the kernels
are precompiled in libwave_b200.so, and "compiling" checks the options and picks the kernel path.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

import torch

from . import _lib, ops
from .lang import DataType, f32


class SchedulingType:
    """Names of the reference's scheduling modes (wave_lang/kernel/wave/scheduling/schedule_enums.py).
    Accepted and ignored: the B200 kernels have one fixed TMA / tcgen05 pipeline."""
    NONE = "none"
    PREFETCH = "prefetch"
    MODULO = "modulo"
    FOUR_STAGE = "four_stage"
    MANUAL = "manual"


@dataclass
class WaveCompileOptions:
    """The subset of the reference's option set (wave_lang/kernel/wave/compile_options.py:18-160)
    that callers of the MXFP4 templates set. Fields that steer AMD code generation are accepted so
    that existing call sites run, and have no effect."""

    # symbol mappings
    subs: dict = field(default_factory=dict)
    dynamic_symbols: list = field(default_factory=list)
    # general / scheduling (no effect)
    postprocess: Optional[str] = None
    canonicalize: bool = True
    func_name: str = "isolated_benchmark"
    schedule: Any = SchedulingType.NONE
    use_scheduling_barriers: bool = False
    multi_buffer_count: Optional[int] = None
    # backend
    backend: str = "cuda"
    device: str = "cuda"
    target: str = "sm_100a"
    num_devices: int = 1
    use_water_backend: bool = False
    # benchmark options
    run_bench: bool = False
    benchmark_batch_size: Optional[int] = None
    benchmark_repetitions: Optional[int] = None
    benchmark_results_file: Optional[str] = None
    profile_python_wrapper: bool = False
    profile_python_cprofile: bool = True  # False: timeit instead of cProfile
    profile_python_warmup: int = 1
    profile_python_repetitions: int = 1000
    # performance options (no effect unless noted)
    wave_runtime: bool = True
    use_buffer_ops: bool = False
    use_global_to_shared: bool = False
    linearize_shared_access: bool = False
    minimize_shared_allocs: bool = True
    reorder_allocs: bool = True
    use_bound_check: bool = False
    specialize: bool = False
    eliminate_epilogue: bool = False
    print_mlir: bool = False
    print_mlir_file: Optional[str] = None
    kernel_hash: Optional[str] = None
    # wave_b200 only: force a kernel path (a PATH_* flag of the C ABI), 0 = choose by shape
    kernel_path: int = _lib.PATH_AUTO
    # wave_b200 only: the caller asserts that b and b_scale are not written by the kernel that precedes the call
    # in the stream (weights of a layer), so the GEMM may start streaming them while that kernel drains
    # (WB200_OVERLAP_PREVIOUS: programmatic dependent launch)
    overlap_previous: bool = False
    # wave_b200 only: for M <= 128 pack a weight's scales per tile of the height that gives every SM the same number of
    # weight tiles (include/wave_b200.h, wb200_decode_tile_rows) instead of per 128 rows; False keeps one packing
    decode_tiled_weight_scales: bool = True


def get_default_arch() -> str:
    """The reference returns the AMD gcnArchName (wave_lang/kernel/wave/utils/run_utils.py:137-156);
    this library has exactly one target."""
    return "sm_100a"


def set_default_run_config(options: WaveCompileOptions) -> WaveCompileOptions:
    """wave_lang/kernel/wave/utils/run_utils.py:183-198: fill in device and target."""
    options.device = "cuda"
    options.target = get_default_arch()
    return options


def validate_options(options: WaveCompileOptions) -> None:
    """Reject option combinations this library cannot honour (the reference's validate_options,
    wave_lang/kernel/wave/compile.py:1489-1500, raises ValueError in the same way)."""
    if options.num_devices < 1:
        raise ValueError(f"num_devices must be at least 1, got {options.num_devices}")
    if options.kernel_path not in (_lib.PATH_AUTO, _lib.PATH_TILE_1CTA, _lib.PATH_TILE_2CTA, _lib.PATH_SKINNY, _lib.PATH_TILE_SPLITK):
        raise ValueError(f"unknown kernel_path {options.kernel_path}")


class ScaledGemmKernel:
    """The callable `wave_compile` returns: `kernel(a, a_scale, b, b_scale, c)` writes c in place and
    returns None (wave_lang/kernel/wave/compile.py:225-339).

    a [M, K/2] (or [B, M, K/2]) and b [N, K/2] are packed E2M1 bytes, a_scale [.., K/32] and
    b_scale [N, K/32] are E8M0 bytes, c is f32 or bf16 as the template says. M, N, K are read from
    the tensors (the reference's dynamic dims, compile.py:256-265); static sizes given at template
    creation are checked against them unless they were declared dynamic.
    """

    def __init__(self, template, options: WaveCompileOptions):
        self.template = template
        self.options = options
        self.asm = ""  # the reference exposes generated code here; nothing is generated at run time
        self._weight_scales = ops.WeightScaleCache()
        self._a_scale_buf: dict[int, torch.Tensor] = {}
        self._workspaces = ops.WorkspacePool()  # this object's own: calls through another object may overlap with these
        self._plans: dict = {}
        self._tile_rows: dict = {}
        self._lib = _lib.load()
        self._static = None
        if template.shape is not None and not options.dynamic_symbols:
            self._static = tuple(template.shape)

    # the reference offers both spellings
    def __call__(self, *args):
        return self.invoke(*args)

    def invoke(self, a, a_scale, b, b_scale, c) -> None:
        if self.options.run_bench and not getattr(self, "_in_bench", False):
            self._in_bench = True
            try:
                self.invoke(a, a_scale, b, b_scale, c)
                run_bench(self.options, self.invoke, a, a_scale, b, b_scale, c)
            finally:
                self._in_bench = False
            return None
        # Fast path: plain tensors whose (shape, dtype, stride, device) signature was validated before.
        # The signature check is what stands between the caller and the C ABI on every call, so it is
        # done once per distinct signature and remembered.
        if type(a_scale) is torch.Tensor and type(b_scale) is torch.Tensor and a.is_cuda:
            # (the stream is part of the signature: the plan holds a workspace, and calls on different streams may overlap)
            sig = (a.shape, a.stride(), a.dtype, a_scale.shape, a_scale.stride(), b.shape, b.stride(), b_scale.shape,
                   c.shape, c.stride(), c.dtype, a.device, torch.cuda.current_stream(a.device).cuda_stream)
            plan = self._plans.get(sig)
            if plan is not None:
                return self._launch(plan, a, a_scale, b, b_scale, c)
        return self._invoke_checked(a, a_scale, b, b_scale, c)

    def _launch(self, plan, a, a_scale, b, b_scale, c) -> None:
        M, N, K, a_buf, ws_ptr, ws_bytes, flags, dtype_code, dev_index, _ws_keepalive = plan
        if M > 128 and ws_bytes and not ops.split_k_pays() and (flags & _lib.PATH_MASK) != _lib.PATH_TILE_SPLITK:
            ws_ptr = ws_bytes = 0  # eager call: stay on the plain tile path (see ops.split_k_pays)
        tile_rows = self._weight_tile_rows(M, N, dev_index)
        b_sf = self._weight_scales.get(b_scale, tile_rows)
        if tile_rows != 128:
            flags |= _lib.B_TILE_ROWS(tile_rows)
        lib = self._lib
        if dev_index == torch.cuda.current_device():
            rc = lib.wb200_mxfp4_gemm_repack_a(M, N, K, a.data_ptr(), a_scale.data_ptr(), a_scale.stride(0) if M > 1 else K // 32, a_buf.data_ptr(),
                                               b.data_ptr(), b_sf.data.data_ptr(), c.data_ptr(), dtype_code, c.stride(0) if M > 1 else N,
                                               ws_ptr, ws_bytes, flags, torch.cuda.current_stream().cuda_stream)
        else:
            with torch.cuda.device(dev_index):
                rc = lib.wb200_mxfp4_gemm_repack_a(M, N, K, a.data_ptr(), a_scale.data_ptr(), a_scale.stride(0) if M > 1 else K // 32,
                                                   a_buf.data_ptr(), b.data_ptr(), b_sf.data.data_ptr(), c.data_ptr(),
                                                   dtype_code, c.stride(0) if M > 1 else N, ws_ptr, ws_bytes, flags,
                                                   torch.cuda.current_stream().cuda_stream)
        if rc:
            _lib.check(rc)

    def _invoke_mxfp8(self, a, a_scale, b, b_scale, c) -> None:
        t = self.template
        for name, x in (("a", a), ("b", b)):
            if x.element_size() != 1 or x.dim() != 2 or not x.is_cuda:
                raise ValueError(f"{name} must be a 2-D CUDA tensor of 8-bit elements, got {x.dtype} {tuple(x.shape)}")
        if c.dtype != t.output_dtype.torch_dtype:
            raise ValueError(f"this kernel writes {t.output_dtype}; got an output tensor of {c.dtype}")
        a, b = a.contiguous(), b.contiguous()  # non-contiguous inputs are copied, as the reference does (run_utils.py:106-109)
        M, K = a.shape
        N = b.shape[0]
        b_fp4 = t.weight_bits == 4
        if b_fp4:
            b = ops._as_u8(b, "b")
            if b.shape[1] * 2 != K:
                raise ValueError(f"b must be packed E2M1 [N, K/2] = [{N}, {K // 2}], got {tuple(b.shape)}")
        if self._static is not None and self._static != (M, N, K):
            raise ValueError(f"kernel was built for (M, N, K) = {self._static}, called with {(M, N, K)}")
        a_sf = a_scale if isinstance(a_scale, ops.PackedScales) else self._pack_activation_scales(a_scale, M, K)
        if isinstance(b_scale, ops.PackedScales):
            b_sf = b_scale
        else:
            idx = a.device.index if a.device.index is not None else torch.cuda.current_device()
            b_sf = self._weight_scales.get(self._check_scale(b_scale, N, K, "b_scale"), self._weight_tile_rows(M, N, idx))
        fmt = _lib.E5M2 if t.element_format == "f8e5m2" else _lib.E4M3
        flags = self.options.kernel_path | self._raster_flags() | (_lib.ACCUMULATE if t.accumulate else 0)
        ops.scaled_gemm_mxfp8_packed(a, a_sf, b, b_sf, c, fmt, flags, b_fp4=b_fp4)

    def _invoke_checked(self, a, a_scale, b, b_scale, c) -> None:
        t = self.template
        if t.element_bits == 8:
            return self._invoke_mxfp8(a, a_scale, b, b_scale, c)
        if a.dim() == 3:  # batched activations, shared weights (tests/kernel/wave_gemm_mxfp_test.py:205-288)
            if c.dim() != 3 or not c.is_contiguous():
                raise ValueError("batched call needs a contiguous 3-D output")
            a2 = a.reshape(-1, a.shape[-1])
            as2 = a_scale if isinstance(a_scale, ops.PackedScales) else a_scale.reshape(-1, a_scale.shape[-1])
            return self.invoke(a2, as2, b, b_scale, c.view(-1, c.shape[-1]))
        for name, x in (("a", a), ("b", b)):
            ops._as_u8(x, name)
            if x.dim() != 2:
                raise ValueError(f"{name} must be 2-D, got shape {tuple(x.shape)}")
        if not c.is_cuda:
            raise ValueError("c must be a CUDA tensor")
        if c.dtype != t.output_dtype.torch_dtype:
            raise ValueError(f"this kernel writes {t.output_dtype}; got an output tensor of {c.dtype}")
        # Non-contiguous inputs are copied, as the reference does (run_utils.py:106-109).
        contiguous_inputs = a.is_contiguous() and b.is_contiguous()
        if not a.is_contiguous():
            a = a.contiguous()
        if not b.is_contiguous():
            b = b.contiguous()
        M, N, K = a.shape[0], b.shape[0], a.shape[1] * 2
        if self._static is not None and self._static != (M, N, K):
            raise ValueError(f"kernel was built for (M, N, K) = {self._static}, called with {(M, N, K)}")
        if t.broadcast_a_scale:
            ops._as_u8(a_scale, "a_scale")
            if tuple(a_scale.shape) != (M,):
                raise ValueError(f"a_scale must be [{M}] (one scale per row), got {tuple(a_scale.shape)}")
            a_scale = ops.repack_scales_broadcast(a_scale, K, out=self._a_scale_buffer(a.device, M, K))
        if t.preshuffled_scales and not (isinstance(a_scale, ops.PackedScales) and isinstance(b_scale, ops.PackedScales)):
            raise ValueError(f"{t.name} takes pre-shuffled scales: pass mxfp_utils.e8m0_shuffle(scale) for a_scale and b_scale")
        flags = self.options.kernel_path | self._raster_flags()
        if t.accumulate:
            flags |= _lib.ACCUMULATE
        if self.options.overlap_previous:
            flags |= _lib.OVERLAP_PREVIOUS
        plain = type(a_scale) is torch.Tensor and type(b_scale) is torch.Tensor
        if plain:
            self._check_scale(a_scale, M, K, "a_scale")
            self._check_scale(b_scale, N, K, "b_scale")
        if (plain and contiguous_inputs and a_scale.stride(1) == 1 and c.dim() == 2 and tuple(c.shape) == (M, N)
                and c.stride(1) == 1 and b.shape[1] * 2 == K):
            # remember this signature: later calls go straight to the combined repack + GEMM entry point
            ws_bytes = ws_ptr = 0
            ws = None  # the plan keeps the workspace tensor alive: it holds its address
            ws_bytes = int(self._lib.wb200_mxfp4_gemm_workspace_bytes(M, N, K))
            if ws_bytes:
                ws = ops._workspace(a.device, ws_bytes, "skinny" if M <= 128 else "splitk", self._workspaces)
                ws_ptr = ws.data_ptr()
            idx = a.device.index if a.device.index is not None else torch.cuda.current_device()
            a_buf = self._a_scale_buffer(a.device, M, K)
            plan = (M, N, K, a_buf, ws_ptr, ws_bytes, flags, ops._DTYPE_CODE[c.dtype], idx, ws)
            sig = (a.shape, a.stride(), a.dtype, a_scale.shape, a_scale.stride(), b.shape, b.stride(), b_scale.shape,
                   c.shape, c.stride(), c.dtype, a.device, torch.cuda.current_stream(a.device).cuda_stream)
            self._plans[sig] = plan
            return self._launch(plan, a, a_scale, b, b_scale, c)
        a_sf = self._pack_activation_scales(a_scale, M, K)
        if isinstance(b_scale, ops.PackedScales):
            b_sf = b_scale
        else:
            idx = a.device.index if a.device.index is not None else torch.cuda.current_device()
            b_sf = self._weight_scales.get(self._check_scale(b_scale, N, K, "b_scale"), self._weight_tile_rows(M, N, idx))
        ops.scaled_gemm_packed(a, a_sf, b, b_sf, c, flags)  # adds the tile-height bits a tiled packing needs

    @staticmethod
    def _check_scale(s, rows, K, name):
        ops._as_u8(s, name)
        if tuple(s.shape) != (rows, K // ops.SCALE_GROUP_SIZE):
            raise ValueError(f"{name} must be [{rows}, {K // ops.SCALE_GROUP_SIZE}], got {tuple(s.shape)}")
        return s

    def _weight_tile_rows(self, M: int, N: int, dev_index: int) -> int:
        """Rows per tile the weight scales are packed for: the decode kernel's balanced tile height for M <= 128 (every
        SM gets the same number of weight tiles, `ops.decode_tile_rows`), 128 otherwise. Weights are packed once per
        (weight, height) and cached, so a weight used at both ends of the M range keeps two packings."""
        if M > 128 or not self.options.decode_tiled_weight_scales:
            return 128
        key = (N, dev_index)
        h = self._tile_rows.get(key)
        if h is None:
            h = self._tile_rows[key] = ops.decode_tile_rows(N, dev_index)
        return h

    def drop_cached_weights(self, b_scale: torch.Tensor | None = None) -> None:
        """Forget the packed copy of `b_scale` (of every weight when None). The kernel repacks a weight's scales on
        first use and reuses the packing while the same tensor object keeps its version; after a write the version
        counter cannot see (a raw-pointer write, a graph replay that refreshes the scales in place), call this
        before the next GEMM. Launch plans that captured the old packing are dropped with it."""
        if b_scale is None:
            self._weight_scales.clear()
        else:
            self._weight_scales.drop(b_scale)
        self._plans.clear()

    def _raster_flags(self) -> int:
        """The template's reorder_workgroups / group_size_n as the tile kernels' raster-group bits. The reference
        counts groups in workgroups of BLOCK_N columns (tagged_mxfp4_gemm.py, _reorder_mxfp4_workgroups); the
        tile kernels here walk 256-column tiles, so the group keeps its width in columns."""
        h = self.template.hints
        if not h.get("reorder_workgroups", True):
            return _lib.GROUP_N_ALL
        g = h.get("group_size_n")
        if g is None:
            return 0
        block_n = int(h.get("block_shape", (256, 256, 256))[1])
        return _lib.GROUP_N(max(1, min(254, (int(g) * block_n) // 256)))

    def _a_scale_buffer(self, device, M, K):
        idx = device.index or 0
        need = ops.packed_scale_bytes(M, K)
        buf = self._a_scale_buf.get(idx)
        if buf is None or buf.numel() < need:
            buf = torch.empty(need, dtype=torch.uint8, device=device)
            self._a_scale_buf[idx] = buf
            self._plans.clear()  # plans hold the old buffer
        return buf

    def _pack_activation_scales(self, a_scale, M, K):
        if isinstance(a_scale, ops.PackedScales):
            return a_scale
        self._check_scale(a_scale, M, K, "a_scale")
        return ops.repack_scales(a_scale, out=self._a_scale_buffer(a_scale.device, M, K))


def invoke_with_profile(options: WaveCompileOptions, invoke, *args, **kwargs):
    """Measure the HOST side of a call, as the reference does for its own wrapper
    (wave_lang/kernel/wave/compile.py:341-365): `profile_python_warmup` untimed calls, then
    `profile_python_repetitions` calls under cProfile (statistics printed, sorted by cumulative time) or, with
    `profile_python_cprofile` off, under timeit (one "Time: ...s, ...s per iteration" line). For a decode-shaped GEMM
    the wrapper costs about as much as the kernel runs, which is what this is for. Launches are asynchronous, so
    what is measured is argument checking, marshalling and the launch calls, not GPU time."""
    for _ in range(options.profile_python_warmup):
        invoke(*args, **kwargs)
    repetitions = options.profile_python_repetitions
    if options.profile_python_cprofile:
        import cProfile

        with cProfile.Profile() as pr:
            for _ in range(repetitions):
                res = invoke(*args, **kwargs)
        pr.print_stats(sort="cumulative")
        return res
    import timeit

    seconds = timeit.timeit(lambda: invoke(*args, **kwargs), number=repetitions)
    print(f"Time: {seconds:.3f}s, {seconds / repetitions:.6f}s per iteration")
    return invoke(*args, **kwargs)


class ScaledGemmKernelWithProfile(ScaledGemmKernel):
    """What `wave_compile` returns when `options.profile_python_wrapper` is set (the reference's
    WaveKernelWithProfile, wave_lang/kernel/wave/compile.py:368-371)."""

    def __call__(self, *args, **kwargs):
        return invoke_with_profile(self.options, self.invoke, *args, **kwargs)


def run_bench(options: WaveCompileOptions, invoke, *args) -> dict:
    """`options.run_bench`: time the kernel on the device after the call, as the reference does by handing the compiled
    module to its benchmark tool (wave_lang/kernel/wave/compile.py:317-329): `benchmark_repetitions` (default 10)
    batches of `benchmark_batch_size` (default 20) launches between CUDA events; the result, in the shape of that
    tool's report, goes to `benchmark_results_file` or is printed."""
    import json

    batch = options.benchmark_batch_size or 20
    reps = options.benchmark_repetitions or 10
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for _ in range(reps):
        e0.record()
        for _ in range(batch):
            invoke(*args)
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3 / batch)
    result = {"benchmarks": [{"name": options.func_name, "real_time": sum(times) / len(times), "min_time": min(times),
                              "time_unit": "us", "iterations": reps, "batch_size": batch}]}
    text = json.dumps(result, sort_keys=True, indent=4)
    if options.benchmark_results_file:
        with open(options.benchmark_results_file, "w") as f:
            f.write(text)
    else:
        print(text)
    return result


def wave_compile(options: WaveCompileOptions, kernel, schedule=None) -> ScaledGemmKernel:
    """wave_lang/kernel/wave/compile.py:1021: (options, kernel[, schedule]) -> callable.
    `schedule` objects from wave_b200.schedules are accepted and have no effect."""
    from .moe import SiluAndMulKernel, SiluAndMulTemplate
    from .templates import ScaledGemmTemplate

    if isinstance(kernel, SiluAndMulTemplate):
        _lib.load()
        return SiluAndMulKernel(kernel, options)
    if not isinstance(kernel, ScaledGemmTemplate):
        raise TypeError("wave_compile here only compiles the MXFP4 scaled-GEMM templates of wave_b200.templates")
    validate_options(options)
    _lib.load()  # fail now, not at the first call, when the CUDA library is missing
    if options.num_devices > 1:
        # the reference returns a multi-device launchable in this case (compile.py:194-201, 1141-1142)
        from .multi_device import MultiDeviceScaledGemm
        if kernel.element_bits != 4 or kernel.broadcast_a_scale or kernel.preshuffled_scales:
            raise ValueError("the multi-device form serves the plain MXFP4 scaled-GEMM templates")
        return MultiDeviceScaledGemm(kernel, options)
    cls = ScaledGemmKernelWithProfile if options.profile_python_wrapper else ScaledGemmKernel
    return cls(kernel, options)
