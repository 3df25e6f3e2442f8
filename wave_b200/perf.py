"""Shape-sweep benchmark of the MXFP4 scaled GEMM: `python -m wave_b200.perf [--validate] [--csv out.csv]`;
`python -m wave_b200.perf --moe` times the steps of the MXFP4 expert MLP.

Same bookkeeping as the reference's benchmark driver (wave_lang/kernel/wave/perf/benchmark_mxfp4.py):
flops = 2 M N K (:78-79), bytes = M K/2 + M K/32 + N K/2 + N K/32 + M N sizeof(c) (:82-85), TFLOP/s from the
mean device time of `iters` back-to-back launches between two CUDA events (:117-138; here the launches are
replayed from a CUDA graph so that the Python launch cost is not in the figure), optional
validation of every shape against a reference GEMM before timing (:163-177). The reference sweeps a
CSV of 167 shapes with K = 16000; here the grid is generated: M in {512 .. 8192}, N in {512 .. 32768},
K = 16000 (not a multiple of the 256-element pipeline stage, so every shape exercises the K tail),
plus the decode and square shapes used elsewhere in this repository. Inputs are the seeded random
codes of `generate_gemm_afp4wfp4_inputs`.
"""

from __future__ import annotations

import argparse
import csv
import sys

import torch


def get_flops(M: int, N: int, K: int) -> int:
    return 2 * M * N * K


def get_byte_count_mxfp4(M: int, N: int, K: int, c_bytes: int = 2) -> int:
    return M * K // 2 + M * K // 32 + N * K // 2 + N * K // 32 + M * N * c_bytes


def runtime_us_to_tflops(M: int, N: int, K: int, us: float) -> float:
    return get_flops(M, N, K) / (us * 1e-6) / 1e12


def default_shapes():
    shapes = [(M, N, 16000) for M in (512, 1024, 2048, 4096, 8192) for N in (512, 2048, 8192, 32768)]
    shapes += [(1024, 1024, 1024), (4096, 4096, 4096), (8192, 8192, 8192), (16384, 16384, 16384)]
    shapes += [(M, 28672, 8192) for M in (1, 16, 64, 128)]
    return shapes


def time_shape(M, N, K, out_dtype=torch.bfloat16, iters: int = 20, validate: bool = False, device="cuda:0"):
    """Mean device microseconds per launch of the GEMM alone (scales packed beforehand)."""
    from . import generate_gemm_afp4wfp4_inputs, ops
    x, w, xs, ws = generate_gemm_afp4wfp4_inputs((M, N, K), device=torch.device(device))
    w_t = w.T.contiguous()
    a_sf, b_sf = ops.repack_scales(xs), ops.repack_scales(ws)
    c = torch.empty(M, N, dtype=out_dtype, device=device)
    for _ in range(3):
        ops.scaled_gemm_packed(x, a_sf, w_t, b_sf, c)
    if validate:
        # row-sampled check against the dequantised f32 product computed by torch on the GPU
        rows = torch.arange(0, M, max(1, M // 64), device=device)
        ref = ops.dequant_mxfp4(x[rows].contiguous(), xs[rows].contiguous()) @ ops.dequant_mxfp4(w_t, ws).T
        torch.testing.assert_close(c[rows].float(), ref, rtol=2e-2, atol=1e-2 * float(ref.abs().max()))
    # `iters` launches captured in one CUDA graph and replayed: the Python launch cost (~15 us per call) would
    # otherwise bound every shape that runs for less than that
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(iters):
            ops.scaled_gemm_packed(x, a_sf, w_t, b_sf, c)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    # warm up for ~30 ms of GPU time (clocks ramp up under load), then time as many replays as fill ~30 ms more
    reps = max(2, int(30.0 / max(e0.elapsed_time(e1), 1e-3)))
    for _ in range(reps):
        graph.replay()
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ops.check_device_status()
    return e0.elapsed_time(e1) * 1e3 / (iters * reps)


def time_moe(tokens=4096, experts=8, top_k=2, K=4096, inter=7168, iters=10, device="cuda:0"):
    """Device time of every step of the MXFP4 expert MLP at the grouped-GEMM benchmark's sizes
    (8 experts x [14336, 4096] gate|up weights, 4096 tokens, top-2): microseconds per step and, for the
    memory-bound steps, the bytes they must move / that time."""
    from . import moe, ops
    from .grouped import moe_scaled_gemm
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(4)
    rnd = lambda *shape: torch.randint(0, 256, shape, dtype=torch.uint8, device=dev, generator=g)  # noqa: E731
    sc = lambda *shape: torch.randint(120, 126, shape, dtype=torch.uint8, device=dev, generator=g)  # noqa: E731
    mlp = moe.MXFP4ExpertMLP([rnd(2 * inter, K // 2) for _ in range(experts)], [sc(2 * inter, K // 32) for _ in range(experts)],
                             [rnd(K, inter // 2) for _ in range(experts)], [sc(K, inter // 32) for _ in range(experts)], top_k)
    x = torch.randn(tokens, K, device=dev, generator=g).to(torch.bfloat16)
    logits = torch.randn(tokens, experts, device=dev, generator=g)
    n = tokens * top_k
    B = mlp.BLOCK
    weight, ids = mlp.route(logits)
    cap = (n + experts * (B - 1) + B - 1) // B * B
    sorted_ids = torch.empty(cap, dtype=torch.int32, device=dev)
    expert_ids = torch.empty(cap // B, dtype=torch.int32, device=dev)
    post = torch.empty(1, dtype=torch.int32, device=dev)
    inverse = torch.empty(n, dtype=torch.int32, device=dev)
    moe.moe_align_block_size(ids, experts, B, sorted_ids, expert_ids, post, inverse)
    R = cap  # every buffer has the worst-case row count; the GEMMs skip the row blocks past the padded total
    a = torch.empty(R, K // 2, dtype=torch.uint8, device=dev)
    a_s = torch.empty(R, K // 32, dtype=torch.uint8, device=dev)
    h = torch.empty(R, 2 * inter, dtype=torch.bfloat16, device=dev)
    y = torch.empty(R, K, dtype=torch.bfloat16, device=dev)
    out = torch.empty(tokens, K, dtype=torch.bfloat16, device=dev)
    moe.quantize_scatter(x, inverse, top_k, a, a_s)
    moe_scaled_gemm(a, a_s, mlp.w1, expert_ids, post, h)
    _, hq, hs = moe.silu_and_mul(h[:, :inter], h[:, inter:], quantize=True, num_rows=post)
    steps = [
        ("moe_align_block_size", lambda: moe.moe_align_block_size(ids, experts, B, sorted_ids, expert_ids, post, inverse), None),
        ("quantise tokens into their sorted rows", lambda: moe.quantize_scatter(x, inverse, top_k, a, a_s),
         tokens * K * 2 + n * (K // 2 + K // 32)),
        ("grouped GEMM gate|up", lambda: moe_scaled_gemm(a, a_s, mlp.w1, expert_ids, post, h), None),
        ("silu_and_mul + quantise", lambda: moe.silu_and_mul(h[:, :inter], h[:, inter:], quantize=True, num_rows=post),
         int(post.item()) * (2 * inter * 2 + inter // 2 + inter // 32)),
        ("grouped GEMM down", lambda: moe_scaled_gemm(hq, hs, mlp.w2, expert_ids, post, y), None),
        ("combine", lambda: moe.combine(y, inverse, weight.reshape(-1), top_k, out), R * K * 2 + tokens * K * 2),
        ("whole forward", lambda: mlp(x, logits), None),
    ]
    rows = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for name, fn, nbytes in steps:
        for _ in range(2):
            fn()
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / iters
        row = {"step": name, "us": round(us, 1)}
        if nbytes:
            row["gbytes_per_s"] = round(nbytes / us / 1e3, 1)
        if "GEMM" in name:
            NN, KK = (2 * inter, K) if "gate" in name else (K, inter)
            row["tflops"] = round(2.0 * n * NN * KK / us / 1e6, 1)  # routed rows only; padding rows are not counted
        rows.append(row)
        print(row, flush=True)
    ops.check_device_status()
    return rows


def time_mxfp8(iters=20, device="cuda:0", b_fp4: bool = False):
    """MXFP8 (E4M3 operands, E8M0 block scales, bf16 output): large tile shapes and the decode shapes, three rotating
    operand sets (> L2 for the decode shapes), launches replayed from a CUDA graph. b_fp4: the mixed pair, E4M3
    activations against packed E2M1 weights (K rounded to a multiple of 128)."""
    from . import ops
    rows = []
    shapes = [(8192, 8192, 8192), (4096, 4096, 4096), (8192, 8192, 16000)] + [(M, 28672, 8192) for M in (1, 16, 64, 128)]
    for M, N, K in shapes:
        if b_fp4:
            K = K // 128 * 128
        g = torch.Generator(device=device).manual_seed(1)
        sets = []
        for _ in range(3):
            a = torch.randn(M, K, device=device, generator=g).to(torch.float8_e4m3fn)
            if b_fp4:
                b = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=device, generator=g)
            else:
                b = torch.randn(N, K, device=device, generator=g).to(torch.float8_e4m3fn)
            a_sf = ops.repack_scales(torch.randint(124, 128, (M, K // 32), dtype=torch.uint8, device=device, generator=g))
            b_sf = ops.repack_scales(torch.randint(124, 128, (N, K // 32), dtype=torch.uint8, device=device, generator=g),
                                     tile_rows=ops.decode_tile_rows(N, device) if M <= 128 else 128)  # weights: packed once, per balanced tile
            sets.append((a, a_sf, b, b_sf, torch.empty(M, N, dtype=torch.bfloat16, device=device)))
        for st in sets:
            ops.scaled_gemm_mxfp8_packed(*st, b_fp4=b_fp4)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for st in sets:
                ops.scaled_gemm_mxfp8_packed(*st, b_fp4=b_fp4)
        graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        reps = max(iters // 3, int(20.0 / max(e0.elapsed_time(e1), 1e-3)))  # ~20 ms of warm-up, then ~20 ms timed
        for _ in range(reps):
            graph.replay()
        e0.record()
        for _ in range(reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (3 * reps)
        nbytes = M * K + M * K // 32 + N * K // (2 if b_fp4 else 1) + N * K // 32 + M * N * 2
        rows.append({"M": M, "N": N, "K": K, "runtime_us": round(us, 1), "tflops": round(runtime_us_to_tflops(M, N, K, us), 1),
                     "gbytes_per_s": round(nbytes / us / 1e3, 1)})
        print(rows[-1], flush=True)
        del sets, graph
    ops.check_device_status()
    return rows


def compare_cublaslt(shapes=((8192, 8192, 8192), (4096, 4096, 4096), (2048, 8192, 8192), (16384, 16384, 16384)), iters=20,
                     device="cuda:0"):
    """Context only, never a product path: the vendor library's block-scaled FP4 GEMM (cuBLASLt through
    torch.nn.functional.scaled_mm, 1x32 blocks, E8M0 scales in the 32x4x4 swizzle, which is the packed layout of
    this library when K is a multiple of 256) on the same operands, timed the same way. Prints both times and the
    largest difference of the results."""
    import torch.nn.functional as F
    from torch.nn.functional import ScalingType, SwizzleType
    from . import ops
    rows = []
    for M, N, K in shapes:
        g = torch.Generator(device=device).manual_seed(1)
        a = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, device=device, generator=g)
        b = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=device, generator=g)
        a_sf = ops.repack_scales(torch.randint(124, 128, (M, K // 32), dtype=torch.uint8, device=device, generator=g))
        b_sf = ops.repack_scales(torch.randint(124, 128, (N, K // 32), dtype=torch.uint8, device=device, generator=g))
        c = torch.empty(M, N, dtype=torch.bfloat16, device=device)
        a4, b4 = a.view(torch.float4_e2m1fn_x2), b.view(torch.float4_e2m1fn_x2)
        sa, sb = a_sf.data.view(torch.float8_e8m0fnu), b_sf.data.view(torch.float8_e8m0fnu)

        def ours():
            ops.scaled_gemm_packed(a, a_sf, b, b_sf, c)
            return c

        def vendor():
            return F.scaled_mm(a4, b4.t(), sa, ScalingType.BlockWise1x32, sb, ScalingType.BlockWise1x32,
                               swizzle_a=SwizzleType.SWIZZLE_32_4_4, swizzle_b=SwizzleType.SWIZZLE_32_4_4,
                               output_dtype=torch.bfloat16)

        diff = float((vendor().float() - ours().float()).abs().max())
        row = {"M": M, "N": N, "K": K, "max_abs_diff": diff}
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for name, fn in (("wave_b200", ours), ("cublaslt", vendor), ("wave_b200 again", ours)):
            for _ in range(3):
                fn()
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / iters
            row[name] = f"{us:.1f} us / {runtime_us_to_tflops(M, N, K, us):.0f} TFLOP/s"
        rows.append(row)
        print(row, flush=True)
    return rows


def time_k_sharded(M=8192, N=8192, k_per_rank=8192, iters=20):
    """Under torchrun (one rank per GPU): the K-sharded GEMM whose tiles are scattered to the owning ranks'
    buffers by the GEMM kernel itself, against the unfused sequence on the same operands (GEMM into a local
    f32 matrix, NCCL reduce-scatter, cast). Prints device microseconds per call, max over ranks."""
    import os
    import torch.distributed as dist
    from . import ops
    from .multi_gpu import KShardedScaledGemm
    from .lang import bf16
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    K = k_per_rank * world
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    a = torch.randint(0, 256, (M, k_per_rank // 2), dtype=torch.uint8, device=dev, generator=g)
    b = torch.randint(0, 256, (N, k_per_rank // 2), dtype=torch.uint8, device=dev, generator=g)
    a_s = torch.randint(124, 128, (M, k_per_rank // 32), dtype=torch.uint8, device=dev, generator=g)
    b_s = torch.randint(124, 128, (N, k_per_rank // 32), dtype=torch.uint8, device=dev, generator=g)
    op = KShardedScaledGemm(M, N, K, bf16)
    op.load_weight_shard(b, b_s)
    a_sf, b_sf = ops.repack_scales(a_s), ops.repack_scales(b_s)
    partial = torch.empty(M, N, dtype=torch.float32, device=dev)
    rows = torch.empty(M // world, N, dtype=torch.float32, device=dev)

    def unfused():
        ops.scaled_gemm_packed(a, a_sf, b, b_sf, partial)
        dist.reduce_scatter_tensor(rows, partial)
        return rows.to(torch.bfloat16)

    def fused():
        return op(a, a_s)

    ref, got = unfused().float(), fused().float()
    torch.cuda.synchronize()
    err = float((ref - got).abs().max() / ref.abs().max())
    out = {}
    def fused_tma():
        op.scatter_flags = 1
        r = op(a, a_s)
        op.scatter_flags = 0
        return r

    for name, fn in (("fused scatter + sum", fused), ("fused, TMA stores", fused_tma), ("gemm + nccl reduce_scatter + cast", unfused), ("gemm alone", lambda: ops.scaled_gemm_packed(a, a_sf, b, b_sf, partial))):
        for _ in range(3):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1e3 / iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[name] = round(float(t[0]), 1)
    if rank == 0:
        flops = 2.0 * M * N * K
        print({"world": world, "M": M, "N": N, "K": K, "us": out, "tflops_fused": round(flops / out["fused scatter + sum"] / 1e6, 1),
               "nvlink_bytes_per_rank": (world - 1) * (M // world) * N * 4, "max_rel_diff_fused_vs_unfused": err}, flush=True)
    ops.check_device_status()
    dist.barrier()
    op.close()
    dist.destroy_process_group()


def _interleaved_times(launchers, rounds=10, launches_per_replay=8):
    """Median us per launch of each launcher; one CUDA graph each, replayed in turn round after round so that every
    setting meets the same clock and power state."""
    import statistics
    graphs = []
    for fn in launchers:
        fn()
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(launches_per_replay):
                fn()
        graphs.append(g)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = [[] for _ in launchers]
    for _ in range(rounds + 2):
        for i, g in enumerate(graphs):
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            times[i].append(e0.elapsed_time(e1) * 1e3 / launches_per_replay)
    return [statistics.median(t[2:]) for t in times]


_rowmajor_scales = {}  # the row-major weight scales of the last _packed_problem, for other packings of them


def _packed_problem(M, N, K, device):
    from . import generate_gemm_afp4wfp4_inputs, ops
    x, w, xs, ws = generate_gemm_afp4wfp4_inputs((M, N, K), device=torch.device(device))
    _rowmajor_scales["b"] = ws
    w_t = w.T.contiguous()
    return x, ops.repack_scales(xs), w_t, ops.repack_scales(ws), torch.empty(M, N, dtype=torch.bfloat16, device=device)


def sweep_raster_group(shapes=((8192, 8192, 8192), (4096, 8192, 8192), (8192, 4096, 8192), (16384, 6656, 16384),
                               (8192, 14336, 8192), (4096, 4096, 4096), (8192, 32768, 16000)),
                       groups=(4, 8, 16, 24, 32, 255), device="cuda:0"):
    """us per launch for each raster group size (N tiles per group; 255 = one group, plain row-major order)."""
    from . import _lib, ops
    for M, N, K in shapes:
        x, a_sf, w_t, b_sf, c = _packed_problem(M, N, K, device)
        fl = [_lib.GROUP_N_ALL if g == 255 else _lib.GROUP_N(g) for g in groups]
        us = _interleaved_times([lambda f=f: ops.scaled_gemm_packed(x, a_sf, w_t, b_sf, c, f) for f in fl])
        print((M, N, K), "N tiles", (N + 255) // 256, " | ".join(f"g={g}: {t:8.1f}" for g, t in zip(groups, us)), flush=True)
    ops.check_device_status()


def tile_variants(M: int, N: int, K: int, device="cuda:0"):
    """us per launch of one shape on every tile path that takes it, next to the automatic choice."""
    from . import _lib, ops
    x, a_sf, w_t, b_sf, c = _packed_problem(M, N, K, device)
    names = {"auto": _lib.PATH_AUTO, "2cta-256": _lib.PATH_TILE_2CTA, "2cta-192": _lib.PATH_TILE_2CTA | _lib.TILE_N192,
             "2cta-128": _lib.PATH_TILE_2CTA | _lib.TILE_N128, "1cta-256": _lib.PATH_TILE_1CTA,
             "1cta-128": _lib.PATH_TILE_1CTA | _lib.TILE_N128}
    launchers = [lambda f=f: ops.scaled_gemm_packed(x, a_sf, w_t, b_sf, c, f) for f in names.values()]
    if M > 128:  # 224-wide tiles read weight scales packed for them
        b_224 = ops.repack_scales(_rowmajor_scales["b"], tile_rows=224)
        names["2cta-224"] = None
        launchers.append(lambda: ops.scaled_gemm_packed(x, a_sf, w_t, b_224, c))
    us = _interleaved_times(launchers)
    print((M, N, K), " | ".join(f"{n}: {t:7.1f} us ({runtime_us_to_tflops(M, N, K, t):6.0f} TF)" for n, t in zip(names, us)), flush=True)
    ops.check_device_status()


def sustained_rate(M: int, N: int, K: int, seconds: float = 2.0, device="cuda:0"):
    """TFLOP/s of one shape launched back to back for `seconds` (after a ramp of a quarter of that), with the SM clock
    and the board power sampled through NVML meanwhile. Operands are Gaussian data quantised on the GPU (what the
    tensor pipe draws depends on the bits it multiplies), three rotating sets.

    With the measurement build of the library (`python -m wave_b200.build --mma-ceiling`, then
    `WAVE_B200_LIB=wave_b200/libwave_b200_mma_ceiling.so python -m wave_b200.perf --sustained 8192 8192 8192`) the
    tile kernels load only their first ring of stages and never read the accumulators: the figure is then the ceiling
    of the scale copies + MMAs alone, for this tile shape, under the same power limit."""
    import statistics
    import threading
    import time
    from . import _lib, ops
    dev = torch.device(device)
    sets = []
    g = torch.Generator(device=dev).manual_seed(1)
    for _ in range(3):
        a, _, a_sf = ops.quantize_mxfp4(torch.randn(M, K, device=dev, generator=g, dtype=torch.bfloat16), want_rowmajor=False)
        b, _, b_sf = ops.quantize_mxfp4(torch.randn(N, K, device=dev, generator=g, dtype=torch.bfloat16), want_rowmajor=False)
        sets.append((a, a_sf, b, b_sf, torch.empty(M, N, dtype=torch.bfloat16, device=dev)))

    def launch_all():
        for a, a_sf, b, b_sf, c in sets:
            ops.scaled_gemm_packed(a, a_sf, b, b_sf, c)

    launch_all()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        launch_all()
    samples, stop = [], [False]

    def sample():
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(dev.index or 0)
            while not stop[0]:
                samples.append((pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM), pynvml.nvmlDeviceGetPowerUsage(h) / 1e3))
                time.sleep(0.002)
        except Exception:
            pass

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    per_replay = max(e0.elapsed_time(e1), 1e-3)
    for _ in range(max(1, int(250.0 * seconds / per_replay))):  # ramp: clocks and temperature settle under load
        graph.replay()
    torch.cuda.synchronize()
    th = threading.Thread(target=sample, daemon=True)
    th.start()
    reps = max(3, int(1000.0 * seconds / per_replay))
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    stop[0] = True
    th.join(timeout=1.0)
    ms = e0.elapsed_time(e1) / (reps * len(sets))
    out = dict(library=str(_lib.library_path()), M=M, N=N, K=K, seconds=round(e0.elapsed_time(e1) / 1e3, 2), kernel_us=round(ms * 1e3, 2),
               tflops=round(runtime_us_to_tflops(M, N, K, ms * 1e3), 1))
    if samples:
        out.update(sm_mhz_median=statistics.median(s[0] for s in samples), watts_median=round(statistics.median(s[1] for s in samples), 1))
    print(out, flush=True)
    return out


def skinny_timeline(M: int, N: int, K: int, launches: int = 12, save: str | None = None, device="cuda:0"):
    """Per-CTA timeline of the skinny kernel (M <= 128), from the marks of the measurement build of the library:
    build it with `python -m wave_b200.build --trace` and run
    `WAVE_B200_LIB=wave_b200/libwave_b200_trace.so python -m wave_b200.perf --timeline M N K`.
    Launches rotate over three weight sets (nothing in L2) and are synchronised one by one, so the figures describe
    an isolated cold launch. Prints microseconds after the first CTA's entry: min / median / max over the CTAs."""
    import ctypes

    import numpy as np

    from . import _lib, ops
    lib = _lib.load()
    if not hasattr(lib, "wb200_trace_read"):
        raise SystemExit("this library has no timeline marks: build with `python -m wave_b200.build --trace` and set WAVE_B200_LIB to it")
    lib.wb200_trace_read.restype = ctypes.c_int
    lib.wb200_trace_read.argtypes = [ctypes.c_void_p, ctypes.c_int]
    dev = torch.device(device)
    sets = []
    for i in range(3):
        g = torch.Generator(device=dev).manual_seed(100 + i)
        a = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, device=dev, generator=g)
        b = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev, generator=g)
        a_s = torch.randint(124, 128, (M, K // 32), dtype=torch.uint8, device=dev, generator=g)
        b_s = torch.randint(124, 128, (N, K // 32), dtype=torch.uint8, device=dev, generator=g)
        sets.append((a, ops.repack_scales(a_s), b, ops.repack_scales(b_s, tile_rows=ops.decode_tile_rows(N, dev)),
                     torch.empty(M, N, dtype=torch.bfloat16, device=dev)))
    ctas = torch.cuda.get_device_properties(dev).multi_processor_count
    records = []
    for it in range(launches):
        a, a_sf, b, b_sf, c = sets[it % 3]
        ops.scaled_gemm_packed(a, a_sf, b, b_sf, c, _lib.PATH_SKINNY)
        buf = np.zeros(ctas * 64, dtype=np.uint64)
        words = lib.wb200_trace_read(buf.ctypes.data, ctas)
        if words <= 0:
            raise SystemExit("wb200_trace_read failed")
        records.append(buf[: ctas * words].reshape(ctas, words).astype(np.int64))
    ops.check_device_status()
    if save:
        np.save(save, np.stack(records))

    def stats(x):
        return f"{x.min():7.2f} {np.median(x):7.2f} {x.max():7.2f}"

    print(f"M={M} N={N} K={K}: us after the first CTA's entry, min / median / max over the CTAs that ran (last {min(4, launches)} launches)")
    for r in records[-4:]:
        live = r[:, 0] > 0
        r = r[live]
        t0 = r[:, 0].min()
        nseg = np.clip(r[:, 2], 1, 8)
        last = 8 + 4 * (nseg - 1)
        rows = np.arange(r.shape[0])
        landed = (r[rows, last + 1] - t0) / 1e3
        done = ((r[rows, last + 3] & ((1 << 62) - 1)) - t0) / 1e3
        print(f"  entry {stats((r[:, 0] - t0) / 1e3)} | first ring issued {stats((r[:, 4] - t0) / 1e3)} | first stage landed {stats((r[:, 3] - t0) / 1e3)}"
              f" | last stage landed {stats(landed)} | last epilogue done {stats(done)} | exit {stats((r[:, 1] - t0) / 1e3)}")
    return records


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--validate", action="store_true")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--csv", default=None)
    ap.add_argument("--mxfp8", action="store_true", help="time the MXFP8 GEMM (tile shapes and decode shapes)")
    ap.add_argument("--mxfp8-fp4-weights", action="store_true", help="time the mixed pair: E4M3 activations, packed E2M1 weights")
    ap.add_argument("--compare-cublaslt", action="store_true", help="context: time cuBLASLt's block-scaled FP4 GEMM on the same operands")
    ap.add_argument("--k-sharded", action="store_true", help="under torchrun: time the K-sharded GEMM against GEMM + NCCL reduce-scatter")
    ap.add_argument("--moe", action="store_true", help="time the steps of the MXFP4 expert MLP instead of the shape sweep")
    ap.add_argument("--timeline", nargs=3, type=int, metavar=("M", "N", "K"),
                    help="per-CTA timeline of the skinny kernel (needs the --trace build of the library, see skinny_timeline)")
    ap.add_argument("--save", default=None, help="with --timeline: write the raw marks to this .npy file")
    ap.add_argument("--sustained", nargs=3, type=int, metavar=("M", "N", "K"),
                    help="one shape back to back for two seconds with clock and power sampled (see sustained_rate)")
    ap.add_argument("--group-sweep", action="store_true", help="time the tile kernel over raster group sizes (WB200_GROUP_N)")
    ap.add_argument("--variants", nargs=3, type=int, action="append", metavar=("M", "N", "K"),
                    help="time one shape on every tile path (may be given several times)")
    args = ap.parse_args(argv)
    if args.timeline:
        skinny_timeline(*args.timeline, save=args.save)
        return
    if args.sustained:
        sustained_rate(*args.sustained)
        return
    if args.group_sweep:
        sweep_raster_group()
        return
    if args.variants:
        for shape in args.variants:
            tile_variants(*shape)
        return
    if args.moe:
        time_moe(iters=args.iters)
        return
    if args.mxfp8 or args.mxfp8_fp4_weights:
        time_mxfp8(iters=args.iters, b_fp4=args.mxfp8_fp4_weights)
        return
    if args.compare_cublaslt:
        compare_cublaslt(iters=args.iters)
        return
    if args.k_sharded:
        time_k_sharded(iters=args.iters)
        return
    rows = []
    for M, N, K in default_shapes():
        us = time_shape(M, N, K, iters=args.iters, validate=args.validate)
        rows.append(dict(M=M, N=N, K=K, runtime_us=round(us, 2), tflops=round(runtime_us_to_tflops(M, N, K, us), 1),
                         gbytes_per_s=round(get_byte_count_mxfp4(M, N, K) / us / 1e3, 1)))
        print(rows[-1], flush=True)
    if args.csv:
        with open(args.csv, "w", newline="") as f:
            wr = csv.DictWriter(f, fieldnames=list(rows[0]))
            wr.writeheader()
            wr.writerows(rows)


if __name__ == "__main__":
    sys.exit(main())
