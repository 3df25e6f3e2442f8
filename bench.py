"""Benchmark of the MXFP4 scaled-GEMM path: `python bench.py --gpus N --steps K --warmup W`.

One step = one pass of the hot path over one synthetic problem: repack of the activation scales
plus the GEMM (weight scales are packed once, before timing). Workloads:

  c2  (default)  M = N = K = 8192, operands quantised from seeded N(0, 1), bf16 output. With N GPUs
                 every rank owns an [8192, K] row shard of b (global N = 8192 * N, weak scaling), a is
                 replicated, and there is no communication in the timed region.
  c3             M = 16, N = 28672, K = 8192 decode shape (weights from N(0, 0.02)), bf16 output.

`--impl reference` times the reference's CPU implementation of the path (the torch oracle port in
oracle/) on this machine's host cores instead, on a bounded slice of the same workload.

Prints one JSON line (rank 0).
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

NOMINAL_FP4_TFLOPS = 9000.0
NOMINAL_HBM_GBS = 8000.0
FALLBACK_BF16_TFLOPS = 1590.0
FALLBACK_HBM_GBS = 6650.0

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from one ncu
# capture (profiles/), scaled to the full workload where the capture ran a smaller case.
NCU_TRAFFIC_BYTES = {"c2": 201.6e6, "c3": 130.7e6}

WORKLOADS = {
    "c2": dict(M=8192, N=8192, K=8192, std_b=1.0, seed_a=1002, seed_b=2002,
               desc="C2 prefill projection: MXFP4 GEMM M=N=K=8192, block 32, operands quantised from seeded N(0,1), bf16 out"),
    "c3": dict(M=16, N=28672, K=8192, std_b=0.02, seed_a=1003, seed_b=2003,
               desc="C3 decode: MXFP4 GEMM M=16, N=28672, K=8192, weights from N(0,0.02), activations from N(0,1), bf16 out"),
}


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm=float(d["hbm_gbs"]), bf16=float(d["bf16_tflops"]), bf16_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    source="MEASURED_PEAKS.json")
    return dict(hbm=FALLBACK_HBM_GBS, bf16=FALLBACK_BF16_TFLOPS, bf16_sustained=1400.0, source="fallback")


def algorithmic_bytes(M, N, K, c_bytes=2):
    # wave_lang/kernel/wave/perf/benchmark_mxfp4.py:82-85
    return M * K // 2 + M * K // 32 + N * K // 2 + N * K // 32 + M * N * c_bytes


def make_operands(w, rank=0):
    """Seeded synthetic operands on the CPU (pinned), quantised with the harness quantiser."""
    from oracle import mxfp4_oracle as orc  # input generation only; nothing here is timed as the product
    ga = torch.Generator().manual_seed(w["seed_a"])
    gb = torch.Generator().manual_seed(w["seed_b"] + 1000 * rank)
    a, a_s = orc.quantize_mxfp4(torch.randn(w["M"], w["K"], generator=ga))
    b, b_s = orc.quantize_mxfp4(torch.randn(w["N"], w["K"], generator=gb) * w["std_b"])
    return [t.pin_memory() if torch.cuda.is_available() else t for t in (a, a_s, b, b_s)]


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.samples, self.reasons, self.stop_flag, self.max_mhz = [], set(), False, None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self.stop_flag:
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                break
            time.sleep(0.002)

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def cpu_reference_run(w, steps, warmup):
    """The reference's CPU path (torch oracle port) on a bounded slice: the first `rows` rows of a
    against all of b. Returns (TFLOP/s, seconds per step, description, threads)."""
    from oracle import mxfp4_oracle as orc
    # torchrun exports OMP_NUM_THREADS=1; the CPU arm is meant to use every host core
    torch.set_num_threads(os.cpu_count() or 1)
    rows = min(w["M"], 512)
    a, a_s, b, b_s = make_operands(w)
    a, a_s = a[:rows], a_s[:rows]
    threads = torch.get_num_threads()
    for _ in range(warmup):
        orc.scaled_gemm(a, a_s, b, b_s)
    # exactly `steps` steps unless they would take more than two minutes of CPU time: then as many as fit
    done = 0
    t0 = time.perf_counter()
    while done < max(steps, 1) and (done == 0 or time.perf_counter() - t0 < 120.0):
        orc.scaled_gemm(a, a_s, b, b_s)
        done += 1
    dt = (time.perf_counter() - t0) / done
    flops = 2.0 * rows * w["N"] * w["K"]
    sample = f"rows 0..{rows - 1} of a against all of b (N={w['N']}, K={w['K']}): dequantise both, f32 torch.mm; {rows}/{w['M']} of the workload's flops"
    return flops / dt / 1e12, dt, sample, threads, done


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-overlap", action="store_true", help="launch every call after the previous one has completed (for comparison)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    w = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    M, N, K = w["M"], w["N"], w["K"]
    metric, unit = "mxfp4_gemm_tflops", "TFLOP/s"
    config = {"workload": w["desc"], "n_shard": f"b row-sharded, {N} rows per GPU (global N = {N * max(world, 1)})",
              "l2": "3 rotating operand/output sets (>126 MB L2) so no step finds its inputs cached"}

    if args.impl == "reference":
        if rank != 0:
            return
        warm = min(args.warmup, 3)
        tf, dt, sample, threads, steps = cpu_reference_run(w, args.steps, warm)
        print(json.dumps({
            "impl": "reference", "metric": metric, "value": tf, "unit": unit, "n_gpus": args.gpus, "steps": steps,
            "warmup": warm, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "mxfp4", "data": "synthetic", "config": config,
            "cpu_baseline": {"value": tf, "unit": unit, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": tf, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }))
        return

    import wave_b200 as wb
    from wave_b200 import ops

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200; wave_b200 has no CPU path (use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    host = make_operands(w, rank)
    SETS = 3
    dsets = [[t.to(dev, non_blocking=True).clone() for t in host] for _ in range(SETS)]
    outs = [torch.empty(M, N, dtype=torch.bfloat16, device=dev) for _ in range(SETS)]
    kernel, options = wb.get_tagged_mxfp4_gemm((M, N, K), output_dtype=wb.bf16)
    # the weights (b, b_scale) are resident and never written inside the loop: consecutive calls may overlap
    # their tails and heads (programmatic dependent launch, wave_b200's overlap_previous option)
    # (measured on one box: the decode kernel gains 5 %, 23.7 against 25.0 us; the 8192-cubed kernel gains nothing)
    options.overlap_previous = M <= 128 and not args.no_overlap
    if options.overlap_previous:
        config["overlap"] = "each launch is a programmatic dependent of the one before it (weights are not written in the loop)"
    gemm = wb.wave_compile(wb.set_default_run_config(options), kernel)
    b_packed = [ops.repack_scales(d[3]) for d in dsets]  # weights: packed once, outside the timed region
    torch.cuda.synchronize()

    def step(i):
        # the call a user makes: activation scales are repacked inside it (every call), the weight
        # scales of each operand set were packed on the first call with that set and are reused
        d = dsets[i % SETS]
        gemm(d[0], d[1], d[2], d[3], outs[i % SETS])

    if M <= 128:
        # Launch-bound shape: the public call is captured once per operand set and replayed
        # (wave_b200.GraphedScaledGemm), as a decode loop would run it.
        from wave_b200.graphs import GraphedScaledGemm
        graphed = [GraphedScaledGemm(gemm, d[0], d[1], d[2], d[3], outs[i]) for i, d in enumerate(dsets)]
        config["launch"] = "CUDA-graph replay of the public call (wave_b200.GraphedScaledGemm)"

        def step(i):  # noqa: F811
            graphed[i % SETS].replay()

    def gemm_only(i):
        ops.scaled_gemm_packed(dsets[i % SETS][0], a_packed[i % SETS], dsets[i % SETS][2], b_packed[i % SETS], outs[i % SETS],
                               _lib_flags)

    from wave_b200 import _lib as _wb_lib
    _lib_flags = _wb_lib.OVERLAP_PREVIOUS if options.overlap_previous else 0

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    a_packed = [ops.repack_scales(d[1]) for d in dsets]

    # -- device-resident timing ---------------------------------------------------------------
    for i in range(args.warmup):
        step(i)
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    ev[0].record()
    for i in range(args.steps):
        step(i)
    ev[1].record()
    barrier()
    # The dominant kernel alone, same operand rotation, back to back between two events: its average
    # launch duration for the roofline (events around single launches would add several microseconds
    # of gaps to a 25-microsecond kernel).
    # The launches are replayed from a CUDA graph (one launch per operand set), so that the host's
    # launch cost (~15 us per call from Python) cannot bound a 25-microsecond kernel.
    for i in range(SETS):
        gemm_only(i)
    torch.cuda.synchronize()
    kgraph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(kgraph):
        for i in range(SETS):
            gemm_only(i)
    kreps = (max(args.steps, 20) + SETS - 1) // SETS
    ksteps = kreps * SETS
    kgraph.replay()
    ev[2].record()
    for _ in range(kreps):
        kgraph.replay()
    ev[3].record()
    barrier()
    sampler.stop_flag = True
    sampler.join(timeout=2)
    ops.check_device_status()
    elapsed_ms = ev[0].elapsed_time(ev[1])
    kernel_ms_avg = ev[2].elapsed_time(ev[3]) / ksteps
    if world > 1:
        t = torch.tensor([elapsed_ms, kernel_ms_avg], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, kernel_ms_avg = float(t[0]), float(t[1])
    ms_per_step = elapsed_ms / args.steps
    flops = 2.0 * M * N * K
    value = flops * world / (ms_per_step * 1e-3) / 1e12

    # -- end to end through the public API with host buffers -----------------------------------
    # Every step copies all four operands from pinned host memory, runs the public call and copies C
    # back; wave_b200.HostScaledGemm overlaps the three stages of successive steps on three streams.
    from wave_b200.host_pipeline import HostScaledGemm
    e2e_steps = max(6, min(args.steps, 30))
    del dsets, outs, a_packed, b_packed
    torch.cuda.empty_cache()
    pipe = HostScaledGemm(M, N, K, wb.bf16, device=dev, depth=3)
    c_hosts = [torch.empty(M, N, dtype=torch.bfloat16).pin_memory() for _ in range(3)]
    for i in range(3):
        pipe.submit(*host, c_hosts[i % 3])
    pipe.drain()
    barrier()
    ev2 = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    ev2[0].record()
    for i in range(e2e_steps):
        pipe.submit(*host, c_hosts[i % 3])
    pipe.join()
    ev2[1].record()
    pipe.drain()
    barrier()
    ops.check_device_status()
    e2e_ms = ev2[0].elapsed_time(ev2[1]) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t[0])
    c_host = c_hosts[0]
    h2d = sum(t.numel() * t.element_size() for t in host)
    d2h = c_host.numel() * c_host.element_size()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = measured_peaks()
    if M <= 128:
        alg = algorithmic_bytes(M, N, K)
        achieved = alg / (kernel_ms_avg * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s", "frac": achieved / peaks["hbm"],
                    "traffic": NCU_TRAFFIC_BYTES[args.workload], "frac_of_nominal": achieved / NOMINAL_HBM_GBS,
                    "peak_source": f"{peaks['source']} HBM copy bandwidth (of measured); nominal 8000 GB/s",
                    "algorithmic_bytes_per_launch": alg, "kernel_ms": kernel_ms_avg}
    else:
        achieved = flops / (kernel_ms_avg * 1e-3) / 1e12
        peak = 4.0 * peaks["bf16"]
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                    "traffic": NCU_TRAFFIC_BYTES[args.workload], "frac_of_nominal": achieved / NOMINAL_FP4_TFLOPS,
                    "peak_source": f"4 x {peaks['source']} cuBLAS bf16 burst {peaks['bf16']:.0f} TFLOP/s (dense FP4 issues at 4x the "
                                   "bf16 rate; no FP4 figure is measured on this pool) (of measured); nominal 9000 TFLOP/s",
                    "algorithmic_flops_per_launch": flops, "kernel_ms": kernel_ms_avg}
    line = {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "mxfp4",
        "data": "synthetic", "config": config, "clocks": sampler.summary(),
        "e2e": {"value": flops * world / (e2e_ms * 1e-3) / 1e12, "unit": unit, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms},
        "gpu_launches": 2 * args.steps + ksteps + 3, "roofline": roofline,
    }
    if world == 1 and not args.no_cpu_baseline:
        tf, dt, sample, threads, _ = cpu_reference_run(w, 1, 1)
        line["cpu_baseline"] = {"value": tf, "unit": unit, "cores": threads, "kind": "port", "sample": sample,
                                "seconds_per_sample": dt}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
