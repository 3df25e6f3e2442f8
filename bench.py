"""Benchmark of the MXFP4 scaled-GEMM path: `python bench.py --gpus N --steps K --warmup W`.

One step = one pass of the hot path over one synthetic problem: repack of the activation scales
plus the GEMM (weight scales are packed once, before timing). The headline workload (`value`):

  c2  (default)  M = N = K = 8192, operands quantised from seeded N(0, 1), bf16 output. With N GPUs
                 every rank owns an [8192, K] row shard of b (global N = 8192 * N, weak scaling), a is
                 replicated, and there is no communication in the timed region.
  c3             M = 16, N = 28672, K = 8192 decode shape (weights from N(0, 0.02)), bf16 output.

The metric has three more parts, carried as sub-records of the same JSON line (all with `--workload c2`):

  sustained      the c2 kernel launched back to back for at least two seconds with the clock sampler running:
                 what the figure is once the power governor has settled, next to the short burst of `value`.
  decode         the HBM-bound half of the metric: M in {1, 4, 16, 64, 128}, N = 28672, K = 8192, the kernel alone
                 replayed from a CUDA graph over three rotating weight sets; roofline for M = 16. (Rank 0 only.)
  sharded        M = 16384, N = 53248, K = 16384, bf16, through wave_b200.multi_gpu.ShardedScaledGemm: rank r
                 holds N / G rows of b, a is replicated before timing; the GEMM (no collective) and the
                 all-gather of C are timed separately; every rank checks a sample of its shard against the
                 CPU oracle outside the timed region.

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

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from one ncu capture of this
# benchmark's workload each (scaled to the full workload where the capture ran a smaller case), with the commit whose
# kernel was captured: the figure describes that kernel, not necessarily the one timed now.
NCU_TRAFFIC = {
    "c2": {"bytes": 200.0e6, "kernel": "mxfp4_gemm_kernel<2,256,bf16>", "captured_at_commit": "49071a8"},
    "c3": {"bytes": 131.1e6, "kernel": "mxfp4_skinny_whole_kernel<16,10,bf16>, 104-row tiles", "captured_at_commit": "49071a8"},
    "c3_m128": {"bytes": 128.9e6, "kernel": "mxfp4_skinny_whole_kernel<128,6,bf16>", "captured_at_commit": "53ffb24"},
}

# Sustained rate of a measurement build of the c2 kernel that keeps only its scale copies and MMAs (operands resident
# in shared memory, accumulators never read): the tensor pipe's ceiling for this tile shape under the board's power
# limit. Measured once with `python -m wave_b200.perf --sustained 8192 8192 8192` against that build; not re-measured here.
MMA_ONLY_CEILING = {"tflops": 6881.0, "sm_mhz_median": 1665, "watts_median": 992, "measured_at_commit": "0cf7fad",
                    "how": "library built with -DWB200_MMA_CEILING, two seconds back to back, same operands and launch protocol"}

WORKLOADS = {
    "c2": dict(M=8192, N=8192, K=8192, std_b=1.0, seed_a=1002, seed_b=2002,
               desc="C2 prefill projection: MXFP4 GEMM M=N=K=8192, block 32, operands quantised from seeded N(0,1), bf16 out"),
    "c3": dict(M=16, N=28672, K=8192, std_b=0.02, seed_a=1003, seed_b=2003,
               desc="C3 decode: MXFP4 GEMM M=16, N=28672, K=8192, weights from N(0,0.02), activations from N(0,1), bf16 out"),
    "c3_m128": dict(M=128, N=28672, K=8192, std_b=0.02, seed_a=1003, seed_b=2003,
                    desc="C3 decode shape at the top of the M <= 128 range: MXFP4 GEMM M=128, N=28672, K=8192, bf16 out"),
}
DECODE = dict(N=28672, K=8192, Ms=(1, 4, 16, 64, 128), std_b=0.02, seed_a=1003, seed_b=2003)
SHARDED = dict(M=16384, N=53248, K=16384, seed_a=1005, seed_b=2005, block=6656)


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


def gpu_quantised(rows, K, seed, std, dev, chunk=8192):
    """Seeded N(0, std) values generated and quantised on the GPU, `chunk` rows at a time (the GPU quantiser is
    bit-exact against the harness quantiser of the oracle; tests/test_gpu_parity.py checks that)."""
    from wave_b200 import ops
    g = torch.Generator(device=dev).manual_seed(seed)
    qs, ss = [], []
    for r0 in range(0, rows, chunk):
        x = torch.randn(min(chunk, rows - r0), K, generator=g, device=dev)
        if std != 1.0:
            x *= std
        q, s, _ = ops.quantize_mxfp4(x, want_rowmajor=True, want_packed=False)
        qs.append(q)
        ss.append(s)
        del x
    return torch.cat(qs), torch.cat(ss)


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while timed regions run. `mark(name)` starts a
    named span; summaries can be asked per span."""

    def __init__(self, index, period_s=0.0005):
        super().__init__(daemon=True)
        self.samples, self.stop_flag, self.max_mhz, self.period = [], False, None, period_s
        self.span = "setup"
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def mark(self, name):
        self.span = name

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
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.samples.append((self.span, mhz, tuple(name for bit, name in names.items() if mask & bit)))
            except Exception:
                break
            time.sleep(self.period)

    def summary(self, spans=None):
        sel = [s for s in self.samples if spans is None or s[0] in spans]
        mhz = sorted(s[1] for s in sel)
        reasons = sorted({r for s in sel for r in s[2]})
        return {"sm_mhz": (mhz[len(mhz) // 2] if mhz else None), "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(mhz)}


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


def timed_replays(graph, launches_per_replay, min_ms, stream_sync=True):
    """Replay `graph` until about `min_ms` of GPU time has passed (after one warm-up replay); ms per launch."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    reps = max(3, int(min_ms / max(e0.elapsed_time(e1), 1e-3)))
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (reps * launches_per_replay), reps * launches_per_replay


def decode_record(dev, peaks, overlap=True):
    """The M <= 128 half of the metric: the skinny kernel alone at N = 28672, K = 8192, three rotating weight sets
    (3 x 117 MB: no launch finds its weights in the 126 MB L2), replayed from a CUDA graph; every launch a
    programmatic dependent of the one before it unless `overlap` is off."""
    from oracle import mxfp4_oracle as orc
    from wave_b200 import _lib, ops
    N, K, SETS, ROUNDS = DECODE["N"], DECODE["K"], 3, 4
    weights = []
    # weight scales packed once, per tile of the height that gives every SM the same number of weight tiles
    tile_rows = ops.decode_tile_rows(N, dev)
    for i in range(SETS):
        q, s = gpu_quantised(N, K, DECODE["seed_b"] + 7 * i, DECODE["std_b"], dev)
        weights.append((q, s, ops.repack_scales(s, tile_rows=tile_rows)))
    act_q, act_s = gpu_quantised(128, K, DECODE["seed_a"], 1.0, dev)
    flags = _lib.PATH_SKINNY | (_lib.OVERLAP_PREVIOUS if overlap else 0)
    out = {"N": N, "K": K, "weight_sets": SETS, "launches_per_graph": SETS * ROUNDS,
           "launch": "CUDA-graph replay of the kernel alone (activation scales packed beforehand)",
           "overlap": "each launch is a programmatic dependent of the one before it" if overlap else "none",
           "weight_tile_rows": tile_rows, "per_m": {}}
    for M in DECODE["Ms"]:
        a, a_s = act_q[:M].contiguous(), act_s[:M].contiguous()
        a_sf = ops.repack_scales(a_s)
        cs = [torch.empty(M, N, dtype=torch.bfloat16, device=dev) for _ in range(SETS)]

        def launch_all(fl):
            # ROUNDS passes over the weight sets per graph: a replay is a chain of launches as long as a decode step's
            # (the overlap of one launch with the next ends where a graph ends)
            for _ in range(ROUNDS):
                for i in range(SETS):
                    ops.scaled_gemm_packed(a, a_sf, weights[i][0], weights[i][2], cs[i], fl)

        launch_all(flags)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            launch_all(flags)
        ms, launches = timed_replays(g, SETS * ROUNDS, 30.0)
        alg = algorithmic_bytes(M, N, K)
        rec = {"kernel_us": ms * 1e3, "GBps": alg / (ms * 1e-3) / 1e9, "frac_of_nominal": alg / (ms * 1e-3) / 1e9 / NOMINAL_HBM_GBS,
               "launches_timed": launches}
        if M == 16:
            g2 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g2):
                launch_all(_lib.PATH_SKINNY)
            ms2, _ = timed_replays(g2, SETS * ROUNDS, 30.0)
            rec["kernel_us_without_overlap"] = ms2 * 1e3
            # sampled oracle comparison (one 2048-column block of set 0), outside the timed region
            ref = orc.scaled_gemm(a.cpu(), a_s.cpu(), weights[0][0][4096:6144].cpu(), weights[0][1][4096:6144].cpu())
            d = orc.bf16_ulp_distance(cs[0][:, 4096:6144].contiguous(), ref)
            rec["parity_ok"] = bool(int(d.max()) <= 1)
            achieved = alg / (ms * 1e-3) / 1e9
            out["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s", "frac": achieved / peaks["hbm"],
                               "frac_of_nominal": achieved / NOMINAL_HBM_GBS, "traffic": NCU_TRAFFIC["c3"]["bytes"],
                               "traffic_source": NCU_TRAFFIC["c3"], "peak_source": f"{peaks['source']} HBM copy bandwidth (of measured); nominal 8000 GB/s",
                               "algorithmic_bytes_per_launch": alg, "kernel_ms": ms, "M": 16}
        out["per_m"][str(M)] = rec
        del g, cs
    ops.check_device_status()
    return out


def sharded_record(dev, rank, world, dist):
    """Config 5 through the sharded launcher: GEMM (no collective) and all-gather timed separately, max over ranks."""
    from oracle import mxfp4_oracle as orc
    import wave_b200 as wb
    from wave_b200 import ops
    from wave_b200.multi_gpu import ShardedScaledGemm
    M, N, K, blk = SHARDED["M"], SHARDED["N"], SHARDED["K"], SHARDED["block"]
    op = ShardedScaledGemm(N, K, wb.bf16)
    n0, n1 = op.n0, op.n1
    # b is defined block by block (6656 rows, the 8-way shard) so that every sharding sees the same matrix
    qs, ss = [], []
    for r0 in range(n0, n1, blk):
        q, s = gpu_quantised(min(blk, n1 - r0), K, SHARDED["seed_b"] * 1000 + r0 // blk, 1.0, dev)
        qs.append(q)
        ss.append(s)
    b_shard, bs_shard = torch.cat(qs), torch.cat(ss)
    del qs, ss
    a, a_s = gpu_quantised(M, K, SHARDED["seed_a"], 1.0, dev)  # replicated: same seed on every rank
    op.load_weight_shard(b_shard, bs_shard)
    stacked = op.slot_buffer(M, dev)
    c_local = stacked[rank][:, : op.local_n]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(2):
        op(a, a_s, out=c_local)
    barrier()
    reps = 6
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    ev[0].record()
    for _ in range(reps):
        op(a, a_s, out=c_local)
    ev[1].record()
    barrier()
    gemm_ms = ev[0].elapsed_time(ev[1]) / reps
    # the exchange on its own: all-gather of the column blocks + the interleaving copy into [M, N]
    full = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    op.gather_slots(stacked, out=full)
    barrier()
    greps = 3
    ev[2].record()
    for _ in range(greps):
        op.gather_slots(stacked, out=full)
    ev[3].record()
    barrier()
    gather_ms = ev[2].elapsed_time(ev[3]) / greps
    # the product's exchange: the block computed in place in a matrix the ranks share over CUDA IPC, then pushed to the
    # peers by the copy engines (no collective library, no interleaving pass)
    so = op.shared_output(M, dev)
    c_inplace = so.tensor[:, n0:n1]
    op(a, a_s, out=c_inplace)
    op.push_blocks(so)
    barrier()
    pev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    pev[0].record()
    for _ in range(greps):
        op.push_blocks(so)
    pev[1].record()
    barrier()
    push_ms = pev[0].elapsed_time(pev[1]) / greps
    push_equal = bool(torch.equal(so.tensor, full))
    barrier()
    so.close()
    del so, c_inplace
    ops.check_device_status()
    # parity, outside the timed regions: 48 sampled rows of a against two 512-column blocks of this rank's shard,
    # on the gathered C (which also checks that the gather put this rank's block where it belongs)
    g = torch.Generator().manual_seed(77 + rank)
    rows = torch.randperm(M, generator=g)[:48].sort().values
    worst, over = 0, 0
    for c0 in (0, max(0, op.local_n - 512)):
        ref = orc.scaled_gemm(a[rows.to(dev)].cpu(), a_s[rows.to(dev)].cpu(), b_shard[c0:c0 + 512].cpu(), bs_shard[c0:c0 + 512].cpu())
        got = full[rows.to(dev)][:, n0 + c0:n0 + c0 + 512].contiguous()
        d = orc.bf16_ulp_distance(got, ref)
        worst, over = max(worst, int(d.max())), over + int((d > 1).sum())
    # one more block that another rank computed (exists only when there is more than one rank): bit-equal across ranks
    stats = torch.tensor([gemm_ms, gather_ms, float(worst), float(over), push_ms, 0.0 if push_equal else 1.0], device=dev, dtype=torch.float64)
    if world > 1:
        t = stats.clone()
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        stats = t
    gemm_ms, gather_ms, worst, over, push_ms, push_bad = (float(x) for x in stats)
    flops = 2.0 * M * N * K
    recv = (world - 1) / world * M * N * 2
    # The same problem through the one-call, one-process form (wave_compile with num_devices = G, the reference's
    # MultiDeviceLaunchable): rank 0 drives all the GPUs of the job while the other ranks wait at a barrier; its
    # result must equal the per-rank launcher's bit for bit.
    native = None
    if world > 1 and torch.cuda.device_count() >= world:  # with one device the call is the plain kernel object
        # The other ranks wait on the HOST (a key in the job's store), with nothing of theirs queued on their GPU: a
        # collective's kernel spinning on GPU g while rank 0's GEMM runs there from another process would time-slice
        # against it.
        torch.cuda.synchronize()
        store = dist.distributed_c10d._get_default_store() if world > 1 else None
        if rank == 0:
            del stacked, b_shard, bs_shard
            torch.cuda.empty_cache()
            qs, ss = [], []
            for r0 in range(0, N, blk):
                q, s = gpu_quantised(min(blk, N - r0), K, SHARDED["seed_b"] * 1000 + r0 // blk, 1.0, dev)
                qs.append(q)
                ss.append(s)
            b_full, bs_full = torch.cat(qs), torch.cat(ss)
            del qs, ss
            kernel, options = wb.get_tagged_mxfp4_gemm((M, N, K), output_dtype=wb.bf16)
            options.num_devices = world
            md = wb.wave_compile(wb.set_default_run_config(options), kernel)
            c1 = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
            for _ in range(2):
                md(a, a_s, b_full, bs_full, c1)
                md.synchronize()
            g_ms, c_ms = [], []
            for _ in range(4):
                md.invoke(a, a_s, b_full, bs_full, c1, timed=True)
                md.synchronize()
                g_ms.append(md.last_gemm_ms)
                c_ms.append(md.last_gather_ms)
            native = {"through": "wave_compile(options with num_devices = G)(a, a_scale, b, b_scale, c): one process, wb200_multi_gpu_* (tensors on GPU 0 in, merged c on GPU 0 out)",
                      "gemm_ms": sum(g_ms) / len(g_ms), "merge_ms": sum(c_ms) / len(c_ms),
                      "merge_note": "2-D copy-engine copies of the column blocks into c on GPU 0 (no collective)",
                      "merge_received_bytes": recv, "merge_GBps": (recv / (sum(c_ms) / len(c_ms) * 1e-3) / 1e9) if world > 1 else None,
                      "bit_equal_to_per_rank_launcher": bool(torch.equal(c1, full)), "timing": "CUDA events per GPU, longest over the GPUs, mean of 4 calls"}
            del md, c1, b_full, bs_full
            torch.cuda.synchronize()
            if store is not None:
                store.set("one_process_launcher_done", "1")
        elif store is not None:
            store.wait(["one_process_launcher_done"])
        barrier()
    out = {"config": f"C5: M={M}, N={N}, K={K}, bf16 out, b row-sharded {world}-way ({op.local_n} rows on rank 0), a replicated before timing",
            "through": "wave_b200.multi_gpu.ShardedScaledGemm (public call: activation-scale repack + GEMM per rank, no collective)",
            "gemm_ms": gemm_ms, "tflops": flops / (gemm_ms * 1e-3) / 1e12, "frac_of_nominal_per_gpu": flops / world / (gemm_ms * 1e-3) / 1e12 / NOMINAL_FP4_TFLOPS,
            "allgather_ms": push_ms, "allgather_received_bytes_per_gpu": recv,
            "allgather_GBps_per_gpu": (recv / (push_ms * 1e-3) / 1e9) if world > 1 else None,
            "allgather_note": "ShardedScaledGemm.push_blocks: every rank's column block, computed in place in a matrix shared over CUDA IPC, copied by the copy engines into every other rank's matrix, then a stream-ordered barrier",
            "allgather_equals_nccl_result": push_bad == 0.0,
            "allgather_nccl_ms": gather_ms, "allgather_nccl_GBps_per_gpu": (recv / (gather_ms * 1e-3) / 1e9) if world > 1 else None,
            "allgather_nccl_note": "the library baseline: NCCL all-gather of the column blocks plus the copy that interleaves them into [M, N]; with one rank only the copy",
            "parity_ok": bool(worst <= 1), "parity_max_ulp": worst, "parity_entries_over_1ulp": over,
            "parity_sample": "per rank: 48 rows of a x 2 blocks of 512 columns of its shard, read from the gathered C, against the CPU oracle",
            "timing": f"CUDA events, {reps} GEMM calls / {greps} gathers, max over ranks", "data": "operands generated and quantised on the GPU (seeded)"}
    if native:
        out["one_process_launcher"] = native
    return out


def copy_ceiling(host, c_host, dev, steps):
    """The bytes of one end-to-end step moved by bare pinned copies, no GEMM: all four operands host-to-device on one
    stream and a C-sized buffer device-to-host on another, back to back. ms per step."""
    dbufs = [torch.empty_like(t, device=dev) for t in host]
    dc = torch.empty(c_host.shape, dtype=c_host.dtype, device=dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def one():
        with torch.cuda.stream(s_in):
            for src, dst in zip(host, dbufs):
                dst.copy_(src, non_blocking=True)
        with torch.cuda.stream(s_out):
            c_host.copy_(dc, non_blocking=True)

    for _ in range(2):
        one()
    torch.cuda.synchronize()
    t0 = torch.cuda.Event(enable_timing=True)
    t1a, t1b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    s_in.wait_event(t0)
    s_out.wait_event(t0)
    for _ in range(steps):
        one()
    t1a.record(s_in)
    t1b.record(s_out)
    torch.cuda.synchronize()
    return max(t0.elapsed_time(t1a), t0.elapsed_time(t1b)) / steps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-overlap", action="store_true", help="launch every call after the previous one has completed (for comparison)")
    ap.add_argument("--only", default="", help="comma-separated sub-records to keep (decode,sharded,sustained,e2e); default all")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    parts = set(p for p in args.only.split(",") if p) or {"decode", "sharded", "sustained", "e2e"}
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
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    host = make_operands(w, rank)
    SETS = 3
    dsets = [[t.to(dev, non_blocking=True).clone() for t in host] for _ in range(SETS)]
    outs = [torch.empty(M, N, dtype=torch.bfloat16, device=dev) for _ in range(SETS)]
    kernel, options = wb.get_tagged_mxfp4_gemm((M, N, K), output_dtype=wb.bf16)
    # the weights (b, b_scale) are resident and never written inside the loop: consecutive calls may overlap
    # their tails and heads (programmatic dependent launch, wave_b200's overlap_previous option); this pays
    # for the short decode kernel, not for the 8192-cubed one
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

    from wave_b200 import _lib as _wb_lib
    _lib_flags = _wb_lib.OVERLAP_PREVIOUS if options.overlap_previous else 0
    a_packed = [ops.repack_scales(d[1]) for d in dsets]

    def gemm_only(i):
        ops.scaled_gemm_packed(dsets[i % SETS][0], a_packed[i % SETS], dsets[i % SETS][2], b_packed[i % SETS], outs[i % SETS],
                               _lib_flags)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # -- device-resident timing ---------------------------------------------------------------
    for i in range(args.warmup):
        step(i)
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    sampler.mark("burst")
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    ev[0].record()
    for i in range(args.steps):
        step(i)
    ev[1].record()
    barrier()
    # The dominant kernel alone, same operand rotation, back to back between two events: its average
    # launch duration for the roofline (events around single launches would add several microseconds
    # of gaps to a 25-microsecond kernel). The launches are replayed from a CUDA graph (one launch per operand
    # set), so that the host's launch cost (~15 us per call from Python) cannot bound a short kernel.
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
    elapsed_ms = ev[0].elapsed_time(ev[1])
    kernel_ms_avg = ev[2].elapsed_time(ev[3]) / ksteps

    # -- the same kernel for at least two seconds: what the number is once clocks and power have settled ------------
    sustained = None
    if "sustained" in parts:
        sampler.mark("sustained_ramp")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ramp = max(1, int(300.0 / (kernel_ms_avg * SETS)))  # ~0.3 s untimed: lets the power governor settle
        for _ in range(ramp):
            kgraph.replay()
        torch.cuda.synchronize()
        sreps = max(1, int(2100.0 / (kernel_ms_avg * SETS)))
        sampler.mark("sustained")
        e0.record()
        for _ in range(sreps):
            kgraph.replay()
        e1.record()
        torch.cuda.synchronize()
        sampler.mark("after")
        s_ms = e0.elapsed_time(e1) / (sreps * SETS)
        sustained = {"seconds": e0.elapsed_time(e1) / 1e3, "launches": sreps * SETS, "kernel_ms": s_ms}
    barrier()
    sampler.mark("after")
    ops.check_device_status()
    if world > 1:
        t = torch.tensor([elapsed_ms, kernel_ms_avg, sustained["kernel_ms"] if sustained else 0.0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, kernel_ms_avg = float(t[0]), float(t[1])
        if sustained:
            sustained["kernel_ms"] = float(t[2])
    ms_per_step = elapsed_ms / args.steps
    flops = 2.0 * M * N * K
    value = flops * world / (ms_per_step * 1e-3) / 1e12

    # -- end to end through the public API with host buffers -----------------------------------
    # Every step copies all four operands from pinned host memory, runs the public call and copies C
    # back; wave_b200.HostScaledGemm overlaps the three stages of successive steps on three streams.
    e2e = None
    del dsets, outs, a_packed, b_packed, kgraph
    torch.cuda.empty_cache()
    if "e2e" in parts:
        from wave_b200.host_pipeline import HostScaledGemm
        e2e_steps = max(6, min(args.steps, 30))
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
        del pipe
        torch.cuda.empty_cache()
        barrier()
        ceil_ms = copy_ceiling(host, c_hosts[0], dev, e2e_steps)
        barrier()
        if world > 1:
            t = torch.tensor([e2e_ms, ceil_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms, ceil_ms = float(t[0]), float(t[1])
        h2d = sum(t.numel() * t.element_size() for t in host)
        d2h = c_hosts[0].numel() * c_hosts[0].element_size()
        e2e = {"value": flops * world / (e2e_ms * 1e-3) / 1e12, "unit": unit, "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "copy_ceiling_ms": ceil_ms,
               "frac_of_copy_ceiling": ceil_ms / e2e_ms,
               "copy_ceiling_note": "the same bytes per step moved by bare pinned copies (four operands in on one stream, C out on another), no GEMM, same run, max over ranks"}
        del c_hosts
    del host

    # -- the other parts of the metric -----------------------------------------------------------
    peaks = measured_peaks()
    decode = None
    if "decode" in parts and args.workload == "c2" and rank == 0:
        sampler.mark("decode")
        decode = decode_record(dev, peaks, overlap=not args.no_overlap)
        sampler.mark("after")
    torch.cuda.empty_cache()
    sharded = None
    if "sharded" in parts and args.workload == "c2":
        barrier()
        sampler.mark("sharded")
        sharded = sharded_record(dev, rank, world, dist)
        sampler.mark("after")
    sampler.stop_flag = True
    sampler.join(timeout=2)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    if M <= 128:
        alg = algorithmic_bytes(M, N, K)
        achieved = alg / (kernel_ms_avg * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s", "frac": achieved / peaks["hbm"],
                    "traffic": NCU_TRAFFIC[args.workload]["bytes"], "traffic_source": NCU_TRAFFIC[args.workload],
                    "frac_of_nominal": achieved / NOMINAL_HBM_GBS,
                    "peak_source": f"{peaks['source']} HBM copy bandwidth (of measured); nominal 8000 GB/s",
                    "algorithmic_bytes_per_launch": alg, "kernel_ms": kernel_ms_avg}
    else:
        achieved = flops / (kernel_ms_avg * 1e-3) / 1e12
        assumed = 4.0 * peaks["bf16"]
        roofline = {"bound": "tensor", "achieved": achieved, "peak": NOMINAL_FP4_TFLOPS, "unit": "TFLOP/s",
                    "frac": achieved / NOMINAL_FP4_TFLOPS, "frac_of_nominal": achieved / NOMINAL_FP4_TFLOPS,
                    "traffic": NCU_TRAFFIC[args.workload]["bytes"], "traffic_source": NCU_TRAFFIC[args.workload],
                    "peak_source": "nominal dense FP4 rate of the part (9000 TFLOP/s): no FP4 peak has been measured on this hardware",
                    "assumed_peak": assumed, "frac_of_assumed_peak": achieved / assumed,
                    "assumed_peak_source": f"assumed 4 x measured bf16 burst ({peaks['source']}: {peaks['bf16']:.0f} TFLOP/s); an assumption, not a measurement",
                    "algorithmic_flops_per_launch": flops, "kernel_ms": kernel_ms_avg}
    clocks_burst = sampler.summary({"burst"})
    if sustained:
        cs = sampler.summary({"sustained"})
        sustained.update({"tflops": flops / (sustained["kernel_ms"] * 1e-3) / 1e12,
                          "frac_of_nominal": flops / (sustained["kernel_ms"] * 1e-3) / 1e12 / NOMINAL_FP4_TFLOPS,
                          "sm_mhz_median": cs["sm_mhz"], "clock_samples": cs["samples"], "reasons": cs["reasons"],
                          "ms_x_mhz": (sustained["kernel_ms"] * cs["sm_mhz"]) if cs["sm_mhz"] else None,
                          "burst_kernel_ms": kernel_ms_avg, "burst_sm_mhz_median": clocks_burst["sm_mhz"],
                          "burst_clock_samples": clocks_burst["samples"],
                          "burst_ms_x_mhz": (kernel_ms_avg * clocks_burst["sm_mhz"]) if clocks_burst["sm_mhz"] else None,
                          "mma_only_ceiling": dict(MMA_ONLY_CEILING, frac_of_it=flops / (sustained["kernel_ms"] * 1e-3) / 1e12 / MMA_ONLY_CEILING["tflops"]),
                          "what": "the c2 kernel alone, replayed from a CUDA graph over the three rotating operand sets, back to back after 0.3 s untimed"})
    # clocks of the line: the samples taken while the timed steps and the kernel-only loop ran (a few milliseconds:
    # few samples); the sustained record carries the clocks of the two-second loop
    clocks = clocks_burst
    clocks["all_timed_regions"] = sampler.summary({"burst", "sustained_ramp", "sustained", "decode", "sharded"})
    line = {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "mxfp4",
        "data": "synthetic", "config": config, "clocks": clocks,
        "gpu_launches": 2 * args.steps, "gpu_launches_note": "activation-scale repack + GEMM per timed step; the kernel-only, sustained, decode and sharded loops launch more",
        "roofline": roofline,
    }
    if e2e:
        line["e2e"] = e2e
    if sustained:
        line["sustained"] = sustained
    if decode:
        line["decode"] = decode
    if sharded:
        line["sharded"] = sharded
    if world == 1 and not args.no_cpu_baseline:
        tf, dt, sample, threads, _ = cpu_reference_run(w, 1, 1)
        line["cpu_baseline"] = {"value": tf, "unit": unit, "cores": threads, "kind": "port", "sample": sample,
                                "seconds_per_sample": dt}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
