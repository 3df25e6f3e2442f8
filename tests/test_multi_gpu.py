"""N-sharded launcher: partitioning properties on the CPU, a world-size-2 gloo run of the shard /
gather logic (the CUDA kernel replaced by the CPU oracle through the launcher's two hooks), and the
real thing on GPUs when more than one is visible."""

import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from wave_b200.multi_gpu import ShardedScaledGemm, shard_bounds  # noqa: E402


@pytest.mark.parametrize("N,world", [(8192, 1), (8192, 8), (53248, 2), (53248, 4), (53248, 8), (1000, 4), (130, 8), (128, 3)])
def test_shard_bounds_cover_n_in_128_row_granules(N, world):
    bounds = [shard_bounds(N, world, r) for r in range(world)]
    assert bounds[0][0] == 0 and bounds[-1][1] == N
    for (a0, a1), (b0, b1) in zip(bounds, bounds[1:]):
        assert a1 == b0 and a0 <= a1
    for n0, n1 in bounds:
        assert (n0 % 128 == 0 or n0 == N) and (n1 % 128 == 0 or n1 == N)  # shards past the end are empty
    widths = [n1 - n0 for n0, n1 in bounds]
    assert max(widths) - min(widths) <= 128 + 127  # as even as 128-row granules allow
    if N % (128 * world) == 0:
        assert len(set(widths)) == 1


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cpu_rank(rank, world, port, N, gather_mode, out_queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, str(ROOT))
    from oracle import mxfp4_oracle as orc
    import wave_b200 as wb

    class CpuStandIn(ShardedScaledGemm):
        def _pack_scales(self, b_scale_shard):
            return b_scale_shard

        def _build_kernel(self):
            def kernel(a, a_scale, b, b_scale, c):
                c.copy_(orc.scaled_gemm(a, a_scale, b, b_scale))
            return kernel

    M, K = 24, 256
    g = torch.Generator().manual_seed(7)  # same operands on every rank
    a = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, generator=g)
    b = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g)
    a_s = torch.randint(124, 131, (M, K // 32), dtype=torch.uint8, generator=g)
    b_s = torch.randint(124, 131, (N, K // 32), dtype=torch.uint8, generator=g)
    op = CpuStandIn(N, K, wb.f32)
    with pytest.raises(ValueError):
        op.load_weight_shard(b[: op.local_n + 1], b_s[: op.local_n + 1])
    op.load_weight_shard(b[op.n0:op.n1], b_s[op.n0:op.n1])
    ref = orc.scaled_gemm(a, a_s, b, b_s)
    local = op(a, a_s)
    ok = torch.equal(local, ref[:, op.n0:op.n1])
    if gather_mode:
        full = op(a, a_s, gather=True)
        ok = ok and torch.equal(full, ref)
    out_queue.put((rank, ok, (op.n0, op.n1)))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("N", [512, 640, 200])  # equal shards, unequal shards, ragged tail
def test_two_cpu_ranks_shard_and_gather(N):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_cpu_rank, args=(r, 2, port, N, True, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _ in results)
    assert results[0][2][1] == results[1][2][0] and results[1][2][1] == N


def _guarded(body, rank, world, port, out_queue):
    """Run a rank's body; whatever happens, the parent gets an answer from this rank (a rank that dies silently
    would leave its peers blocked in a collective and the parent waiting for the queue)."""
    try:
        body(rank, world, port, out_queue)
    except BaseException as e:  # noqa: BLE001 - reported to the parent, which fails the test
        out_queue.put((rank, False, repr(e)))
        raise


def _run_gpu_ranks(target, world, timeout_s):
    """Start one child per GPU, collect one answer per rank, and never leave a child behind: children are daemons,
    and any that is still alive after the answers are in (or after the wait ran out) is terminated, then killed."""
    import datetime  # noqa: F401
    import queue as queue_mod
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=target, args=(r, world, port, q), daemon=True) for r in range(world)]
    for p in procs:
        p.start()
    results = []
    try:
        for _ in procs:
            try:
                results.append(q.get(timeout=timeout_s))
            except queue_mod.Empty:
                break
            if results[-1][1] is False:
                break  # one rank failed: the others may be blocked in a collective; do not wait for them
    finally:
        for p in procs:
            p.join(timeout=30 if len(results) == len(procs) and all(r[1] for r in results) else 2)
        for p in procs:
            if p.is_alive():
                p.terminate()
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
                p.join(timeout=10)
    assert len(results) == world, f"only {len(results)} of {world} ranks answered: {results}"
    assert all(r[1] for r in results), f"rank failures: {[r for r in results if not r[1]]}"


def _gpu_rank_body(rank, world, port, out_queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=120))
    sys.path.insert(0, str(ROOT))
    from oracle import mxfp4_oracle as orc
    import wave_b200 as wb
    dev = torch.device("cuda", rank)
    M, N, K = 300, 1024 * world, 1024
    g = torch.Generator().manual_seed(11)
    a = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, generator=g)
    b = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g)
    a_s = torch.randint(124, 131, (M, K // 32), dtype=torch.uint8, generator=g)
    b_s = torch.randint(124, 131, (N, K // 32), dtype=torch.uint8, generator=g)
    op = ShardedScaledGemm(N, K, wb.bf16)
    op.load_weight_shard(b[op.n0:op.n1].to(dev), b_s[op.n0:op.n1].to(dev))
    ref = orc.scaled_gemm(a, a_s, b, b_s)
    local = op(a.to(dev), a_s.to(dev))
    full = op(a.to(dev), a_s.to(dev), gather=True)
    torch.cuda.synchronize()
    ok = int(orc.bf16_ulp_distance(local, ref[:, op.n0:op.n1]).max()) <= 1
    ok = ok and int(orc.bf16_ulp_distance(full, ref).max()) <= 1
    # each shard equals the same columns of a single-GPU run bit for bit (same kernel, same K order)
    kernel, options = wb.get_tagged_mxfp4_gemm((M, N, K), output_dtype=wb.bf16)
    single = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    wb.wave_compile(options, kernel)(a.to(dev), a_s.to(dev), b.to(dev), b_s.to(dev), single)
    ok = ok and torch.equal(single, full)
    # the exchange step on its own gives the same matrix
    stacked = op.slot_buffer(M, dev)
    stacked[rank][:, : op.local_n].copy_(local)
    ok = ok and torch.equal(op.gather_slots(stacked), full)
    # the same exchange with copy-engine pushes into matrices the ranks share over CUDA IPC: compute in place, push
    so = op.shared_output(M, dev)
    for _ in range(2):
        so.tensor.fill_(float("nan"))
        torch.cuda.synchronize()
        dist.barrier()  # nobody pushes into a matrix that is still being filled
        op(a.to(dev), a_s.to(dev), out=so.tensor[:, op.n0:op.n1])
        pushed = op.push_blocks(so)
        torch.cuda.synchronize()
        ok = ok and torch.equal(pushed, full)
    dist.barrier()
    so.close()
    out_queue.put((rank, bool(ok), ""))
    dist.barrier()
    dist.destroy_process_group()


def _gpu_rank(rank, world, port, out_queue):  # top level: spawn pickles the target by name
    _guarded(_gpu_rank_body, rank, world, port, out_queue)


@pytest.mark.gpu
def test_gpu_ranks_shard_and_gather():
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    _run_gpu_ranks(_gpu_rank, world, timeout_s=300)


# ---------------------------------------------------------------------------------------------
# K-sharded variant: partial products scattered by rows, summed in rank order
# ---------------------------------------------------------------------------------------------
def _k_operands(M, N, K, seed):
    g = torch.Generator().manual_seed(seed)  # same operands on every rank
    a = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, generator=g)
    b = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g)
    a_s = torch.randint(124, 131, (M, K // 32), dtype=torch.uint8, generator=g)
    b_s = torch.randint(124, 131, (N, K // 32), dtype=torch.uint8, generator=g)
    return a, a_s, b, b_s


def _cpu_rank_ksharded(rank, world, port, M, K, out_queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, str(ROOT))
    from oracle import mxfp4_oracle as orc
    import wave_b200 as wb
    from wave_b200.multi_gpu import KShardedScaledGemm

    class CpuStandIn(KShardedScaledGemm):
        """Same partitioning, slot order and double buffering; the GEMM is the oracle, the scatter is send/recv."""

        def _pack_scales(self, scale):
            return scale

        def _exchange_buffers(self, device):
            self._recv = torch.zeros(2, self.world_size, self.rows_max, self.N, dtype=torch.float32)
            return None

        def _scatter_gemm(self, a, a_scale, parity):
            part = orc.scaled_gemm(a, a_scale, self._b, self._b_sf)
            reqs, keep = [], []
            for d, (m0, m1) in enumerate(self.row_bounds):
                if d == self.rank:
                    self._recv[parity, self.rank, : m1 - m0] = part[m0:m1]
                elif m1 > m0:
                    keep.append(part[m0:m1].contiguous())
                    reqs.append(dist.isend(keep[-1], d))
            rows = self.m1 - self.m0
            bufs = {}
            for s in range(self.world_size):
                if s != self.rank and rows:
                    bufs[s] = torch.empty(rows, self.N)
                    reqs.append(dist.irecv(bufs[s], s))
            for r in reqs:
                r.wait()
            for s, t in bufs.items():
                self._recv[parity, s, :rows] = t

        def _barrier(self):
            dist.barrier()

        def _reduce(self, parity, out):
            rows = self.m1 - self.m0
            acc = self._recv[parity, 0, :rows].clone()
            for s in range(1, self.world_size):
                acc += self._recv[parity, s, :rows]
            out.copy_(acc)

    N = 96
    a, a_s, b, b_s = _k_operands(M, N, K, seed=13)
    op = CpuStandIn(M, N, K, wb.f32)
    k0, k1 = op.k0, op.k1
    with pytest.raises(ValueError):
        op.load_weight_shard(b[:, : k1 // 2 - k0 // 2 + 1], b_s[:, k0 // 32:k1 // 32])
    op.load_weight_shard(b[:, k0 // 2:k1 // 2], b_s[:, k0 // 32:k1 // 32])
    ref = orc.scaled_gemm(a, a_s, b, b_s)
    tol = orc.f32_tolerance(orc.dequant_mxfp4(a, a_s), orc.dequant_mxfp4(b, b_s), ref, K)
    ok = True
    for _ in range(3):  # alternating receive buffers
        rows = op(a[:, k0 // 2:k1 // 2], a_s[:, k0 // 32:k1 // 32])
        ok = ok and bool(((rows - ref[op.m0:op.m1]).abs() <= tol[op.m0:op.m1]).all())
    full = op(a[:, k0 // 2:k1 // 2], a_s[:, k0 // 32:k1 // 32], gather=True)
    ok = ok and bool(((full - ref).abs() <= tol).all())
    out_queue.put((rank, ok, (op.k0, op.k1), (op.m0, op.m1)))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("M,K", [(256, 512), (300, 1024), (100, 768)])  # equal parts, ragged rows, one rank without rows / uneven K
def test_two_cpu_ranks_k_sharded(M, K):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_cpu_rank_ksharded, args=(r, 2, port, M, K, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _, _ in results)
    assert results[0][2][0] == 0 and results[0][2][1] == results[1][2][0] and results[1][2][1] == K
    assert results[0][3][0] == 0 and results[0][3][1] == results[1][3][0] and results[1][3][1] == M
    assert results[0][2][1] % 256 == 0 and (results[0][3][1] % 128 == 0 or results[0][3][1] == M)


def _gpu_rank_ksharded_body(rank, world, port, out_queue):
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=120))
    sys.path.insert(0, str(ROOT))
    from oracle import mxfp4_oracle as orc
    import wave_b200 as wb
    from wave_b200.multi_gpu import KShardedScaledGemm
    dev = torch.device("cuda", rank)
    ok = True
    for (M, N, K) in [(512, 768, 1024 * world), (300, 1000, 512 * world + 256)]:
        a, a_s, b, b_s = _k_operands(M, N, K, seed=17)
        op = KShardedScaledGemm(M, N, K, wb.bf16)
        k0, k1 = op.k0, op.k1
        op.load_weight_shard(b[:, k0 // 2:k1 // 2].to(dev), b_s[:, k0 // 32:k1 // 32].to(dev))
        ref = orc.scaled_gemm(a, a_s, b, b_s)
        tol = orc.f32_tolerance(orc.dequant_mxfp4(a, a_s), orc.dequant_mxfp4(b, b_s), ref, K)
        ad, asd = a[:, k0 // 2:k1 // 2].to(dev), a_s[:, k0 // 32:k1 // 32].to(dev)
        first = None
        for _ in range(3):
            rows = op(ad, asd)
            torch.cuda.synchronize()
            r = ref[op.m0:op.m1]
            # the bar: within 1 bf16 ulp of the rounded reference, or, where the sum of the ranks' f32 partial products
            # cancels far below its terms, inside the f32 bound (which has an absolute part) plus the bf16 rounding
            # of the result (half an ulp: |r| * 2^-9)
            ulp = orc.bf16_ulp_distance(rows, r)
            bad = (ulp > 1) & ~((rows.float().cpu() - r).abs() <= tol[op.m0:op.m1] + r.abs() * 2.0 ** -9)
            ok = ok and not bool(bad.any())
            if first is None:
                first = rows.clone()
            ok = ok and torch.equal(first, rows)  # fixed slot order: the same bits every call
        full = op(ad, asd, gather=True)
        torch.cuda.synchronize()
        ok = ok and torch.equal(full[op.m0:op.m1], first)
        ulp = orc.bf16_ulp_distance(full, ref)
        ok = ok and not bool(((ulp > 1) & ~((full.float().cpu() - ref).abs() <= tol + ref.abs() * 2.0 ** -9)).any())
        wb.ops.check_device_status()
        dist.barrier()
        op.close()
    out_queue.put((rank, bool(ok), ""))
    dist.barrier()
    dist.destroy_process_group()


def _gpu_rank_ksharded(rank, world, port, out_queue):
    _guarded(_gpu_rank_ksharded_body, rank, world, port, out_queue)


@pytest.mark.gpu
def test_gpu_ranks_k_sharded_scatter_and_sum():
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    _run_gpu_ranks(_gpu_rank_ksharded, world, timeout_s=180)


# ---------------------------------------------------------------------------------------------
# one process, several GPUs: the reference's single-call multi-device form
# ---------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("where", ["device0", "host"])
def test_one_call_multi_device_gemm(where):
    """wave_compile(options with num_devices = G)(a, a_scale, b, b_scale, c) with the tensors in one place, as
    tests/kernel/dist_gemm_test.py:60-101 calls the reference's distributed GEMM: b is split over the GPUs, every
    GPU computes its column block, c comes back merged. Checked against the oracle and, bit for bit, against the
    single-GPU kernel (same kernel, same K order)."""
    G = min(torch.cuda.device_count(), 4)
    if G < 2:
        pytest.skip("needs at least 2 GPUs")
    sys.path.insert(0, str(ROOT))
    from oracle import mxfp4_oracle as orc
    import wave_b200 as wb
    for (M, N, K, dtype) in [(300, 1024 * G + 256, 1024, wb.bf16), (16, 4096, 2048, wb.f32)]:
        g = torch.Generator().manual_seed(23)
        a = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, generator=g)
        b = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g)
        a_s = torch.randint(124, 131, (M, K // 32), dtype=torch.uint8, generator=g)
        b_s = torch.randint(124, 131, (N, K // 32), dtype=torch.uint8, generator=g)
        ref = orc.scaled_gemm(a, a_s, b, b_s)
        kernel, options = wb.get_tagged_mxfp4_gemm((M, N, K), output_dtype=dtype)
        options.num_devices = G
        gemm = wb.wave_compile(wb.set_default_run_config(options), kernel)
        if where == "host":
            t = [x.pin_memory() for x in (a, a_s, b, b_s)]
            c = torch.empty(M, N, dtype=dtype.torch_dtype).pin_memory()
        else:
            t = [x.to("cuda:0") for x in (a, a_s, b, b_s)]
            c = torch.full((M, N), float("nan"), dtype=dtype.torch_dtype, device="cuda:0")
        for _ in range(2):  # the second call reuses the sharded weights
            gemm(*t, c)
            gemm.synchronize()
        if dtype is wb.bf16:
            assert int(orc.bf16_ulp_distance(c, ref).max()) <= 1
        else:
            tol = orc.f32_tolerance(orc.dequant_mxfp4(a, a_s), orc.dequant_mxfp4(b, b_s), ref, K)
            assert bool(((c.float().cpu() - ref).abs() <= tol).all())
        k1, o1 = wb.get_tagged_mxfp4_gemm((M, N, K), output_dtype=dtype)
        single = torch.empty(M, N, dtype=dtype.torch_dtype, device="cuda:0")
        wb.wave_compile(o1, k1)(*[x.to("cuda:0") for x in (a, a_s, b, b_s)], single)
        torch.cuda.synchronize()
        assert torch.equal(single.cpu(), c.cpu())
