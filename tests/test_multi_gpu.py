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


def _gpu_rank(rank, world, port, out_queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
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
    out_queue.put((rank, bool(ok)))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.gpu
def test_gpu_ranks_shard_and_gather():
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gpu_rank, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(ok for _, ok in results)
