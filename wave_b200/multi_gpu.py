"""N-sharded scaled GEMM over the GPUs of one node, one process per GPU.

The reference distributes a GEMM by tiling M and/or N over IREE devices inside one process: its
`DeviceConstraint` (wave_lang/kernel/wave/constraints.py:1105-1180) makes the host wrapper slice
the inputs per device, dispatch one kernel per device and merge the output slices
(wave_lang/kernel/compiler/host_utils.py:158-330, wave_lang/runtime/multi_device_launch.py:38-273,
template wave_lang/kernel/wave/templates/dist_gemm.py:20-119). There is no collective in it.

Here each rank of a `torch.distributed` job owns the rows [r * N/G, (r+1) * N/G) of b and b_scale
(a column block of C) and keeps them resident; a and a_scale are replicated. The compute path has
no communication at all. Only when the caller asks for the full C on every rank is one NCCL
all-gather issued over NVLink, after the GEMM, on the same stream.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from . import ops
from .compile import wave_compile
from .lang import as_output_dtype
from .templates import get_tagged_mxfp4_gemm


def shard_bounds(N: int, world_size: int, rank: int, granule: int = 128) -> tuple[int, int]:
    """Rows of b owned by `rank`: N is dealt in multiples of `granule` rows (the scale-factor atom
    height), as evenly as possible, earlier ranks taking the remainder; the last non-empty shard
    takes the ragged tail."""
    blocks = (N + granule - 1) // granule
    base, extra = divmod(blocks, world_size)
    b0 = rank * base + min(rank, extra)
    b1 = b0 + base + (1 if rank < extra else 0)
    return min(b0 * granule, N), min(b1 * granule, N)


class ShardedScaledGemm:
    """Column-sharded MXFP4 GEMM: rank r computes C[:, n0_r:n1_r] = A · B[n0_r:n1_r]^T.

    Usage, inside an initialised process group (backend nccl on GPUs, gloo for host-side tests of
    the partitioning):

        op = ShardedScaledGemm(N, K, output_dtype=wave_b200.bf16)
        op.load_weight_shard(b[n0:n1], b_scale[n0:n1])     # this rank's rows, kept resident
        c_local = op(a, a_scale)                           # [M, n1 - n0], no communication
        c_full = op(a, a_scale, gather=True)               # [M, N] on every rank, one all-gather
    """

    def __init__(self, N: int, K: int, output_dtype, group: Optional[dist.ProcessGroup] = None):
        self.N, self.K = N, K
        self.group = group
        self.world_size = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.out = as_output_dtype(output_dtype)
        self.n0, self.n1 = shard_bounds(N, self.world_size, self.rank)
        self.bounds = [shard_bounds(N, self.world_size, r) for r in range(self.world_size)]
        self._b = None
        self._b_sf = None
        self._kernel = None

    @property
    def local_n(self) -> int:
        return self.n1 - self.n0

    def load_weight_shard(self, b_shard: torch.Tensor, b_scale_shard: torch.Tensor) -> None:
        """Keep this rank's rows of b ([local_n, K/2]) and pack their scales once."""
        if tuple(b_shard.shape) != (self.local_n, self.K // 2):
            raise ValueError(f"rank {self.rank} owns rows [{self.n0}, {self.n1}) of b: expected shape "
                             f"{(self.local_n, self.K // 2)}, got {tuple(b_shard.shape)}")
        if tuple(b_scale_shard.shape) != (self.local_n, self.K // ops.SCALE_GROUP_SIZE):
            raise ValueError(f"b_scale shard must be {(self.local_n, self.K // ops.SCALE_GROUP_SIZE)}, "
                             f"got {tuple(b_scale_shard.shape)}")
        self._b = b_shard.contiguous()
        self._b_sf = self._pack_scales(b_scale_shard) if self.local_n else None
        self._kernel = self._build_kernel()

    # The two hooks below are the only places that touch the CUDA library, so that the partitioning
    # and gathering logic can be exercised by CPU ranks with stand-ins.
    def _pack_scales(self, b_scale_shard: torch.Tensor):
        return ops.repack_scales(b_scale_shard)

    def _build_kernel(self):
        kernel, options = get_tagged_mxfp4_gemm((0, self.local_n, self.K), output_dtype=self.out)
        options.dynamic_symbols = ["M"]
        return wave_compile(options, kernel)

    def __call__(self, a: torch.Tensor, a_scale: torch.Tensor, gather: bool = False,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self._kernel is None:
            raise RuntimeError("load_weight_shard() must be called before the first GEMM")
        M = a.shape[0]
        if not gather:
            c = out if out is not None else torch.empty(M, self.local_n, dtype=self.out.torch_dtype, device=a.device)
            if self.local_n:
                self._kernel(a, a_scale, self._b, self._b_sf, c)
            return c
        # Full C on every rank. Every rank computes into its slot of a [world, M, widest shard] buffer
        # (narrower shards leave the tail columns of their slot unused), one all-gather fills the other
        # slots, and one strided copy per shard lays the column blocks side by side.
        wmax = max(n1 - n0 for n0, n1 in self.bounds)
        stacked = torch.empty(self.world_size, M, wmax, dtype=self.out.torch_dtype, device=a.device)
        if self.local_n:
            self._kernel(a, a_scale, self._b, self._b_sf, stacked[self.rank][:, : self.local_n])
        if self.world_size > 1:
            dist.all_gather_into_tensor(stacked.view(-1), stacked[self.rank].reshape(-1), group=self.group)
        full = out if out is not None else torch.empty(M, self.N, dtype=self.out.torch_dtype, device=a.device)
        if all(n1 - n0 == wmax for n0, n1 in self.bounds):
            full.view(M, self.world_size, wmax).copy_(stacked.permute(1, 0, 2))
        else:
            for r, (n0, n1) in enumerate(self.bounds):
                if n1 > n0:
                    full[:, n0:n1].copy_(stacked[r][:, : n1 - n0])
        return full
