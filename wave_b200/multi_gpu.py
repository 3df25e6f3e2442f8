"""N-sharded (and K-sharded) scaled GEMM over the GPUs of one node, one process per GPU.

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
        # Full C on every rank: every rank computes into its slot of a [world, M, widest shard] buffer (narrower
        # shards leave the tail columns of their slot unused); gather_slots does the rest.
        stacked = self.slot_buffer(M, a.device)
        if self.local_n:
            self._kernel(a, a_scale, self._b, self._b_sf, stacked[self.rank][:, : self.local_n])
        return self.gather_slots(stacked, out=out)

    def shared_output(self, M: int, device) -> SharedOutput:
        """A full-width [M, N] output on every rank that the other ranks can write (collective). Compute into
        `out.tensor[:, n0:n1]` (pass it as `out=`), then `push_blocks(out)`."""
        return SharedOutput(M, self.N, self.out.torch_dtype, device, self.group)

    def push_blocks(self, out: SharedOutput) -> torch.Tensor:
        """The exchange without a collective library: this rank's column block of `out.tensor`, already computed in
        place, is copied by the copy engines into the same columns of every other rank's matrix (one 2-D copy per
        peer, on the current stream, starting with the next rank so that the ranks do not all write to the same peer
        at once); a stream-ordered barrier follows, after which `out.tensor` holds the whole C on every rank. No
        interleaving pass: the blocks land where they belong. A rank that is still reading `out.tensor` when a peer
        pushes the NEXT call's block would see it change: alternate two SharedOutputs, or order the calls."""
        from . import _lib
        lib = _lib.load()
        if self.local_n and self.world_size > 1:
            esz = out.row_bytes // out.N
            off, width = self.n0 * esz, self.local_n * esz
            stream = torch.cuda.current_stream(out.device).cuda_stream
            with torch.cuda.device(out.device):
                for i in range(1, self.world_size):
                    r = (self.rank + i) % self.world_size
                    _lib.check(lib.wb200_copy_2d(out.peers[r] + off, out.row_bytes, out.ptr + off, out.row_bytes, width, out.M, stream))
        if self.world_size > 1:
            dist.all_reduce(out._flag, group=self.group)  # stream-ordered: every rank's copies have landed
        return out.tensor

    def slot_buffer(self, M: int, device) -> torch.Tensor:
        """[world, M, widest shard] buffer of the output type; rank r's GEMM result belongs in slot r."""
        wmax = max(n1 - n0 for n0, n1 in self.bounds)
        return torch.empty(self.world_size, M, wmax, dtype=self.out.torch_dtype, device=device)

    def gather_slots(self, stacked: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The exchange step on its own: this rank's slot of `stacked` holds its column block of C; one all-gather
        fills the other slots, and one strided copy per shard lays the column blocks side by side in [M, N].
        The reference merges per-device output slices the same way, without a collective, inside one process
        (wave_lang/kernel/compiler/host_utils.py:330-376)."""
        M, wmax = stacked.shape[1], stacked.shape[2]
        if self.world_size > 1:
            dist.all_gather_into_tensor(stacked.view(-1), stacked[self.rank].reshape(-1), group=self.group)
        full = out if out is not None else torch.empty(M, self.N, dtype=self.out.torch_dtype, device=stacked.device)
        if all(n1 - n0 == wmax for n0, n1 in self.bounds):
            full.view(M, self.world_size, wmax).copy_(stacked.permute(1, 0, 2))
        else:
            for r, (n0, n1) in enumerate(self.bounds):
                if n1 > n0:
                    full[:, n0:n1].copy_(stacked[r][:, : n1 - n0])
        return full


class _DeviceArray:
    """Lets torch view device memory it did not allocate (a buffer made by wb200_peer_buffer_create)."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 2}


class SharedOutput:
    """An [M, N] output matrix per rank that the OTHER ranks can write: allocated by the library (cudaMalloc, so that
    it can be exported), exchanged as CUDA IPC handles, mapped by every peer. `ShardedScaledGemm.push_blocks` uses
    it to build the full C on every rank with nothing but copy-engine copies: every rank computes its column block
    in place and copies it into the same columns of every other rank's matrix. Collective to create and to close."""

    def __init__(self, M: int, N: int, torch_dtype: torch.dtype, device, group=None):
        import ctypes
        from . import _lib
        self.M, self.N, self.dtype, self.group = M, N, torch_dtype, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.device(device)
        esz = torch.empty(0, dtype=torch_dtype).element_size()
        self.row_bytes = N * esz
        lib = _lib.load()
        handle = ctypes.create_string_buffer(64)
        base = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(lib.wb200_peer_buffer_create(M * N * esz, ctypes.byref(base), handle))
        self.ptr = base.value
        self._opened = []
        self.peers = [self.ptr] * self.world  # base address of every rank's matrix as seen from this process
        if self.world > 1:
            gathered = [None] * self.world
            dist.all_gather_object(gathered, handle.raw, group=group)
            with torch.cuda.device(self.device):
                for r in range(self.world):
                    if r == self.rank:
                        continue
                    p = ctypes.c_void_p()
                    _lib.check(lib.wb200_peer_buffer_open(ctypes.create_string_buffer(gathered[r], 64), ctypes.byref(p)))
                    self._opened.append(p.value)
                    self.peers[r] = p.value
        words = {2: "<i2", 4: "<f4"}[esz]
        t = torch.as_tensor(_DeviceArray(self.ptr, (M, N), words), device=self.device)
        self.tensor = t.view(torch_dtype) if t.dtype != torch_dtype else t
        self._flag = torch.zeros(1, dtype=torch.int32, device=self.device)

    def close(self) -> None:
        """Unmap the peers' matrices and free this rank's. Call on every rank, after a barrier; the tensor is dead afterwards."""
        from . import _lib
        lib = _lib.load()
        for p in self._opened:
            lib.wb200_peer_buffer_close(p)
        self._opened = []
        if self.ptr:
            lib.wb200_peer_buffer_destroy(self.ptr)
            self.ptr = None


class KShardedScaledGemm:
    """K-sharded MXFP4 GEMM: rank r holds the K columns [k0_r, k1_r) of a and b (multiples of 256 elements),
    C = sum over ranks of a_r · b_r^T, and rank r ends up with the rows [m0_r, m1_r) of C (multiples of 128).

    The reference distributes a GEMM by M / N tiles only (wave_lang/kernel/wave/templates/dist_gemm.py:49-50);
    this is the second sharding axis, the one a row-parallel linear layer needs. Compute and exchange are one
    step: every rank runs ONE persistent GEMM launch (`wb200_mxfp4_gemm_scatter_rows`) whose tiles are stored,
    as they finish, straight into the receive buffer of the rank that owns those rows — the peers' buffers are
    mapped for this rank's device with CUDA IPC, so the f32 partial products cross NVLink while the remaining tiles
    are still being computed. A stream-ordered barrier follows, then each rank adds the `world` slots of its
    receive buffer in rank order (`wb200_sum_slots`, deterministic) and rounds once to the output type.
    Two receive buffers alternate between calls, so a rank may start scattering call i+1 while a peer still
    sums call i.

        op = KShardedScaledGemm(M, N, K, wave_b200.bf16)
        op.load_weight_shard(b[:, k0/2:k1/2], b_scale[:, k0/32:k1/32])     # this rank's K columns of b
        c_rows = op(a[:, k0/2:k1/2], a_scale[:, k0/32:k1/32])              # [m1 - m0, N]
        c_full = op(..., gather=True)                                      # [M, N] on every rank (one all-gather)
    """

    def __init__(self, M: int, N: int, K: int, output_dtype, group: Optional[dist.ProcessGroup] = None):
        self.M, self.N, self.K = M, N, K
        self.group = group
        self.world_size = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.out = as_output_dtype(output_dtype)
        self.k0, self.k1 = shard_bounds(K, self.world_size, self.rank, granule=256)
        self.row_bounds = [shard_bounds(M, self.world_size, r, granule=128) for r in range(self.world_size)]
        self.m0, self.m1 = self.row_bounds[self.rank]
        self.rows_max = max(m1 - m0 for m0, m1 in self.row_bounds)
        self._b = self._b_sf = None
        self._calls = 0
        self._peers = None
        self.scatter_flags = 0  # 1: TMA stores instead of ordinary stores to the peers' buffers

    @property
    def local_k(self) -> int:
        return self.k1 - self.k0

    def load_weight_shard(self, b_cols: torch.Tensor, b_scale_cols: torch.Tensor) -> None:
        """Keep this rank's K columns of b ([N, local_k/2]) and of its scales ([N, local_k/32], packed once)."""
        if tuple(b_cols.shape) != (self.N, self.local_k // 2) or \
                tuple(b_scale_cols.shape) != (self.N, self.local_k // ops.SCALE_GROUP_SIZE):
            raise ValueError(f"rank {self.rank} owns K columns [{self.k0}, {self.k1}): expected b {(self.N, self.local_k // 2)} "
                             f"and scales {(self.N, self.local_k // ops.SCALE_GROUP_SIZE)}, got {tuple(b_cols.shape)} and "
                             f"{tuple(b_scale_cols.shape)}")
        self._b = b_cols.contiguous()
        self._b_sf = self._pack_scales(b_scale_cols.contiguous()) if self.local_k else None
        if self._peers is None:
            self._peers = self._exchange_buffers(self._b.device)

    # ---- the hooks below are the only places that touch CUDA; CPU ranks replace them in tests ----------
    def _pack_scales(self, scale: torch.Tensor):
        return ops.repack_scales(scale)

    def _exchange_buffers(self, device):
        """Allocate this rank's receive buffers [2, world, rows_max, N] f32 and map every peer's for THIS device.
        Returns the base address of every rank's buffer as seen from this process."""
        import ctypes
        from . import _lib
        lib = _lib.load()
        self._slot_elems = self.rows_max * self.N
        nbytes = 2 * self.world_size * self._slot_elems * 4
        handle = ctypes.create_string_buffer(64)
        base = ctypes.c_void_p()
        with torch.cuda.device(device):
            _lib.check(lib.wb200_peer_buffer_create(nbytes, ctypes.byref(base), handle))
        self._recv_ptr = base.value
        self._opened = []
        if self.world_size == 1:
            return [self._recv_ptr]
        gathered = [None] * self.world_size
        dist.all_gather_object(gathered, handle.raw, group=self.group)
        self._flag = torch.zeros(1, dtype=torch.int32, device=device)
        peers = []
        with torch.cuda.device(device):
            for r in range(self.world_size):
                if r == self.rank:
                    peers.append(self._recv_ptr)
                    continue
                p = ctypes.c_void_p()
                _lib.check(lib.wb200_peer_buffer_open(ctypes.create_string_buffer(gathered[r], 64), ctypes.byref(p)))
                self._opened.append(p.value)
                peers.append(p.value)
        return peers

    def close(self) -> None:
        """Unmap the peers' buffers and free this rank's. Call on every rank, after a barrier."""
        from . import _lib
        lib = _lib.load()
        for p in getattr(self, "_opened", []):
            lib.wb200_peer_buffer_close(p)
        self._opened = []
        if getattr(self, "_recv_ptr", None):
            lib.wb200_peer_buffer_destroy(self._recv_ptr)
            self._recv_ptr = None

    def _slot_ptr(self, owner: int, parity: int, source: int) -> int:
        return self._peers[owner] + ((parity * self.world_size + source) * self._slot_elems) * 4

    def _scatter_gemm(self, a: torch.Tensor, a_scale: torch.Tensor, parity: int) -> None:
        """Partial products of this rank's K columns, rows of rank d written to slot [parity, self.rank] of d's buffer."""
        import ctypes
        from . import _lib
        lib = _lib.load()
        a_sf = ops.repack_scales(a_scale)
        W = self.world_size
        offsets = (ctypes.c_int * (W + 1))(*([m0 for m0, _ in self.row_bounds] + [self.row_bounds[-1][1]]))
        ptrs = (ctypes.c_void_p * W)(*[self._slot_ptr(d, parity, self.rank) for d in range(W)])
        with torch.cuda.device(a.device):
            _lib.check(lib.wb200_mxfp4_gemm_scatter_rows(W, offsets, self.N, self.local_k, a.data_ptr(), a_sf.data.data_ptr(),
                                                         self._b.data_ptr(), self._b_sf.data.data_ptr(), ptrs, ops._DTYPE_CODE[torch.float32],
                                                         self.N, self.scatter_flags, torch.cuda.current_stream().cuda_stream))
        self._keep = (a, a_sf)  # alive until the next call: the launch is asynchronous

    def _barrier(self) -> None:
        """Stream-ordered: returns (on the stream) once every rank's scatter has finished."""
        if self.world_size > 1:
            dist.all_reduce(self._flag, group=self.group)

    def _reduce(self, parity: int, out: torch.Tensor) -> None:
        from . import _lib
        lib = _lib.load()
        rows = self.m1 - self.m0
        if rows == 0:
            return
        with torch.cuda.device(out.device):
            _lib.check(lib.wb200_sum_slots(self._slot_ptr(self.rank, parity, 0), self.world_size, self._slot_elems, rows * self.N,
                                           out.data_ptr(), ops._DTYPE_CODE[out.dtype], torch.cuda.current_stream().cuda_stream))

    # -----------------------------------------------------------------------------------------------------
    def __call__(self, a_cols: torch.Tensor, a_scale_cols: torch.Tensor, gather: bool = False) -> torch.Tensor:
        if self._b is None:
            raise RuntimeError("load_weight_shard() must be called before the first GEMM")
        if tuple(a_cols.shape) != (self.M, self.local_k // 2) or \
                tuple(a_scale_cols.shape) != (self.M, self.local_k // ops.SCALE_GROUP_SIZE):
            raise ValueError(f"rank {self.rank} takes a {(self.M, self.local_k // 2)} and scales "
                             f"{(self.M, self.local_k // ops.SCALE_GROUP_SIZE)}, got {tuple(a_cols.shape)} and {tuple(a_scale_cols.shape)}")
        parity = self._calls & 1
        self._calls += 1
        if self.local_k:
            self._scatter_gemm(a_cols.contiguous(), a_scale_cols.contiguous(), parity)
        self._barrier()
        rows = self.m1 - self.m0
        if not gather:
            c = torch.empty(rows, self.N, dtype=self.out.torch_dtype, device=a_cols.device)
            self._reduce(parity, c)
            return c
        stacked = torch.zeros(self.world_size, self.rows_max, self.N, dtype=self.out.torch_dtype, device=a_cols.device)
        self._reduce(parity, stacked[self.rank][:rows])
        if self.world_size > 1:
            dist.all_gather_into_tensor(stacked.view(-1), stacked[self.rank].reshape(-1).clone(), group=self.group)
        full = torch.empty(self.M, self.N, dtype=self.out.torch_dtype, device=a_cols.device)
        for r, (m0, m1) in enumerate(self.row_bounds):
            if m1 > m0:
                full[m0:m1].copy_(stacked[r][: m1 - m0])
        return full
