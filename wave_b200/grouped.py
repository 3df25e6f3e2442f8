"""Grouped (per-expert) MXFP4 GEMM: the MoE shape of the scaled-GEMM path.

The reference has no MXFP4 MoE kernel: its MoE test drives an f16/bf16 GEMM per expert from a
Python loop (tests/kernel/moe_test.py:183-240, wave_lang/kernel/wave/templates/moe.py:17-86).
Here the rows routed to each expert are gathered into one activation matrix, every expert keeps its
own weight matrix and packed scales resident, and one call computes

    c[row_offsets[e] : row_offsets[e+1], :] = a[rows of e] @ b_e^T        for every expert e.

The activation scales are packed per expert, each expert's block starting at a 128-row boundary of
the packed array, because a scale-factor atom covers 128 consecutive rows of one GEMM.
"""

from __future__ import annotations

import ctypes
from typing import Sequence

import torch

from . import _lib, ops
from .lang import as_output_dtype


class ExpertWeights:
    """Weights of all experts, prepared once: contiguous packed bytes and packed scales per expert."""

    def __init__(self, b_list: Sequence[torch.Tensor], b_scale_list: Sequence[torch.Tensor]):
        if len(b_list) != len(b_scale_list) or not b_list:
            raise ValueError("need one scale tensor per expert weight")
        self.N, half_k = b_list[0].shape
        self.K = half_k * 2
        self.b = []
        self.b_sf = []
        for e, (b, s) in enumerate(zip(b_list, b_scale_list)):
            ops._as_u8(b, f"b[{e}]")
            if tuple(b.shape) != (self.N, self.K // 2) or tuple(s.shape) != (self.N, self.K // ops.SCALE_GROUP_SIZE):
                raise ValueError(f"expert {e}: expected b {(self.N, self.K // 2)} and scales "
                                 f"{(self.N, self.K // ops.SCALE_GROUP_SIZE)}, got {tuple(b.shape)} and {tuple(s.shape)}")
            self.b.append(b.contiguous())
            self.b_sf.append(ops.repack_scales(s))
        n = len(self.b)
        self._b_ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in self.b])
        self._sf_ptrs = (ctypes.c_void_p * n)(*[p.data.data_ptr() for p in self.b_sf])

    def __len__(self) -> int:
        return len(self.b)


def route_top_k(router_logits: torch.Tensor, k: int = 2):
    """Rows per expert for top-k routing: returns (token index of every routed row, expert-major and
    ascending by token inside an expert; row_offsets [E+1] as a Python list). Bookkeeping on the
    routing decision only; the activations themselves are gathered by the caller."""
    E = router_logits.shape[1]
    top = router_logits.topk(k, dim=1).indices  # [T, k]
    tokens = torch.arange(router_logits.shape[0], device=router_logits.device).unsqueeze(1).expand_as(top)
    expert = top.reshape(-1)
    order = torch.sort(expert * router_logits.shape[0] + tokens.reshape(-1)).indices  # expert-major, token ascending
    counts = torch.bincount(expert, minlength=E).tolist()
    offsets = [0]
    for cnt in counts:
        offsets.append(offsets[-1] + cnt)
    return tokens.reshape(-1)[order], offsets


def grouped_scaled_gemm(a: torch.Tensor, a_scale: torch.Tensor, experts: ExpertWeights, row_offsets: Sequence[int],
                        c: torch.Tensor) -> None:
    """a [R, K/2] gathered activations (rows of expert e at row_offsets[e]:row_offsets[e+1]),
    a_scale [R, K/32] row-major, c [R, N] f32 or bf16, written in place on the current stream."""
    lib = _lib.load()
    E = len(experts)
    if len(row_offsets) != E + 1 or row_offsets[0] != 0 or row_offsets[-1] != a.shape[0]:
        raise ValueError("row_offsets must have one entry per expert plus one, start at 0 and end at the row count of a")
    as_output_dtype(c.dtype)
    ops._as_u8(a, "a")
    if not a.is_contiguous():
        a = a.contiguous()
    K, N = experts.K, experts.N
    if a.shape[1] * 2 != K or tuple(a_scale.shape) != (a.shape[0], K // ops.SCALE_GROUP_SIZE):
        raise ValueError("a / a_scale do not match the experts' K")
    if tuple(c.shape) != (a.shape[0], N) or c.stride(1) != 1:
        raise ValueError(f"c must be [{a.shape[0]}, {N}] with unit column stride")
    # activation scales: one packed block per expert, starting at a 128-row block boundary
    block_offsets = [0]
    for e in range(E):
        block_offsets.append(block_offsets[-1] + (row_offsets[e + 1] - row_offsets[e] + 127) // 128)
    atom_row_bytes = ops.packed_scale_bytes(128, K)
    a_sf = torch.empty(max(block_offsets[-1], 1) * atom_row_bytes, dtype=torch.uint8, device=a.device)
    offs = (ctypes.c_int * (E + 1))(*row_offsets)
    boffs = (ctypes.c_int * (E + 1))(*block_offsets)
    if a_scale.stride(1) != 1:
        a_scale = a_scale.contiguous()
    with torch.cuda.device(a.device):
        stream = torch.cuda.current_stream().cuda_stream
        if E <= 32:  # one launch packs every expert's block
            _lib.check(lib.wb200_repack_scales_grouped(a_scale.data_ptr(), a_scale.stride(0), E, offs, boffs, K,
                                                       a_sf.data_ptr(), stream))
        else:
            for e in range(E):
                r0, r1 = row_offsets[e], row_offsets[e + 1]
                if r1 > r0:
                    ops.repack_scales(a_scale[r0:r1], out=a_sf[block_offsets[e] * atom_row_bytes:])
        _lib.check(lib.wb200_mxfp4_grouped_gemm(E, offs, boffs, N, K, a.data_ptr(), a_sf.data_ptr(), experts._b_ptrs,
                                                experts._sf_ptrs, c.data_ptr(), ops._DTYPE_CODE[c.dtype], c.stride(0),
                                                torch.cuda.current_stream().cuda_stream))


def moe_scaled_gemm(a: torch.Tensor, a_scale: torch.Tensor, experts: ExpertWeights, expert_ids: torch.Tensor,
                    num_rows: torch.Tensor, c: torch.Tensor) -> None:
    """Grouped GEMM over the row layout of `moe_align_block_size(..., block_size=256, ...)`, driven by its device
    outputs: a [R, K/2] / a_scale [R, K/32] hold the routed rows of all experts (R a multiple of 256, every expert
    padded to whole 256-row blocks), expert_ids [>= R/256] int32 the expert of each block, num_rows [1] int32 the
    padded total. c [R, N]; row blocks at or past num_rows are left untouched. No host synchronisation."""
    lib = _lib.load()
    ops._as_u8(a, "a")
    R = a.shape[0]
    K, N = experts.K, experts.N
    if R % 256 or a.shape[1] * 2 != K or tuple(a_scale.shape) != (R, K // ops.SCALE_GROUP_SIZE) or not a.is_contiguous():
        raise ValueError("a must be contiguous [R, K/2] with R a multiple of 256, a_scale [R, K/32]")
    if tuple(c.shape) != (R, N) or c.stride(1) != 1:
        raise ValueError(f"c must be [{R}, {N}] with unit column stride")
    if expert_ids.dtype != torch.int32 or num_rows.dtype != torch.int32 or expert_ids.numel() < R // 256:
        raise ValueError("expert_ids (one int32 per 256-row block) and num_rows (int32) must be device tensors")
    as_output_dtype(c.dtype)
    a_sf = ops.repack_scales(a_scale)
    with torch.cuda.device(a.device):
        _lib.check(lib.wb200_mxfp4_moe_gemm(len(experts), R, expert_ids.data_ptr(), num_rows.data_ptr(), N, K, a.data_ptr(),
                                            a_sf.data.data_ptr(), experts._b_ptrs, experts._sf_ptrs, c.data_ptr(),
                                            ops._DTYPE_CODE[c.dtype], c.stride(0), torch.cuda.current_stream().cuda_stream))
