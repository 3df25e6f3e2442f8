"""Mixture-of-experts steps around the grouped MXFP4 GEMM, and the expert MLP built from them.

The reference's MoE is a Python loop over experts calling an f16/bf16 GEMM, `silu_and_mul` and a
second GEMM per expert, followed by a weighted sum (tests/kernel/moe_test.py:183-260; kernels in
wave_lang/kernel/wave/templates/moe.py). Its block-alignment step exists as a torch function
(tests/kernel/moe/torch_kernels.py:10-97). Here every step is a CUDA kernel behind the C ABI and the
two projections are grouped MXFP4 GEMMs over all experts at once:

    route -> moe_align_block_size(256) -> quantise tokens -> gather rows -> grouped GEMM (gate|up)
          -> silu_and_mul fused with MXFP4 quantisation -> grouped GEMM (down) -> weighted combine

The grouped GEMMs read the routing (expert of every 256-row block, padded row count) from the device arrays
the alignment kernel wrote, so a forward pass has no host synchronisation.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib, ops
from .grouped import ExpertWeights, moe_scaled_gemm
from .lang import DataType, TORCH_DTYPE_TO_WAVE, bf16, f32


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def moe_align_block_size(topk_ids: torch.Tensor, num_experts: int, block_size: int, sorted_ids: torch.Tensor,
                         expert_ids: torch.Tensor, num_tokens_post_pad: torch.Tensor,
                         inverse: torch.Tensor | None = None) -> None:
    """Same arguments and outputs as moe_align_block_size_pytorch (tests/kernel/moe/torch_kernels.py:10-97):
    all outputs are int32 tensors pre-allocated by the caller; `inverse` [topk_ids.numel()] is an extra."""
    lib = _lib.load()
    if topk_ids.dtype not in (torch.int32, torch.int64) or not topk_ids.is_cuda:
        raise ValueError("topk_ids must be an int32 or int64 CUDA tensor")
    ids = topk_ids.contiguous()
    for name, t in (("sorted_ids", sorted_ids), ("expert_ids", expert_ids), ("num_tokens_post_pad", num_tokens_post_pad)):
        if t.dtype != torch.int32 or not t.is_contiguous() or t.device != ids.device:
            raise ValueError(f"{name} must be a contiguous int32 tensor on the device of topk_ids")
    if inverse is not None and (inverse.dtype != torch.int32 or inverse.numel() < ids.numel() or not inverse.is_contiguous()):
        raise ValueError("inverse must be a contiguous int32 tensor with one entry per routed pair")
    with torch.cuda.device(ids.device):
        _lib.check(lib.wb200_moe_align_block_size(ids.data_ptr(), int(ids.dtype == torch.int64), ids.numel(), num_experts,
                                                  block_size, sorted_ids.data_ptr(), sorted_ids.numel(),
                                                  expert_ids.data_ptr(), expert_ids.numel(), num_tokens_post_pad.data_ptr(),
                                                  inverse.data_ptr() if inverse is not None else None, _stream()))


def gather_rows(src: torch.Tensor, sorted_ids: torch.Tensor, num_ids: int, top_k: int, out: torch.Tensor) -> None:
    """out[p] = src[sorted_ids[p] // top_k] for real entries, zero rows for padding entries (uint8 matrices)."""
    lib = _lib.load()
    ops._as_u8(src, "src")
    ops._as_u8(out, "out")
    if src.dim() != 2 or out.dim() != 2 or src.shape[1] != out.shape[1] or src.stride(1) != 1 or out.stride(1) != 1:
        raise ValueError("src and out must be 2-D uint8 matrices with rows of the same length")
    if out.shape[0] > sorted_ids.numel():
        raise ValueError("sorted_ids is shorter than out")
    with torch.cuda.device(src.device):
        _lib.check(lib.wb200_moe_gather_rows(src.data_ptr(), src.stride(0), src.shape[1], sorted_ids.data_ptr(), out.shape[0],
                                             num_ids, top_k, out.data_ptr(), out.stride(0), _stream()))


def quantize_scatter(x: torch.Tensor, dst_rows: torch.Tensor, top_k: int, q: torch.Tensor, scale: torch.Tensor) -> None:
    """Quantise x [T, K] (f32 / bf16) to MXFP4 and write row t to rows dst_rows[t * top_k + j] of q [R, K/2] and
    scale [R, K/32] (both contiguous uint8): tokens go straight to their expert-sorted rows."""
    lib = _lib.load()
    if x.dtype not in ops._DTYPE_CODE or x.dim() != 2 or not x.is_cuda:
        raise ValueError("x must be a 2-D f32 or bf16 CUDA tensor")
    if x.stride(1) != 1:
        x = x.contiguous()
    T, K = x.shape
    if dst_rows.dtype != torch.int32 or dst_rows.numel() != T * top_k or not dst_rows.is_contiguous():
        raise ValueError("dst_rows must be a contiguous int32 tensor with tokens * top_k entries")
    ops._as_u8(q, "q")
    ops._as_u8(scale, "scale")
    if not (q.is_contiguous() and scale.is_contiguous()) or q.shape[1] != K // 2 or scale.shape[1] != K // 32 or \
            q.shape[0] != scale.shape[0]:
        raise ValueError("q must be contiguous [R, K/2] and scale contiguous [R, K/32]")
    with torch.cuda.device(x.device):
        _lib.check(lib.wb200_moe_quantize_scatter(x.data_ptr(), ops._DTYPE_CODE[x.dtype], x.stride(0) if T > 1 else K, T, K,
                                                  top_k, dst_rows.data_ptr(), q.data_ptr(), scale.data_ptr(), _stream()))


def silu_and_mul(x1: torch.Tensor, x2: torch.Tensor, out: torch.Tensor | None = None, quantize: bool = False,
                 num_rows: torch.Tensor | None = None):
    """out = silu(x1) * x2 ([rows, n], f32 or bf16, unit column stride; x1 and x2 may be column blocks of one
    matrix). With quantize=True also returns (codes [rows, n/2], scales [rows, n/32]) of the f32 result
    quantised to MXFP4 in the same pass; `out` may then be omitted. num_rows: int32 device tensor, rows at or
    past its value are skipped."""
    lib = _lib.load()
    if x1.dtype not in ops._DTYPE_CODE or x2.dtype != x1.dtype or x1.shape != x2.shape or x1.dim() != 2:
        raise ValueError("x1 and x2 must be 2-D f32 or bf16 tensors of the same shape and type")
    if x1.stride(1) != 1 or x2.stride(1) != 1 or not x1.is_cuda:
        raise ValueError("x1 and x2 must be CUDA tensors with unit column stride")
    rows, n = x1.shape
    if out is None and not quantize:
        out = torch.empty(rows, n, dtype=x1.dtype, device=x1.device)
    if out is not None and (out.dtype != x1.dtype or tuple(out.shape) != (rows, n) or out.stride(1) != 1):
        raise ValueError("out must match x1 in shape and type, with unit column stride")
    q = s = None
    if quantize:
        q = torch.empty(rows, n // 2, dtype=torch.uint8, device=x1.device)
        s = torch.empty(rows, n // 32, dtype=torch.uint8, device=x1.device)
    ld = lambda t: t.stride(0) if rows > 1 else n  # noqa: E731
    with torch.cuda.device(x1.device):
        _lib.check(lib.wb200_silu_and_mul(x1.data_ptr(), x2.data_ptr(), ld(x1), ld(x2), ops._DTYPE_CODE[x1.dtype], rows, n,
                                          out.data_ptr() if out is not None else None, ld(out) if out is not None else n,
                                          q.data_ptr() if quantize else None, s.data_ptr() if quantize else None, None,
                                          num_rows.data_ptr() if num_rows is not None else None, _stream()))
    return (out, q, s) if quantize else out


def combine(y: torch.Tensor, row_of: torch.Tensor, weight: torch.Tensor, top_k: int, out: torch.Tensor) -> None:
    """out[t] = sum_j weight[t, j] * y[row_of[t, j]] (f32 accumulation, slot order)."""
    lib = _lib.load()
    if y.dtype not in ops._DTYPE_CODE or out.dtype != y.dtype or y.stride(1) != 1 or out.stride(1) != 1:
        raise ValueError("y and out must be f32 or bf16 matrices of the same type with unit column stride")
    tokens, cols = out.shape
    if row_of.dtype != torch.int32 or weight.dtype != torch.float32 or row_of.numel() != tokens * top_k or \
            weight.numel() != tokens * top_k or not row_of.is_contiguous() or not weight.is_contiguous():
        raise ValueError("row_of (int32) and weight (f32) must be contiguous with tokens * top_k entries")
    with torch.cuda.device(y.device):
        _lib.check(lib.wb200_moe_combine(y.data_ptr(), y.stride(0), ops._DTYPE_CODE[y.dtype], row_of.data_ptr(),
                                         weight.data_ptr(), tokens, top_k, cols, out.data_ptr(), out.stride(0), _stream()))


@dataclass
class SiluAndMulTemplate:
    """What get_silu_and_mul_kernel returns in place of the reference's traced kernel."""
    shape: tuple
    datatype: DataType


def get_silu_and_mul_kernel(m: int, n: int, datatype):
    """(kernel, hyperparams) for out[M, N] = silu(x1) * x2 — wave_lang/kernel/wave/templates/moe.py:89-145.
    `wave_compile(options, kernel)` returns a callable (x1, x2, out)."""
    dt = datatype if isinstance(datatype, DataType) else TORCH_DTYPE_TO_WAVE.get(datatype)
    assert dt in (f32, bf16), f"Unsupported datatype: {datatype}"
    return SiluAndMulTemplate((m, n), dt), {"M": m, "N": n}


class SiluAndMulKernel:
    def __init__(self, template: SiluAndMulTemplate, options):
        self.template, self.options, self.asm = template, options, ""

    def __call__(self, x1, x2, out) -> None:
        if tuple(x1.shape) != tuple(self.template.shape) or x1.dtype != self.template.datatype.torch_dtype:
            raise ValueError(f"kernel was built for {self.template.shape} {self.template.datatype}")
        silu_and_mul(x1, x2, out)

    invoke = __call__


class MXFP4ExpertMLP:
    """Top-k routed expert MLP with MXFP4 weights: y = sum_j w_j * down_e(silu(gate_e(x)) * up_e(x)).

    w1 [E][2 I, K/2] holds gate rows then up rows (the fused w1 of torch_ref_moe,
    tests/kernel/moe_test.py:108-121), w2 [E][K_out, I/2]; scales row-major per expert.
    Routing weights are softmax(logits) in f32, top-k (tests/kernel/moe_test.py:111-112).
    """

    BLOCK = 256  # rows per routing block = rows of one CTA-pair tile: every tile belongs to one expert

    def __init__(self, w1, w1_scale, w2, w2_scale, top_k: int = 2):
        self.w1 = ExpertWeights(w1, w1_scale)
        self.w2 = ExpertWeights(w2, w2_scale)
        if len(self.w1) != len(self.w2) or self.w1.N % 2 or self.w2.K * 2 != self.w1.N:
            raise ValueError("w1 must be [E][2 I, K/2] and w2 [E][K_out, I/2] for the same E and I")
        self.top_k = top_k
        self.E, self.K, self.I = len(self.w1), self.w1.K, self.w1.N // 2

    def route(self, router_logits: torch.Tensor):
        score = torch.softmax(router_logits, dim=-1, dtype=torch.float32)
        weight, ids = torch.topk(score, self.top_k)
        return weight.contiguous(), ids.contiguous()

    def forward(self, x: torch.Tensor, router_logits: torch.Tensor) -> torch.Tensor:
        """Everything is sized by the worst case of the routing (tokens * top_k + E * 255 rows) and driven by the
        device outputs of the block alignment, so the call never waits for the GPU."""
        T, dev = x.shape[0], x.device
        n = T * self.top_k
        B = self.BLOCK
        weight, ids = self.route(router_logits)
        cap = (n + self.E * (B - 1) + B - 1) // B * B
        sorted_ids = torch.empty(cap, dtype=torch.int32, device=dev)
        expert_ids = torch.empty(cap // B, dtype=torch.int32, device=dev)
        post_pad = torch.empty(1, dtype=torch.int32, device=dev)
        inverse = torch.empty(n, dtype=torch.int32, device=dev)
        moe_align_block_size(ids, self.E, B, sorted_ids, expert_ids, post_pad, inverse)
        # Tokens are quantised once and written straight to their sorted rows. Padding rows are never written:
        # every output row of a GEMM depends on its own input row only, and `combine` reads routed rows only,
        # so whatever the padding rows hold stays in the padding rows.
        a = torch.empty(cap, self.K // 2, dtype=torch.uint8, device=dev)
        a_s = torch.empty(cap, self.K // 32, dtype=torch.uint8, device=dev)
        quantize_scatter(x, inverse, self.top_k, a, a_s)
        h = torch.empty(cap, 2 * self.I, dtype=torch.bfloat16, device=dev)
        moe_scaled_gemm(a, a_s, self.w1, expert_ids, post_pad, h)
        _, hq, hs = silu_and_mul(h[:, :self.I], h[:, self.I:], quantize=True, num_rows=post_pad)
        y = torch.empty(cap, self.w2.N, dtype=torch.bfloat16, device=dev)
        moe_scaled_gemm(hq, hs, self.w2, expert_ids, post_pad, y)
        out = torch.empty(T, self.w2.N, dtype=torch.bfloat16, device=dev)
        combine(y, inverse, weight.reshape(-1), self.top_k, out)
        return out

    __call__ = forward
