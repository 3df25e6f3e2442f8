"""MXFP helpers with the reference's names (wave_lang/kernel/wave/utils/mxfp_utils.py), GPU-side.

Input generation and the two "preshuffle" entry points callers of the reference use. The
reference GEMM itself (`torchScaledGemmMXFP4`) is a CPU oracle and deliberately not part of this
package; the tests hold their own restatement of it.
"""

from __future__ import annotations

import torch
from torch import Tensor

from . import ops
from .ops import SCALE_GROUP_SIZE, PackedScales  # noqa: F401  (re-exported)


def generate_gemm_afp4wfp4_inputs(shape, device=None, scale_range=(124, 128)):
    """Seeded random packed-FP4 operands and E8M0 scales, as mxfp_utils.py:20-57: the same seed (5),
    draws and shapes; returns x [M, K/2], w [K/2, N] (a transposed view: pass `w.T.contiguous()` to
    the kernel), x_scales [M, K/32], w_scales [N, K/32]. `scale_range` is [lo, hi)."""
    if device is None:
        device = torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu")
    M, N, K = shape
    torch.manual_seed(5)
    x_low = torch.randint(0, 16, (M, K // 2), dtype=torch.uint8, device=device)
    x_high = torch.randint(0, 16, (M, K // 2), dtype=torch.uint8, device=device)
    x = x_low | (x_high << 4)
    w_low = torch.randint(0, 16, (N, K // 2), dtype=torch.uint8, device=device)
    w_high = torch.randint(0, 16, (N, K // 2), dtype=torch.uint8, device=device)
    w = (w_low | (w_high << 4)).T
    lo, hi = scale_range
    x_scales = torch.randint(lo, hi, (K // SCALE_GROUP_SIZE, M), dtype=torch.uint8, device=device)
    w_scales = torch.randint(lo, hi, (K // SCALE_GROUP_SIZE, N), dtype=torch.uint8, device=device)
    return x, w, x_scales.T.contiguous(), w_scales.T.contiguous()


def e8m0_shuffle(scale: Tensor) -> PackedScales:
    """Pre-shuffle a [rows, K/32] E8M0 scale matrix for the `*_preshuffle_*` templates.

    The reference permutes into the AMD scaled-MFMA layout on the host (mxfp_utils.py:113-128).
    The B200 counterpart is the tcgen05 scale-factor layout, produced by a CUDA kernel; the result
    is a PackedScales object that the preshuffle templates take in place of the scale tensor.
    """
    return ops.repack_scales(scale)


def b_preshuffle(b: Tensor) -> Tensor:
    """The reference reorders 16-row x 32-byte tiles of b for direct global reads on AMD
    (mxfp_utils.py:98-110). TMA with the 128-byte swizzle reads row-major b at full speed, so on
    B200 this is the identity; it exists so that call sites need no change."""
    return b


def mxfp4_dequant(q: Tensor, scale: Tensor) -> Tensor:
    """E2M1 x 2^(scale-127) as f32 on the GPU: the dequantised operand of mxfp_utils.py:60-95,135-142."""
    return ops.dequant_mxfp4(q, scale)


def quantize_mxfp4(x: Tensor):
    """f32 / bf16 [rows, K] -> (codes, row-major scales, PackedScales) on the GPU; see ops.quantize_mxfp4."""
    return ops.quantize_mxfp4(x)
