"""CPU oracle for the MXFP8 scaled GEMM — TEST INFRASTRUCTURE, not a product path.

Restates the reference's own CPU functions for this variant, which live in its test file:
`generate_gemm_afp8wfp8_inputs` (tests/kernel/wave_gemm_mxfp_test.py:64-77) and
`torchScaledGemmMXFP8` (tests/kernel/wave_gemm_mxfp_test.py:80-91). Only `tests/` may import this module.

Parity is pinned: `tests/golden/make_golden.py` executes those two reference functions themselves
(their source is read from the reference tree at generation time) and stores their outputs in
`tests/golden/gemm_mxfp8_seed5_64x96x128.npz`; `tests/test_oracle.py` checks this file against them.
"""

from __future__ import annotations

import torch

from .mxfp4_oracle import SCALE_GROUP_SIZE, e8m0_to_f32


def generate_gemm_afp8wfp8_inputs(shape, seed: int = 5, dtype=torch.float8_e5m2):
    """tests/kernel/wave_gemm_mxfp_test.py:64-77 on the CPU: x [M, K] f8, w [K, N] f8 (a transposed view of
    [N, K]), scales uniform in [124, 128) generated as [K/32, rows] and transposed (views, not contiguous)."""
    M, N, K = shape
    torch.manual_seed(seed)                                                         # :66
    x = torch.randn((M, K), dtype=torch.float32).to(dtype)                          # :68
    w = torch.randn((N, K), dtype=torch.float32).to(dtype)                          # :69
    w = w.T                                                                         # :70
    x_scales = torch.randint(124, 128, (K // SCALE_GROUP_SIZE, M), dtype=torch.uint8)   # :72
    w_scales = torch.randint(124, 128, (K // SCALE_GROUP_SIZE, N), dtype=torch.uint8)   # :73
    return x, w, x_scales.T, w_scales.T                                             # :74-77


def dequant_mxfp8(x: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """[R, K] f8 and [R, K/32] E8M0 -> [R, K] f32 (:82-86: value * 2^(scale - 127), exact in f32)."""
    s = scales.repeat_interleave(SCALE_GROUP_SIZE, dim=1).to(torch.float32)
    return x.to(torch.float32) * e8m0_to_f32(s)


def torch_scaled_gemm_mxfp8(x, w, x_scales, w_scales) -> torch.Tensor:
    """tests/kernel/wave_gemm_mxfp_test.py:80-91: w is [K, N], w_scales [N, K/32]."""
    x_f32 = dequant_mxfp8(x, x_scales)                                              # :82-87
    w_f32 = w.to(torch.float32) * e8m0_to_f32(
        w_scales.repeat_interleave(SCALE_GROUP_SIZE, dim=1).to(torch.float32)).T   # :88-90
    return torch.mm(x_f32, w_f32)                                                   # :91


def torch_scaled_gemm_mxfp8_mxfp4(x, w_codes, x_scales, w_scales) -> torch.Tensor:
    """The mixed pair of the same scaled MMA: 8-bit activations x [M, K] against packed E2M1 weights w_codes [N, K/2]
    (the kernel's layout), each with E8M0 block scales: dequantise both as the reference's two oracles do
    (tests/kernel/wave_gemm_mxfp_test.py:80-91 for the 8-bit side, wave_lang/kernel/wave/utils/mxfp_utils.py:131-143 for
    the 4-bit side), then one f32 torch.mm. The reference has no test of this pair; its scaled MMA takes it
    (wave_lang/kernel/wave/constraints.py:79-86)."""
    from .mxfp4_oracle import dequant_mxfp4
    return torch.mm(dequant_mxfp8(x, x_scales), dequant_mxfp4(w_codes, w_scales).T)


def quantize_mxfp8(x: torch.Tensor, dtype=torch.float8_e5m2):
    """f32 [R, K] -> (f8 [R, K], scales [R, K/32] uint8). Not in the reference (its MXFP8 test feeds random values,
    tests/kernel/wave_gemm_mxfp_test.py:64-77); the block rule of the MXFP4 harness quantiser carried over:
    e = floor(log2(amax)) - emax_elem (8 for E4M3, whose largest value is 448 = 1.75 * 2^8; 15 for E5M2, 57344 =
    1.75 * 2^15), scale byte clamp(e + 127, 0, 254), amax == 0 -> 127; values x * 2^-e clamped to the largest
    finite value and rounded to nearest even by the type conversion. A block that holds a NaN or an infinity gets
    scale byte 255 (E8M0's NaN) and zero codes, as in the MXFP4 quantiser."""
    R, K = x.shape
    assert K % SCALE_GROUP_SIZE == 0
    emax, vmax = (8, 448.0) if dtype == torch.float8_e4m3fn else (15, 57344.0)
    xb = x.reshape(R, K // 32, 32).to(torch.float32)
    bad = ~torch.isfinite(xb).all(dim=2)
    xb = torch.where(bad.unsqueeze(2), torch.zeros_like(xb), xb)
    amax = xb.abs().amax(dim=2)
    e = torch.floor(torch.log2(torch.where(amax > 0, amax, torch.ones_like(amax)))) - float(emax)
    e = torch.where(amax > 0, e, torch.zeros_like(e))
    sb = torch.clamp(e + 127.0, 0, 254)
    y = torch.clamp(xb / torch.pow(torch.tensor(2.0), sb - 127.0).unsqueeze(2), -vmax, vmax)
    sb = torch.where(bad, torch.full_like(sb, 255.0), sb)
    return y.reshape(R, K).to(dtype), sb.to(torch.uint8)
