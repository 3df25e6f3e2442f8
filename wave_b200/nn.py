"""A linear layer on the MXFP4 path: weights held as packed E2M1 codes with their scales already in
the layout the GEMM reads, activations quantised on the fly.

Counterpart of the reference's module wrappers around its kernels (wave_lang/kernel/wave/nn/linear.py:147
`WaveLinear`, nn/quant_linear.py:196 `WaveQuantLinear`, which is FP8 per-tensor); the reference has
no MXFP4 module. forward(x) = dequant(quantise(x)) @ dequant(W)^T, output bf16 or f32.
"""

from __future__ import annotations

import torch

from . import ops
from .lang import as_output_dtype


class MXFP4Linear(torch.nn.Module):
    def __init__(self, weight_codes: torch.Tensor, weight_scales: torch.Tensor, output_dtype=torch.bfloat16):
        """weight_codes [N, K/2] uint8, weight_scales [N, K/32] uint8 (row-major E8M0), both on the GPU."""
        super().__init__()
        ops._as_u8(weight_codes, "weight_codes")
        self.out_features, half_k = weight_codes.shape
        self.in_features = half_k * 2
        self.output_dtype = as_output_dtype(output_dtype).torch_dtype
        self.register_buffer("weight_codes", weight_codes.contiguous())
        self.register_buffer("weight_scales", weight_scales.contiguous())
        self._packed = ops.repack_scales(self.weight_scales)  # once
        # decode calls (at most 128 rows) read a second packing, per tile of the height that gives every SM the same number
        # of weight tiles; made on first use, and only where that height differs from 128
        self._packed_decode = None

    @classmethod
    def from_float(cls, weight: torch.Tensor, output_dtype=torch.bfloat16) -> "MXFP4Linear":
        """Quantise an f32 / bf16 [N, K] weight on the GPU."""
        q, s, _ = ops.quantize_mxfp4(weight, want_rowmajor=True, want_packed=False)
        return cls(q, s, output_dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        q, _, sf = ops.quantize_mxfp4(x2, want_rowmajor=False, want_packed=True)
        out = torch.empty(x2.shape[0], self.out_features, dtype=self.output_dtype, device=x.device)
        packed = self._packed
        if x2.shape[0] <= 128:
            if self._packed_decode is None:
                h = ops.decode_tile_rows(self.out_features, x.device)
                self._packed_decode = self._packed if h == 128 else ops.repack_scales(self.weight_scales, tile_rows=h)
            packed = self._packed_decode
        ops.scaled_gemm_packed(q, sf, self.weight_codes, packed, out)
        return out.reshape(*lead, self.out_features)
