"""Scaled-MMA instruction kinds accepted by the templates.

The reference names AMD intrinsics here (wave_lang/kernel/wave/constraints.py:79-86). Their
members are kept so that calls written for the reference run unchanged; whichever is passed, the
B200 kernels issue `tcgen05.mma.kind::mxf4.block_scale` (128 or 256 x N x 64, E8M0 scales per 32).
"""

from enum import Enum


class ScaledMMAType(Enum):
    # reference members (CDNA4, GFX1250)
    F32_16x16x128_F8F6F4 = 0x1340
    F32_32x32x64_F8F6F4 = 0x1341
    GFX1250_F32_16x16x128_F8F6F4 = 0x1940
    # the instruction this library issues
    SM100_F32_128xNx64_MXF4 = 0xB200
