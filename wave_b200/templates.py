"""MXFP4 scaled-GEMM kernel templates with the reference's names and signatures.

In the reference these functions build a traced DSL kernel plus its symbol table
(wave_lang/kernel/wave/templates/gemm.py:134-205, wave_lang/kernel/wave/templates/tagged_mxfp4_gemm.py).
Here they return a small descriptor that `wave_compile` turns into a launcher of the precompiled
sm_100a kernels. Tile, wave and address-space arguments describe AMD work distribution; they are
accepted, recorded, and have no effect on B200, where the tile shape is fixed by tcgen05.mma
(128 or 256 rows x 128/256 columns x 256 K elements per stage).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

from . import _lib
from .compile import SchedulingType, WaveCompileOptions
from .constraints import ScaledMMAType
from .lang import SHARED_ADDRESS_SPACE, DataType, as_output_dtype, f32


@dataclass
class ScaledGemmTemplate:
    """What a template function returns in place of the reference's traced kernel."""

    name: str
    shape: Optional[tuple]                 # (M, N, K) given at creation, or None
    output_dtype: DataType = f32
    accumulate: bool = False               # split-K contract: add into caller-initialised c
    num_splits: int = 1
    preshuffled_scales: bool = False       # scale arguments are PackedScales from e8m0_shuffle
    preshuffled_b: bool = False            # b went through b_preshuffle (identity on B200)
    broadcast_a_scale: bool = False        # a_scale is [M]: one scale per row for all of K
    element_bits: int = 4                  # 4: packed E2M1 (MXFP4); 8: one byte per element (MXFP8)
    element_format: str = "f4e2m1fn"       # MXFP8: "f8e5m2" or "f8e4m3fn"
    weight_bits: int = 0                   # 8-bit kernels only: 4 = b is packed E2M1 (the mixed f8 x f4 pair); 0 = as a
    hints: dict = field(default_factory=dict)


def _hyperparams(shape, block_shape, extra=None):
    h = {"M": shape[0], "N": shape[1], "K": shape[2],
         "BLOCK_M": block_shape[0], "BLOCK_N": block_shape[1], "BLOCK_K": block_shape[2]}
    if extra:
        h.update(extra)
    return h


def get_scaled_gemm_kernel(shape, mfma_variant: ScaledMMAType, block_shape=None, waves_per_block=None):
    """(kernel, hyperparams) for c[M, N] f32 = a * b^T — wave_lang/kernel/wave/templates/gemm.py:134-205.

    Use as the reference does:
        kernel, hyper = get_scaled_gemm_kernel(shape, ScaledMMAType.F32_16x16x128_F8F6F4)
        gemm = wave_compile(WaveCompileOptions(subs=hyper), kernel)
        gemm(a, a_scale, b, b_scale, c)
    """
    if not isinstance(mfma_variant, ScaledMMAType):
        raise TypeError("mfma_variant must be a ScaledMMAType")
    block_shape = block_shape or (32, 32, 256)
    waves_per_block = waves_per_block or (2, 2)
    tpl = ScaledGemmTemplate("scaled_gemm", tuple(shape), f32,
                             hints={"mfma_variant": mfma_variant, "block_shape": tuple(block_shape),
                                    "waves_per_block": tuple(waves_per_block)})
    return tpl, _hyperparams(shape, block_shape, {"ADDRESS_SPACE": SHARED_ADDRESS_SPACE})


def get_broadcasted_scale_gemm_mxfp4(shape, mfma_variant: ScaledMMAType):
    """(kernel, hyperparams) for the kernel whose a_scale is [M], broadcast along K before the scaled MMA —
    wave_lang/kernel/wave/templates/test_kernels.py:75-140 (tested by tests/kernel/wave_gemm_mxfp_test.py:594-634)."""
    if not isinstance(mfma_variant, ScaledMMAType):
        raise TypeError("mfma_variant must be a ScaledMMAType")
    tpl = ScaledGemmTemplate("broadcasted_scale_scaled_mma", tuple(shape), f32, broadcast_a_scale=True,
                             hints={"mfma_variant": mfma_variant, "block_shape": (32, 32, 256)})
    return tpl, _hyperparams(shape, (32, 32, 256), {"ADDRESS_SPACE": SHARED_ADDRESS_SPACE})


def get_scaled_gemm_mxfp8_kernel(shape, mfma_variant: ScaledMMAType, element_format: str = "f8e5m2", output_dtype=f32,
                                 weight_format: str | None = None):
    """(kernel, hyperparams) for the MXFP8 scaled GEMM: a [M, K], b [N, K] bytes of f8e5m2 (or f8e4m3fn),
    E8M0 scales [rows, K/32], c [M, N]. The reference has this kernel only inside its test
    (tests/kernel/wave_gemm_mxfp_test.py:416-501: same signature as the MXFP4 kernel with K instead of K/2
    columns and a bitcast to f8e5m2); this function gives it the template form of get_scaled_gemm_kernel.

    weight_format = "f4e2m1fn": the mixed pair of the same scaled MMA (F32_16x16x128_F8F6F4 takes f8, f6 and f4
    operands; in the reference's DSL it is the same kernel with b bitcast to f4e2m1fn): a stays 8-bit, b is packed E2M1
    [N, K/2] exactly as for the MXFP4 GEMM; K must be a multiple of 128."""
    if not isinstance(mfma_variant, ScaledMMAType):
        raise TypeError("mfma_variant must be a ScaledMMAType")
    if element_format not in ("f8e5m2", "f8e4m3fn"):
        raise ValueError(f"unknown 8-bit element format {element_format}")
    if weight_format not in (None, element_format, "f4e2m1fn"):
        raise ValueError(f"weights are {element_format} like the activations, or f4e2m1fn (got {weight_format})")
    if weight_format == "f4e2m1fn" and shape[2] % 128:
        raise ValueError(f"4-bit weights under 8-bit activations need K % 128 == 0 (K = {shape[2]})")
    tpl = ScaledGemmTemplate("scaled_gemm_mxfp8" if weight_format != "f4e2m1fn" else "scaled_gemm_mxfp8_mxfp4", tuple(shape),
                             as_output_dtype(output_dtype), element_bits=8, element_format=element_format,
                             weight_bits=4 if weight_format == "f4e2m1fn" else 8,
                             hints={"mfma_variant": mfma_variant, "block_shape": (32, 32, 256)})
    return tpl, _hyperparams(shape, (32, 32, 256), {"ADDRESS_SPACE": SHARED_ADDRESS_SPACE})


def _tagged(name, shape, block_shape, wave_shape, mfma_variant, output_dtype, reorder_workgroups=True,
            group_size_n=None, **flags):
    out = as_output_dtype(output_dtype)
    hints = {"mfma_variant": mfma_variant, "block_shape": tuple(block_shape), "wave_shape": tuple(wave_shape),
             "reorder_workgroups": bool(reorder_workgroups)}
    if group_size_n is not None:
        if int(group_size_n) < 1:
            raise ValueError(f"group_size_n must be at least 1, got {group_size_n}")
        hints["group_size_n"] = int(group_size_n)
    tpl = ScaledGemmTemplate(name, tuple(shape), out, hints=hints, **flags)
    options = WaveCompileOptions(subs=_hyperparams(shape, block_shape), canonicalize=True,
                                 schedule=SchedulingType.MANUAL, use_global_to_shared=True,
                                 minimize_shared_allocs=False)
    return tpl, options


def get_tagged_mxfp4_gemm(shape=(1024, 1024, 8192), block_shape=(256, 256, 256), wave_shape=(2, 2),
                          mfma_variant=ScaledMMAType.F32_16x16x128_F8F6F4, a_address_space=SHARED_ADDRESS_SPACE,
                          b_address_space=SHARED_ADDRESS_SPACE, reorder_workgroups=True, group_size_n=None,
                          output_dtype=f32):
    """(kernel, options); f32 or bf16 output — wave_lang/kernel/wave/templates/tagged_mxfp4_gemm.py:38-145.

    `reorder_workgroups` / `group_size_n` set the order in which the tile kernels visit the output tiles, as in
    the reference (groups of group_size_n workgroups along N, each swept down M): a group keeps its width in
    columns, group_size_n * BLOCK_N. group_size_n = None (the default here; the reference's is 32, tuned for its
    hardware) leaves the kernel's own group of 16 tiles of 256 columns; reorder_workgroups = False walks the
    tiles row by row. The result does not depend on either."""
    return _tagged("tagged_mxfp4_gemm", shape, block_shape, wave_shape, mfma_variant, output_dtype,
                   reorder_workgroups, group_size_n)


def get_tagged_mxfp4_gemm_preshuffle_scales(shape=(1024, 1024, 8192), block_shape=(256, 256, 256), wave_shape=(2, 2),
                                            mfma_variant=ScaledMMAType.F32_16x16x128_F8F6F4,
                                            a_address_space=SHARED_ADDRESS_SPACE, reorder_workgroups=True,
                                            group_size_n=None, output_dtype=f32):
    """Scales arrive pre-shuffled: pass the result of `mxfp_utils.e8m0_shuffle` for a_scale and b_scale
    (tagged_mxfp4_gemm.py:334-365). On B200 the shuffle is the tcgen05 scale-factor repack."""
    return _tagged("tagged_mxfp4_gemm_preshuffle_scales", shape, block_shape, wave_shape, mfma_variant, output_dtype,
                   reorder_workgroups, group_size_n,
                   preshuffled_scales=True)


def get_tagged_mxfp4_gemm_preshuffle_scales_and_B(shape=(1024, 1024, 8192), block_shape=(256, 256, 256),
                                                  wave_shape=(2, 2),
                                                  mfma_variant=ScaledMMAType.F32_16x16x128_F8F6F4,
                                                  a_address_space=SHARED_ADDRESS_SPACE, reorder_workgroups=True,
                                                  group_size_n=None, output_dtype=f32):
    """tagged_mxfp4_gemm.py:368-403: pre-shuffled scales and pre-shuffled b."""
    return _tagged("tagged_mxfp4_gemm_preshuffle_scales_and_B", shape, block_shape, wave_shape, mfma_variant, output_dtype,
                   reorder_workgroups, group_size_n, preshuffled_scales=True, preshuffled_b=True)


def get_tagged_mxfp4_gemm_preshuffle_b(shape=(1024, 1024, 8192), block_shape=(256, 256, 256), wave_shape=(2, 2),
                                       mfma_variant=ScaledMMAType.F32_16x16x128_F8F6F4,
                                       a_address_space=SHARED_ADDRESS_SPACE, reorder_workgroups=True,
                                       group_size_n=None, output_dtype=f32):
    """tagged_mxfp4_gemm.py:950-991."""
    return _tagged("tagged_mxfp4_gemm_preshuffle_b", shape, block_shape, wave_shape, mfma_variant, output_dtype,
                   reorder_workgroups, group_size_n,
                   preshuffled_scales=True, preshuffled_b=True)


def get_tagged_mxfp4_gemm_preshuffle_b_wide_store(shape=(1024, 1024, 8192), block_shape=(256, 256, 256),
                                                  wave_shape=(2, 2),
                                                  mfma_variant=ScaledMMAType.F32_16x16x128_F8F6F4,
                                                  a_address_space=SHARED_ADDRESS_SPACE, reorder_workgroups=True,
                                                  group_size_n=None, output_dtype=f32):
    """tagged_mxfp4_gemm.py:994-1035; every epilogue here already stores 16 bytes per thread."""
    return _tagged("tagged_mxfp4_gemm_preshuffle_b_wide_store", shape, block_shape, wave_shape, mfma_variant, output_dtype,
                   reorder_workgroups, group_size_n, preshuffled_scales=True, preshuffled_b=True)


def _splitk(name, shape, num_splits, block_shape, wave_shape, mfma_variant, output_type, **flags):
    # Same preconditions and messages as tagged_mxfp4_gemm.py:636-645.
    k_per_split = math.ceil(shape[2] / num_splits)
    if k_per_split < block_shape[2]:
        raise ValueError(
            f"K per split ({k_per_split}) is less than BLOCK_K ({block_shape[2]}). "
            f"Reduce num_splits or BLOCK_K so that each split has at least BLOCK_K elements.")
    if k_per_split % block_shape[2] != 0:
        raise ValueError(f"k_per_split ({k_per_split}) must be a multiple of BLOCK_K ({block_shape[2]}).")
    tpl, options = _tagged(name, shape, block_shape, wave_shape, mfma_variant, output_type, accumulate=True,
                           num_splits=num_splits, **flags)
    return tpl, options


def get_tagged_splitk_mxfp4_gemm(shape, num_splits=2, block_shape=(128, 128, 256), wave_shape=(2, 2),
                                 mfma_variant=ScaledMMAType.F32_16x16x128_F8F6F4,
                                 a_address_space=SHARED_ADDRESS_SPACE, output_type=f32):
    """Split-K GEMM that ADDS into c; the caller zero-initialises c (tagged_mxfp4_gemm.py:819-858).

    The reference sums per-split partials with atomics in the output type. Here the K range is split
    by the kernel itself (stream-K for M <= 128), partials stay in f32 and are added in a fixed
    order; `num_splits` is validated and otherwise ignored.
    """
    return _splitk("tagged_splitk_mxfp4_gemm", shape, num_splits, block_shape, wave_shape, mfma_variant, output_type)


def get_tagged_splitk_mxfp4_gemm_preshuffle_scales(shape, num_splits=2, block_shape=(128, 128, 256),
                                                   wave_shape=(2, 2),
                                                   mfma_variant=ScaledMMAType.F32_16x16x128_F8F6F4,
                                                   a_address_space=SHARED_ADDRESS_SPACE, output_type=f32):
    """tagged_mxfp4_gemm.py:861-903."""
    return _splitk("tagged_splitk_mxfp4_gemm_preshuffle_scales", shape, num_splits, block_shape, wave_shape,
                   mfma_variant, output_type, preshuffled_scales=True)


def get_tagged_splitk_mxfp4_gemm_preshuffle_b(shape, num_splits=2, block_shape=(128, 128, 256), wave_shape=(2, 2),
                                              mfma_variant=ScaledMMAType.F32_16x16x128_F8F6F4,
                                              a_address_space=SHARED_ADDRESS_SPACE, output_type=f32):
    """tagged_mxfp4_gemm.py:906-947."""
    return _splitk("tagged_splitk_mxfp4_gemm_preshuffle_b", shape, num_splits, block_shape, wave_shape,
                   mfma_variant, output_type, preshuffled_scales=True, preshuffled_b=True)


def reorder_mxfp4_workgroups(m_tiles: int, n_tiles: int, group_size_n: int, flat_id: int):
    """Tile order of the persistent kernels, as a host function for tests: tile ids run through
    groups of `group_size_n` N tiles, each group swept down M with N fastest. Same purpose as the
    reference's _reorder_mxfp4_workgroups (tagged_mxfp4_gemm.py:1038-1089): consecutive ids share
    A rows and a bounded set of B rows, so they hit in L2."""
    per_group = group_size_n * m_tiles
    g, r = divmod(flat_id, per_group)
    n0 = g * group_size_n
    gw = min(group_size_n, n_tiles - n0)
    mt, j = divmod(r, gw)
    return mt, n0 + j
