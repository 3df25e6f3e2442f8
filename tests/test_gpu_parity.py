"""GPU parity: the CUDA kernels, called through the C ABI and through the template API, against the
CPU oracle and the golden vectors made from the reference. Mirrors the reference's own MXFP4 tests
(tests/kernel/wave_gemm_mxfp_test.py, tests/kernel/wave_gemm_test.py:3640-3690).

Tolerances (stated by the task this library serves):
  * dequantised operands and repacked scales: bit-exact;
  * f32 output: |c - ref| <= 1e-5 * |ref| + 1e-5 * sqrt(K) * max|row of dequant(a)| * max|row of dequant(b)|;
  * bf16 output: within 1 bf16 ulp of the f32 reference rounded to bf16.
"""

import ctypes
import functools

import numpy as np
import pytest
import torch

import wave_b200 as wb
from conftest import GOLDEN
from oracle import mxfp4_oracle as orc
from wave_b200 import _lib, ops

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def check_f32(c, a, a_s, b, b_s, ref=None):
    K = a.shape[1] * 2
    if ref is None:
        ref = orc.scaled_gemm(a, a_s, b, b_s)
    tol = orc.f32_tolerance(orc.dequant_mxfp4(a, a_s), orc.dequant_mxfp4(b, b_s), ref, K)
    err = (c.float().cpu() - ref).abs()
    bad = ~(err <= tol)
    assert not bool(bad.any()), f"{int(bad.sum())} of {bad.numel()} outside tolerance, max err {float(err.max())}"


def check_bf16(c, ref):
    d = orc.bf16_ulp_distance(c, ref)
    assert int(d.max()) <= 1, f"{int((d > 1).sum())} of {d.numel()} differ by more than 1 bf16 ulp (max {int(d.max())})"


def check(c, a, a_s, b, b_s, ref=None):
    if ref is None:
        ref = orc.scaled_gemm(a, a_s, b, b_s)
    if c.dtype == torch.float32:
        check_f32(c, a, a_s, b, b_s, ref)
    else:
        check_bf16(c, ref)
    ops.check_device_status()


def random_problem(M, N, K, seed, lo=124, hi=131):
    g = torch.Generator().manual_seed(seed)
    a = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, generator=g)
    b = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g)
    a_s = torch.randint(lo, hi, (M, K // 32), dtype=torch.uint8, generator=g)
    b_s = torch.randint(lo, hi, (N, K // 32), dtype=torch.uint8, generator=g)
    return a, a_s, b, b_s


def quantized_problem(M, N, K, seed_a, seed_b, std_b=1.0):
    a, a_s = orc.quantize_mxfp4(torch.randn(M, K, generator=torch.Generator().manual_seed(seed_a)))
    b, b_s = orc.quantize_mxfp4(torch.randn(N, K, generator=torch.Generator().manual_seed(seed_b)) * std_b)
    return a, a_s, b, b_s


def run(a, a_s, b, b_s, out_dtype=torch.float32, path=_lib.PATH_AUTO, fill=float("nan")):
    kernel, options = wb.get_tagged_mxfp4_gemm((a.shape[0], b.shape[0], a.shape[1] * 2),
                                               output_dtype=wb.TORCH_DTYPE_TO_WAVE[out_dtype])
    options.kernel_path = path
    gemm = wb.wave_compile(wb.set_default_run_config(options), kernel)
    c = torch.full((a.shape[0], b.shape[0]), fill, dtype=out_dtype, device=DEV)  # kernel must overwrite all of c
    gemm(a.to(DEV), a_s.to(DEV), b.to(DEV), b_s.to(DEV), c)
    return c


# ---------------------------------------------------------------------------------------------
# scale repack and dequantisation: bit-exact
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("rows,K", [(128, 256), (1024, 1024), (100, 96), (300, 8192), (16, 8192), (257, 1184),
                                    (1, 32), (4096, 16384)])
def test_repack_scales_bit_exact(rows, K):
    s = torch.randint(0, 256, (rows, K // 32), dtype=torch.uint8)
    got = ops.repack_scales(s.to(DEV))
    assert torch.equal(got.data.cpu(), orc.pack_scales(s))
    assert got.data.numel() == ops.packed_scale_bytes(rows, K)


def test_repack_scales_strided_source():
    s = torch.randint(0, 256, (70, 40), dtype=torch.uint8)
    view = s.to(DEV)[:, 3:19]  # row stride 40, 16 K-blocks, misaligned start
    got = ops.repack_scales(view)
    assert torch.equal(got.data.cpu(), orc.pack_scales(s[:, 3:19].contiguous()))


@pytest.mark.parametrize("rows,K", [(64, 256), (33, 96), (1000, 4096)])
def test_dequant_bit_exact_all_codes(rows, K):
    q = torch.randint(0, 256, (rows, K // 2), dtype=torch.uint8)
    s = torch.randint(0, 256, (rows, K // 32), dtype=torch.uint8)  # includes 0, 254 and the NaN code 255
    got = wb.mxfp4_dequant(q.to(DEV), s.to(DEV)).cpu()
    exp = orc.dequant_mxfp4(q, s)
    same = (got.view(torch.int32) == exp.view(torch.int32)) | (got.isnan() & exp.isnan())
    assert bool(same.all()), f"{int((~same).sum())} mismatches"


def test_dequant_golden_edges():
    g = np.load(GOLDEN / "gemm_wide_scales_48x80x256.npz")
    a = torch.from_numpy(g["a"])
    for scale_key, deq_key in (("a_scale", "a_deq"), ("edge_scale", "edge_deq")):
        got = wb.mxfp4_dequant(a.to(DEV), torch.from_numpy(g[scale_key]).to(DEV)).cpu().numpy()
        exp = g[deq_key]
        assert bool(((got.view(np.int32) == exp.view(np.int32)) | (np.isnan(got) & np.isnan(exp))).all())


# ---------------------------------------------------------------------------------------------
# golden GEMM vectors from the reference
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_golden_seed5_small(out_dtype):
    g = np.load(GOLDEN / "gemm_seed5_64x96x128.npz")
    x, w, xs, ws = (torch.from_numpy(g[k]) for k in ("x", "w", "x_scales", "w_scales"))
    c = run(x, xs, w.T.contiguous(), ws, out_dtype)
    check(c, x, xs, w.T.contiguous(), ws, ref=torch.from_numpy(g["out"]))


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_golden_wide_scales(out_dtype):
    g = np.load(GOLDEN / "gemm_wide_scales_48x80x256.npz")
    a, b, a_s, b_s = (torch.from_numpy(g[k]) for k in ("a", "b", "a_scale", "b_scale"))
    c = run(a, a_s, b, b_s, out_dtype)
    check(c, a, a_s, b, b_s, ref=torch.from_numpy(g["out"]))


def test_reference_test_shape_1024_seed5_f32():
    """testScaledGemmMXFP4 (wave_gemm_mxfp_test.py:94-201) at (1024, 1024, 1024), written as the reference writes it."""
    shape = (1024, 1024, 1024)
    kernel, hyper = wb.get_scaled_gemm_kernel(shape, wb.ScaledMMAType.F32_16x16x128_F8F6F4)
    options = wb.WaveCompileOptions(subs=hyper, canonicalize=True, schedule=wb.SchedulingType.NONE)
    gemm = wb.wave_compile(wb.set_default_run_config(options), kernel)
    x, w, x_scales, w_scales = wb.generate_gemm_afp4wfp4_inputs(shape, device=torch.device("cpu"))
    ox, ow, oxs, ows = orc.generate_gemm_afp4wfp4_inputs(shape)
    assert torch.equal(x, ox) and torch.equal(w, ow) and torch.equal(x_scales, oxs) and torch.equal(w_scales, ows)
    out = torch.zeros(x.shape[0], w.shape[1], dtype=torch.float32, device=DEV)
    w_t = w.T.contiguous()
    gemm(x.to(DEV), x_scales.to(DEV), w_t.to(DEV), w_scales.to(DEV), out)
    torch_out = orc.torch_scaled_gemm_mxfp4(x, w, x_scales, w_scales)
    torch.testing.assert_close(torch_out, out.cpu(), check_dtype=False)  # the reference's own (default) tolerance
    check(out, x, x_scales, w_t, w_scales, ref=torch_out)
    g = np.load(GOLDEN / "gemm_seed5_1024_sample.npz")
    torch.testing.assert_close(out.cpu()[::64, ::64], torch.from_numpy(g["out_sample"]), rtol=1e-5, atol=1e-3)


def test_config1_1024_cubed_wide_scales_f32():
    """Scales uniform in [124, 130], codes uniform over all 16 values, f32 output."""
    x, w, xs, ws = orc.generate_gemm_afp4wfp4_inputs((1024, 1024, 1024), scale_lo=124, scale_hi=131)
    w_t = w.T.contiguous()
    check(run(x, xs, w_t, ws, torch.float32), x, xs, w_t, ws)


# ---------------------------------------------------------------------------------------------
# every kernel path, ragged and aligned shapes, both output types
# ---------------------------------------------------------------------------------------------
TILE_PATHS = [_lib.PATH_TILE_1CTA, _lib.PATH_TILE_1CTA | _lib.TILE_N128, _lib.PATH_TILE_2CTA,
              _lib.PATH_TILE_2CTA | _lib.TILE_N128, _lib.PATH_TILE_1CTA | _lib.TILE_N192,
              _lib.PATH_TILE_2CTA | _lib.TILE_N192]


@pytest.mark.parametrize("flags", TILE_PATHS)
@pytest.mark.parametrize("shape", [(128, 128, 256), (256, 512, 1024), (1000, 1100, 992), (130, 260, 32),
                                   (1024, 1600, 2048), (512, 1920, 1024), (3, 5, 64)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_tile_paths(flags, shape, out_dtype):
    M, N, K = shape
    a, a_s, b, b_s = random_problem(M, N, K, seed=M + N + K)
    ad, asd, bd, bsd = a.to(DEV), a_s.to(DEV), b.to(DEV), b_s.to(DEV)
    c = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.scaled_gemm_packed(ad, ops.repack_scales(asd), bd, ops.repack_scales(bsd), c, flags)
    check(c, a, a_s, b, b_s)


@pytest.mark.parametrize("M", [1, 4, 16, 17, 64, 100, 128])
@pytest.mark.parametrize("N,K", [(1024, 2048), (1000, 992), (4096, 512)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_skinny_path(M, N, K, out_dtype):
    a, a_s, b, b_s = random_problem(M, N, K, seed=7 * M + N)
    c = run(a, a_s, b, b_s, out_dtype, path=_lib.PATH_SKINNY)
    check(c, a, a_s, b, b_s)
    # the same launch again gives the same bits (fixed-order reduction; counters left clean)
    c2 = run(a, a_s, b, b_s, out_dtype, path=_lib.PATH_SKINNY)
    assert torch.equal(c.view(torch.int16 if out_dtype == torch.bfloat16 else torch.int32),
                       c2.view(torch.int16 if out_dtype == torch.bfloat16 else torch.int32))


@pytest.mark.parametrize("shape", [(1024, 2304, 512), (640, 5120, 256)])
def test_raster_group_changes_the_tile_order_not_the_result(shape):
    """WB200_GROUP_N (the templates' reorder_workgroups / group_size_n): every group size gives the bits of the default."""
    M, N, K = shape
    a, a_s, b, b_s = random_problem(M, N, K, seed=4242)
    ad, bd = a.to(DEV), b.to(DEV)
    asp, bsp = ops.repack_scales(a_s.to(DEV)), ops.repack_scales(b_s.to(DEV))
    for path in (_lib.PATH_TILE_1CTA, _lib.PATH_TILE_2CTA):
        base = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.scaled_gemm_packed(ad, asp, bd, bsp, base, path)
        check(base, a, a_s, b, b_s)
        for group in (_lib.GROUP_N(1), _lib.GROUP_N(3), _lib.GROUP_N(32), _lib.GROUP_N(254), _lib.GROUP_N_ALL):
            c = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
            ops.scaled_gemm_packed(ad, asp, bd, bsp, c, path | group)
            assert torch.equal(c.view(torch.int16), base.view(torch.int16))


def test_template_group_size_reaches_the_kernel():
    """get_tagged_mxfp4_gemm(group_size_n=..., reorder_workgroups=...) compiles to the matching raster flags and
    still matches the oracle."""
    M, N, K = 512, 2048, 512
    a, a_s, b, b_s = random_problem(M, N, K, seed=77)
    for kwargs, want in ((dict(group_size_n=4), _lib.GROUP_N(4)), (dict(group_size_n=8, block_shape=(256, 128, 256)), _lib.GROUP_N(4)),
                         (dict(reorder_workgroups=False), _lib.GROUP_N_ALL), (dict(), 0)):
        tpl, options = wb.templates.get_tagged_mxfp4_gemm((M, N, K), output_dtype=wb.bf16, **kwargs)
        gemm = wb.wave_compile(options, tpl)
        assert gemm._raster_flags() == want
        c = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        gemm(a.to(DEV), a_s.to(DEV), b.to(DEV), b_s.to(DEV), c)
        check(c, a, a_s, b, b_s)


def test_many_tiles_per_cta_and_accumulator_reuse():
    """More tiles than SMs on every path, so each CTA runs several tiles through both accumulators."""
    M, N, K = 2048, 6144, 512
    a, a_s, b, b_s = random_problem(M, N, K, seed=99)
    ref = orc.scaled_gemm(a, a_s, b, b_s)
    ad, bd = a.to(DEV), b.to(DEV)
    asp, bsp = ops.repack_scales(a_s.to(DEV)), ops.repack_scales(b_s.to(DEV))
    for flags in TILE_PATHS:
        for out_dtype in (torch.bfloat16, torch.float32):
            c = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
            ops.scaled_gemm_packed(ad, asp, bd, bsp, c, flags)
            check(c, a, a_s, b, b_s, ref=ref)


def test_output_column_block_with_row_pitch():
    """c may be a column block of a wider matrix (what the N-sharded launcher writes into)."""
    M, N, K = 256, 384, 512
    a, a_s, b, b_s = random_problem(M, N, K, seed=5)
    wide = torch.full((M, 1024), -7.0, dtype=torch.bfloat16, device=DEV)
    ad, bd = a.to(DEV), b.to(DEV)
    ops.scaled_gemm_packed(ad, ops.repack_scales(a_s.to(DEV)), bd, ops.repack_scales(b_s.to(DEV)), wide[:, 256:640])
    check_bf16(wide[:, 256:640].contiguous(), orc.scaled_gemm(a, a_s, b, b_s))
    assert bool((wide[:, :256] == -7.0).all()) and bool((wide[:, 640:] == -7.0).all())


def test_unaligned_output_falls_back_to_scalar_stores():
    M, N, K = 130, 70, 256
    a, a_s, b, b_s = random_problem(M, N, K, seed=11)
    wide = torch.zeros(M, 75, dtype=torch.float32, device=DEV)  # row pitch 300 bytes: not a multiple of 16
    ops.scaled_gemm_packed(a.to(DEV), ops.repack_scales(a_s.to(DEV)), b.to(DEV), ops.repack_scales(b_s.to(DEV)),
                           wide[:, 3:73], _lib.PATH_TILE_1CTA)
    check_f32(wide[:, 3:73].contiguous(), a, a_s, b, b_s)


# ---------------------------------------------------------------------------------------------
# reference API variants
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("shape,num_splits", [((256, 256, 256), 2), ((256, 256, 512), 4), ((256, 256, 1024), 4),
                                              ((512, 512, 1024), 4)])
@pytest.mark.parametrize("output_type", [torch.float32, torch.bfloat16])
def test_splitk_adds_into_c(shape, num_splits, output_type):
    """testSplitKMxfp4Gemm (wave_gemm_test.py:3640-3690): zero-initialised c, result added in."""
    kernel, options = wb.get_tagged_splitk_mxfp4_gemm(shape, num_splits=num_splits, block_shape=(128, 128, 128),
                                                      output_type=wb.TORCH_DTYPE_TO_WAVE[output_type])
    gemm = wb.wave_compile(wb.set_default_run_config(options), kernel, wb.get_mxfp4_dbuf_schedule(True, 1))
    x, w, xs, ws = orc.generate_gemm_afp4wfp4_inputs(shape)
    ref = orc.torch_scaled_gemm_mxfp4(x, w, xs, ws)
    w_t = w.T.contiguous()
    c = torch.zeros(shape[0], shape[1], dtype=output_type, device=DEV)
    gemm(x.to(DEV), xs.to(DEV), w_t.to(DEV), ws.to(DEV), c)
    check(c, x, xs, w_t, ws, ref=ref)  # far inside the reference's rtol 1e-3 / atol 1e-2 (f32) and atol 4.0 (bf16)
    if output_type == torch.float32:
        gemm(x.to(DEV), xs.to(DEV), w_t.to(DEV), ws.to(DEV), c)  # second call accumulates: c == 2 * ref
        torch.testing.assert_close(c.cpu(), 2 * ref, rtol=1e-5, atol=1e-2)


def test_splitk_skinny_accumulates():
    M, N, K = 16, 512, 2048
    a, a_s, b, b_s = random_problem(M, N, K, seed=21)
    kernel, options = wb.get_tagged_splitk_mxfp4_gemm((M, N, K), num_splits=2)
    gemm = wb.wave_compile(options, kernel)
    c = torch.ones(M, N, dtype=torch.float32, device=DEV)
    gemm(a.to(DEV), a_s.to(DEV), b.to(DEV), b_s.to(DEV), c)
    ref = orc.scaled_gemm(a, a_s, b, b_s) + 1.0
    check_f32(c, a, a_s, b, b_s, ref=ref)


def test_batched_activations_shared_weights():
    """testScaledBatchedGemmMXFP4 (wave_gemm_mxfp_test.py:205-339): a is [B, M, K/2], b is shared."""
    B, M, N, K = 4, 96, 256, 512
    a, a_s, b, b_s = random_problem(B * M, N, K, seed=31)
    kernel, options = wb.get_tagged_mxfp4_gemm((B * M, N, K))
    options.dynamic_symbols = ["M", "N", "K"]
    gemm = wb.wave_compile(options, kernel)
    c = torch.empty(B, M, N, dtype=torch.float32, device=DEV)
    gemm(a.view(B, M, -1).to(DEV), a_s.view(B, M, -1).to(DEV), b.to(DEV), b_s.to(DEV), c)
    check_f32(c.view(B * M, N), a, a_s, b, b_s)


def test_preshuffled_scale_templates():
    shape = (256, 384, 1024)
    a, a_s, b, b_s = random_problem(*shape, seed=41)
    ref = orc.scaled_gemm(a, a_s, b, b_s)
    for make in (wb.get_tagged_mxfp4_gemm_preshuffle_scales, wb.get_tagged_mxfp4_gemm_preshuffle_scales_and_B,
                 wb.get_tagged_mxfp4_gemm_preshuffle_b, wb.get_tagged_mxfp4_gemm_preshuffle_b_wide_store):
        kernel, options = make(shape, output_dtype=wb.bf16)
        gemm = wb.wave_compile(options, kernel)
        c = torch.empty(shape[0], shape[1], dtype=torch.bfloat16, device=DEV)
        gemm(a.to(DEV), wb.e8m0_shuffle(a_s.to(DEV)), wb.b_preshuffle(b.to(DEV)), wb.e8m0_shuffle(b_s.to(DEV)), c)
        check_bf16(c, ref)
        with pytest.raises(ValueError, match="pre-shuffled"):
            gemm(a.to(DEV), a_s.to(DEV), b.to(DEV), b_s.to(DEV), c)


def test_call_time_errors():
    kernel, options = wb.get_tagged_mxfp4_gemm((64, 64, 64))
    gemm = wb.wave_compile(options, kernel)
    a = torch.zeros(64, 32, dtype=torch.uint8, device=DEV)
    s = torch.zeros(64, 2, dtype=torch.uint8, device=DEV)
    with pytest.raises(ValueError, match="writes f32"):
        gemm(a, s, a, s, torch.zeros(64, 64, dtype=torch.bfloat16, device=DEV))
    with pytest.raises(ValueError, match="was built for"):
        gemm(a[:32], s[:32], a, s, torch.zeros(32, 64, device=DEV))
    with pytest.raises(ValueError, match="a_scale must be"):
        gemm(a, s[:, :1], a, s, torch.zeros(64, 64, device=DEV))
    with pytest.raises(ValueError, match="uint8 or int8"):
        gemm(a.float(), s, a, s, torch.zeros(64, 64, device=DEV))
    with pytest.raises(ValueError, match="workspace"):
        _lib.check(_lib.load().wb200_mxfp4_gemm(16, 64, 64, a.data_ptr(), a.data_ptr(), a.data_ptr(), a.data_ptr(),
                                                a.data_ptr(), 0, 64, None, 0, _lib.PATH_SKINNY, None))
    assert ctypes.c_int(_lib.load().wb200_version()).value >= 1000


def test_noncontiguous_inputs_are_copied():
    M, N, K = 64, 128, 256
    a, a_s, b, b_s = random_problem(M, N, K, seed=51)
    a_wide = torch.zeros(M, K, dtype=torch.uint8, device=DEV)
    a_wide[:, ::2] = a.to(DEV)
    c = torch.empty(M, N, device=DEV)
    kernel, options = wb.get_tagged_mxfp4_gemm((M, N, K))
    wb.wave_compile(options, kernel)(a_wide[:, ::2], a_s.to(DEV), b.to(DEV), b_s.to(DEV), c)
    check_f32(c, a, a_s, b, b_s)


# ---------------------------------------------------------------------------------------------
# full-size configurations: sampled oracle rows plus size-independent properties
# ---------------------------------------------------------------------------------------------
def test_config2_8192_cubed_bf16_whole_matrix_and_scaling_property():
    """M = N = K = 8192, operands quantised from N(0, 1), bf16 output. The whole output is compared with the
    oracle, 512 rows of A at a time (the reference's tests compare whole outputs too,
    tests/kernel/wave_gemm_mxfp_test.py:184-201), and through an exact property: raising every A scale by one
    doubles C bit for bit (power-of-two scaling is exact)."""
    M = N = K = 8192
    a, a_s, b, b_s = quantized_problem(M, N, K, 1002, 2002)
    ad, asd, bd, bsd = a.to(DEV), a_s.to(DEV), b.to(DEV), b_s.to(DEV)
    kernel, options = wb.get_tagged_mxfp4_gemm((M, N, K), output_dtype=wb.bf16)
    gemm = wb.wave_compile(options, kernel)
    c = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    gemm(ad, asd, bd, bsd, c)
    c_host = c.cpu()
    b_deq = orc.dequant_mxfp4(b, b_s)  # once: 256 MB of f32
    for r0 in range(0, M, 512):
        ref = orc.dequant_mxfp4(a[r0:r0 + 512], a_s[r0:r0 + 512]) @ b_deq.T
        check_bf16(c_host[r0:r0 + 512], ref)
    del b_deq
    c2 = torch.empty_like(c)
    gemm(ad, asd + 1, bd, bsd, c2)
    assert torch.equal((c.float() * 2).to(torch.bfloat16), c2)
    ops.check_device_status()


@functools.lru_cache(maxsize=1)
def _config3_operands():
    N, K = 28672, 8192
    a, a_s = orc.quantize_mxfp4(torch.randn(128, K, generator=torch.Generator().manual_seed(1003)))
    b, b_s = orc.quantize_mxfp4(torch.randn(N, K, generator=torch.Generator().manual_seed(2003)) * 0.02)
    return a, a_s, b, b_s


@pytest.mark.parametrize("M", [1, 4, 16, 64, 128])
def test_config3_decode_shapes_bf16(M):
    """N = 28672, K = 8192, weights from N(0, 0.02), activations from N(0, 1); column blocks of the
    oracle are checked (the full dequantised weight matrix would be 0.9 GB)."""
    N = 28672
    a, a_s, b, b_s = _config3_operands()
    a, a_s = a[:M].contiguous(), a_s[:M].contiguous()
    c = run(a, a_s, b, b_s, torch.bfloat16)
    # every column block at M = 16 (the shape the bandwidth target is quoted on), three of them otherwise
    blocks = range(0, N, 2048) if M == 16 else (0, 12288, N - 2048)
    for n0 in blocks:
        ref = orc.scaled_gemm(a, a_s, b[n0:n0 + 2048], b_s[n0:n0 + 2048])
        check_bf16(c[:, n0:n0 + 2048].contiguous(), ref)
    ops.check_device_status()


@pytest.mark.parametrize("M,N,K,out_dtype,accumulate", [
    (16, 28672, 2048, torch.bfloat16, False),   # one static round, 76 dealt tiles in main / closer parts
    (16, 28672 + 72, 1024, torch.float32, False),  # ragged last tile among the dealt ones
    (100, 19200, 1536, torch.bfloat16, False),  # 150 tiles: 2 dealt tiles only
    (4, 18944, 512, torch.float32, True),       # a whole number of rounds; accumulate into c
    (16, 38000, 256, torch.bfloat16, False),    # one K block per tile: nothing to cut
])
def test_skinny_path_with_dealt_parts(M, N, K, out_dtype, accumulate):
    """Shapes with at least as many N tiles as SMs: the kernel that deals whole N tiles from an atomic counter.
    Checked against the oracle; and because which CTA computes which tile varies from run to run while each
    tile's sum over K does not, repeated launches must give the same bits."""
    a, a_s, b, b_s = random_problem(M, N, K, seed=M + N + K, lo=124, hi=128)
    ref = orc.scaled_gemm(a, a_s, b, b_s)
    ad, bd = a.to(DEV), b.to(DEV)
    a_sf, b_sf = ops.repack_scales(a_s.to(DEV)), ops.repack_scales(b_s.to(DEV))
    flags = _lib.PATH_SKINNY | (_lib.ACCUMULATE if accumulate else 0)
    outs = []
    for _ in range(4):
        c = torch.full((M, N), 1.0 if accumulate else float("nan"), dtype=out_dtype, device=DEV)
        ops.scaled_gemm_packed(ad, a_sf, bd, b_sf, c, flags)
        outs.append(c)
    check(outs[0], a, a_s, b, b_s, ref + 1.0 if accumulate else ref)
    bits = torch.int16 if out_dtype == torch.bfloat16 else torch.int32
    for c in outs[1:]:
        assert torch.equal(outs[0].view(bits), c.view(bits))


@pytest.mark.parametrize("rows,K,tile_rows", [(300, 768, 104), (28672 // 8, 512, 104), (97, 96, 96), (1000, 256, 8), (256, 1024, 128),
                                              (224, 256, 224), (1000, 288, 224), (8192, 512, 224)])
def test_tiled_weight_scale_packing_is_bit_exact(rows, K, tile_rows):
    s = torch.randint(0, 255, (rows, K // 32), dtype=torch.uint8, generator=torch.Generator().manual_seed(rows + tile_rows))
    packed = ops.repack_scales(s.to(DEV), tile_rows=tile_rows)
    assert packed.tile_rows == tile_rows
    assert torch.equal(packed.data.cpu(), orc.pack_scales_tiled(s, tile_rows))


@pytest.mark.parametrize("M", [1, 16, 40, 128])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_decode_kernel_with_weight_scales_packed_per_balanced_tile(M, out_dtype):
    """N = 28672 (the decode configuration's N): the balanced tile height is below 128 on any part whose SM count
    does not divide 224; the GEMM on scales packed for it matches the oracle, and gives the bits of the usual packing
    (every output column's sum over K is made in the same order either way)."""
    N, K = 28672, 256
    h = ops.decode_tile_rows(N)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    assert h % 8 == 0 and 8 <= h <= 128
    if 224 % sms:
        assert h < 128 and -(-N // h) <= -(-224 // sms) * sms  # every SM gets at most `rounds` tiles
    a, a_s, b, b_s = random_problem(M, N, K, seed=500 + M)
    ad, bd = a.to(DEV), b.to(DEV)
    a_sf = ops.repack_scales(a_s.to(DEV))
    usual, tiled = ops.repack_scales(b_s.to(DEV)), ops.repack_scales(b_s.to(DEV), tile_rows=h)
    c0 = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    c1 = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.scaled_gemm_packed(ad, a_sf, bd, usual, c0, _lib.PATH_SKINNY)
    ops.scaled_gemm_packed(ad, a_sf, bd, tiled, c1, _lib.PATH_SKINNY)
    check(c1, a, a_s, b, b_s)
    bits = torch.int16 if out_dtype == torch.bfloat16 else torch.int32
    assert torch.equal(c0.view(bits), c1.view(bits))
    # accumulate form and a ragged N on the same packing rule
    N2 = N - 200
    h2 = ops.decode_tile_rows(N2)
    t2 = ops.repack_scales(b_s[:N2].to(DEV), tile_rows=h2)
    c2 = torch.ones(M, N2, dtype=out_dtype, device=DEV)
    ops.scaled_gemm_packed(ad, a_sf, bd[:N2].contiguous(), t2, c2, _lib.PATH_SKINNY | _lib.ACCUMULATE)
    check(c2, a, a_s, b[:N2], b_s[:N2], orc.scaled_gemm(a, a_s, b[:N2], b_s[:N2]) + 1.0)


@pytest.mark.parametrize("shape", [(256, 224, 256), (300, 1000, 288), (1024, 2304, 1024), (2048, 4096, 512)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_224_wide_tiles_on_weight_scales_packed_for_them(shape, out_dtype):
    """CTA-pair tiles of 224 columns: two accumulators side by side in tensor memory (no hand-over between tiles), read
    from weight scales packed two atom rows per 224-row tile. Same bits as the 256-wide kernel (each output's sum over
    K is made in the same order)."""
    M, N, K = shape
    a, a_s, b, b_s = random_problem(M, N, K, seed=M + N)
    ad, bd, a_sf = a.to(DEV), b.to(DEV), ops.repack_scales(a_s.to(DEV))
    c224 = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.scaled_gemm_packed(ad, a_sf, bd, ops.repack_scales(b_s.to(DEV), tile_rows=224), c224)
    check(c224, a, a_s, b, b_s)
    c256 = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.scaled_gemm_packed(ad, a_sf, bd, ops.repack_scales(b_s.to(DEV)), c256, _lib.PATH_TILE_2CTA)
    bits = torch.int16 if out_dtype == torch.bfloat16 else torch.int32
    assert torch.equal(c224.view(bits), c256.view(bits))
    with pytest.raises(Exception):  # forcing another width on scales packed for 224 is refused
        ops.scaled_gemm_packed(ad, a_sf, bd, ops.repack_scales(b_s.to(DEV), tile_rows=224), c224, _lib.PATH_TILE_2CTA | _lib.TILE_N128)
    ops.check_device_status()


def test_tiled_weight_scales_are_refused_where_no_kernel_reads_them():
    N, K = 28672, 256
    h = ops.decode_tile_rows(N)
    if h == 128:
        pytest.skip("this part's SM count divides the tile count: no tiled packing")
    a, a_s, b, b_s = random_problem(256, N, K, seed=9)
    tiled = ops.repack_scales(b_s.to(DEV), tile_rows=h)
    c = torch.empty(256, N, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError):  # M > 128: the tile kernels read 128-row blocks
        ops.scaled_gemm_packed(a.to(DEV), ops.repack_scales(a_s.to(DEV)), b.to(DEV), tiled, c)
    lib = _lib.load()
    small = ops.repack_scales(b_s[:1024].to(DEV), tile_rows=h)  # fewer tiles than SMs
    c16 = torch.empty(16, 1024, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(Exception) as err:
        ops.scaled_gemm_packed(a[:16].to(DEV), ops.repack_scales(a_s[:16].to(DEV)), b[:1024].to(DEV), small, c16, _lib.PATH_SKINNY)
    assert "wb200_repack_scales" in str(err.value)
    assert lib.wb200_packed_scale_bytes_tiled(100, 256, 100) == 0  # not a multiple of 8
    ops.check_device_status()


def test_template_call_packs_weight_scales_for_the_decode_kernel():
    """The reference-facing call at M <= 128 uses the balanced packing by itself and keeps the usual one for M > 128
    of the same weight; both match the oracle."""
    N, K = 28672, 256
    a, a_s, b, b_s = random_problem(256, N, K, seed=77)
    tpl, options = wb.templates.get_tagged_mxfp4_gemm((16, N, K), output_dtype=wb.bf16)
    tpl.shape = None  # dynamic M
    gemm = wb.wave_compile(options, tpl)
    bd, bsd = b.to(DEV), b_s.to(DEV)
    for M in (16, 256, 16):
        c = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        gemm(a[:M].to(DEV), a_s[:M].to(DEV), bd, bsd, c)
        check(c, a[:M], a_s[:M], b, b_s)
    h = ops.decode_tile_rows(N)
    heights = sorted({k[-1] for k in gemm._weight_scales._entries})
    assert heights == sorted({h, 128})


def test_two_streams_run_skinny_gemms_at_the_same_time():
    """Two decode-shaped GEMMs launched on two streams with nothing ordering them: each call gets its own
    workspace (counters and partial tiles belong to one running GEMM), so both match the oracle however the
    GPU interleaves them."""
    M, N, K = 16, 20480, 1024
    probs = [random_problem(M, N, K, seed=s, lo=124, hi=128) for s in (11, 12)]
    refs = [orc.scaled_gemm(*p) for p in probs]
    kernel, options = wb.get_tagged_mxfp4_gemm((M, N, K), output_dtype=wb.bf16)
    gemm = wb.wave_compile(options, kernel)  # ONE kernel object, used from both streams
    dev = [[t.to(DEV) for t in p] for p in probs]
    outs = [torch.empty(M, N, dtype=torch.bfloat16, device=DEV) for _ in probs]
    streams = [torch.cuda.Stream(DEV) for _ in probs]
    torch.cuda.synchronize()
    for rep in range(20):
        for i, st in enumerate(streams):
            with torch.cuda.stream(st):
                gemm(*dev[i], outs[i])
    torch.cuda.synchronize()
    for i in range(2):
        check_bf16(outs[i], refs[i])
    ops.check_device_status()


# ---------------------------------------------------------------------------------------------
# grouped (MoE) GEMM
# ---------------------------------------------------------------------------------------------
def _moe_problem(E, N, K, tokens, seed):
    from wave_b200 import grouped
    g = torch.Generator().manual_seed(seed)
    x, x_s = orc.quantize_mxfp4(torch.randn(tokens, K, generator=g))
    weights = [orc.quantize_mxfp4(torch.randn(N, K, generator=torch.Generator().manual_seed(seed + 1 + e)) * 0.02)
               for e in range(E)]
    logits = torch.randn(tokens, E, generator=g)
    rows, offsets = grouped.route_top_k(logits, 2)
    return x, x_s, weights, rows, offsets


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_grouped_gemm_ragged_experts(out_dtype):
    """Top-2 routing over 5 experts gives ragged per-expert row counts (one expert is starved on purpose)."""
    from wave_b200 import grouped
    E, N, K, tokens = 5, 640, 1024, 300
    x, x_s, weights, rows, offsets = _moe_problem(E, N, K, tokens, seed=61)
    # starve the last expert: move its rows to expert 0 by re-routing (keeps the offsets consistent)
    assert offsets[-1] == 2 * tokens and len(offsets) == E + 1
    a, a_s = x[rows], x_s[rows]
    experts = grouped.ExpertWeights([w.to(DEV) for w, _ in weights], [s.to(DEV) for _, s in weights])
    c = torch.full((a.shape[0], N), float("nan"), dtype=out_dtype, device=DEV)
    grouped.grouped_scaled_gemm(a.to(DEV), a_s.to(DEV), experts, offsets, c)
    for e in range(E):
        r0, r1 = offsets[e], offsets[e + 1]
        if r1 == r0:
            continue
        w, s = weights[e]
        check(c[r0:r1].contiguous(), a[r0:r1], a_s[r0:r1], w, s)


def test_grouped_gemm_with_an_empty_expert():
    from wave_b200 import grouped
    E, N, K = 3, 256, 512
    g = torch.Generator().manual_seed(71)
    a = torch.randint(0, 256, (200, K // 2), dtype=torch.uint8, generator=g)
    a_s = torch.randint(124, 131, (200, K // 32), dtype=torch.uint8, generator=g)
    ws = [(torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g),
           torch.randint(124, 131, (N, K // 32), dtype=torch.uint8, generator=g)) for _ in range(E)]
    offsets = [0, 130, 130, 200]  # expert 1 gets no rows
    experts = grouped.ExpertWeights([w.to(DEV) for w, _ in ws], [s.to(DEV) for _, s in ws])
    c = torch.full((200, N), float("nan"), dtype=torch.float32, device=DEV)
    grouped.grouped_scaled_gemm(a.to(DEV), a_s.to(DEV), experts, offsets, c)
    for e in (0, 2):
        r0, r1 = offsets[e], offsets[e + 1]
        check_f32(c[r0:r1].contiguous(), a[r0:r1], a_s[r0:r1], ws[e][0], ws[e][1])
    with pytest.raises(ValueError):
        grouped.grouped_scaled_gemm(a.to(DEV), a_s.to(DEV), experts, [0, 100, 200], c)


def test_config4_moe_8_experts_bf16_sampled():
    """8 experts of [14336, 4096], 4096 tokens, top-2: every expert's block is checked on sampled rows and
    a column block of the oracle."""
    from wave_b200 import grouped
    E, N, K, tokens = 8, 14336, 4096, 4096
    x, x_s = orc.quantize_mxfp4(torch.randn(tokens, K, generator=torch.Generator().manual_seed(1004)))
    weights = [orc.quantize_mxfp4(torch.randn(N, K, generator=torch.Generator().manual_seed(2004 + e)) * 0.02)
               for e in range(E)]
    logits = torch.randn(tokens, E, generator=torch.Generator().manual_seed(3004))
    rows, offsets = grouped.route_top_k(logits, 2)
    assert offsets[-1] == 8192
    a, a_s = x[rows], x_s[rows]
    experts = grouped.ExpertWeights([w.to(DEV) for w, _ in weights], [s.to(DEV) for _, s in weights])
    c = torch.empty(a.shape[0], N, dtype=torch.bfloat16, device=DEV)
    grouped.grouped_scaled_gemm(a.to(DEV), a_s.to(DEV), experts, offsets, c)
    for e in range(E):
        r0, r1 = offsets[e], offsets[e + 1]
        sample = torch.arange(r0, r1, max(1, (r1 - r0) // 48))
        w, s = weights[e]
        n0 = (e * 1792) % (N - 2048)
        ref = orc.scaled_gemm(a[sample], a_s[sample], w[n0:n0 + 2048], s[n0:n0 + 2048])
        check_bf16(c[sample.to(DEV)][:, n0:n0 + 2048].contiguous(), ref)
        # the rows at both ends of the expert's block, against all columns of a narrow slice
        edge = torch.tensor([r0, r1 - 1])
        ref_e = orc.scaled_gemm(a[edge], a_s[edge], w[:512], s[:512])
        check_bf16(c[edge.to(DEV)][:, :512].contiguous(), ref_e)
    ops.check_device_status()


def test_grouped_repack_matches_per_group_repack():
    import ctypes
    lib = _lib.load()
    K = 1184  # 37 K-blocks: ragged along K too
    offsets = [0, 130, 130, 131, 400, 1000]
    s = torch.randint(0, 256, (offsets[-1], K // 32), dtype=torch.uint8)
    blocks = [0]
    for g in range(len(offsets) - 1):
        blocks.append(blocks[-1] + (offsets[g + 1] - offsets[g] + 127) // 128)
    per_block = ops.packed_scale_bytes(128, K)
    out = torch.zeros(blocks[-1] * per_block, dtype=torch.uint8, device=DEV)
    E = len(offsets) - 1
    sd = s.to(DEV)
    _lib.check(lib.wb200_repack_scales_grouped(sd.data_ptr(), sd.stride(0), E, (ctypes.c_int * (E + 1))(*offsets),
                                               (ctypes.c_int * (E + 1))(*blocks), K, out.data_ptr(),
                                               torch.cuda.current_stream().cuda_stream))
    got = out.cpu()
    for g in range(E):
        r0, r1 = offsets[g], offsets[g + 1]
        if r1 > r0:
            exp = orc.pack_scales(s[r0:r1])
            assert torch.equal(got[blocks[g] * per_block: blocks[g] * per_block + exp.numel()], exp), g


# ---------------------------------------------------------------------------------------------
# activation quantiser and the linear module built on it
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,K", [(128, 256), (100, 96), (300, 8192), (1, 32), (257, 1184)])
def test_quantizer_bit_exact_against_oracle(rows, K, dtype):
    g = torch.Generator().manual_seed(rows + K)
    x = torch.randn(rows, K, generator=g) * torch.exp(torch.randn(rows, 1, generator=g) * 3)  # wide range of row scales
    x[0, :32] = 0.0                                                 # an all-zero block
    x[-1, :32] = 0.0
    x[-1, :8] = torch.tensor([6.0, 0.25, 0.75, 2.5, 5.0, -0.25, -1.25, 3.5]) * 4  # midpoints (ties) after scaling by 4
    x = x.to(dtype)
    q, s, packed = wb.quantize_mxfp4(x.to(DEV))
    eq, es = orc.quantize_mxfp4(x.float())
    assert torch.equal(s.cpu(), es)
    assert torch.equal(q.cpu(), eq)
    assert torch.equal(packed.data.cpu(), orc.pack_scales(es))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_quantizer_marks_blocks_with_nan_or_inf(dtype):
    """A NaN or an infinity in a block gives scale byte 255 (E8M0's NaN) and codes 0, bit-exact against the oracle;
    read back through the reference's dequantisation rule the block is NaN, every other block is untouched, and a
    GEMM on it returns NaN for the row instead of finite numbers."""
    rows, K, N = 40, 512, 256
    g = torch.Generator().manual_seed(31)
    x = torch.randn(rows, K, generator=g)
    planted = {(1, 40): float("nan"), (2, 70): float("-inf"), (3, 0): float("inf"), (39, 511): float("nan"), (5, 100): float("inf")}
    x[5, 101] = float("nan")  # both kinds in one block
    for (r, k), v in planted.items():
        x[r, k] = v
    x = x.to(dtype)
    q, s, packed = wb.quantize_mxfp4(x.to(DEV))
    eq, es = orc.quantize_mxfp4(x.float())
    assert torch.equal(s.cpu(), es) and torch.equal(q.cpu(), eq)
    assert torch.equal(packed.data.cpu(), orc.pack_scales(es))
    bad = torch.zeros(rows, K // 32, dtype=torch.bool)
    for (r, k) in planted:
        bad[r, k // 32] = True
    assert torch.equal(s.cpu() == 255, bad)
    deq = orc.dequant_mxfp4(q.cpu(), s.cpu()).reshape(rows, K // 32, 32)
    assert torch.equal(torch.isnan(deq).all(dim=2), bad) and torch.equal(torch.isnan(deq).any(dim=2), bad)
    w, w_s = orc.quantize_mxfp4(torch.randn(N, K, generator=g))
    c = torch.zeros(rows, N, dtype=torch.float32, device=DEV)
    ops.scaled_gemm_packed(q, packed, w.to(DEV), ops.repack_scales(w_s.to(DEV)), c)
    nan_rows = bad.any(dim=1)
    assert torch.equal(torch.isnan(c).all(dim=1).cpu(), nan_rows) and torch.equal(torch.isnan(c).any(dim=1).cpu(), nan_rows)


def test_weight_scale_cache_belongs_to_the_tensor_not_the_address():
    """A new scale tensor that the allocator puts at a freed tensor's address must be repacked, an in-place write
    must be seen, and drop_cached_weights forgets a packing that a raw write made stale."""
    M, N, K = 64, 256, 512
    a, a_s, b, b_s = random_problem(M, N, K, seed=11)
    tpl, options = wb.templates.get_tagged_mxfp4_gemm((M, N, K), output_dtype=wb.bf16)
    gemm = wb.wave_compile(options, tpl)
    ad, asd, bd = a.to(DEV), a_s.to(DEV), b.to(DEV)
    c = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    s1 = b_s.to(DEV)
    ptr = s1.data_ptr()
    gemm(ad, asd, bd, s1, c)
    check(c, a, a_s, b, b_s)
    del s1
    other = (b_s.to(torch.int16) + 1).clamp(max=131).to(torch.uint8)
    s2 = other.to(DEV)  # same shape: the caching allocator hands the freed block out again
    if s2.data_ptr() != ptr:
        pytest.skip("the allocator did not reuse the address")
    gemm(ad, asd, bd, s2, c)
    check(c, a, a_s, b, other)
    s2.copy_(b_s.to(DEV))  # in-place write: version counter moves
    gemm(ad, asd, bd, s2, c)
    check(c, a, a_s, b, b_s)
    # a write the version counter does not see (here through a detached alias of the memory)
    alias = torch.as_strided(s2.detach().view(-1).data, s2.shape, s2.stride())
    version = s2._version
    alias.data.copy_(other.to(DEV))
    if s2._version == version:
        gemm.drop_cached_weights(s2)
    gemm(ad, asd, bd, s2, c)
    check(c, a, a_s, b, other)


def test_mxfp4_linear_module_matches_oracle():
    torch.manual_seed(5)
    N, K = 768, 1024
    w = torch.randn(N, K) * 0.02
    x = torch.randn(3, 50, K)
    layer = wb.MXFP4Linear.from_float(w.to(DEV), output_dtype=torch.bfloat16)
    y = layer(x.to(DEV))
    assert y.shape == (3, 50, N) and y.dtype == torch.bfloat16
    wq, ws = orc.quantize_mxfp4(w)
    xq, xs = orc.quantize_mxfp4(x.reshape(-1, K))
    assert torch.equal(layer.weight_codes.cpu(), wq) and torch.equal(layer.weight_scales.cpu(), ws)
    check_bf16(y.reshape(-1, N), orc.scaled_gemm(xq, xs, wq, ws))


def test_mxfp4_linear_decode_batch_uses_the_balanced_packing():
    """A layer wide enough for the whole-tile decode kernel: small batches read the per-tile packing, large ones the usual
    one, both match the oracle."""
    torch.manual_seed(6)
    N, K = 28672, 256
    w = torch.randn(N, K) * 0.02
    layer = wb.MXFP4Linear.from_float(w.to(DEV), output_dtype=torch.bfloat16)
    wq, ws = orc.quantize_mxfp4(w)
    for rows in (4, 200, 4):
        x = torch.randn(rows, K)
        y = layer(x.to(DEV))
        xq, xs = orc.quantize_mxfp4(x)
        check_bf16(y, orc.scaled_gemm(xq, xs, wq, ws))
    assert layer._packed_decode.tile_rows == ops.decode_tile_rows(N) and layer._packed.tile_rows == 128
    ops.check_device_status()


def test_host_pipelined_gemm_on_pinned_buffers():
    """Five calls through the three-stream host pipeline with three device buffer sets: every result
    must belong to its own call's operands (no buffer reused before its result left the device)."""
    from wave_b200.host_pipeline import HostScaledGemm
    M, N, K = 200, 384, 512
    pipe = HostScaledGemm(M, N, K, wb.bf16, device=DEV, depth=3)
    problems = [random_problem(M, N, K, seed=80 + i) for i in range(5)]
    pinned = [[t.pin_memory() for t in p] for p in problems]
    outs = [torch.empty(M, N, dtype=torch.bfloat16).pin_memory() for _ in problems]
    for (a, a_s, b, b_s), c in zip(pinned, outs):
        pipe.submit(a, a_s, b, b_s, c)
    pipe.drain()
    for (a, a_s, b, b_s), c in zip(problems, outs):
        check_bf16(c, orc.scaled_gemm(a, a_s, b, b_s))
    with pytest.raises(ValueError, match="pinned"):
        pipe.submit(*problems[0], outs[0])
    ops.check_device_status()


# ---------------------------------------------------------------------------------------------
# the reference's own test shapes, and a seeded sweep of odd shapes
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("shape", [(1024, 1024, 8192), (1024, 1600, 8192), (1024, 1920, 8192), (1024, 3072, 8192)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_reference_macrotile_shapes_seed5(shape, out_dtype):
    """Shapes of testScaledGemmMXFP4ManualDoubleBuf / ...PreshuffleMacrotiles / ...8WavePingpong
    (wave_gemm_mxfp_test.py:637-680, 778-1085, 1088-1260), inputs from the reference's seed-5 generator,
    compared as the reference compares (default assert_close) and with this library's tolerances."""
    x, w, xs, ws = orc.generate_gemm_afp4wfp4_inputs(shape)
    w_t = w.T.contiguous()
    ref = orc.torch_scaled_gemm_mxfp4(x, w, xs, ws)
    kernel, options = wb.get_tagged_mxfp4_gemm_preshuffle_b(shape, (128, 256, 256), wave_shape=(1, 4),
                                                            output_dtype=wb.TORCH_DTYPE_TO_WAVE[out_dtype])
    gemm = wb.wave_compile(wb.set_default_run_config(options), kernel, wb.get_mxfp4_asymmetric_schedule())
    out = torch.zeros(shape[0], shape[1], dtype=out_dtype, device=DEV)
    gemm(x.to(DEV), wb.e8m0_shuffle(xs.to(DEV)), wb.b_preshuffle(w_t.to(DEV)), wb.e8m0_shuffle(ws.to(DEV)), out)
    torch.testing.assert_close(ref, out.cpu(), check_dtype=False)
    check(out, x, xs, w_t, ws, ref=ref)


def test_seeded_sweep_of_odd_shapes():
    """40 random (M, N, K) with K a multiple of 32 and nothing else aligned, automatic path choice,
    alternating output types; scales over a wider range than the fixed tests."""
    rng = torch.Generator().manual_seed(2024)
    for i in range(40):
        M = int(torch.randint(1, 700, (1,), generator=rng))
        N = int(torch.randint(1, 900, (1,), generator=rng))
        K = 32 * int(torch.randint(1, 40, (1,), generator=rng))
        a, a_s, b, b_s = random_problem(M, N, K, seed=1000 + i, lo=118, hi=136)
        out_dtype = torch.float32 if i % 2 else torch.bfloat16
        kernel, options = wb.get_tagged_mxfp4_gemm((M, N, K), output_dtype=wb.TORCH_DTYPE_TO_WAVE[out_dtype])
        c = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
        wb.wave_compile(options, kernel)(a.to(DEV), a_s.to(DEV), b.to(DEV), b_s.to(DEV), c)
        ref = orc.scaled_gemm(a, a_s, b, b_s)
        if out_dtype == torch.float32:
            try:
                check_f32(c, a, a_s, b, b_s, ref)
            except AssertionError as e:
                raise AssertionError(f"shape {(M, N, K)} f32: {e}") from e
        else:
            # With scales spread over 18 binades some outputs are sums that cancel to far below their
            # terms; there the f32 bound (which has an absolute part) governs, and the bf16 result may
            # sit more than one ulp from the rounded reference. Everywhere else: 1 ulp.
            ulp = orc.bf16_ulp_distance(c, ref)
            tol = orc.f32_tolerance(orc.dequant_mxfp4(a, a_s), orc.dequant_mxfp4(b, b_s), ref, K)
            half_ulp = ref.abs() * 2.0 ** -8
            bad = (ulp > 1) & ~((c.float().cpu() - ref).abs() <= tol + half_ulp)
            assert not bool(bad.any()), f"shape {(M, N, K)} bf16: {int(bad.sum())} outside both bounds"
            assert float((ulp > 1).float().mean()) < 1e-3, f"shape {(M, N, K)} bf16: too many entries beyond 1 ulp"
        ops.check_device_status()


def test_nan_scale_propagates_like_the_reference():
    """Scale code 255 is NaN in the reference (mxfp_utils.py:92-94): the rows and columns it touches are
    NaN in the output, everything else is unaffected."""
    M, N, K = 64, 96, 256
    a, a_s, b, b_s = random_problem(M, N, K, seed=3)
    a_s[5, 2] = 255
    b_s[7, 0] = 255
    ref = orc.scaled_gemm(a, a_s, b, b_s)
    c = run(a, a_s, b, b_s, torch.float32).cpu()
    assert torch.equal(c.isnan(), ref.isnan()) and bool(ref.isnan()[5].all()) and bool(ref.isnan()[:, 7].all())
    ok = ~ref.isnan()
    tol = orc.f32_tolerance(orc.dequant_mxfp4(a, a_s).nan_to_num(0), orc.dequant_mxfp4(b, b_s).nan_to_num(0), ref.nan_to_num(0), K)
    assert bool(((c - ref).abs()[ok] <= tol[ok]).all())


def test_cuda_graph_replay_of_a_decode_call():
    from wave_b200.graphs import GraphedScaledGemm
    M, N, K = 16, 2048, 1024
    a, a_s, b, b_s = random_problem(M, N, K, seed=91)
    a2, a2_s, _, _ = random_problem(M, N, K, seed=92)
    kernel, options = wb.get_tagged_mxfp4_gemm((M, N, K), output_dtype=wb.bf16)
    gemm = wb.wave_compile(options, kernel)
    ad, asd, bd, bsd = a.to(DEV), a_s.to(DEV), b.to(DEV), b_s.to(DEV)
    c = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    g = GraphedScaledGemm(gemm, ad, asd, bd, bsd, c)
    g.replay()
    check_bf16(c, orc.scaled_gemm(a, a_s, b, b_s))
    ad.copy_(a2.to(DEV)); asd.copy_(a2_s.to(DEV))          # new activations in the same buffers
    g.replay()
    check_bf16(c, orc.scaled_gemm(a2, a2_s, b, b_s))
    ops.check_device_status()


def test_bounded_wait_reports_timeout_and_context_stays_usable():
    """A wait that nothing satisfies gives up after its limit, the kernel ends normally, the status word
    carries the code, and the next GEMM on the same context is correct."""
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.wb200_selftest_wait_timeout(2_000_000, stream))  # ~1 ms
    with pytest.raises(_lib.DeviceTimeoutError, match="wait 7"):
        ops.check_device_status()
    ops.check_device_status()  # the word was cleared
    assert lib.wb200_selftest_wait_timeout(10 ** 12, stream) == _lib.WB200_ERR_INVALID_ARG
    a, a_s, b, b_s = random_problem(256, 256, 512, seed=17)
    check(run(a, a_s, b, b_s, torch.float32), a, a_s, b, b_s)


def test_single_row_operands_with_arbitrary_size_one_stride():
    """M = 1 through the reference's generator: `x_scales.T.contiguous()` of a [K/32, 1] tensor is a
    [1, K/32] tensor whose row stride is 1, not K/32."""
    shape = (1, 512, 1024)
    x, w, xs, ws = orc.generate_gemm_afp4wfp4_inputs(shape)
    assert xs.shape == (1, 32)
    w_t = w.T.contiguous()
    kernel, options = wb.get_tagged_mxfp4_gemm(shape, output_dtype=wb.bf16)
    gemm = wb.wave_compile(options, kernel)
    c = torch.empty(1, 512, dtype=torch.bfloat16, device=DEV)
    xs_dev = xs.to(DEV).T.contiguous().T  # keeps the odd stride on the device
    for _ in range(2):  # first call: checked path; second: remembered-signature path
        gemm(x.to(DEV), xs_dev, w_t.to(DEV), ws.to(DEV), c)
        check_bf16(c, orc.torch_scaled_gemm_mxfp4(x, w, xs, ws))


def test_broadcasted_scale_gemm_as_the_reference_tests_it():
    """testBroadcastedScaleGemmMXFP4 (tests/kernel/wave_gemm_mxfp_test.py:594-634): a_scale is the first
    column of the generated scales, shape [M]; the oracle gets it repeated along K."""
    shape = (512, 512, 512)
    kernel, hyper = wb.get_broadcasted_scale_gemm_mxfp4(shape, wb.ScaledMMAType.F32_16x16x128_F8F6F4)
    options = wb.WaveCompileOptions(subs=hyper, canonicalize=True, schedule=wb.SchedulingType.NONE)
    gemm = wb.wave_compile(wb.set_default_run_config(options), kernel)
    x, w, x_scales, w_scales = orc.generate_gemm_afp4wfp4_inputs(shape)
    compact = x_scales[:, 0].contiguous()
    out = torch.zeros(shape[0], shape[1], dtype=torch.float32, device=DEV)
    w_t = w.T.contiguous()
    gemm(x.to(DEV), compact.to(DEV), w_t.to(DEV), w_scales.to(DEV), out)
    full = compact.view(-1, 1).repeat(1, x_scales.shape[-1]).contiguous()
    torch_out = orc.torch_scaled_gemm_mxfp4(x, w, full, w_scales)
    torch.testing.assert_close(torch_out, out.cpu(), check_dtype=False)
    check(out, x, full, w_t, w_scales, ref=torch_out)
    # the packed form is bit-identical to packing the repeated scales, also for a strided, ragged source
    wide = torch.randint(0, 256, (300, 3), dtype=torch.uint8)
    got = ops.repack_scales_broadcast(wide.to(DEV)[:, 1], 1184)
    assert torch.equal(got.data.cpu(), orc.pack_scales(wide[:, 1:2].repeat(1, 1184 // 32).contiguous()))
    with pytest.raises(ValueError):
        gemm(x.to(DEV), x_scales.to(DEV), w_t.to(DEV), w_scales.to(DEV), out)


@pytest.mark.parametrize("ways", [8, 2])
def test_config5_one_shard_of_the_sharded_gemm_bf16_sampled(ways):
    """M = 16384, N = 53248, K = 16384 sharded over `ways` GPUs by rows of b: one GPU's shard
    (N / ways = 6656 or 26624 rows) at full size. Operands are seeded f32 N(0, 1) matrices (seeds 1005 / 2005)
    quantised on the GPU (the quantiser is bit-exact against the oracle's, tested above); the oracle is evaluated for
    sampled rows of a against sampled row blocks of the shard, and the whole shard is checked through the exact
    doubling property. Bar: 1 bf16 ulp of the rounded f32 reference. An entry further away passes only where the f32
    bound holds (a sum that cancels far below its terms, so that the accumulation order moves it across more than one
    bf16 step); such entries are counted and reported, and there may be at most one in ten thousand."""
    M, N, K = 16384, 53248, 16384
    n_shard = N // ways
    assert n_shard % 256 == 0
    g = torch.Generator(device=DEV).manual_seed(1005)
    a, a_s, _ = ops.quantize_mxfp4(torch.randn(M, K, device=DEV, generator=g, dtype=torch.float32), want_packed=False)
    g.manual_seed(2005)
    b, b_s, _ = ops.quantize_mxfp4(torch.randn(n_shard, K, device=DEV, generator=g, dtype=torch.float32), want_packed=False)
    kernel, options = wb.get_tagged_mxfp4_gemm((M, n_shard, K), output_dtype=wb.bf16)
    gemm = wb.wave_compile(options, kernel)
    c = torch.empty(M, n_shard, dtype=torch.bfloat16, device=DEV)
    gemm(a, a_s, b, b_s, c)
    rows = torch.arange(0, M, 683, device=DEV)
    escaped = checked = 0
    for n0 in (0, (n_shard // 2) // 256 * 256 + 128, n_shard - 1024):
        ref = orc.scaled_gemm(a[rows].cpu(), a_s[rows].cpu(), b[n0:n0 + 1024].cpu(), b_s[n0:n0 + 1024].cpu())
        got = c[rows][:, n0:n0 + 1024].contiguous()
        ulp = orc.bf16_ulp_distance(got, ref)
        tol = orc.f32_tolerance(orc.dequant_mxfp4(a[rows].cpu(), a_s[rows].cpu()),
                                orc.dequant_mxfp4(b[n0:n0 + 1024].cpu(), b_s[n0:n0 + 1024].cpu()), ref, K)
        within_f32 = (got.float().cpu() - ref).abs() <= tol
        failed = (ulp > 1) & ~within_f32
        assert not bool(failed.any()), f"{int(failed.sum())} entries beyond 1 bf16 ulp and beyond the f32 bound (max {int(ulp.max())} ulp)"
        escaped += int(((ulp > 1) & within_f32).sum())
        checked += ulp.numel()
    if escaped:
        import warnings
        warnings.warn(f"config 5, {ways}-way shard: {escaped} of {checked} sampled entries are more than 1 bf16 ulp from the "
                      "rounded reference and pass by the f32 bound")
    assert escaped * 10000 <= checked
    c2 = torch.empty_like(c)
    gemm(a, a_s + 1, b, b_s, c2)
    assert torch.equal((c.float() * 2).to(torch.bfloat16), c2)
    ops.check_device_status()


@pytest.mark.parametrize("shape", [(512, 512, 16000), (256, 512, 4096), (1000, 300, 8192), (300, 260, 2560), (2048, 512, 16000)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_split_k_tile_path(shape, out_dtype):
    """Few output tiles and a long K (the small-N end of the reference's benchmark shapes,
    perf/mxfp4_shapes_macrotiles.csv): K slices x tiles in one launch, partial products added in slice order."""
    M, N, K = shape
    a, a_s, b, b_s = random_problem(M, N, K, seed=M + N + K, lo=125, hi=129)
    ad, bd = a.to(DEV), b.to(DEV)
    asp, bsp = ops.repack_scales(a_s.to(DEV)), ops.repack_scales(b_s.to(DEV))
    ref = orc.scaled_gemm(a, a_s, b, b_s)
    c = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.scaled_gemm_packed(ad, asp, bd, bsp, c, _lib.PATH_TILE_SPLITK)
    check(c, a, a_s, b, b_s, ref=ref)
    auto = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.scaled_gemm_packed(ad, asp, bd, bsp, auto)  # the automatic choice (split-K from three slices up)
    check(auto, a, a_s, b, b_s, ref=ref)
    if out_dtype == torch.float32:  # the split-K templates' contract: add into a caller-initialised c
        base = torch.randn(M, N)
        acc = base.to(DEV)
        ops.scaled_gemm_packed(ad, asp, bd, bsp, acc, _lib.PATH_TILE_SPLITK | _lib.ACCUMULATE)
        tol = orc.f32_tolerance(orc.dequant_mxfp4(a, a_s), orc.dequant_mxfp4(b, b_s), ref, K)
        assert bool(((acc.cpu() - (ref + base)).abs() <= tol + 1e-6 * base.abs()).all())
    ops.check_device_status()


def test_split_k_is_the_automatic_choice_under_graph_capture_only():
    """Eager Python calls keep the plain tile path (the split-K launch costs more host time than it saves on
    the GPU for a slow host); a call captured into a CUDA graph takes split-K. Both match the oracle; the
    captured one equals the forced split-K result bit for bit."""
    M, N, K = 512, 512, 8192
    a, a_s, b, b_s = random_problem(M, N, K, seed=77, lo=125, hi=129)
    ad, bd = a.to(DEV), b.to(DEV)
    asp, bsp = ops.repack_scales(a_s.to(DEV)), ops.repack_scales(b_s.to(DEV))
    forced = torch.empty(M, N, dtype=torch.float32, device=DEV)
    plain = torch.empty_like(forced)
    eager = torch.empty_like(forced)
    captured = torch.empty_like(forced)
    ops.scaled_gemm_packed(ad, asp, bd, bsp, forced, _lib.PATH_TILE_SPLITK)
    ops.scaled_gemm_packed(ad, asp, bd, bsp, plain, _lib.PATH_TILE_2CTA | _lib.TILE_N128)
    ops.scaled_gemm_packed(ad, asp, bd, bsp, eager)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ops.scaled_gemm_packed(ad, asp, bd, bsp, captured)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(eager, plain) and torch.equal(captured, forced)
    check(captured, a, a_s, b, b_s)
    check(eager, a, a_s, b, b_s)


def test_split_k_tile_path_refuses_what_it_cannot_do():
    a, a_s, b, b_s = random_problem(4096, 4096, 1024, seed=1)
    c = torch.empty(4096, 4096, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError):  # plenty of tiles: not a split-K shape
        ops.scaled_gemm_packed(a.to(DEV), ops.repack_scales(a_s.to(DEV)), b.to(DEV), ops.repack_scales(b_s.to(DEV)), c,
                               _lib.PATH_TILE_SPLITK)


@pytest.mark.parametrize("shape", [(16, 4096, 2048), (100, 1000, 992), (512, 768, 1024)])
def test_overlap_previous_chain_gives_the_same_bits(shape):
    """Back-to-back calls flagged WB200_OVERLAP_PREVIOUS (each launched as a programmatic dependent of the one
    before it, sharing scratch and workspace) against the same calls launched one after the other."""
    M, N, K = shape
    kernel, options = wb.get_tagged_mxfp4_gemm(shape, output_dtype=wb.bf16)
    plain = wb.wave_compile(wb.set_default_run_config(options), kernel)
    kernel2, options2 = wb.get_tagged_mxfp4_gemm(shape, output_dtype=wb.bf16)
    options2.overlap_previous = True
    chained = wb.wave_compile(wb.set_default_run_config(options2), kernel2)
    probs = [random_problem(M, N, K, seed=500 + i) for i in range(4)]
    dev_probs = [[t.to(DEV) for t in p] for p in probs]
    ref_out = [torch.empty(M, N, dtype=torch.bfloat16, device=DEV) for _ in probs]
    for p, c in zip(dev_probs, ref_out):
        plain(p[0], p[1], p[2], p[3], c)
        torch.cuda.synchronize()
    outs = [torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV) for _ in probs]
    for rep in range(3):  # no synchronisation between the calls
        for p, c in zip(dev_probs, outs):
            chained(p[0], p[1], p[2], p[3], c)
    torch.cuda.synchronize()
    for c, r in zip(outs, ref_out):
        assert torch.equal(c.view(torch.int16), r.view(torch.int16))
    check_bf16(outs[0], orc.scaled_gemm(*probs[0]))
    ops.check_device_status()


def test_run_bench_option_reports_kernel_time(tmp_path):
    """options.run_bench: after the call the kernel is timed on the device and the report goes to
    benchmark_results_file (the reference hands its module to a benchmark tool, compile.py:317-329)."""
    import json
    a, a_s, b, b_s = random_problem(128, 256, 512, seed=3)
    kernel, options = wb.get_tagged_mxfp4_gemm((128, 256, 512), output_dtype=wb.bf16)
    options.run_bench, options.benchmark_batch_size, options.benchmark_repetitions = True, 5, 3
    options.benchmark_results_file = str(tmp_path / "bench.json")
    gemm = wb.wave_compile(options, kernel)
    c = torch.empty(128, 256, dtype=torch.bfloat16, device=DEV)
    gemm(a.to(DEV), a_s.to(DEV), b.to(DEV), b_s.to(DEV), c)
    check(c, a, a_s, b, b_s)
    rep = json.loads((tmp_path / "bench.json").read_text())["benchmarks"][0]
    assert rep["time_unit"] == "us" and rep["iterations"] == 3 and 0 < rep["min_time"] <= rep["real_time"] < 1e5
