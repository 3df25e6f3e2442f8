"""GPU parity of the MXFP8 scaled GEMM (8-bit E5M2 / E4M3 operands, E8M0 block scales) against the CPU oracle
and the golden vector made from the reference's own functions. Mirrors testScaledGemmMXFP8
(tests/kernel/wave_gemm_mxfp_test.py:416-501), whose tolerance is atol 2e-3, rtol 1e-3; the checks here also
apply the tighter f32 / bf16 criteria used for MXFP4 (products of dequantised operands are exact in f32, only
the summation order differs)."""

import numpy as np
import pytest
import torch

import wave_b200 as wb
from conftest import GOLDEN
from oracle import mxfp4_oracle as orc
from oracle import mxfp8_oracle as orc8
from wave_b200 import _lib, ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def check(c, a, a_s, b, b_s, ref=None):
    """a [M, K], b [N, K] f8 tensors on the CPU; c on the GPU."""
    ad, bd = orc8.dequant_mxfp8(a, a_s), orc8.dequant_mxfp8(b, b_s)
    if ref is None:
        ref = ad @ bd.T
    if c.dtype == torch.float32:
        tol = orc.f32_tolerance(ad, bd, ref, a.shape[1])
        err = (c.cpu() - ref).abs()
        assert bool((err <= tol).all()), f"{int((err > tol).sum())} outside tolerance, max err {float(err.max())}"
    else:
        # 1 bf16 ulp of the rounded reference; where a sum cancels to a value far below its terms, the f32
        # summation-order tolerance plus half an ulp applies instead (few entries: under 0.1 %)
        ulp = orc.bf16_ulp_distance(c, ref)
        tol = orc.f32_tolerance(ad, bd, ref, a.shape[1])
        bad = (ulp > 1) & ~((c.float().cpu() - ref).abs() <= tol + ref.abs() * 2.0 ** -8)
        assert not bool(bad.any()), f"{int(bad.sum())} entries outside both bounds"
        assert float((ulp > 1).float().mean()) < 1e-3, "too many entries beyond 1 bf16 ulp"
    ops.check_device_status()


def problem(M, N, K, seed, dtype=torch.float8_e5m2, lo=124, hi=131):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(M, K, generator=g).to(dtype)
    b = torch.randn(N, K, generator=g).to(dtype)
    a_s = torch.randint(lo, hi, (M, K // 32), dtype=torch.uint8, generator=g)
    b_s = torch.randint(lo, hi, (N, K // 32), dtype=torch.uint8, generator=g)
    return a, a_s, b, b_s


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_golden_small(out_dtype):
    g = np.load(GOLDEN / "gemm_mxfp8_seed5_64x96x128.npz")
    x = torch.from_numpy(g["x"]).view(torch.float8_e5m2)
    w_t = torch.from_numpy(g["w"]).view(torch.float8_e5m2)  # [N, K]
    xs, ws = torch.from_numpy(g["x_scales"]), torch.from_numpy(g["w_scales"])
    kernel, hyper = wb.get_scaled_gemm_mxfp8_kernel((64, 96, 128), wb.ScaledMMAType.F32_16x16x128_F8F6F4, output_dtype=out_dtype)
    gemm = wb.wave_compile(wb.WaveCompileOptions(subs=hyper, canonicalize=True, schedule=wb.SchedulingType.NONE), kernel)
    out = torch.zeros(64, 96, dtype=out_dtype, device=DEV)
    gemm(x.to(DEV).view(torch.int8), xs.to(DEV), w_t.to(DEV).view(torch.int8), ws.to(DEV), out)
    ref = torch.from_numpy(g["out"])
    torch.testing.assert_close(ref, out.cpu().float(), atol=2e-3 if out_dtype == torch.float32 else 0.5, rtol=1e-3 if out_dtype == torch.float32 else 1e-2)
    check(out, x, xs, w_t, ws, ref=ref)


def test_reference_test_shape_1024_as_the_reference_writes_it():
    shape = (1024, 1024, 1024)
    kernel, hyper = wb.get_scaled_gemm_mxfp8_kernel(shape, wb.ScaledMMAType.F32_16x16x128_F8F6F4)
    options = wb.set_default_run_config(wb.WaveCompileOptions(subs=hyper, canonicalize=True, schedule=wb.SchedulingType.NONE))
    gemm = wb.wave_compile(options, kernel)
    x, w, x_scales, w_scales = orc8.generate_gemm_afp8wfp8_inputs(shape)
    out = torch.zeros(x.shape[0], w.shape[1], dtype=torch.float32, device=DEV)
    w_t = w.T.contiguous()
    # x_scales / w_scales are transposed views, as in the reference test
    gemm(x.to(DEV).view(torch.int8), x_scales.to(DEV), w_t.to(DEV).view(torch.int8), w_scales.to(DEV), out)
    torch_out = orc8.torch_scaled_gemm_mxfp8(x, w, x_scales, w_scales)
    torch.testing.assert_close(torch_out, out.cpu(), atol=2e-3, rtol=1e-3, check_dtype=False)
    check(out, x, x_scales, w_t, w_scales, ref=torch_out)


PATHS = [_lib.PATH_TILE_1CTA, _lib.PATH_TILE_1CTA | _lib.TILE_N128, _lib.PATH_TILE_2CTA, _lib.PATH_TILE_2CTA | _lib.TILE_N128]


@pytest.mark.parametrize("flags", PATHS)
@pytest.mark.parametrize("shape", [(128, 128, 128), (256, 512, 1024), (1000, 1100, 992), (130, 260, 32), (3, 5, 64),
                                   (2048, 3072, 512)])
@pytest.mark.parametrize("out_dtype,elem", [(torch.float32, torch.float8_e5m2), (torch.bfloat16, torch.float8_e4m3fn)])
def test_paths_and_shapes(flags, shape, out_dtype, elem):
    M, N, K = shape
    a, a_s, b, b_s = problem(M, N, K, seed=M + N + K, dtype=elem)
    c = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.scaled_gemm_mxfp8_packed(a.to(DEV), ops.repack_scales(a_s.to(DEV)), b.to(DEV), ops.repack_scales(b_s.to(DEV)), c,
                                 flags=flags)
    check(c, a, a_s, b, b_s)


def test_accumulate_and_errors():
    a, a_s, b, b_s = problem(256, 384, 512, seed=4)
    ad, bd = a.to(DEV), b.to(DEV)
    asp, bsp = ops.repack_scales(a_s.to(DEV)), ops.repack_scales(b_s.to(DEV))
    base = torch.randn(256, 384)
    c = base.to(DEV)
    ops.scaled_gemm_mxfp8_packed(ad, asp, bd, bsp, c, flags=_lib.ACCUMULATE)
    ref = orc8.dequant_mxfp8(a, a_s) @ orc8.dequant_mxfp8(b, b_s).T
    torch.testing.assert_close(c.cpu(), ref + base, rtol=1e-5, atol=1e-3)
    with pytest.raises(ValueError):
        ops.scaled_gemm_mxfp8_packed(ad.view(torch.uint8), asp, bd.view(torch.uint8), bsp, c)  # format not given
    with pytest.raises(RuntimeError):
        ops.scaled_gemm_mxfp8_packed(ad, asp, bd, bsp, c, flags=_lib.PATH_SKINNY)


def test_full_size_8192_sampled():
    """The reference test's large shape (8192^3): seeded inputs made on the GPU, sampled rows checked against
    the dequantised f32 product."""
    M = N = K = 8192
    g = torch.Generator(device=DEV).manual_seed(5)
    a = torch.randn(M, K, device=DEV, generator=g).to(torch.float8_e5m2)
    b = torch.randn(N, K, device=DEV, generator=g).to(torch.float8_e5m2)
    a_s = torch.randint(124, 128, (M, K // 32), dtype=torch.uint8, device=DEV, generator=g)
    b_s = torch.randint(124, 128, (N, K // 32), dtype=torch.uint8, device=DEV, generator=g)
    c = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ops.scaled_gemm_mxfp8_packed(a, ops.repack_scales(a_s), b, ops.repack_scales(b_s), c)
    rows = torch.arange(0, M, 331, device=DEV)
    check(c[rows], a[rows].cpu(), a_s[rows].cpu(), b.cpu(), b_s.cpu())


@pytest.mark.parametrize("dtype", [torch.float8_e5m2, torch.float8_e4m3fn])
@pytest.mark.parametrize("rows,K,src", [(64, 256, torch.float32), (300, 1184, torch.bfloat16), (1, 32, torch.float32)])
def test_quantize_mxfp8_bit_exact_and_feeds_the_gemm(dtype, rows, K, src):
    g = torch.Generator().manual_seed(rows + K)
    x = (torch.randn(rows, K, generator=g) * torch.logspace(-6, 6, rows).unsqueeze(1)).to(src)
    x[0, :32] = 0  # an all-zero block
    q, s, packed = ops.quantize_mxfp8(x.to(DEV), dtype)
    q_ref, s_ref = orc8.quantize_mxfp8(x.float(), dtype)
    assert torch.equal(s.cpu(), s_ref)
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))
    assert torch.equal(packed.data.cpu(), orc.pack_scales(s_ref))
    if rows >= 64:  # the quantised activations against quantised weights through the GEMM
        w, w_s = orc8.quantize_mxfp8(torch.randn(96, K, generator=g), dtype)
        c = torch.empty(rows, 96, dtype=torch.float32, device=DEV)
        ops.scaled_gemm_mxfp8_packed(q, packed, w.to(DEV), ops.repack_scales(w_s.to(DEV)), c)
        check(c, q_ref, s_ref, w, w_s)


@pytest.mark.parametrize("dtype", [torch.float8_e5m2, torch.float8_e4m3fn])
def test_quantize_mxfp8_marks_blocks_with_nan_or_inf(dtype):
    """Scale byte 255 and zero codes for a block that holds a NaN or an infinity; other blocks bit-exact as before."""
    rows, K = 33, 256
    x = torch.randn(rows, K, generator=torch.Generator().manual_seed(8))
    x[0, 5], x[7, 100], x[32, 255], x[9, 64] = float("nan"), float("inf"), float("-inf"), float("nan")
    q, s, packed = ops.quantize_mxfp8(x.to(DEV), dtype)
    q_ref, s_ref = orc8.quantize_mxfp8(x, dtype)
    assert torch.equal(s.cpu(), s_ref) and torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))
    assert torch.equal(packed.data.cpu(), orc.pack_scales(s_ref))
    bad = torch.zeros(rows, K // 32, dtype=torch.bool)
    for r, k in ((0, 5), (7, 100), (32, 255), (9, 64)):
        bad[r, k // 32] = True
    assert torch.equal(s.cpu() == 255, bad)
    assert int(q.cpu().view(torch.uint8).reshape(rows, K // 32, 32)[bad].max()) == 0


@pytest.mark.parametrize("M", [1, 16, 40, 100, 128])
@pytest.mark.parametrize("N,K", [(1024, 2048), (1000, 992), (4096, 384)])
@pytest.mark.parametrize("out_dtype,elem", [(torch.float32, torch.float8_e5m2), (torch.bfloat16, torch.float8_e4m3fn)])
def test_skinny_path_mxfp8(M, N, K, out_dtype, elem):
    """M <= 128 with 8-bit operands: the stream-K weight-streaming kernel (chosen automatically, and forced)."""
    a, a_s, b, b_s = problem(M, N, K, seed=3 * M + N + K, dtype=elem)
    ad, bd = a.to(DEV), b.to(DEV)
    asp, bsp = ops.repack_scales(a_s.to(DEV)), ops.repack_scales(b_s.to(DEV))
    c = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.scaled_gemm_mxfp8_packed(ad, asp, bd, bsp, c)
    check(c, a, a_s, b, b_s)
    forced = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.scaled_gemm_mxfp8_packed(ad, asp, bd, bsp, forced, flags=_lib.PATH_SKINNY)
    assert torch.equal(forced.view(torch.int16 if out_dtype == torch.bfloat16 else torch.int32),
                       c.view(torch.int16 if out_dtype == torch.bfloat16 else torch.int32))
    tiles = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.scaled_gemm_mxfp8_packed(ad, asp, bd, bsp, tiles, flags=_lib.PATH_TILE_1CTA)
    check(tiles, a, a_s, b, b_s)


def test_decode_shape_mxfp8_sampled():
    """M = 16, N = 28672, K = 8192 with E4M3 operands (235 MB of weights): column blocks against the oracle."""
    M, N, K = 16, 28672, 8192
    g = torch.Generator(device=DEV).manual_seed(9)
    a = torch.randn(M, K, device=DEV, generator=g).to(torch.float8_e4m3fn)
    b = (torch.randn(N, K, device=DEV, generator=g) * 0.5).to(torch.float8_e4m3fn)
    a_s = torch.randint(124, 129, (M, K // 32), dtype=torch.uint8, device=DEV, generator=g)
    b_s = torch.randint(120, 126, (N, K // 32), dtype=torch.uint8, device=DEV, generator=g)
    c = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ops.scaled_gemm_mxfp8_packed(a, ops.repack_scales(a_s), b, ops.repack_scales(b_s), c)
    for n0 in (0, 14336, N - 1024):
        check(c[:, n0:n0 + 1024].contiguous(), a.cpu(), a_s.cpu(), b[n0:n0 + 1024].cpu(), b_s[n0:n0 + 1024].cpu())


def test_overlapped_chain_of_mxfp8_decode_calls_gives_the_same_bits():
    M, N, K = 16, 4096, 2048
    probs = [problem(M, N, K, seed=900 + i, dtype=torch.float8_e4m3fn) for i in range(3)]
    dev = [(a.to(DEV), ops.repack_scales(a_s.to(DEV)), b.to(DEV), ops.repack_scales(b_s.to(DEV))) for a, a_s, b, b_s in probs]
    ref = [torch.empty(M, N, dtype=torch.bfloat16, device=DEV) for _ in probs]
    for p, c in zip(dev, ref):
        ops.scaled_gemm_mxfp8_packed(*p, c)
        torch.cuda.synchronize()
    outs = [torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV) for _ in probs]
    for _ in range(3):
        for p, c in zip(dev, outs):
            ops.scaled_gemm_mxfp8_packed(*p, c, flags=_lib.OVERLAP_PREVIOUS)
    torch.cuda.synchronize()
    for c, r in zip(outs, ref):
        assert torch.equal(c.view(torch.int16), r.view(torch.int16))
    ops.check_device_status()


# ---------------------------------------------------------------------------------------------
# the mixed pair: 8-bit activations, packed E2M1 weights (kind::mxf8f6f4 with two operand formats)
# ---------------------------------------------------------------------------------------------
def mixed_problem(M, N, K, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    a = (torch.randn(M, K, generator=g) * 2).to(dtype)
    b = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g)  # every E2M1 code, both signs of zero included
    a_s = torch.randint(123, 131, (M, K // 32), dtype=torch.uint8, generator=g)
    b_s = torch.randint(123, 131, (N, K // 32), dtype=torch.uint8, generator=g)
    return a, a_s, b, b_s


def check_mixed(c, a, a_s, b, b_s):
    ad, bd = orc8.dequant_mxfp8(a, a_s), orc.dequant_mxfp4(b, b_s)
    ref = orc8.torch_scaled_gemm_mxfp8_mxfp4(a, b, a_s, b_s)
    tol = orc.f32_tolerance(ad, bd, ref, a.shape[1])
    if c.dtype == torch.float32:
        err = (c.cpu() - ref).abs()
        assert bool((err <= tol).all()), f"{int((err > tol).sum())} outside tolerance, max err {float(err.max())}"
    else:
        ulp = orc.bf16_ulp_distance(c, ref)
        bad = (ulp > 1) & ~((c.float().cpu() - ref).abs() <= tol)
        assert not bool(bad.any()), f"{int(bad.sum())} entries beyond 1 bf16 ulp and beyond the f32 bound"
        assert float((ulp > 1).float().mean()) < 1e-3
    ops.check_device_status()


@pytest.mark.parametrize("elem", [torch.float8_e4m3fn, torch.float8_e5m2])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("flags,shape", [
    (_lib.PATH_TILE_1CTA, (256, 256, 512)), (_lib.PATH_TILE_1CTA | _lib.TILE_N128, (130, 520, 128)),
    (_lib.PATH_TILE_2CTA, (512, 512, 1024)), (_lib.PATH_TILE_2CTA | _lib.TILE_N128, (300, 1000, 384)),
    (_lib.PATH_SKINNY, (1, 1024, 2048)), (_lib.PATH_SKINNY, (16, 1000, 384)), (_lib.PATH_SKINNY, (100, 4096, 256)),
    (_lib.PATH_SKINNY, (40, 128 * 230, 128)), (_lib.PATH_AUTO, (2048, 2304, 1024))])
def test_fp8_activations_against_fp4_weights(flags, shape, out_dtype, elem):
    """The weights cross HBM as packed E2M1 and are expanded into the MMA's 8-bit containers by the copy engine; the
    result equals dequantised activations times dequantised weights, on every path the 8-bit GEMM has."""
    M, N, K = shape
    a, a_s, b, b_s = mixed_problem(M, N, K, M + N + K, elem)
    c = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.scaled_gemm_mxfp8_packed(a.to(DEV), ops.repack_scales(a_s.to(DEV)), b.to(DEV), ops.repack_scales(b_s.to(DEV)), c,
                                 flags=flags, b_fp4=True)
    check_mixed(c, a, a_s, b, b_s)


def test_mixed_pair_equals_the_mxfp8_gemm_on_expanded_weights():
    """Every E2M1 value is an E4M3 value: converting the weights to E4M3 bytes and running the plain MXFP8 GEMM must give
    the same bits as the mixed pair on the packed weights (same scales, same instruction, same order of sums)."""
    M, N, K = 384, 768, 512
    a, a_s, b, b_s = mixed_problem(M, N, K, 3, torch.float8_e4m3fn)
    expanded = orc.mxfp4_to_f32(b).to(torch.float8_e4m3fn)
    assert torch.equal(expanded.float(), orc.mxfp4_to_f32(b))
    a_sf, b_sf = ops.repack_scales(a_s.to(DEV)), ops.repack_scales(b_s.to(DEV))
    for out_dtype in (torch.float32, torch.bfloat16):
        c_mixed = torch.empty(M, N, dtype=out_dtype, device=DEV)
        c_plain = torch.empty(M, N, dtype=out_dtype, device=DEV)
        ops.scaled_gemm_mxfp8_packed(a.to(DEV), a_sf, b.to(DEV), b_sf, c_mixed, b_fp4=True)
        ops.scaled_gemm_mxfp8_packed(a.to(DEV), a_sf, expanded.to(DEV), b_sf, c_plain)
        bits = torch.int32 if out_dtype == torch.float32 else torch.int16
        assert torch.equal(c_mixed.view(bits), c_plain.view(bits))
    ops.check_device_status()


def test_mixed_pair_through_the_template_and_its_argument_errors():
    M, N, K = 200, 384, 256
    a, a_s, b, b_s = mixed_problem(M, N, K, 21, torch.float8_e5m2)
    kernel, hyper = wb.get_scaled_gemm_mxfp8_kernel((M, N, K), wb.ScaledMMAType.F32_16x16x128_F8F6F4, weight_format="f4e2m1fn")
    gemm = wb.wave_compile(wb.WaveCompileOptions(subs=hyper), kernel)
    c = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
    gemm(a.to(DEV).view(torch.int8), a_s.to(DEV), b.to(DEV).view(torch.int8), b_s.to(DEV), c)
    check_mixed(c, a, a_s, b, b_s)
    with pytest.raises(ValueError):  # K must be a multiple of 128
        wb.get_scaled_gemm_mxfp8_kernel((M, N, 160), wb.ScaledMMAType.F32_16x16x128_F8F6F4, weight_format="f4e2m1fn")
    with pytest.raises(ValueError):  # b in the 8-bit layout [N, K] where packed [N, K/2] is expected
        gemm(a.to(DEV), a_s.to(DEV), torch.zeros(N, K, dtype=torch.uint8, device=DEV), b_s.to(DEV), c)
    lib = _lib.load()
    a_sf, b_sf = ops.repack_scales(a_s.to(DEV)), ops.repack_scales(b_s.to(DEV))
    rc = lib.wb200_mxfp8_gemm(M, N, 160, a.to(DEV).data_ptr(), a_sf.data.data_ptr(), b.to(DEV).data_ptr(), b_sf.data.data_ptr(),
                              c.data_ptr(), 0, N, _lib.E5M2 | _lib.B_FP4, None, 0, 0, None)
    assert rc == _lib.WB200_ERR_UNSUPPORTED and b"128" in lib.wb200_last_error()


@pytest.mark.parametrize("M", [1, 16, 100])
@pytest.mark.parametrize("b_fp4", [False, True])
def test_8bit_decode_kernel_on_weight_scales_packed_per_balanced_tile(M, b_fp4):
    """N = 28672 with the balanced tile height (as for MXFP4), 8-bit and mixed operands: matches the oracle, and gives the
    bits of the usual packing wherever both run the whole-tile kernel."""
    N, K = 28672, 256
    h = ops.decode_tile_rows(N)
    if h == 128:
        pytest.skip("this part's SM count divides the tile count")
    if b_fp4:
        a, a_s, b, b_s = mixed_problem(M, N, K, 70 + M, torch.float8_e4m3fn)
    else:
        a, a_s, b, b_s = problem(M, N, K, 70 + M, torch.float8_e4m3fn)
    ad, bd, a_sf = a.to(DEV), b.to(DEV), ops.repack_scales(a_s.to(DEV))
    outs = []
    for b_sf in (ops.repack_scales(b_s.to(DEV)), ops.repack_scales(b_s.to(DEV), tile_rows=h)):
        c = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
        ops.scaled_gemm_mxfp8_packed(ad, a_sf, bd, b_sf, c, flags=_lib.PATH_SKINNY, b_fp4=b_fp4)
        outs.append(c)
    for c in outs:
        (check_mixed if b_fp4 else check)(c, a, a_s, b, b_s)
    if M > 16:  # up to 16 rows the usual packing takes the K-split kernel, whose partial sums are added in another order
        assert torch.equal(outs[0].view(torch.int32), outs[1].view(torch.int32))


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_mixed_pair_golden_small(out_dtype):
    """Against the output stored from the reference's own functions (its f8e5m2 activations, its packed E2M1 weights)."""
    g = np.load(GOLDEN / "gemm_mxfp8_mxfp4_seed5_64x96x128.npz")
    x = torch.from_numpy(g["x"]).view(torch.float8_e5m2)
    w, xs, ws = torch.from_numpy(g["w"]), torch.from_numpy(g["x_scales"]), torch.from_numpy(g["w_scales"])
    ref = torch.from_numpy(g["out"])
    c = torch.full((64, 96), float("nan"), dtype=out_dtype, device=DEV)
    ops.scaled_gemm_mxfp8_packed(x.to(DEV), ops.repack_scales(xs.to(DEV)), w.to(DEV), ops.repack_scales(ws.to(DEV)), c, b_fp4=True)
    if out_dtype == torch.float32:
        torch.testing.assert_close(c.cpu(), ref, atol=2e-3, rtol=1e-3)  # the reference's tolerance for its 8-bit test
    check_mixed(c, x, xs, w, ws)
