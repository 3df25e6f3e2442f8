"""Host-side checks that need no GPU: the C ABI loads and exports what the header declares,
argument validation, error classes, and the template / option surface."""

import ctypes
import re
from pathlib import Path

import pytest
import torch

import wave_b200 as wb
from wave_b200 import _lib, templates

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib(built_library):
    return _lib.load()


def test_header_symbols_are_exported(lib):
    header = (ROOT / "include" / "wave_b200.h").read_text()
    declared = set(re.findall(r"\b(wb200_[a-z0-9_]+)\s*\(", header))
    assert declared == set(_lib.EXPORTED_SYMBOLS)
    for name in declared:
        assert getattr(lib, name) is not None
    assert lib.wb200_version() >= 1000


def test_header_status_codes_match_binding():
    header = (ROOT / "include" / "wave_b200.h").read_text()
    for name in ("WB200_ERR_INVALID_ARG", "WB200_ERR_ALIGNMENT", "WB200_ERR_WORKSPACE", "WB200_ERR_UNSUPPORTED",
                 "WB200_ERR_DEVICE_TIMEOUT", "WB200_ERR_CUDA"):
        m = re.search(rf"#define {name} \((-?\d+)\)", header)
        assert m and int(m.group(1)) == getattr(_lib, name)
    for name, val in (("WB200_PATH_SKINNY", _lib.PATH_SKINNY), ("WB200_TILE_N128", _lib.TILE_N128),
                      ("WB200_ACCUMULATE", _lib.ACCUMULATE)):
        m = re.search(rf"#define {name} (0x[0-9a-fA-F]+|\d+)u", header)
        assert m and int(m.group(1), 0) == val


def test_packed_scale_bytes(lib):
    assert lib.wb200_packed_scale_bytes(128, 256) == 1024          # 1 row block x 2 atoms
    assert lib.wb200_packed_scale_bytes(1, 32) == 1024             # padded to one stage
    assert lib.wb200_packed_scale_bytes(129, 8192) == 2 * 64 * 512
    assert lib.wb200_packed_scale_bytes(0, 256) == 0


def test_argument_validation_returns_codes_and_messages(lib):
    buf = (ctypes.c_uint8 * 4096)()
    p = ctypes.addressof(buf)
    p16 = (p + 15) & ~15
    # K not a multiple of 32
    assert lib.wb200_mxfp4_gemm(16, 16, 48, p16, p16, p16, p16, p16, 0, 16, 0, 0, 0, None) == _lib.WB200_ERR_INVALID_ARG
    assert b"multiple of the scale group size" in lib.wb200_last_error()
    # null pointer
    assert lib.wb200_mxfp4_gemm(16, 16, 64, None, p16, p16, p16, p16, 0, 16, 0, 0, 0, None) == _lib.WB200_ERR_INVALID_ARG
    # unknown dtype
    assert lib.wb200_mxfp4_gemm(16, 16, 64, p16, p16, p16, p16, p16, 7, 16, 0, 0, 0, None) == _lib.WB200_ERR_INVALID_ARG
    # ldc < N
    assert lib.wb200_mxfp4_gemm(16, 32, 64, p16, p16, p16, p16, p16, 0, 16, 0, 0, 0, None) == _lib.WB200_ERR_INVALID_ARG
    # misaligned operand
    assert lib.wb200_mxfp4_gemm(16, 16, 64, p16 + 4, p16, p16, p16, p16, 0, 16, 0, 0, 0, None) == _lib.WB200_ERR_ALIGNMENT
    # repack: bad K, null, short stride
    assert lib.wb200_repack_scales(p16, 1, 16, 40, p16, None) == _lib.WB200_ERR_INVALID_ARG
    assert lib.wb200_repack_scales(None, 2, 16, 64, p16, None) == _lib.WB200_ERR_INVALID_ARG
    assert lib.wb200_repack_scales(p16, 1, 16, 64, p16, None) == _lib.WB200_ERR_INVALID_ARG
    with pytest.raises(ValueError):
        _lib.check(_lib.WB200_ERR_INVALID_ARG)


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU failure mode")
def test_fails_loudly_without_a_gpu(lib):
    buf = (ctypes.c_uint8 * 8192)()
    p16 = (ctypes.addressof(buf) + 15) & ~15
    rc = lib.wb200_mxfp4_gemm(16, 16, 64, p16, p16, p16, p16, p16, 0, 16, 0, 0, 0, None)
    assert rc == _lib.WB200_ERR_CUDA
    with pytest.raises(RuntimeError):
        _lib.check(rc)
    # the Python layer refuses CPU tensors instead of computing on the host
    kernel, options = wb.get_tagged_mxfp4_gemm((16, 16, 64))
    gemm = wb.wave_compile(options, kernel)
    a = torch.zeros(16, 32, dtype=torch.uint8)
    s = torch.zeros(16, 2, dtype=torch.uint8)
    with pytest.raises(ValueError, match="no CPU path"):
        gemm(a, s, a, s, torch.zeros(16, 16))


def test_missing_library_is_an_error(monkeypatch, tmp_path):
    monkeypatch.setenv("WAVE_B200_LIB", str(tmp_path / "nope.so"))
    monkeypatch.setattr(_lib, "_lib", None)
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.load()


def test_template_surface_matches_reference_names(lib):
    kernel, hyper = wb.get_scaled_gemm_kernel((1024, 1024, 1024), wb.ScaledMMAType.F32_16x16x128_F8F6F4)
    assert hyper["M"] == 1024 and hyper["BLOCK_K"] == 256 and kernel.output_dtype is wb.f32
    options = wb.set_default_run_config(wb.WaveCompileOptions(subs=hyper, canonicalize=True))
    assert options.target == "sm_100a"
    gemm = wb.wave_compile(options, kernel)
    assert callable(gemm) and gemm.options is options and isinstance(gemm.asm, str)

    kernel, options = wb.get_tagged_mxfp4_gemm((1024, 1024, 8192), (256, 256, 256), wave_shape=(1, 4),
                                               b_address_space=wb.GLOBAL_ADDRESS_SPACE, output_dtype=wb.bf16)
    options.minimize_shared_allocs = True
    options.linearize_shared_access = True
    options.use_buffer_ops = True
    gemm = wb.wave_compile(wb.set_default_run_config(options), kernel, wb.get_mxfp4_asymmetric_schedule())
    assert gemm.template.output_dtype is wb.bf16

    with pytest.raises(AssertionError, match="Unsupported output dtype"):
        wb.get_tagged_mxfp4_gemm((64, 64, 64), output_dtype=wb.i8)
    with pytest.raises(TypeError):
        wb.wave_compile(wb.WaveCompileOptions(), object())
    with pytest.raises(ValueError):
        wb.wave_compile(wb.WaveCompileOptions(num_devices=0), kernel)
    # num_devices > 1 asks for the multi-device launcher (wave_lang/kernel/wave/compile.py:194-201): without that many
    # GPUs it fails loudly, it does not fall back to anything
    if torch.cuda.device_count() < 2:
        with pytest.raises(RuntimeError, match="GPU"):
            wb.wave_compile(wb.WaveCompileOptions(num_devices=2), kernel)


def test_splitk_preconditions_match_reference():
    # tagged_mxfp4_gemm.py:636-645
    with pytest.raises(ValueError, match="is less than BLOCK_K"):
        wb.get_tagged_splitk_mxfp4_gemm((256, 256, 256), num_splits=4, block_shape=(128, 128, 128))
    with pytest.raises(ValueError, match="must be a multiple of BLOCK_K"):
        wb.get_tagged_splitk_mxfp4_gemm((256, 256, 768), num_splits=2, block_shape=(128, 128, 256))
    k, o = wb.get_tagged_splitk_mxfp4_gemm((256, 256, 512), num_splits=4, block_shape=(128, 128, 128),
                                           output_type=wb.TORCH_DTYPE_TO_WAVE[torch.bfloat16])
    assert k.accumulate and k.num_splits == 4 and k.output_dtype is wb.bf16


def test_tile_order_is_a_permutation_grouped_by_n():
    for mt, nt, g in ((64, 32, 16), (7, 5, 16), (3, 37, 16), (10, 33, 8)):
        seen = [templates.reorder_mxfp4_workgroups(mt, nt, g, t) for t in range(mt * nt)]
        assert sorted(seen) == [(m, n) for m in range(mt) for n in range(nt)]
        # a run of `g` consecutive ids inside a full group shares one M tile
        if nt >= g:
            assert len({m for m, _ in seen[:g]}) == 1


def test_raster_group_flags_follow_the_template_arguments():
    header = (ROOT / "include" / "wave_b200.h").read_text()
    assert re.search(r"#define WB200_GROUP_N_SHIFT 8\b", header) and re.search(r"#define WB200_GROUP_N_MASK 0xFF00u", header)
    assert _lib.GROUP_N(1) == 0x100 and _lib.GROUP_N(254) == 0xFE00 and _lib.GROUP_N_ALL == 0xFF00
    with pytest.raises(ValueError):
        _lib.GROUP_N(255)
    with pytest.raises(ValueError):
        _lib.GROUP_N(0)
    shape = (1024, 1024, 8192)
    for kwargs, want in ((dict(), 0), (dict(group_size_n=32), _lib.GROUP_N(32)), (dict(group_size_n=1000), _lib.GROUP_N(254)),
                         (dict(group_size_n=4, block_shape=(128, 128, 256)), _lib.GROUP_N(2)),
                         (dict(group_size_n=1, block_shape=(128, 128, 256)), _lib.GROUP_N(1)),
                         (dict(group_size_n=8, reorder_workgroups=False), _lib.GROUP_N_ALL)):
        tpl, options = templates.get_tagged_mxfp4_gemm_preshuffle_b(shape, **kwargs)
        assert wb.wave_compile(options, tpl)._raster_flags() == want
    with pytest.raises(ValueError):
        templates.get_tagged_mxfp4_gemm(shape, group_size_n=0)


def test_perf_formulas_match_the_reference_benchmark_driver():
    """flops and byte counts of wave_lang/kernel/wave/perf/benchmark_mxfp4.py:78-92."""
    from wave_b200 import perf
    M, N, K = 8192, 28672, 16000
    assert perf.get_flops(M, N, K) == 2 * M * N * K
    assert perf.get_byte_count_mxfp4(M, N, K) == M * K // 2 + M * K // 32 + N * K // 2 + N * K // 32 + M * N * 2
    assert abs(perf.runtime_us_to_tflops(8192, 8192, 8192, 122.17) - 9000) < 1
    shapes = perf.default_shapes()
    assert (8192, 8192, 8192) in shapes and all(k % 32 == 0 for _, _, k in shapes)



def test_native_shard_bounds_match_the_python_rule(lib):
    """The native launcher and the torch.distributed launcher must agree on who owns which rows of b."""
    from wave_b200 import multi_device, multi_gpu
    for N in (128, 1000, 8192, 53248, 28672 + 5):
        for G in (1, 2, 3, 4, 8):
            got = [multi_device.shard_bounds(N, G, g) for g in range(G)]
            assert got == [multi_gpu.shard_bounds(N, G, g) for g in range(G)]
            assert got[0][0] == 0 and got[-1][1] == N and all(a[1] == b[0] for a, b in zip(got, got[1:]))
            assert all(n0 % 128 == 0 for n0, n1 in got if n1 > n0)
    import ctypes as C
    n0, n1 = C.c_int(), C.c_int()
    assert lib.wb200_multi_gpu_shard_bounds(0, 2, 0, 128, C.byref(n0), C.byref(n1)) == _lib.WB200_ERR_INVALID_ARG
    assert lib.wb200_multi_gpu_shard_bounds(1024, 2, 2, 128, C.byref(n0), C.byref(n1)) == _lib.WB200_ERR_INVALID_ARG
    h = C.c_void_p()
    assert lib.wb200_multi_gpu_create(0, None, C.byref(h)) == _lib.WB200_ERR_INVALID_ARG
    assert lib.wb200_multi_gpu_num_devices(None) == 0 and lib.wb200_multi_gpu_destroy(None) == 0


def test_profile_python_wrapper_times_the_host_side(capsys):
    """options.profile_python_wrapper: warm-up calls, then the repetitions under timeit or cProfile, as the reference's
    invoke_with_profile (wave_lang/kernel/wave/compile.py:341-365). Exercised on a stand-in for invoke: no GPU needed."""
    from wave_b200 import compile as wc
    calls = []
    opts = wb.WaveCompileOptions(profile_python_wrapper=True, profile_python_cprofile=False, profile_python_warmup=2,
                                 profile_python_repetitions=5)
    assert wc.invoke_with_profile(opts, lambda x: calls.append(x) or "done", 7) == "done"
    assert len(calls) == 2 + 5 + 1  # warm-up, timed, and the call whose result is returned
    assert "per iteration" in capsys.readouterr().out
    opts.profile_python_cprofile = True
    calls.clear()
    wc.invoke_with_profile(opts, lambda x: calls.append(x), 7)
    assert len(calls) == 2 + 5 and "cumulative" in capsys.readouterr().out
    kernel, options = wb.get_tagged_mxfp4_gemm((64, 64, 64))
    options.profile_python_wrapper = True
    assert isinstance(wb.wave_compile(options, kernel), wc.ScaledGemmKernelWithProfile)
