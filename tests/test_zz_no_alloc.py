"""The allocation-free skinny entry point against the regular one, through the C ABI.

`wb200_mxfp4_gemm_skinny_noalloc` serves callers that cannot allocate device memory when they
call (a host with a fixed memory plan, a latency-critical decode loop, a plug-in boundary that
passes tensors only): its stream-K scratch is a fixed array inside the library instead of a
caller workspace. It must give the same result as `wb200_mxfp4_gemm` on its skinny path, call
after call, because every call reuses the same array. This file sorts last on purpose, so that
a run that stops at the first failure has already run every other test.
"""

import ctypes

import pytest
import torch

from oracle import mxfp4_oracle as orc
from wave_b200 import _lib, ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _problem(M, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    a = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, generator=g)
    b = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g)
    a_s = torch.randint(124, 131, (M, K // 32), dtype=torch.uint8, generator=g)
    b_s = torch.randint(124, 131, (N, K // 32), dtype=torch.uint8, generator=g)
    return a, a_s, b, b_s


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K", [(16, 4096, 2048), (5, 1000, 992)])
def test_noalloc_matches_workspace_path_on_two_calls_in_a_row(M, N, K, out_dtype):
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    code = _lib.WB200_F32 if out_dtype == torch.float32 else _lib.WB200_BF16
    a, a_s, b, b_s = _problem(M, N, K, seed=M * 1000 + N)
    ad, bd = a.to(DEV), b.to(DEV)
    a_sf, b_sf = ops.repack_scales(a_s.to(DEV)), ops.repack_scales(b_s.to(DEV))

    # existing entry point, skinny path, caller-provided workspace
    expected = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.scaled_gemm_packed(ad, a_sf, bd, b_sf, expected, _lib.PATH_SKINNY)

    # new entry point: no workspace argument, twice in a row on the same stream
    outs = []
    for _ in range(2):
        c = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
        _lib.check(lib.wb200_mxfp4_gemm_skinny_noalloc(M, N, K, ad.data_ptr(), a_sf.data.data_ptr(), bd.data_ptr(),
                                                       b_sf.data.data_ptr(), c.data_ptr(), code, N, 0, stream))
        outs.append(c)
    ops.check_device_status()

    ref = orc.scaled_gemm(a, a_s, b, b_s)
    for c in outs:
        # same kernel, same order of additions: the two entry points agree bit for bit ...
        assert torch.equal(c.view(torch.int16 if out_dtype == torch.bfloat16 else torch.int32),
                           expected.view(torch.int16 if out_dtype == torch.bfloat16 else torch.int32))
        # ... and both are inside the tolerance the parity tests use against the oracle
        if out_dtype == torch.bfloat16:
            assert int(orc.bf16_ulp_distance(c, ref).max()) <= 1
        else:
            tol = orc.f32_tolerance(orc.dequant_mxfp4(a, a_s), orc.dequant_mxfp4(b, b_s), ref, K)
            assert bool(((c.cpu() - ref).abs() <= tol).all())


def test_noalloc_rejects_sizes_beyond_its_scratch_array():
    lib = _lib.load()
    buf = torch.zeros(1 << 16, dtype=torch.uint8, device=DEV)
    p = buf.data_ptr()
    for M, N in ((17, 1024), (16, 65536 + 128)):
        rc = lib.wb200_mxfp4_gemm_skinny_noalloc(M, N, 64, p, p, p, p, p, 0, N, 0, None)
        assert rc == _lib.WB200_ERR_UNSUPPORTED
        assert b"built-in scratch array" in lib.wb200_last_error()
    assert lib.wb200_mxfp4_gemm_skinny_noalloc(16, 1024, 64, p, p, p, p, p, 0, 1024, _lib.PATH_SKINNY, None) == _lib.WB200_ERR_INVALID_ARG
    assert ctypes.c_int(lib.wb200_version()).value >= 1000
