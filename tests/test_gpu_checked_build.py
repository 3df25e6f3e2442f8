"""Out-of-bounds and alignment checks without compute-sanitizer.

Two layers, the ones the reference gets from `use_bound_check` (generate_bound_checks.py) and its in-bounds
static checks:
  * host canaries: every output is a window inside a larger buffer filled with a canary pattern, and every
    workspace has canary bytes behind it; after the GEMM the window matches the oracle and no canary changed.
    Runs on the shipped library, small shapes on every kernel path;
  * the debug-checked build of the library (-DWB200_CHECKS): the same cases in a child process that loads
    libwave_b200_checks.so, with the device-side predicate record read back: no predicate may have failed,
    and the self-test shows that a failed predicate is recorded without trapping.
"""

import ctypes
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
DEV = "cuda:0"
CANARY_BF16 = -12345.0   # exactly representable in bf16 and f32; no GEMM case below produces it
CANARY_BYTE = 0xA5


def _cases():
    from wave_b200 import _lib
    tile = [(_lib.PATH_TILE_1CTA, "1cta"), (_lib.PATH_TILE_1CTA | _lib.TILE_N128, "1cta-128"), (_lib.PATH_TILE_2CTA, "2cta"),
            (_lib.PATH_TILE_2CTA | _lib.TILE_N192, "2cta-192"), (_lib.PATH_TILE_2CTA | _lib.TILE_N128, "2cta-128")]
    out = []
    for flags, name in tile:
        for shape in ((256, 256, 512), (200, 136, 288), (130, 520, 64)):
            out.append((name, flags, shape))
    for shape in ((1, 256, 512), (16, 200, 288), (100, 136, 96), (128, 256, 512), (16, 128 * 150, 64), (40, 128 * 149 + 8, 96), (8, 128 * 230, 64)):
        out.append(("skinny", _lib.PATH_SKINNY, shape))
    out.append(("split-k", _lib.PATH_TILE_SPLITK, (256, 256, 4096)))
    out.append(("split-k", _lib.PATH_TILE_SPLITK, (200, 136, 2080)))
    return out


def run_canary_cases(expect_checked_build) -> int:
    """Every case: c is rows [3, 3 + M) x columns [8, 8 + N) of a canary-filled buffer, the workspace is followed by
    canary bytes. Returns the number of cases run; raises AssertionError on any mismatch."""
    sys.path.insert(0, str(ROOT))
    from oracle import mxfp4_oracle as orc
    from wave_b200 import _lib, ops
    lib = _lib.load()
    record = (ctypes.c_ulonglong * 3)()
    rc = lib.wb200_debug_checks(record, 0)
    if expect_checked_build is None:  # whichever build this process loaded
        expect_checked_build = rc == _lib.WB200_OK
    assert (rc == _lib.WB200_OK) == expect_checked_build, f"debug_checks returned {rc}"
    selftest = expect_checked_build and "--child" in sys.argv  # the self-test leaves a record: only where it is reset afterwards
    before = record[2]
    if selftest:
        assert lib.wb200_debug_checks(record, 1) == _lib.WB200_OK
        assert lib.wb200_debug_checks_selftest(None) == _lib.WB200_OK
        assert lib.wb200_debug_checks(record, 1) == _lib.WB200_OK
        assert (record[0] & 0xFFFFFFFF, record[0] >> 32, record[1], record[2]) == (99, 0, 1, 1), list(record)
        ops.check_device_status()  # the context is intact: no wait timed out, nothing trapped
        before = 0
    n = 0
    for name, flags, (M, N, K) in _cases():
        for dtype in (torch.bfloat16, torch.float32):
            g = torch.Generator().manual_seed(M * 7 + N * 3 + K)
            a = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, generator=g)
            b = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g)
            a_s = torch.randint(124, 131, (M, K // 32), dtype=torch.uint8, generator=g)
            b_s = torch.randint(124, 131, (N, K // 32), dtype=torch.uint8, generator=g)
            ref = orc.scaled_gemm(a, a_s, b, b_s)
            esz = 2 if dtype == torch.bfloat16 else 4
            ld = ((8 + N + 8) * esz + 15) // 16 * 16 // esz  # a row pitch that keeps 16-byte alignment
            big = torch.full((M + 6, ld), CANARY_BF16, dtype=dtype, device=DEV)
            c = big[3:3 + M, 8:8 + N]
            ws_bytes = int(lib.wb200_mxfp4_gemm_workspace_bytes(M, N, K))
            ws = torch.full((ws_bytes + 4096,), CANARY_BYTE, dtype=torch.uint8, device=DEV)
            if ws_bytes:  # 0: the shape needs no workspace on any path (the canary tail is still checked)
                assert lib.wb200_workspace_init(ws.data_ptr(), ws_bytes, None) == _lib.WB200_OK
            a_d, b_d = a.to(DEV), b.to(DEV)
            a_sf, b_sf = ops.repack_scales(a_s.to(DEV)), ops.repack_scales(b_s.to(DEV))
            rc = lib.wb200_mxfp4_gemm(M, N, K, a_d.data_ptr(), a_sf.data.data_ptr(), b_d.data_ptr(), b_sf.data.data_ptr(),
                                      c.data_ptr(), ops._DTYPE_CODE[dtype], ld, ws.data_ptr() if ws_bytes else None, ws_bytes, flags, None)
            assert rc == _lib.WB200_OK, f"{name} {(M, N, K)}: rc {rc}: {lib.wb200_last_error().decode()}"
            ops.check_device_status()
            where = f"{name} {(M, N, K)} {dtype}"
            out = big.cpu()
            window = out[3:3 + M, 8:8 + N]
            if dtype == torch.float32:
                tol = orc.f32_tolerance(orc.dequant_mxfp4(a, a_s), orc.dequant_mxfp4(b, b_s), ref, K)
                assert bool(((window - ref).abs() <= tol).all()), where
            else:
                assert int(orc.bf16_ulp_distance(window.contiguous(), ref).max()) <= 1, where
            frame = out.clone()
            frame[3:3 + M, 8:8 + N] = CANARY_BF16
            assert bool((frame == CANARY_BF16).all()), f"{where}: wrote outside c"
            assert bool((ws[ws_bytes:] == CANARY_BYTE).all().item()), f"{where}: wrote past the workspace"
            # the packed scale arrays are read-only operands: unchanged
            assert torch.equal(b_sf.data.cpu(), orc.pack_scales(b_s)), where
            n += 1
    if expect_checked_build:
        assert lib.wb200_debug_checks(record, 0) == _lib.WB200_OK
        assert record[2] == before, f"{record[2] - before} predicate(s) failed; first: code {record[0] & 0xFFFFFFFF} CTA {record[0] >> 32} detail {record[1]}"
    return n


@pytest.mark.gpu
def test_outputs_and_workspaces_stay_inside_their_buffers():
    assert run_canary_cases(expect_checked_build=None) >= 40


@pytest.mark.gpu
def test_same_cases_under_the_debug_checked_build():
    lib = ROOT / "wave_b200" / "libwave_b200_checks.so"
    if not lib.exists():
        pytest.fail("libwave_b200_checks.so is missing: run `python -m wave_b200.build --checks` (build() makes it)")
    env = dict(os.environ, WAVE_B200_LIB=str(lib))
    res = subprocess.run([sys.executable, str(Path(__file__).resolve()), "--child"], env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert "cases ok under the checked build" in res.stdout


def test_checked_build_exports_the_same_symbols():
    """CPU: the debug-checked library, when built, exports everything the header declares (it is a drop-in)."""
    lib = ROOT / "wave_b200" / "libwave_b200_checks.so"
    if not lib.exists():
        pytest.skip("debug-checked library not built here")
    sys.path.insert(0, str(ROOT))
    from wave_b200 import _lib
    handle = ctypes.CDLL(str(lib))
    for name in _lib.EXPORTED_SYMBOLS:
        getattr(handle, name)


if __name__ == "__main__" and "--child" in sys.argv:
    count = run_canary_cases(expect_checked_build=True)
    print(f"{count} cases ok under the checked build")
