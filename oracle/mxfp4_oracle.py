"""CPU oracle for the MXFP4 scaled GEMM — TEST INFRASTRUCTURE, not a product path.

A restatement, in torch on the CPU, of the reference's own CPU implementation of the path
(`wave_lang/kernel/wave/utils/mxfp_utils.py`). Only `tests/`, `__graft_entry__.smoke()` and the
CPU-baseline / reference legs of `bench.py` may import this module; the library itself has no CPU
path and fails loudly without its CUDA extension.

Parity is pinned: `tests/golden/make_golden.py` imports the reference module itself (in the build
container, where the reference tree is mounted) and stores its outputs on seeded inputs;
`tests/test_oracle.py` checks every function here against those stored outputs.

Reference lines restated by each function are cited in its docstring.
"""

from __future__ import annotations

import math

import numpy as np
import torch

# wave_lang/kernel/wave/utils/mxfp_utils.py:17
SCALE_GROUP_SIZE = 32

# wave_lang/kernel/wave/utils/mxfp_utils.py:65-82 — E2M1 code -> value, sign in bit 3.
E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)


def generate_gemm_afp4wfp4_inputs(shape, scale_lo: int = 124, scale_hi: int = 128, seed: int = 5):
    """Seeded random packed-FP4 operands and E8M0 scales.

    Follows wave_lang/kernel/wave/utils/mxfp_utils.py:20-57 call for call (same generator, same
    draw order, same shapes), so that with the defaults the tensors equal the reference's:
    x [M, K/2] uint8, w [K/2, N] uint8 (a transposed VIEW, as the reference returns it),
    x_scales [M, K/32], w_scales [N, K/32]. `scale_hi` is exclusive.
    """
    M, N, K = shape
    torch.manual_seed(seed)
    x_low = torch.randint(0, 16, (M, K // 2), dtype=torch.uint8)
    x_high = torch.randint(0, 16, (M, K // 2), dtype=torch.uint8)
    x = x_low | (x_high << 4)
    w_low = torch.randint(0, 16, (N, K // 2), dtype=torch.uint8)
    w_high = torch.randint(0, 16, (N, K // 2), dtype=torch.uint8)
    w = (w_low | (w_high << 4)).T
    x_scales = torch.randint(scale_lo, scale_hi, (K // SCALE_GROUP_SIZE, M), dtype=torch.uint8)
    w_scales = torch.randint(scale_lo, scale_hi, (K // SCALE_GROUP_SIZE, N), dtype=torch.uint8)
    return x, w, x_scales.T.contiguous(), w_scales.T.contiguous()


def mxfp4_to_f32(x: torch.Tensor) -> torch.Tensor:
    """Packed E2M1 [R, K/2] uint8 -> [R, K] f32; even k is the low nibble.

    wave_lang/kernel/wave/utils/mxfp_utils.py:60-83.
    """
    lut = torch.tensor(E2M1_VALUES, dtype=torch.float32)
    out = torch.empty(x.shape[0], x.shape[1] * 2, dtype=torch.float32)
    out[:, ::2] = lut[(x & 0xF).to(torch.int64)]
    out[:, 1::2] = lut[(x >> 4).to(torch.int64)]
    return out


def e8m0_to_f32(x: torch.Tensor) -> torch.Tensor:
    """E8M0 code (any numeric dtype) -> 2**(x - 127) as f32; code 255 is NaN.

    wave_lang/kernel/wave/utils/mxfp_utils.py:86-95.
    """
    xf = x.to(torch.float32)
    out = torch.pow(torch.tensor(2.0, dtype=torch.float32), xf - 127.0)
    out[xf == 255] = float("nan")
    return out


def dequant_mxfp4(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """[R, K/2] codes and [R, K/32] scales -> dequantised [R, K] f32 operand.

    The operand the reference feeds its matmul: wave_lang/kernel/wave/utils/mxfp_utils.py:135-143.
    """
    vals = mxfp4_to_f32(q)
    s = e8m0_to_f32(scale.repeat_interleave(SCALE_GROUP_SIZE, dim=1).to(torch.float32))
    return vals * s


def torch_scaled_gemm_mxfp4(x, w, x_scales, w_scales) -> torch.Tensor:
    """The reference GEMM: dequantise, then an f32 torch.mm. `w` is [K/2, N] as the reference passes it.

    wave_lang/kernel/wave/utils/mxfp_utils.py:131-143.
    """
    x_f32 = mxfp4_to_f32(x)
    w_f32 = mxfp4_to_f32(w.T).T
    xs = e8m0_to_f32(x_scales.repeat_interleave(SCALE_GROUP_SIZE, dim=1).to(torch.float32))
    ws = e8m0_to_f32(w_scales.repeat_interleave(SCALE_GROUP_SIZE, dim=1).to(torch.float32))
    return torch.mm(x_f32 * xs, w_f32 * ws.T)


def scaled_gemm(a, a_scale, b, b_scale, n_chunk: int = 4096) -> torch.Tensor:
    """Same as torch_scaled_gemm_mxfp4 with b in the kernel's [N, K/2] layout, evaluated in column
    chunks of C so that large N does not need the whole dequantised b at once."""
    a_deq = dequant_mxfp4(a, a_scale)
    N = b.shape[0]
    out = torch.empty(a.shape[0], N, dtype=torch.float32)
    for n0 in range(0, N, n_chunk):
        n1 = min(N, n0 + n_chunk)
        out[:, n0:n1] = torch.mm(a_deq, dequant_mxfp4(b[n0:n1], b_scale[n0:n1]).T)
    return out


# ---------------------------------------------------------------------------------------------
# Layout oracle for the scale repack (no counterpart in the reference: its e8m0_shuffle,
# mxfp_utils.py:113-128, targets the AMD layout; this states the tcgen05 scale-factor layout)
# ---------------------------------------------------------------------------------------------
SF_PAD = 127


def pack_scales(scale: torch.Tensor) -> torch.Tensor:
    """[rows, K/32] uint8 -> flat uint8 array of 512-byte atoms.

    One atom holds 128 rows x 4 K-blocks; the byte of (row r, K-block j) inside its atom is
    (r % 32) * 16 + (r // 32) * 4 + j; atoms of one 128-row block are contiguous along K; the
    atom count along K is rounded up to an even number; padding bytes are 127.
    """
    s = scale.numpy()
    rows, kb = s.shape
    rb = (rows + 127) // 128
    ka = 2 * ((kb * 32 + 255) // 256)
    padded = np.full((rb * 128, ka * 4), SF_PAD, dtype=np.uint8)
    padded[:rows, :kb] = s
    # [rb, r/32 (4), r%32 (32), ka, j (4)] -> [rb, ka, r%32, r/32, j]
    v = padded.reshape(rb, 4, 32, ka, 4).transpose(0, 3, 2, 1, 4)
    return torch.from_numpy(np.ascontiguousarray(v).reshape(-1))


def pack_scales_tiled(scale: torch.Tensor, tile_rows: int) -> torch.Tensor:
    """Weight-scale packing per tile of `tile_rows` rows. Up to 128 (a multiple of 8; the decode kernel's tiles): every
    tile gets an atom row of its own, its rows in atom rows 0 .. tile_rows - 1 and the padding byte above. 224 (the
    tile kernel's 224-column tiles): two atom rows per tile, rows 0..127 and 128..223 of the tile. Inside an atom the
    layout is `pack_scales`'s; tile_rows = 128 is `pack_scales` itself."""
    assert tile_rows == 224 or (tile_rows % 8 == 0 and 8 <= tile_rows <= 128)
    rows, kb = scale.shape
    tiles = (rows + tile_rows - 1) // tile_rows
    span = (tile_rows + 127) // 128 * 128  # rows of packed storage per tile
    spread = torch.full((tiles * span, kb), SF_PAD, dtype=torch.uint8)
    for t in range(tiles):
        part = scale[t * tile_rows:min(rows, (t + 1) * tile_rows)]
        spread[t * span:t * span + part.shape[0]] = part
    return pack_scales(spread)


# ---------------------------------------------------------------------------------------------
# The reference's AMD pre-shuffles, stated as index maps (mxfp_utils.py:98-128). The B200 kernels do not use
# these layouts; they are restated so that data a caller holds in them can be recognised and undone.
# ---------------------------------------------------------------------------------------------
def amd_e8m0_shuffle(scale: torch.Tensor) -> torch.Tensor:
    """wave_lang/kernel/wave/utils/mxfp_utils.py:113-128. The scale matrix, zero-padded to multiples of
    (256, 8), is read as [R, 2, 16, C, 2, 4] (row = 32 R + 16 h + l, column = 8 C + 4 g + e) and written out in the
    order [R, C, e, l, g, h]; the result is clipped back to the input shape."""
    s = scale.numpy()
    m, n = s.shape
    sm, sn = (m + 255) // 256 * 256, (n + 7) // 8 * 8
    src = np.zeros((sm, sn), dtype=s.dtype)
    src[:m, :n] = s
    flat = np.empty(sm * sn, dtype=s.dtype)
    r, c = np.divmod(np.arange(sm * sn), sn)
    R, h, l = r // 32, (r // 16) % 2, r % 16
    C, g, e = c // 8, (c // 4) % 2, c % 4
    dst = ((((R * (sn // 8) + C) * 4 + e) * 16 + l) * 2 + g) * 2 + h
    flat[dst] = src.reshape(-1)
    return torch.from_numpy(np.ascontiguousarray(flat.reshape(sm, sn)[:m, :n]))


def amd_b_preshuffle(b: torch.Tensor) -> torch.Tensor:
    """wave_lang/kernel/wave/utils/mxfp_utils.py:98-110. Inside every 16-row x 32-byte tile the bytes move from
    [row, half, byte] order to [half, row, byte] order (half = which 16 bytes of the 32)."""
    x = b.numpy()
    N, kp = x.shape
    r, c = np.divmod(np.arange(N * kp), kp)
    tile_r, row = r // 16, r % 16
    tile_c, half, byte = c // 32, (c // 16) % 2, c % 16
    dst = (((tile_r * (kp // 32) + tile_c) * 2 + half) * 16 + row) * 16 + byte
    flat = np.empty(N * kp, dtype=x.dtype)
    flat[dst] = x.reshape(-1)
    return torch.from_numpy(flat.reshape(N, kp))


def amd_b_unshuffle(b_shuffled: torch.Tensor) -> torch.Tensor:
    """Inverse of amd_b_preshuffle: the row-major [N, K/2] bytes the B200 kernels read."""
    x = b_shuffled.numpy()
    N, kp = x.shape
    r, c = np.divmod(np.arange(N * kp), kp)
    tile_r, row = r // 16, r % 16
    tile_c, half, byte = c // 32, (c // 16) % 2, c % 16
    src = (((tile_r * (kp // 32) + tile_c) * 2 + half) * 16 + row) * 16 + byte
    return torch.from_numpy(np.ascontiguousarray(x.reshape(-1)[src].reshape(N, kp)))


# ---------------------------------------------------------------------------------------------
# Harness quantiser (not in the reference, which only feeds random codes): f32 -> MXFP4
# ---------------------------------------------------------------------------------------------
def quantize_mxfp4(x: torch.Tensor):
    """f32 [R, K] -> (codes [R, K/2] uint8, scales [R, K/32] uint8).

    Per 32-element block: e = floor(log2(amax)) - 2 (E2M1's largest value is 6 = 1.5 * 2^2), scale
    byte clamp(e + 127, 0, 254), amax == 0 -> e = 0; values x * 2^-e clamped to [-6, 6] and rounded
    to the nearest E2M1 value, ties to the even code; low nibble = even k. A block that holds a NaN or an
    infinity gets scale byte 255 (the E8M0 NaN that `e8m0_to_f32` reads back as NaN,
    wave_lang/kernel/wave/utils/mxfp_utils.py:86-95; the OCP MX block rule) and codes 0.
    """
    R, K = x.shape
    assert K % SCALE_GROUP_SIZE == 0
    packed = torch.empty(R, K // 2, dtype=torch.uint8)
    scales = torch.empty(R, K // 32, dtype=torch.uint8)
    two = torch.tensor(2.0)
    # Midpoints between neighbouring E2M1 magnitudes. A value on a midpoint goes to the neighbour
    # with the even code: above an even code it stays (strict >), above an odd code it moves up (>=).
    strict = (0.25, 1.25, 2.5, 5.0)
    inclusive = (0.75, 1.75, 3.5)
    for r0 in range(0, R, 1024):
        xb = x[r0:r0 + 1024].reshape(-1, K // 32, 32).to(torch.float32)
        bad = ~torch.isfinite(xb).all(dim=2)
        xb = torch.where(bad.unsqueeze(2), torch.zeros_like(xb), xb)
        amax = xb.abs().amax(dim=2)
        e = torch.floor(torch.log2(torch.where(amax > 0, amax, torch.ones_like(amax)))) - 2.0
        e = torch.where(amax > 0, e, torch.zeros_like(e))
        sb = torch.clamp(e + 127.0, 0, 254)
        y = torch.clamp(xb / torch.pow(two, sb - 127.0).unsqueeze(2), -6.0, 6.0)
        y = torch.where(bad.unsqueeze(2), torch.zeros_like(y), y)  # +0: code 0 whatever the sign of the input
        sb = torch.where(bad, torch.full_like(sb, 255.0), sb)
        mag = y.abs()
        idx = torch.zeros_like(mag, dtype=torch.uint8)
        for t in strict:
            idx += (mag > t).to(torch.uint8)
        for t in inclusive:
            idx += (mag >= t).to(torch.uint8)
        code = (idx | (torch.signbit(y).to(torch.uint8) << 3)).reshape(-1, K)
        packed[r0:r0 + 1024] = code[:, 0::2] | (code[:, 1::2] << 4)
        scales[r0:r0 + 1024] = sb.to(torch.uint8)
    return packed, scales


# ---------------------------------------------------------------------------------------------
# Tolerances of the parity bar
# ---------------------------------------------------------------------------------------------
def f32_tolerance(a_deq: torch.Tensor, b_deq: torch.Tensor, ref: torch.Tensor, K: int) -> torch.Tensor:
    """|c - ref| must stay below rtol 1e-5 * |ref| + 1e-5 * sqrt(K) * amax_ij with
    amax_ij = max_k |A_ik| * max_k |B_jk| over the dequantised rows."""
    amax = a_deq.abs().amax(dim=1, keepdim=True) * b_deq.abs().amax(dim=1, keepdim=True).T
    return 1e-5 * ref.abs() + 1e-5 * math.sqrt(K) * amax


def bf16_ulp_distance(c_bf16: torch.Tensor, ref_f32: torch.Tensor) -> torch.Tensor:
    """Distance, in bf16 units in the last place, between c and the reference rounded to bf16.
    The 16-bit patterns are mapped to a monotonic integer line so that +0 and -0 coincide."""
    def ordered(t):
        bits = t.contiguous().view(torch.int16).to(torch.int32) & 0xFFFF
        return torch.where(bits >= 0x8000, 0x8000 - bits, bits)
    return (ordered(c_bf16.cpu()) - ordered(ref_f32.to(torch.bfloat16))).abs()
