// Activation quantiser: f32 or bf16 [rows, K] -> packed E2M1 codes [rows, K/2] plus E8M0 scales,
// written row-major ([rows, K/32], the reference's a_scale layout) and/or directly in the tcgen05
// scale-factor layout, so that the GEMM needs no separate repack pass over the scales.
//
// The reference only has this as a stated direction ("fused dynamic quantization",
// wave_lang/kernel/wave/templates/test_kernels.py:74; its tests feed random codes,
// wave_lang/kernel/wave/utils/mxfp_utils.py:20-57). Rule, per 32-element block:
//   e = floor(log2(amax)) - 2 (E2M1's largest value is 6 = 1.5 * 2^2), scale byte clamp(e + 127, 0, 254),
//   amax == 0 -> byte 127; y = x * 2^-(byte - 127), clamped to [-6, 6], rounded to the nearest E2M1
//   value, a value on a midpoint going to the neighbour with the even code; even k in the low nibble.
//   A block that holds a NaN or an infinity gets scale byte 255 (E8M0's NaN: the OCP MX rule, and what the
//   reference's dequantisation reads as NaN, mxfp_utils.py:86-95) and codes 0, so that the GEMM's outputs for
//   that row are NaN instead of plausible finite numbers.
//
// HBM-bound: 4 lanes share one block (8 values each), so a warp reads 512 contiguous bytes of bf16
// per load instruction and writes 128 contiguous bytes of codes; the E2M1 rounding is the hardware conversion.
#pragma once
#include "scales.cuh"
#include <cuda_bf16.h>

namespace wb {

// Two f32 -> one byte of E2M1 codes (lo in the low nibble), by the hardware conversion: round to
// nearest with ties to the even code (of the magnitudes {0, .5, 1, 1.5, 2, 3, 4, 6}: 0.25 -> 0, 0.75 -> 1,
// 1.25 -> 1, 1.75 -> 2, 2.5 -> 2, 3.5 -> 4, 5 -> 4), saturating at +-6, sign in bit 3.
__device__ __forceinline__ uint32_t e2m1x2_code(float lo, float hi) {
  uint16_t r;
  asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; mov.b16 %0, {t, 0}; }" : "=h"(r) : "f"(hi), "f"(lo));
  return uint32_t(r);
}

// Bit pattern of the largest |v| over the 32 values held by a group of 32 / VPL neighbouring lanes. For
// non-negative floats the unsigned order of the bit patterns is the numeric order, with the infinity above
// every finite value and every NaN above the infinity: an integer maximum keeps a NaN that fmaxf would drop.
template <int VPL>
__device__ __forceinline__ uint32_t block_amax_bits(const float (&v)[VPL]) {
  uint32_t m = 0;
#pragma unroll
  for (int j = 0; j < VPL; ++j) m = max(m, __float_as_uint(fabsf(v[j])));
#pragma unroll
  for (int o = 1; o < 32 / VPL; o <<= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
  return m;
}

// Scale byte and codes of the 32 values held by a group of 32 / VPL neighbouring lanes (v: the VPL consecutive
// values of this lane; VPL = 4 or 8). All lanes of a warp must call it together (shuffles).
template <int VPL>
__device__ __forceinline__ void mxfp4_encode_values(const float (&v)[VPL], uint32_t& packed, int& sb) {
  static_assert(VPL == 4 || VPL == 8, "4 or 8 values per lane");
  const uint32_t amax_bits = block_amax_bits<VPL>(v);
  if ((amax_bits >> 23) == 0xffu) {  // an infinity or a NaN somewhere in the block
    sb = 255;
    packed = 0;
    return;
  }
  // floor(log2(amax)) is the unbiased exponent field for normal numbers; subnormal maxima fall
  // below the clamp at 0 either way
  sb = 127;
  if (amax_bits != 0u) {
    sb = int(amax_bits >> 23) - 2;
    sb = max(0, min(254, sb));
  }
  // y = x * 2^(127 - sb), exact; 2^127 and 2^-127 are both representable
  const int ie = 127 - sb;  // -127 .. 127
  const float inv = (ie == -127) ? __int_as_float(0x00400000) : __int_as_float((ie + 127) << 23);
  packed = 0;
#pragma unroll
  for (int j = 0; j < VPL / 2; ++j) packed |= e2m1x2_code(v[2 * j] * inv, v[2 * j + 1] * inv) << (8 * j);
}

// Stores what mxfp4_encode_values produced for row r, K block kb (lane `sub` of the group).
template <int VPL>
__device__ __forceinline__ void mxfp4_store_block(uint32_t packed, int sb, int r, int kb, int sub, int K, int kblocks,
                                                  int k_atoms, uint8_t* __restrict__ q, uint8_t* __restrict__ scale_rm,
                                                  uint8_t* __restrict__ scale_packed) {
  uint8_t* dst = q + (long long)r * (K / 2) + kb * 16;
  if constexpr (VPL == 4) reinterpret_cast<uint16_t*>(dst)[sub] = uint16_t(packed);
  else reinterpret_cast<uint32_t*>(dst)[sub] = packed;
  if (sub == 0) {
    if (scale_rm) scale_rm[(long long)r * kblocks + kb] = uint8_t(sb);
    if (scale_packed) {
      const size_t off = (size_t(r >> 7) * k_atoms + (kb >> 2)) * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (kb & 3);
      scale_packed[off] = uint8_t(sb);
    }
  }
}

// Quantises the 32 values of row r, K block kb held by a group of 32 / VPL neighbouring lanes and stores codes
// and scale. All lanes of a warp must call it together; inactive groups pass active = false and store nothing.
template <int VPL>
__device__ __forceinline__ void mxfp4_encode_group(const float (&v)[VPL], bool active, int r, int kb, int sub, int K,
                                                   int kblocks, int k_atoms, uint8_t* __restrict__ q,
                                                   uint8_t* __restrict__ scale_rm, uint8_t* __restrict__ scale_packed) {
  uint32_t packed;
  int sb;
  mxfp4_encode_values<VPL>(v, packed, sb);
  if (active) mxfp4_store_block<VPL>(packed, sb, r, kb, sub, K, kblocks, k_atoms, q, scale_rm, scale_packed);
}

// 8 consecutive values from 16-byte aligned memory.
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 t = *reinterpret_cast<const uint4*>(p);
  v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xffff0000u);
  v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xffff0000u);
  v[4] = __uint_as_float(t.z << 16); v[5] = __uint_as_float(t.z & 0xffff0000u);
  v[6] = __uint_as_float(t.w << 16); v[7] = __uint_as_float(t.w & 0xffff0000u);
}

// Four lanes per 32-element block, 8 values (16 bytes of bf16, 32 of f32) each; grid (rows,
// ceil(kblocks / 64)): a CTA covers 64 consecutive blocks of one row. x rows are 16-byte aligned.
template <typename InT>
__global__ void __launch_bounds__(256)
quantize_mxfp4_kernel(const InT* __restrict__ x, long long ldx, int rows, int K, uint8_t* __restrict__ q,
                      uint8_t* __restrict__ scale_rm, uint8_t* __restrict__ scale_packed, int k_atoms) {
  const int sub = threadIdx.x & 3;
  const int kblocks = K >> 5;
  const int r = blockIdx.x;
  const int kb = blockIdx.y * 64 + (threadIdx.x >> 2);
  const bool active = r < rows && kb < kblocks;
  float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (active) load8(x + (long long)r * ldx + kb * 32 + sub * 8, v);
  mxfp4_encode_group<8>(v, active, r, kb, sub, K, kblocks, k_atoms, q, scale_rm, scale_packed);
}

// MXFP8 counterpart: f32 or bf16 [rows, K] -> one byte per element (E4M3 when fmt == 0, E5M2 when fmt == 1) plus
// E8M0 scales, e = floor(log2(amax)) - 8 (E4M3: largest value 448) or - 15 (E5M2: 57344); the rounding and the
// saturation are the hardware conversion's (cvt.rn.satfinite). Same thread layout as the MXFP4 quantiser.
__device__ __forceinline__ uint32_t f8x2_code(float lo, float hi, int fmt) {
  uint16_t r;
  if (fmt == 0) asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  else asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return uint32_t(r);
}

template <typename InT>
__global__ void __launch_bounds__(256)
quantize_mxfp8_kernel(const InT* __restrict__ x, long long ldx, int rows, int K, int fmt, uint8_t* __restrict__ q,
                      uint8_t* __restrict__ scale_rm, uint8_t* __restrict__ scale_packed, int k_atoms) {
  const int sub = threadIdx.x & 3;
  const int kblocks = K >> 5;
  const int r = blockIdx.x;
  const int kb = blockIdx.y * 64 + (threadIdx.x >> 2);
  const bool active = r < rows && kb < kblocks;
  float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (active) load8(x + (long long)r * ldx + kb * 32 + sub * 8, v);
  const uint32_t amax_bits = block_amax_bits<8>(v);
  const bool not_finite = (amax_bits >> 23) == 0xffu;  // an infinity or a NaN in the block: scale byte 255, codes 0
  int sb = not_finite ? 255 : 127;
  if (!not_finite && amax_bits != 0u) {
    sb = int(amax_bits >> 23) - (fmt == 0 ? 8 : 15);
    sb = max(0, min(254, sb));
  }
  const int ie = 127 - sb;
  const float inv = (ie <= -127) ? __int_as_float(0x00400000) : __int_as_float((ie + 127) << 23);
  if (!active) return;
  uint2 out = make_uint2(0u, 0u);
  if (!not_finite) {
    out.x = f8x2_code(v[0] * inv, v[1] * inv, fmt) | (f8x2_code(v[2] * inv, v[3] * inv, fmt) << 16);
    out.y = f8x2_code(v[4] * inv, v[5] * inv, fmt) | (f8x2_code(v[6] * inv, v[7] * inv, fmt) << 16);
  }
  *reinterpret_cast<uint2*>(q + (long long)r * K + kb * 32 + sub * 8) = out;
  if (sub == 0) {
    if (scale_rm) scale_rm[(long long)r * kblocks + kb] = uint8_t(sb);
    if (scale_packed) {
      const size_t off = (size_t(r >> 7) * k_atoms + (kb >> 2)) * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (kb & 3);
      scale_packed[off] = uint8_t(sb);
    }
  }
}

// Quantise-and-scatter for routed tokens: row t of x is quantised once and written to the `copies` output rows
// dst_rows[t * copies + j] (negative entries are skipped): the tokens of a mixture-of-experts layer go straight
// to their expert-sorted rows without a separate gather pass. Scales are written row-major.
template <typename InT>
__global__ void __launch_bounds__(256)
quantize_scatter_mxfp4_kernel(const InT* __restrict__ x, long long ldx, int rows, int K, int copies,
                              const int* __restrict__ dst_rows, uint8_t* __restrict__ q, uint8_t* __restrict__ scale_rm) {
  const int sub = threadIdx.x & 3;
  const int kblocks = K >> 5;
  const int r = blockIdx.x;
  const int kb = blockIdx.y * 64 + (threadIdx.x >> 2);
  const bool active = r < rows && kb < kblocks;
  float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (active) load8(x + (long long)r * ldx + kb * 32 + sub * 8, v);
  uint32_t packed;
  int sb;
  mxfp4_encode_values<8>(v, packed, sb);
  if (!active) return;
  for (int j = 0; j < copies; ++j) {
    const int dst = dst_rows[r * copies + j];
    if (dst >= 0) mxfp4_store_block<8>(packed, sb, dst, kb, sub, K, kblocks, 0, q, scale_rm, nullptr);
  }
}

// Fills the padding bytes of a packed scale array (rows past `rows` in the last 128-row block, K blocks
// past K/32 in the last atoms) with the neutral byte; the quantiser above writes only real positions.
__global__ void __launch_bounds__(256)
fill_scale_padding_kernel(uint8_t* __restrict__ scale_packed, int rows, int kblocks, int k_atoms, int row_blocks) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)row_blocks * k_atoms * 512;
  if (idx >= total) return;
  const int within = int(idx & 511);
  const long long atom = idx >> 9;
  const int rb = int(atom / k_atoms), ka = int(atom - (long long)rb * k_atoms);
  const int r = rb * 128 + ((within >> 2) & 3) * 32 + (within >> 4);
  const int kb = ka * 4 + (within & 3);
  if (r >= rows || kb >= kblocks) scale_packed[idx] = WB_SF_PAD;
}

}  // namespace wb
