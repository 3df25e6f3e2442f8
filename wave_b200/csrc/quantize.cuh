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
//
// HBM-bound: 8 lanes share one block (4 values each), so a warp reads 512 contiguous bytes (f32)
// per load instruction and writes 64 contiguous bytes of codes.
#pragma once
#include "scales.cuh"
#include <cuda_bf16.h>

namespace wb {

__device__ __forceinline__ uint32_t e2m1_code(float y) {
  const float m = fabsf(y);
  // midpoints between neighbouring magnitudes {0, .5, 1, 1.5, 2, 3, 4, 6}: strict above an even
  // code, inclusive above an odd one (ties to the even code)
  uint32_t idx = (m > 0.25f) + (m >= 0.75f) + (m > 1.25f) + (m >= 1.75f) + (m > 2.5f) + (m >= 3.5f) + (m > 5.0f);
  return idx | ((__float_as_uint(y) >> 31) << 3);
}

// Quantises the 32 values held by a group of 8 lanes (v: 4 consecutive values of lane `sub`) of row r,
// K block kb, and stores codes and scale. All 8 lanes of a group must call it together (shuffles);
// inactive groups pass active = false and store nothing.
__device__ __forceinline__ void mxfp4_encode_group(const float (&v)[4], bool active, int r, int kb, int sub, int K,
                                                   int kblocks, int k_atoms, uint8_t* __restrict__ q,
                                                   uint8_t* __restrict__ scale_rm, uint8_t* __restrict__ scale_packed) {
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  // floor(log2(amax)) is the unbiased exponent field for normal numbers; subnormal maxima fall
  // below the clamp at 0 either way
  int sb = 127;
  if (amax > 0.f) {
    sb = int((__float_as_uint(amax) >> 23) & 0xff) - 2;
    sb = max(0, min(254, sb));
  }
  // y = x * 2^(127 - sb), exact; 2^127 and 2^-127 are both representable
  const int ie = 127 - sb;  // -127 .. 127
  const float inv = (ie == -127) ? __int_as_float(0x00400000) : __int_as_float((ie + 127) << 23);
  uint32_t packed = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float y = fminf(fmaxf(v[j] * inv, -6.0f), 6.0f);
    packed |= e2m1_code(y) << (4 * j);
  }
  if (!active) return;
  reinterpret_cast<uint16_t*>(q + (long long)r * (K / 2) + kb * 16)[sub] = uint16_t(packed);
  if (sub == 0) {
    if (scale_rm) scale_rm[(long long)r * kblocks + kb] = uint8_t(sb);
    if (scale_packed) {
      const size_t off = (size_t(r >> 7) * k_atoms + (kb >> 2)) * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (kb & 3);
      scale_packed[off] = uint8_t(sb);
    }
  }
}

template <typename InT>
__global__ void __launch_bounds__(256)
quantize_mxfp4_kernel(const InT* __restrict__ x, long long ldx, int rows, int K, uint8_t* __restrict__ q,
                      uint8_t* __restrict__ scale_rm, uint8_t* __restrict__ scale_packed, int k_atoms) {
  // one group of 8 lanes per 32-element block; blocks of a row are consecutive groups
  const long long group = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 3;
  const int sub = threadIdx.x & 7;
  const int kblocks = K >> 5;
  const long long total = (long long)rows * kblocks;
  const bool active = group < total;
  const int r = active ? int(group / kblocks) : 0;
  const int kb = active ? int(group - (long long)r * kblocks) : 0;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  if (active) {
    const InT* src = x + (long long)r * ldx + kb * 32 + sub * 4;
    if constexpr (sizeof(InT) == 4) {
      const float4 t = *reinterpret_cast<const float4*>(src);
      v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    } else {
      const uint2 t = *reinterpret_cast<const uint2*>(src);
      v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xffff0000u);
      v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xffff0000u);
    }
  }
  mxfp4_encode_group(v, active, r, kb, sub, K, kblocks, k_atoms, q, scale_rm, scale_packed);
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
