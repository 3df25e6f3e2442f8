// Scale-factor repack and the dequantisation test aid.
//
// repack_scales_kernel takes the reference's row-major E8M0 scales ([rows, K/32] uint8, the
// a_scale / b_scale arguments of wave_lang/kernel/wave/templates/gemm.py:171-175) and writes
// the layout tcgen05.mma reads block scales in. It stands where the reference has its host-side
// e8m0_shuffle permutation for the AMD scale layout
// (wave_lang/kernel/wave/utils/mxfp_utils.py:113-128).
//
// Output layout: 512-byte atoms, one per (128-row block, 4 consecutive K blocks), atoms of one
// row block contiguous along K. Inside an atom the scale of row r (0..127), K block j (0..3)
// sits at byte (r % 32) * 16 + (r / 32) * 4 + j. The atom count along K is padded to an even
// number (one pipeline stage = 256 K elements = 2 atoms) and rows are padded to 128; padding
// bytes are 127 (scale 1.0, never the NaN code 255), they only ever multiply zero-filled data.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace wb {

static constexpr uint8_t WB_SF_PAD = 127;

__host__ __device__ inline int sf_row_blocks(int rows) { return (rows + 127) / 128; }
__host__ __device__ inline int sf_k_atoms(int K) { return 2 * ((K + 255) / 256); }
__host__ __device__ inline size_t sf_packed_bytes(int rows, int K) {
  return size_t(sf_row_blocks(rows)) * sf_k_atoms(K) * 512;
}

// One thread block moves 128 rows x 32 K-blocks through shared memory: reads are 16 bytes per
// thread along K, writes are 4 KiB contiguous. Rows [row_base, row_base + 128) of src, clipped at
// row_limit, go to the 128-row block whose first atom is at dst_block. With `broadcast` src holds one
// scale per row, used for every K block of that row (the a_scale [M] argument of the reference's
// broadcast-scale kernel, wave_lang/kernel/wave/templates/test_kernels.py:98-116).
__device__ __forceinline__ void repack_tile(const uint8_t* __restrict__ src, long long src_row_stride, int row_base,
                                            int row_limit, int kblocks, int k_atoms, int atom0,
                                            uint8_t* __restrict__ dst_block, bool broadcast = false) {
  __shared__ __align__(16) uint8_t tile[128][32 + 4];  // +4 keeps 32-bit reads aligned and spreads banks
  const int t = threadIdx.x;
  {
    const int r = t >> 1;
    const int half = t & 1;
    const int row = row_base + r;
    const int kb0 = atom0 * 4 + half * 16;
    const uint8_t* s = src + (long long)row * src_row_stride + (broadcast ? 0 : kb0);
    const bool row_ok = row < row_limit;
    if (!broadcast && row_ok && kb0 + 16 <= kblocks && ((reinterpret_cast<uintptr_t>(s) & 15) == 0)) {
      const uint4 v = *reinterpret_cast<const uint4*>(s);
      uint32_t* d = reinterpret_cast<uint32_t*>(&tile[r][half * 16]);
      d[0] = v.x; d[1] = v.y; d[2] = v.z; d[3] = v.w;
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j)
        tile[r][half * 16 + j] = (row_ok && kb0 + j < kblocks) ? s[broadcast ? 0 : j] : WB_SF_PAD;
    }
  }
  __syncthreads();
  {
    const int a = t >> 5;    // atom inside this block's run of 8
    const int r32 = t & 31;  // 16-byte row of the atom
    if (atom0 + a < k_atoms) {
      uint4 v;
      v.x = *reinterpret_cast<const uint32_t*>(&tile[r32][a * 4]);
      v.y = *reinterpret_cast<const uint32_t*>(&tile[32 + r32][a * 4]);
      v.z = *reinterpret_cast<const uint32_t*>(&tile[64 + r32][a * 4]);
      v.w = *reinterpret_cast<const uint32_t*>(&tile[96 + r32][a * 4]);
      uint8_t* d = dst_block + size_t(atom0 + a) * 512 + r32 * 16;
      *reinterpret_cast<uint4*>(d) = v;
    }
  }
}

// grid (ceil(k_atoms / 8), row_blocks), 256 threads.
__global__ void __launch_bounds__(256)
repack_scales_kernel(const uint8_t* __restrict__ src, long long src_row_stride, int rows, int kblocks,
                     int k_atoms, uint8_t* __restrict__ dst, bool broadcast, bool dependent, int block_rows = 128) {
  // a GEMM launched behind this kernel as a programmatic dependent may start its set-up now; it waits for
  // this kernel's completion before it reads dst
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // launched as a programmatic dependent itself: the kernel before it may still be reading dst or writing src
  if (dependent) asm volatile("griddepcontrol.wait;" ::: "memory");
  // block_rows != 128: a packing per tile of block_rows weight rows. Up to 128: one atom row per tile (the decode
  // kernel's tiles; rows block_rows..127 of every atom hold the padding byte). Above 128 (224: the tile kernel's
  // 224-column tiles): two atom rows per tile, rows 0..127 and 128..block_rows-1 of the tile.
  const int rb = blockIdx.y;
  const int per_tile = (block_rows + 127) / 128;
  const int tile = rb / per_tile, part = rb - tile * per_tile;
  const int row_base = tile * block_rows + part * 128;
  const int row_end = tile * block_rows + min(block_rows, (part + 1) * 128);
  repack_tile(src, src_row_stride, row_base, min(rows, row_end), kblocks, k_atoms, blockIdx.x * 8,
              dst + size_t(rb) * k_atoms * 512, broadcast);
}

// Grouped form: the rows of group g are src rows [row_start[g], row_start[g+1]) and its packed block
// starts at 128-row block block_start[g] of dst (every group starts on a block boundary, because
// a scale-factor atom covers 128 consecutive rows of ONE GEMM). grid (ceil(k_atoms / 8), total blocks).
constexpr int kMaxRepackGroups = 32;
struct RepackGroups {
  int num_groups;
  int row_start[kMaxRepackGroups + 1];
  int block_start[kMaxRepackGroups + 1];
};
__global__ void __launch_bounds__(256)
repack_scales_grouped_kernel(const uint8_t* __restrict__ src, long long src_row_stride, const RepackGroups tab,
                             int kblocks, int k_atoms, uint8_t* __restrict__ dst) {
  const int rb = blockIdx.y;
  int g = 0;
  while (g + 1 < tab.num_groups && rb >= tab.block_start[g + 1]) ++g;
  const int row_base = tab.row_start[g] + (rb - tab.block_start[g]) * 128;
  repack_tile(src, src_row_stride, row_base, tab.row_start[g + 1], kblocks, k_atoms, blockIdx.x * 8,
              dst + size_t(rb) * k_atoms * 512);
}

// out[r, k] = E2M1(code(r, k)) * 2^(scale(r, k / 32) - 127), the dequantised operand of
// wave_lang/kernel/wave/utils/mxfp_utils.py:60-95,135-142: even k in the low nibble, scale 255 is NaN.
__global__ void __launch_bounds__(256)
dequant_mxfp4_kernel(const uint8_t* __restrict__ q, const uint8_t* __restrict__ scale, int rows, int K,
                     float* __restrict__ out) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // one packed byte each
  const long long total = (long long)rows * (K / 2);
  if (idx >= total) return;
  const int r = int(idx / (K / 2));
  const int kbyte = int(idx - (long long)r * (K / 2));
  const uint8_t byte = q[idx];
  const uint8_t s = scale[(long long)r * (K / 32) + (kbyte / 16)];
  // 2^(s-127): s = 0 is the subnormal 2^-127, s = 255 is NaN.
  const float sc = (s == 255) ? __int_as_float(0x7fc00000)
                              : (s == 0 ? __int_as_float(0x00400000) : __int_as_float(int(s) << 23));
  const float mag[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
  const int lo = byte & 0xF, hi = byte >> 4;
  float vlo = mag[lo & 7], vhi = mag[hi & 7];
  if (lo & 8) vlo = -vlo;
  if (hi & 8) vhi = -vhi;
  float2 o;
  o.x = vlo * sc;
  o.y = vhi * sc;
  reinterpret_cast<float2*>(out)[idx] = o;
}

}  // namespace wb
