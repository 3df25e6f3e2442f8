// The steps either side of the grouped (per-expert) MXFP4 GEMM in a mixture-of-experts MLP:
//
//   moe_align_block_size   routed (token, slot) pairs -> rows sorted by expert, every expert padded to
//                          whole blocks. Same outputs as the reference's moe_align_block_size_pytorch
//                          (tests/kernel/moe/torch_kernels.py:10-97), integer work, bit-exact.
//   moe_gather_rows        copy the packed codes / scales of each routed token to its sorted row.
//   silu_and_mul           out = x1 / (1 + exp(-x1)) * x2, the reference's get_silu_and_mul_kernel
//                          (wave_lang/kernel/wave/templates/moe.py:89-145; checked there against
//                          gate * up / (1 + exp(-gate)), tests/kernel/moe_test.py:39-40), optionally
//                          quantised to MXFP4 in the same pass so that the down projection reads codes.
//   moe_combine            out[t] = sum_j weight[t, j] * y[row of (t, j)]: the weighted sum at the end of
//                          the reference's MoE (tests/kernel/moe_test.py:123-127).
//
// All four are HBM- or latency-bound integer / elementwise work: coalesced 16-byte accesses, no
// tensor cores.
#pragma once
#include "ptx.cuh"
#include "quantize.cuh"

namespace wb {

constexpr int kMoeMaxExperts = 256;

// One CTA of 1024 threads. ids: [n] expert of every routed (token, slot) pair in flat order.
// sorted_ids [sorted_cap]: flat indices grouped by expert, ascending inside an expert, each expert's
// run padded with the value n to a multiple of block_size; the rest of the array is n as well.
// expert_ids [total / block_size]: expert of every block. inverse [n] (may be null): position of
// flat index i in sorted_ids. Ids outside [0, E) are skipped.
template <typename IdT>
__global__ void __launch_bounds__(1024)
moe_align_block_size_kernel(const IdT* __restrict__ ids, int n, int E, int block_size, int sorted_cap,
                            int* __restrict__ sorted_ids, int* __restrict__ expert_ids,
                            int* __restrict__ num_tokens_post_pad, int* __restrict__ inverse) {
  __shared__ int counts[kMoeMaxExperts];
  __shared__ int running[kMoeMaxExperts];
  __shared__ int warp_counts[32][kMoeMaxExperts];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < sorted_cap; i += blockDim.x) sorted_ids[i] = n;
  for (int e = tid; e < E; e += blockDim.x) counts[e] = 0;
  for (int i = tid; i < 32 * kMoeMaxExperts; i += blockDim.x) (&warp_counts[0][0])[i] = 0;
  __syncthreads();
  for (int i = tid; i < n; i += blockDim.x) {
    const long long e = (long long)ids[i];
    if (e >= 0 && e < E) atomicAdd(&counts[int(e)], 1);
  }
  __syncthreads();
  if (tid == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) {
      running[e] = at;
      at += (counts[e] + block_size - 1) / block_size * block_size;
    }
    *num_tokens_post_pad = at;
  }
  __syncthreads();
  for (int e = tid; e < E; e += blockDim.x) {
    const int b0 = running[e] / block_size, nb = (counts[e] + block_size - 1) / block_size;
    for (int b = 0; b < nb; ++b) expert_ids[b0 + b] = e;
  }
  // Stable scatter, one chunk of blockDim elements at a time: position = start of the expert +
  // elements of that expert in earlier chunks + in lower warps of this chunk + in lower lanes.
  for (int base = 0; base < n; base += blockDim.x) {
    const int i = base + tid;
    long long e64 = (i < n) ? (long long)ids[i] : -1;
    const int e = (e64 >= 0 && e64 < E) ? int(e64) : -1;
    const unsigned same = __match_any_sync(0xffffffffu, e);
    const int rank = __popc(same & ((1u << lane) - 1u));
    if (e >= 0 && rank == 0) warp_counts[warp][e] = __popc(same);
    __syncthreads();
    if (e >= 0) {
      int at = running[e] + rank;
      for (int w = 0; w < warp; ++w) at += warp_counts[w][e];
      sorted_ids[at] = i;
      if (inverse) inverse[i] = at;
    } else if (i < n && inverse) {
      inverse[i] = -1;
    }
    __syncthreads();
    for (int x = tid; x < E; x += blockDim.x) {
      int s = 0;
      for (int w = 0; w < 32; ++w) {
        s += warp_counts[w][x];
        warp_counts[w][x] = 0;
      }
      running[x] += s;
    }
    __syncthreads();
  }
}

// dst[p, :] = src[sorted_ids[p] / top_k, :] for sorted_ids[p] < n_valid, zero otherwise. Rows are
// row_bytes long; one warp per row. vec: bases, pitches and row_bytes are multiples of 16 bytes.
__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(const uint8_t* __restrict__ src, long long src_pitch, int row_bytes,
                       const int* __restrict__ sorted_ids, int num_rows, int n_valid, int top_k,
                       uint8_t* __restrict__ dst, long long dst_pitch, int vec) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= num_rows) return;
  const int lane = threadIdx.x & 31;
  const int id = sorted_ids[row];
  const bool real = id >= 0 && id < n_valid;
  const uint8_t* s = src + (long long)(real ? id / top_k : 0) * src_pitch;
  uint8_t* d = dst + (long long)row * dst_pitch;
  if (vec) {
    const int nvec = row_bytes >> 4;
    for (int v = lane; v < nvec; v += 32)
      reinterpret_cast<uint4*>(d)[v] = real ? reinterpret_cast<const uint4*>(s)[v] : make_uint4(0u, 0u, 0u, 0u);
  } else {
    for (int v = lane; v < row_bytes; v += 32) d[v] = real ? s[v] : uint8_t(0);
  }
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
  reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
  *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]),
                                            pack_bf16x2(v[6], v[7]));
}

// y = x1 / (1 + exp(-x1)) * x2 in f32. Four lanes share 32 consecutive columns (8 each), as in the
// quantiser; `out` (same type as the inputs, may be null) gets y rounded once; q / scales (may be
// null; need n % 32 == 0) get y quantised to MXFP4 from the f32 value, not from the rounded one.
// VEC: all three matrices have 16-byte aligned bases and pitches, so 8 values move as one or two accesses.
// Every group of 4 lanes works on kSiluUnroll consecutive blocks of 32 columns and issues all their
// loads before any arithmetic. grid (rows, ceil(nblocks / (64 U))): a CTA covers 64 U blocks of one row.
constexpr int kSiluUnroll = 2;
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
silu_and_mul_kernel(const T* __restrict__ x1, const T* __restrict__ x2, long long ld1, long long ld2, int rows, int n,
                    T* __restrict__ out, long long ldo, uint8_t* __restrict__ q, uint8_t* __restrict__ scale_rm,
                    uint8_t* __restrict__ scale_packed, int k_atoms, const int* __restrict__ row_limit) {
  constexpr int U = kSiluUnroll;
  // rows at or past *row_limit (a device value: the padded row count of a routed batch) are left alone
  if (row_limit) rows = min(rows, __ldg(row_limit));
  const int g0 = blockIdx.y * 64 + (threadIdx.x >> 2);
  const int sub = threadIdx.x & 3;
  const int nblocks = (n + 31) >> 5;
  const int r = blockIdx.x;
  bool active[U], full[U];
  float g[U][8], u[U][8];
#pragma unroll
  for (int i = 0; i < U; ++i) {
    const int kb = g0 * U + i;
    active[i] = r < rows && kb < nblocks;
    const int c0 = kb * 32 + sub * 8;
    full[i] = VEC && c0 + 8 <= n;
#pragma unroll
    for (int j = 0; j < 8; ++j) g[i][j] = u[i][j] = 0.f;
    if (active[i]) {
      const T* p1 = x1 + (long long)r * ld1 + c0;
      const T* p2 = x2 + (long long)r * ld2 + c0;
      if (full[i]) {
        load8(p1, g[i]);
        load8(p2, u[i]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (c0 + j < n) { g[i][j] = to_f32<T>(p1[j]); u[i][j] = to_f32<T>(p2[j]); }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < U; ++i) {
    const int kb = g0 * U + i;
    const int c0 = kb * 32 + sub * 8;
    float y[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) y[j] = __fdividef(g[i][j], 1.0f + __expf(-g[i][j])) * u[i][j];  // ~1e-6 relative
    if (out && active[i]) {
      T* po = out + (long long)r * ldo + c0;
      if (full[i]) {
        store8(po, y);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (c0 + j < n) po[j] = from_f32<T>(y[j]);
      }
    }
    if (q) mxfp4_encode_group<8>(y, active[i], r, kb, sub, n, nblocks, k_atoms, q, scale_rm, scale_packed);
  }
}

// out[t, c] = sum_j weight[t * top_k + j] * y[row_of[t * top_k + j], c], accumulated in f32 in slot
// order; pairs with row_of < 0 are skipped. One thread per (token, 4 columns).
template <typename T>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const T* __restrict__ y, long long ldy, const int* __restrict__ row_of,
                   const float* __restrict__ weight, int tokens, int top_k, int cols, T* __restrict__ out,
                   long long ldo) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int cvec = (cols + 3) >> 2;
  if (idx >= (long long)tokens * cvec) return;
  const int t = int(idx / cvec);
  const int c0 = int(idx - (long long)t * cvec) * 4;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int j = 0; j < top_k; ++j) {
    const int row = row_of[t * top_k + j];
    if (row < 0) continue;
    const float w = weight[t * top_k + j];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (c0 + i < cols) acc[i] += w * to_f32<T>(y[(long long)row * ldy + c0 + i]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (c0 + i < cols) out[(long long)t * ldo + c0 + i] = from_f32<T>(acc[i]);
}

// out[i] = slots[0][i] + slots[1][i] + ... in slot order (f32), rounded once to the output type: the
// reduction step of the K-sharded GEMM, whose ranks deposit f32 partial tiles in one slot each.
template <typename T>
__global__ void __launch_bounds__(256)
sum_slots_kernel(const float* __restrict__ slots, int num_slots, long long slot_stride, long long count, T* __restrict__ out) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= count) return;
  if (i + 4 <= count) {
    float4 acc = *reinterpret_cast<const float4*>(slots + i);
    for (int s = 1; s < num_slots; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(slots + s * slot_stride + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if constexpr (sizeof(T) == 4) {
      *reinterpret_cast<float4*>(out + i) = acc;
    } else {
      *reinterpret_cast<uint2*>(out + i) = make_uint2(pack_bf16x2(acc.x, acc.y), pack_bf16x2(acc.z, acc.w));
    }
  } else {
    for (long long j = i; j < count; ++j) {
      float acc = slots[j];
      for (int s = 1; s < num_slots; ++s) acc += slots[s * slot_stride + j];
      out[j] = from_f32<T>(acc);
    }
  }
}

// c[r, :] (+)= slots[0][r, :] + slots[1][r, :] + ... in slot order (f32), rounded once to the output type:
// the reduction of the tile path's split-K. Slots are dense [M, N] f32 matrices; c has row pitch ldc.
template <typename T>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ slots, int num_slots, long long slot_stride, int M, int N, T* __restrict__ c,
                     long long ldc, int accumulate) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int nvec = (N + 3) >> 2;
  if (idx >= (long long)M * nvec) return;
  const int r = int(idx / nvec), c0 = int(idx - (long long)r * nvec) * 4;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const float* src = slots + (long long)r * N + c0;
  if (c0 + 4 <= N && (N & 3) == 0) {
    for (int s = 0; s < num_slots; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(src + s * slot_stride);
      acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
    }
  } else {
    for (int s = 0; s < num_slots; ++s)
      for (int j = 0; j < 4; ++j)
        if (c0 + j < N) acc[j] += src[s * slot_stride + j];
  }
  T* dst = c + (long long)r * ldc + c0;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (c0 + j < N) dst[j] = from_f32<T>(accumulate ? acc[j] + to_f32<T>(dst[j]) : acc[j]);
}

}  // namespace wb
