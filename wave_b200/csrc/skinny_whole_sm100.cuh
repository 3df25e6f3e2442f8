// Skinny (M <= 128) MXFP4 / MXFP8 GEMM, whole-tile variant: used when there are at least as many 128-row
// N tiles as SMs and the last wave of tiles is not tiny.
//
// Same operand swap and per-stage pipeline as skinny_sm100.cuh (tensor-memory lanes = 128 weight rows,
// accumulator columns = the M activation rows padded to NP; TMA ring; tcgen05.mma kind::mxf4 / mxf8f6f4),
// but the work is not cut along K at all. One CTA per SM takes whole N tiles from ONE atomic counter (its
// first tile is its own index, so the first loads need no round trip), streams the tile's whole K through
// the ring, and writes C directly. This is the data-parallel half of the reference's hybrid stream-K GEMM
// (wave_lang/kernel/wave/templates/gemm.py:538-1366) with the remainder balanced by dealing instead of by
// cutting K:
//   * no partial tiles, so no workspace traffic, no fix-up, no memory fences, and a result that is
//     accumulated in one place in K order: bit-identical from run to run whichever CTA takes a tile;
//   * an SM whose share of the memory system is slower simply takes fewer tiles; while the second wave
//     runs on the SMs that came back first, each of them pulls well over its 1/148 share of HBM, so the
//     total stays bandwidth-bound (measured: M = 128, N = 28672, K = 8192 in 28.6 us against 36 us for the
//     K-split kernel, whose 64 KB partial tiles cost it 5-15 us of epilogue; M <= 16: the same 24 us);
//   * the epilogue transposes 16-row chunks of the accumulator through shared memory; a chunk leaves through one
//     TMA store, or, where C is accumulated into or not 16-byte aligned, as 16 bytes per thread along n.
// The producer hands the tile numbers to the MMA and epilogue warps through a small queue in shared
// memory (mbarrier-guarded), since only it talks to the counter.
#pragma once
#include "ptx.cuh"
#include "skinny_sm100.cuh"
#include <cuda_bf16.h>

namespace wb {

constexpr int kWholeWorkCounter = 1023;  // counters[1023]: the tile dispenser (the K-split kernel uses counters[tile], tile < SMs)
constexpr int kWholeItemQueue = 8;       // depth of the in-CTA queue of tile numbers

// SBUFS: staging buffers of the epilogue (2: a chunk is staged while the one before is still being stored; 1 where the
// ring needs the room).
template <int NP_, int STAGES_, int EB = 4, int WR = 128, int SBUFS = 2>
struct SkinnyWholeCfg {
  using Base = SkinnyCfg<NP_, STAGES_, EB, WR>;
  static_assert(SBUFS == 1 || SBUFS == 2, "one or two staging buffers");
  static constexpr int STAGE_BYTES = Base::STAGE_BYTES;
  static constexpr int STAGING_BUF_BYTES = 16 * 128 * 4;  // 16 output rows x 128 columns of f32
  static constexpr int STAGING_BYTES = SBUFS * STAGING_BUF_BYTES;
  static constexpr int NUM_BARRIERS = 2 * STAGES_ + 4 + 2 * kWholeItemQueue;
  static constexpr int MISC_BYTES = 64 + kWholeItemQueue * 4;
  static constexpr int SMEM_BYTES = 1024 + STAGES_ * STAGE_BYTES + STAGING_BYTES + NUM_BARRIERS * 8 + MISC_BYTES;
  static_assert(SMEM_BYTES <= 232448, "over the dynamic shared memory a CTA may ask for");
};

struct SkinnyWholeParams {
  void* c;
  unsigned int* counters;  // zero before the first launch; the kernel leaves them zero
  int M, N, K;
  int ldc;
  int tiles_n;   // ceil(N / tile_rows)
  int tile_rows; // weight rows per tile: 128, or fewer (a multiple of 8) when the weight scales were packed per tile of
                 // that height (wb200_repack_scales_tiled) so that every SM gets the same number of tiles
  int num_kb;    // ceil(K / BK)
  int accumulate;
  int dependent;
  int elem_format;
  int c_vec;     // C's base and row pitch allow 16-byte accesses
  int tma_store; // write C with TMA stores from the staged chunk (needs c_vec, no accumulate, a staging buffer pair that
                 // holds two chunks in the output type)
  int* status;
};

template <int NP, int STAGES, typename OutT, int EB = 4, int WR = 128, int SBUFS = 2>
__global__ void __launch_bounds__(192, 1)
mxfp4_skinny_whole_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                          const __grid_constant__ CUtensorMap tmSFW, const __grid_constant__ CUtensorMap tmSFX,
                          const __grid_constant__ CUtensorMap tmC, const SkinnyWholeParams p) {
  using Base = SkinnyCfg<NP, STAGES, EB, WR>;
  using Cfg = SkinnyWholeCfg<NP, STAGES, EB, WR, SBUFS>;
  constexpr int IQ = kWholeItemQueue;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  pdl_launch_dependents();  // a kernel launched behind this one as a programmatic dependent may take SMs as they free up
#ifdef WB200_TRACE
  if (threadIdx.x == 0) WB_TRACE_SET(0, trace_now());  // timeline marks as in skinny_sm100.cuh; a "segment" is a tile here
#endif
  if (warp == 0 && lane < 4)  // the copy engine fetches a descriptor on first use: start that now
    prefetch_tensormap(lane == 0 ? &tmW : lane == 1 ? &tmSFW : lane == 2 ? &tmX : &tmSFX);
  if (warp == 2 && lane == 0 && p.tma_store) prefetch_tensormap(&tmC);

  const uint32_t staging_base = smem_base + STAGES * Cfg::STAGE_BYTES;
  const uint32_t bar_base = staging_base + Cfg::STAGING_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto acc_full_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
  auto acc_empty_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + 2 + s); };
  auto item_full_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + 4 + s); };
  auto item_empty_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + 4 + IQ + s); };
  uint32_t* misc = reinterpret_cast<uint32_t*>(smem_gen + STAGES * Cfg::STAGE_BYTES + Cfg::STAGING_BYTES + Cfg::NUM_BARRIERS * 8);
  uint32_t* tmem_slot = misc;
  volatile uint32_t* abort_flag = misc + 1;
  volatile int* item_q = reinterpret_cast<volatile int*>(misc + 16);
  WaitCtx ctx{abort_flag, p.status};

  if (warp == 0) {
    // the barriers, dealt over the lanes; arrival counts by kind
    for (int b = lane; b < Cfg::NUM_BARRIERS; b += 32) {
      uint32_t count = 1;                                  // full / empty stage, accumulator full, tile number written
      const int q = b - 2 * STAGES;
      if (q >= 2 && q < 4) count = 4;                       // accumulator drained: one arrival per epilogue warp
      else if (q >= 4 + IQ && q < 4 + 2 * IQ) count = 5;    // tile number read by the MMA warp and the four epilogue warps
      mbar_init(bar_base + 8u * b, count);
    }
    if (lane == 0) *abort_flag = 0u;
    fence_mbar_init();
    __syncwarp();
  }

  // Consumers' side of the queue: entry number `seq` (a tile number, or -1 for "no more"), freed as soon as it is read.
  auto next_tile = [&](int seq) -> int {
    const int s = seq & (IQ - 1);
    mbar_wait(item_full_bar(s), uint32_t(seq / IQ) & 1u, ctx, WB_DEV_TIMEOUT_MMA_FULL);
    const int tile = (*abort_flag) ? -1 : item_q[s];
    __syncwarp();
    if (lane == 0) mbar_arrive(item_empty_bar(s));
    return tile;
  };

  // ---------------------------------------------------------------------------------- producer state
  uint32_t p_stage = 0, p_phase = 0;
  uint64_t stream_policy = 0, keep_policy = 0;
  // part 0: all four loads of a stage; part 1: only the weights and their scales (no arrival on the barrier
  // yet); part 2: the arrival with the stage's byte count plus the activations and their scales.
  auto load_stage = [&](int tile, int kb, uint32_t stage, int part) {
    const uint32_t sW = smem_base + stage * Cfg::STAGE_BYTES;
    const uint32_t sX = sW + Base::W_BYTES;
    const uint32_t sSFW = sX + Base::X_BYTES;
    const uint32_t sSFX = sSFW + Base::SF_BYTES;
    const uint32_t fb = full_bar(stage);
    if (elect_one()) {
      // a tile of fewer than 128 rows fills the head of the stage's weight area; the MMA still multiplies 128 rows
      // (whatever bits the rest holds: every E2M1 code is finite, the scales of those lanes are the padding byte)
      // and the epilogue keeps the tile's own columns
      // (4-bit weights expanded by the copy engine, EB == 8 only, count with their packed size: 64 bytes per row)
      if (part != 1)
        mbar_expect_tx(fb, Cfg::STAGE_BYTES - Base::W_BYTES + uint32_t(p.tile_rows) * ((EB == 8 && (p.elem_format & 0x10)) ? 64u : 128u));
      if (part != 2) {
        tma_load_2d_hint(sW, &tmW, kb * 128, tile * p.tile_rows, fb, stream_policy);
        tma_load_2d(sSFW, &tmSFW, kb * (Base::SF_ATOMS * 128), tile, fb);
      }
      if (part != 1) {
        tma_load_2d_hint(sX, &tmX, kb * 128, 0, fb, keep_policy);
        tma_load_2d(sSFX, &tmSFX, kb * (Base::SF_ATOMS * 128), 0, fb);
      }
    }
    __syncwarp();
  };
  // Warp 0 has just initialised the barriers: it starts the first ring of loads of this CTA's first tile (its own
  // index) right away, before the CTA-wide synchronisation that waits for the tensor-memory allocation. When the
  // kernel was launched as a programmatic dependent, only the weight loads go out now; the activation loads follow
  // the dependency wait.
  int head = 0;
  if (warp == 0) {
    stream_policy = l2_policy_evict_first();  // weights are read once
    keep_policy = l2_policy_evict_last();     // activations are re-read by every CTA
    head = min(STAGES, p.num_kb);
    for (int i = 0; i < head; ++i) load_stage(int(blockIdx.x), i, uint32_t(i), p.dependent ? 1 : 0);
#ifdef WB200_TRACE
    if (lane == 0) WB_TRACE_SET(4, trace_now());
#endif
  }
  if (warp == 1) {
    tmem_alloc<1>(smem_u32(tmem_slot), Base::TMEM_COLS);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // The whole warp walks the loop; one elected lane issues the copies.
    if (p.dependent) pdl_wait();  // the activations' scales, and the counter, belong to the kernels before this one until now
    int seq = 0;
    auto emit = [&](int tile) {
      const int s = seq & (IQ - 1);
      if (seq >= IQ) mbar_wait(item_empty_bar(s), uint32_t(seq / IQ - 1) & 1u, ctx, WB_DEV_TIMEOUT_PRODUCER);
      if (lane == 0) {
        item_q[s] = tile;
        mbar_arrive(item_full_bar(s));  // release: the entry is visible to whoever sees the phase complete
      }
      __syncwarp();
      ++seq;
    };
    auto run_tile = [&](int tile) {
      emit(tile);
      for (int kb = 0; kb < p.num_kb; ++kb) {
        if (head > 0) {  // this stage's weights are already on their way
          --head;
          if (p.dependent) load_stage(tile, kb, p_stage, 2);
        } else {
          mbar_wait(empty_bar(p_stage), p_phase ^ 1u, ctx, WB_DEV_TIMEOUT_PRODUCER);
          load_stage(tile, kb, p_stage, 0);
        }
        if (++p_stage == STAGES) { p_stage = 0; p_phase ^= 1u; }
      }
    };
    run_tile(int(blockIdx.x));
    // Further tiles: one atomic per tile, drawn only when the loads of the previous tile are all issued (drawing
    // ahead would commit this CTA to a tile that a faster CTA could take); the loads in the ring cover the round trip.
    const int dealt = p.tiles_n - int(gridDim.x);
    unsigned int* work = p.counters + kWholeWorkCounter;
    for (;;) {
      unsigned int raw = 0;
      if (lane == 0) raw = atomicAdd(work, 1u);
      raw = __shfl_sync(0xffffffffu, raw, 0);
      if (raw >= (unsigned int)dealt || *abort_flag) {
        // every CTA draws exactly one value past the end; the last of them leaves the counter at zero
        if (lane == 0 && raw == (unsigned int)(dealt + int(gridDim.x) - 1)) *work = 0u;
        break;
      }
      run_tile(int(gridDim.x) + int(raw));
    }
#ifdef WB200_TRACE
    if (lane == 0) WB_TRACE_SET(2, (unsigned long long)seq);
#endif
    emit(-1);
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t idesc = (EB == 4) ? make_idesc_mxf4(128, NP) : make_idesc_mxf8(128, NP, weight_format_of(p.elem_format), act_format_of(p.elem_format));
    uint32_t stage = 0, phase = 0, sf_set = 0;
    for (int seq = 0;; ++seq) {
      const int tile = next_tile(seq);
      if (tile < 0) break;
      const int as = seq & 1;
      if (seq >= 2)
        mbar_wait(acc_empty_bar(as), uint32_t((seq - 2) >> 1) & 1u, ctx, WB_DEV_TIMEOUT_MMA_ACC);
      tc_fence_after_sync();
      const uint32_t d_tmem = tmem_base + (as ? Base::ACC_COL1 : 0);
      for (int kb = 0; kb < p.num_kb; ++kb) {
        const uint32_t t_sfw = tmem_base + Base::SF_COL + sf_set * 16;
        const uint32_t t_sfx = t_sfw + 8;
        if (++sf_set == Base::SF_SETS) sf_set = 0;
        mbar_wait(full_bar(stage), phase, ctx, WB_DEV_TIMEOUT_MMA_FULL);
        tc_fence_after_sync();
#ifdef WB200_TRACE
        if (lane == 0) {
          if (seq == 0 && kb == 0) WB_TRACE_SET(3, trace_now());
          if (kb == p.num_kb - 1) { WB_TRACE_SEG(seq, 0, (unsigned long long)tile); WB_TRACE_SEG(seq, 1, trace_now()); }
        }
#endif
        const uint32_t sW = smem_base + stage * Cfg::STAGE_BYTES;
        const uint32_t sX = sW + Base::W_BYTES;
        const uint32_t sSFW = sX + Base::X_BYTES;
        const uint32_t sSFX = sSFW + Base::SF_BYTES;
        const uint64_t w_desc = make_desc_k_sw128(sW);
        const uint64_t x_desc = make_desc_k_sw128(sX);
        const uint64_t sfw_desc = make_desc_sf_atom(sSFW);
        const uint64_t sfx_desc = make_desc_sf_atom(sSFX);
        if (elect_one()) {
#pragma unroll
          for (int a = 0; a < Base::SF_ATOMS; ++a) {
            utccp_sf_atom<1>(t_sfw + a * 4, sfw_desc + uint64_t(a * 32));
            utccp_sf_atom<1>(t_sfx + a * 4, sfx_desc + uint64_t(a * 32));
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if constexpr (EB == 4)
              mma_mxf4<1>(d_tmem, w_desc + uint64_t(k * 2), x_desc + uint64_t(k * 2),
                          idesc_with_sf_id(idesc, (k & 1) * 2), t_sfw + (k >> 1) * 4, t_sfx + (k >> 1) * 4,
                          (kb > 0 || k > 0) ? 1u : 0u);
            else  // 32 8-bit values per instruction, one scale each: byte k of the atom's column
              mma_mxf8<1>(d_tmem, w_desc + uint64_t(k * 2), x_desc + uint64_t(k * 2), idesc_with_sf_id(idesc, k), t_sfw,
                          t_sfx, (kb > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit<1>(empty_bar(stage));
          if (kb == p.num_kb - 1) tc_commit<1>(acc_full_bar(as));
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps 2..5
    const int quad = warp & 3;
    const int nl = quad * 32 + lane;      // weight row inside the tile = tensor-memory lane
    const int t = int(threadIdx.x) - 64;  // 0..127
    if (p.dependent) pdl_wait();  // C may still be read by the kernels before this one
    OutT* __restrict__ C = reinterpret_cast<OutT*>(p.c);
    // Every thread owns two 32-byte pieces of a 16-row chunk: rows (t / 16) and (t / 16) + 8, columns 8 (t % 16) .. + 7.
    const int prow = t >> 4, pcol = (t & 15) * 8;
    const int nchunks = (p.M + 15) >> 4;  // 16-row chunks of the accumulator that hold real output rows
    uint32_t chunk_ctr = 0;
    for (int seq = 0;; ++seq) {
      const int tile = next_tile(seq);
      if (tile < 0) break;
      const int as = seq & 1;
      const int n = tile * p.tile_rows + pcol;  // first of this thread's eight columns
      const bool keep = pcol < p.tile_rows;     // tile_rows is a multiple of 8: a piece is all inside or all outside
      mbar_wait(acc_full_bar(as), uint32_t(seq >> 1) & 1u, ctx, WB_DEV_TIMEOUT_EPILOGUE);
      tc_fence_after_sync();
#ifdef WB200_TRACE
      if (t == 0) WB_TRACE_SEG(seq, 2, trace_now());
#endif
      const uint32_t t_acc = tmem_base + (uint32_t(quad * 32) << 16) + (as ? Base::ACC_COL1 : 0);
      if (p.tma_store) {
        // Every 16-row chunk is transposed into a dense [16][tile_rows] block of the output type in one of two
        // staging buffers and leaves through one TMA store (clipped at M and N by the copy engine). The stores are
        // asynchronous: no thread waits for global memory, only, before a buffer is staged again, for the store
        // that last read it to have read it (checked by the issuing thread ahead of the chunk's barrier).
        constexpr uint32_t kHalf = uint32_t(Cfg::STAGING_BYTES) / 2;
        const uint32_t pitch = uint32_t(p.tile_rows) * uint32_t(sizeof(OutT));
#pragma unroll 1
        for (int ch = 0; ch < nchunks; ++ch) {
          uint32_t r[16];
          tmem_ld_32x16(t_acc + ch * 16, r);
          tmem_ld_wait();
          if (ch == nchunks - 1) {  // accumulator fully read: hand it back to the MMA warp
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty_bar(as));
          }
          const uint32_t buf = staging_base + (chunk_ctr & 1u) * kHalf;
          ++chunk_ctr;
          if (nl < p.tile_rows) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const uint32_t dst = buf + uint32_t(j) * pitch + uint32_t(nl) * uint32_t(sizeof(OutT));
              if constexpr (sizeof(OutT) == 4) {
                asm volatile("st.shared.b32 [%0], %1;" ::"r"(dst), "r"(r[j]) : "memory");
              } else {
                const uint16_t h = __bfloat16_as_ushort(__float2bfloat16_rn(__uint_as_float(r[j])));
                asm volatile("st.shared.b16 [%0], %1;" ::"r"(dst), "h"(h) : "memory");
              }
            }
          }
          fence_proxy_async_smem();
          if (t == 0) bulk_wait_group_read<0>();  // the previous chunk's store has read the other buffer
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (t == 0) {
            tma_store_2d(&tmC, buf, tile * p.tile_rows, ch * 16);
            bulk_commit_group();
          }
        }
#ifdef WB200_TRACE
        if (t == 0) WB_TRACE_SEG(seq, 3, trace_now() | (1ull << 63));
#endif
        continue;
      }
#pragma unroll 1
      for (int ch = 0; ch < nchunks; ++ch) {
        const int c0 = ch * 16;
        uint32_t r[16];
        tmem_ld_32x16(t_acc + c0, r);
        tmem_ld_wait();
        if (ch == nchunks - 1) {  // accumulator fully read: hand it back to the MMA warp
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_empty_bar(as));
        }
        // transpose through shared memory: staging[m][n], one 512-byte row per output row of the chunk
        const uint32_t buf = staging_base + (SBUFS == 2 ? (chunk_ctr & 1u) : 0u) * uint32_t(Cfg::STAGING_BUF_BYTES);
        ++chunk_ctr;
#pragma unroll
        for (int j = 0; j < 16; ++j)
          asm volatile("st.shared.b32 [%0], %1;" ::"r"(buf + uint32_t(j * 128 + nl) * 4u), "r"(r[j]) : "memory");
        asm volatile("bar.sync 1, 128;" ::: "memory");
        // (the buffer is written again two chunks from now; the barrier of the chunk in between orders that write
        // after the reads below)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int mi = prow + 8 * i;
          const int m = c0 + mi;
          if (m >= p.M || n >= p.N || !keep) continue;
          const uint32_t src = buf + uint32_t(mi * 128 + pcol) * 4u;
          float4 lo, hi;
          asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(lo.x), "=f"(lo.y), "=f"(lo.z), "=f"(lo.w) : "r"(src) : "memory");
          asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(hi.x), "=f"(hi.y), "=f"(hi.z), "=f"(hi.w) : "r"(src + 16u) : "memory");
          OutT* dst = C + size_t(m) * p.ldc + n;
          if (!WB_CHECK(m >= 0 && m < p.M && n >= 0 && n < p.N, kCheckOutputIndex, (long long)m << 32 | unsigned(n))) continue;
          if (p.c_vec && n + 8 <= p.N) {
            if constexpr (sizeof(OutT) == 4) {
              float4* d4 = reinterpret_cast<float4*>(dst);
              if (p.accumulate) {
                const float4 o0 = d4[0], o1 = d4[1];
                lo.x += o0.x; lo.y += o0.y; lo.z += o0.z; lo.w += o0.w;
                hi.x += o1.x; hi.y += o1.y; hi.z += o1.z; hi.w += o1.w;
              }
              d4[0] = lo;
              d4[1] = hi;
            } else {
              uint4* d4 = reinterpret_cast<uint4*>(dst);
              if (p.accumulate) {
                const uint4 o = *d4;
                lo.x += __uint_as_float(o.x << 16); lo.y += __uint_as_float(o.x & 0xffff0000u);
                lo.z += __uint_as_float(o.y << 16); lo.w += __uint_as_float(o.y & 0xffff0000u);
                hi.x += __uint_as_float(o.z << 16); hi.y += __uint_as_float(o.z & 0xffff0000u);
                hi.z += __uint_as_float(o.w << 16); hi.w += __uint_as_float(o.w & 0xffff0000u);
              }
              *d4 = make_uint4(pack_bf16x2(lo.x, lo.y), pack_bf16x2(lo.z, lo.w), pack_bf16x2(hi.x, hi.y), pack_bf16x2(hi.z, hi.w));
            }
          } else {
            const float e[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
            for (int k = 0; k < 8; ++k) {
              if (n + k >= p.N) break;
              if constexpr (sizeof(OutT) == 4) dst[k] = p.accumulate ? dst[k] + e[k] : e[k];
              else dst[k] = __float2bfloat16_rn(p.accumulate ? __bfloat162float(dst[k]) + e[k] : e[k]);
            }
          }
        }
        // one staging buffer: every thread has read its pieces before the next chunk is staged
        if constexpr (SBUFS == 1) asm volatile("bar.sync 1, 128;" ::: "memory");
      }
#ifdef WB200_TRACE
      if (t == 0) WB_TRACE_SEG(seq, 3, trace_now() | (1ull << 63));
#endif
    }
  }

  if (threadIdx.x == 64 && p.tma_store) bulk_wait_group<0>();  // this thread's stores have left shared memory and landed
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, Base::TMEM_COLS);
  }
#ifdef WB200_TRACE
  if (threadIdx.x == 0) WB_TRACE_SET(1, trace_now());
#endif
}

}  // namespace wb
