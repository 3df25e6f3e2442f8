// Skinny (M <= 128) MXFP4 GEMM for sm_100a: the weight-streaming, HBM-bound regime.
//
// Takes the role of the reference's split-K template
// (wave_lang/kernel/wave/templates/tagged_mxfp4_gemm.py:611-816: grid z = num_splits, partial
// accumulators added into C with atomics) with two differences that the 1-ulp bf16 bar needs:
// partial sums stay in f32 and are added in a fixed order, so the result does not depend on
// arrival order and C needs no zero-initialisation.
//
//   * operands are swapped, as the reference's wide-store variant does
//     (tagged_mxfp4_gemm.py:538-583): the 128 accumulator rows (tensor-memory lanes) hold 128
//     weight rows n, the accumulator columns hold the M activation rows padded to NP in
//     {16, 32, 64, 128}; a warp then writes 32 consecutive n of one output row at a time;
//   * stream-K: the (N tile x K block) units are split evenly over one CTA per SM, each CTA
//     streams a contiguous run of units through a deep TMA pipeline so that b is read exactly
//     once at full bandwidth;
//   * a CTA whose run covers a whole tile writes C directly; otherwise it writes an f32 partial
//     to the workspace and bumps the tile's counter; the CTA that arrives last adds the partials
//     in CTA order, converts once and writes C. A CTA that finds all other contributions already
//     published skips the write of its own. Nobody spins on another CTA.
#pragma once
#include "ptx.cuh"
#include <cuda_bf16.h>

namespace wb {

// Per-CTA timeline of a launch, compiled in with -DWB200_TRACE only (`python -m wave_b200.build --trace`): a
// measurement aid that writes globaltimer marks to a device array which wb200_trace_read copies out. Words per CTA:
// [0] entry, [1] exit, [2] segments, [3] first stage landed, [4] first ring of loads issued, then per segment (up to
// kTraceSegments): tile, last stage landed, accumulator seen complete by the epilogue, epilogue done (bit 62: this CTA
// knew it was last and reduced from registers; bit 63: whole tile).
#ifdef WB200_TRACE
constexpr int kTraceSegments = 8;
constexpr int kTraceHead = 8;
constexpr int kTraceWords = kTraceHead + 4 * kTraceSegments;
__device__ unsigned long long g_skinny_trace[256 * kTraceWords];
__device__ __forceinline__ unsigned long long trace_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define WB_TRACE_SET(idx, val) do { g_skinny_trace[size_t(blockIdx.x) * kTraceWords + (idx)] = (val); } while (0)
#define WB_TRACE_SEG(seg, field, val) do { if ((seg) < kTraceSegments) g_skinny_trace[size_t(blockIdx.x) * kTraceWords + kTraceHead + 4 * (seg) + (field)] = (val); } while (0)
#else
#define WB_TRACE_SET(idx, val) do { } while (0)
#define WB_TRACE_SEG(seg, field, val) do { } while (0)
#endif

// EB: bits per operand element, 4 (MXFP4) or 8 (MXFP8); a stage is one 128-byte swizzle row of every operand row
// either way: 256 or 128 K elements, 2 or 1 scale-factor atoms per 128 rows.
// WR: weight rows a stage has room for. 128 = a whole MMA tile; the whole-tile kernel also runs with 104 when its tiles
// are at most 104 rows high (the MMA then reads the rows above from the bytes that follow in the stage, which it never
// keeps), so that the ring holds more stages.
template <int NP_, int STAGES_, int EB = 4, int WR = 128>
struct SkinnyCfg {
  static_assert(EB == 4 || EB == 8, "operand elements are 4 or 8 bits");
  static_assert(WR % 8 == 0 && WR >= 64 && WR <= 128, "weight rows per stage: whole 8-row swizzle groups");
  static constexpr int NP = NP_;  // padded M = MMA N
  static constexpr int STAGES = STAGES_;
  static constexpr int BK = 1024 / EB;
  static constexpr int SF_ATOMS = BK / 128;
  static constexpr int W_BYTES = WR * 128;
  static constexpr int X_BYTES = NP * 128;
  static constexpr int SF_BYTES = SF_ATOMS * 512;
  static constexpr int STAGE_BYTES = W_BYTES + X_BYTES + 2 * SF_BYTES;
  static constexpr int NUM_BARRIERS = 2 * STAGES + 4;
  static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + NUM_BARRIERS * 8 + 64;
  static constexpr int TMEM_COLS = 512;
  static constexpr int ACC_COL1 = NP;
  // ring of scale-factor column sets (8 columns for the weights, 8 for the activations each), so
  // that the tcgen05.cp of one unit does not wait for the MMAs of the previous unit
  static constexpr int SF_COL = 256;
  static constexpr int SF_SETS = 8;
  static_assert(STAGE_BYTES % 1024 == 0, "stages must keep the 1024-byte swizzle alignment");
};

constexpr int kSkinnyCounterWords = 4096;  // 32-bit tile counters at the head of every workspace

struct SkinnyParams {
  void* c;
  float* partials;         // [2 * gridDim.x][M][128] f32
  unsigned int* counters;  // [tiles_n], zero before the first launch; the kernel re-zeroes them
  int M, N, K;
  int ldc;
  int tiles_n;   // ceil(N / 128)
  int num_kb;    // ceil(K / 256)
  int accumulate;  // add to the values already in C instead of overwriting them
  int dependent;   // launched as the programmatic dependent of the kernel that writes the activations' packed scales
  int elem_format; // 8-bit operands only: 0 = E4M3, 1 = E5M2
  int* status;
};

// Units [u0, u1) of CTA c when `total` units are dealt as evenly as possible to `g` CTAs.
__host__ __device__ __forceinline__ void skinny_range(long long total, int g, int c, int& u0, int& u1) {
  u0 = int((total * c) / g);
  u1 = int((total * (c + 1)) / g);
}
// CTA that owns unit u under skinny_range.
__device__ __forceinline__ int skinny_owner(long long total, int g, int u) {
  int c = int(((long long)(u + 1) * g - 1) / total);
  // guard against rounding at the boundaries
  int a, b;
  skinny_range(total, g, c, a, b);
  while (u < a) { --c; skinny_range(total, g, c, a, b); }
  while (u >= b) { ++c; skinny_range(total, g, c, a, b); }
  return c;
}

template <int NP, int STAGES, typename OutT, int EB = 4>
__global__ void __launch_bounds__(192, 1)
mxfp4_skinny_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                    const __grid_constant__ CUtensorMap tmSFW, const __grid_constant__ CUtensorMap tmSFX,
                    const SkinnyParams p) {
  using Cfg = SkinnyCfg<NP, STAGES, EB>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  pdl_launch_dependents();  // a kernel launched behind this one as a programmatic dependent may take SMs as they free up
#ifdef WB200_TRACE
  if (threadIdx.x == 0) WB_TRACE_SET(0, trace_now());
#endif

  const uint32_t bar_base = smem_base + STAGES * Cfg::STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto acc_full_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
  auto acc_empty_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + 2 + s); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + STAGES * Cfg::STAGE_BYTES + Cfg::NUM_BARRIERS * 8);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile uint32_t* last_flag = tmem_slot + 2;
  volatile uint32_t* known_last_flag = tmem_slot + 3;
  WaitCtx ctx{abort_flag, p.status};

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(acc_full_bar(s), 1);
      mbar_init(acc_empty_bar(s), 4);
    }
    *abort_flag = 0u;
    fence_mbar_init();
  }
  const long long total_units = (long long)p.tiles_n * p.num_kb;
  int u0, u1;
  skinny_range(total_units, gridDim.x, blockIdx.x, u0, u1);

  // This CTA's run of units, cut into segments: one per tile it touches, in ascending tile order. A
  // run may start and end in the middle of a tile; those partial segments need the cross-CTA fix-up.
  // (Processing the partial segments first, so that the fix-up overlaps the streaming of the whole
  // tiles, was measured and is slower: 27.1 us against 25.0 us at M = 16, N = 28672, K = 8192.)
  const int nkb = p.num_kb;
  const int first_tile = u0 / nkb;
  const int last_tile = (u1 > u0) ? (u1 - 1) / nkb : first_tile;
  const int nseg = (u1 > u0) ? last_tile - first_tile + 1 : 0;
  const int head_kbs = u0 - first_tile * nkb;
  const int tail_kbe = u1 - last_tile * nkb;
  auto segment = [&](int j, int& tile, int& kbs, int& kbe) {
    tile = first_tile + j;
    kbs = (j == 0) ? head_kbs : 0;
    kbe = (j == nseg - 1) ? tail_kbe : nkb;
  };

  // Producer state. Warp 0 has just initialised the barriers, so it starts the first ring of loads
  // right away, before the CTA-wide synchronisation that waits for the tensor-memory allocation:
  // the weight stream is what bounds this kernel, and its first bytes need not wait for that.
  uint32_t p_stage = 0, p_phase = 0;
  int p_seg = 0, p_tile = 0, p_kb = 0, p_kbe = 0, p_issued = 0;
  if (nseg > 0) segment(0, p_tile, p_kb, p_kbe);
  uint64_t stream_policy = 0, keep_policy = 0;
  // part 0: all four loads of a stage; part 1: only the weights and their scales (no arrival on the barrier
  // yet); part 2: the arrival with the stage's byte count plus the activations and their scales.
  auto produce = [&](int max_units, bool wait_for_slot, int part) {
    while (p_seg < nseg && p_issued < max_units) {
      if (wait_for_slot) mbar_wait(empty_bar(p_stage), p_phase ^ 1u, ctx, WB_DEV_TIMEOUT_PRODUCER);
      const uint32_t sW = smem_base + p_stage * Cfg::STAGE_BYTES;
      const uint32_t sX = sW + Cfg::W_BYTES;
      const uint32_t sSFW = sX + Cfg::X_BYTES;
      const uint32_t sSFX = sSFW + Cfg::SF_BYTES;
      const uint32_t fb = full_bar(p_stage);
      if (elect_one()) {
        // 4-bit weights expanded by the copy engine (EB == 8 only) count with their packed size
        if (part != 1) mbar_expect_tx(fb, Cfg::STAGE_BYTES - ((EB == 8 && (p.elem_format & 0x10)) ? Cfg::W_BYTES / 2 : 0));
        if (part != 2) {
          tma_load_2d_hint(sW, &tmW, p_kb * 128, p_tile * 128, fb, stream_policy);
          tma_load_2d(sSFW, &tmSFW, p_kb * (Cfg::SF_ATOMS * 128), p_tile, fb);
        }
        if (part != 1) {
          tma_load_2d_hint(sX, &tmX, p_kb * 128, 0, fb, keep_policy);
          tma_load_2d(sSFX, &tmSFX, p_kb * (Cfg::SF_ATOMS * 128), 0, fb);
        }
      }
      __syncwarp();
      ++p_issued;
      if (++p_kb == p_kbe) {
        if (++p_seg < nseg) segment(p_seg, p_tile, p_kb, p_kbe);
      }
      if (++p_stage == STAGES) { p_stage = 0; p_phase ^= 1u; }
    }
  };
  if (warp == 0) {
    __syncwarp();  // lane 0 initialised the barriers above
    stream_policy = l2_policy_evict_first();  // weights are read once
    keep_policy = l2_policy_evict_last();     // activations are re-read by every CTA
    // The first pass over the ring needs no free-slot wait. When this kernel was launched as the programmatic
    // dependent of the kernel that packs the activations' scales, the pass runs in two parts: the weight loads
    // go out at once, the activation loads follow the dependency wait. Otherwise the four loads of a stage go
    // out together (the copy engine takes them in order: a stage completes sooner that way).
    if (p.dependent) {
      const uint32_t s_stage = p_stage, s_phase = p_phase;
      const int s_seg = p_seg, s_tile = p_tile, s_kb = p_kb, s_kbe = p_kbe;
      produce(STAGES, false, 1);
      p_stage = s_stage; p_phase = s_phase; p_seg = s_seg; p_tile = s_tile; p_kb = s_kb; p_kbe = s_kbe; p_issued = 0;
      pdl_wait();
      produce(STAGES, false, 2);
    } else {
      produce(STAGES, false, 0);
    }
#ifdef WB200_TRACE
    if (lane == 0) { WB_TRACE_SET(4, trace_now()); WB_TRACE_SET(2, (unsigned long long)nseg); }
#endif
  }
  if (warp == 1) {
    tmem_alloc<1>(smem_u32(tmem_slot), Cfg::TMEM_COLS);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // The whole warp walks the loop; one elected lane issues the copies.
    produce(0x7fffffff, true, 0);
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t idesc = (EB == 4) ? make_idesc_mxf4(128, NP) : make_idesc_mxf8(128, NP, weight_format_of(p.elem_format), act_format_of(p.elem_format));
    uint32_t stage = 0, phase = 0, sf_set = 0;
    for (int seg = 0; seg < nseg; ++seg) {
      int tile, kbs, kbe;
      segment(seg, tile, kbs, kbe);
      const int as = seg & 1;
      if (seg >= 2)
        mbar_wait(acc_empty_bar(as), uint32_t((seg - 2) >> 1) & 1u, ctx, WB_DEV_TIMEOUT_MMA_ACC);
      tc_fence_after_sync();
      const uint32_t d_tmem = tmem_base + (as ? Cfg::ACC_COL1 : 0);
      for (int kb = kbs; kb < kbe; ++kb) {
        const uint32_t t_sfw = tmem_base + Cfg::SF_COL + sf_set * 16;
        const uint32_t t_sfx = t_sfw + 8;
        if (++sf_set == Cfg::SF_SETS) sf_set = 0;
        mbar_wait(full_bar(stage), phase, ctx, WB_DEV_TIMEOUT_MMA_FULL);
        tc_fence_after_sync();
#ifdef WB200_TRACE
        if (lane == 0) {
          if (seg == 0 && kb == kbs) WB_TRACE_SET(3, trace_now());
          if (kb == kbe - 1) { WB_TRACE_SEG(seg, 0, (unsigned long long)tile); WB_TRACE_SEG(seg, 1, trace_now()); }
        }
#endif
        const uint32_t sW = smem_base + stage * Cfg::STAGE_BYTES;
        const uint32_t sX = sW + Cfg::W_BYTES;
        const uint32_t sSFW = sX + Cfg::X_BYTES;
        const uint32_t sSFX = sSFW + Cfg::SF_BYTES;
        const uint64_t w_desc = make_desc_k_sw128(sW);
        const uint64_t x_desc = make_desc_k_sw128(sX);
        const uint64_t sfw_desc = make_desc_sf_atom(sSFW);
        const uint64_t sfx_desc = make_desc_sf_atom(sSFX);
        if (elect_one()) {
#pragma unroll
          for (int a = 0; a < Cfg::SF_ATOMS; ++a) {
            utccp_sf_atom<1>(t_sfw + a * 4, sfw_desc + uint64_t(a * 32));
            utccp_sf_atom<1>(t_sfx + a * 4, sfx_desc + uint64_t(a * 32));
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if constexpr (EB == 4)
              mma_mxf4<1>(d_tmem, w_desc + uint64_t(k * 2), x_desc + uint64_t(k * 2),
                          idesc_with_sf_id(idesc, (k & 1) * 2), t_sfw + (k >> 1) * 4, t_sfx + (k >> 1) * 4,
                          (kb > kbs || k > 0) ? 1u : 0u);
            else  // 32 8-bit values per instruction, one scale each: byte k of the atom's column
              mma_mxf8<1>(d_tmem, w_desc + uint64_t(k * 2), x_desc + uint64_t(k * 2), idesc_with_sf_id(idesc, k), t_sfw,
                          t_sfx, (kb > kbs || k > 0) ? 1u : 0u);
          }
          tc_commit<1>(empty_bar(stage));
          if (kb == kbe - 1) tc_commit<1>(acc_full_bar(as));
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps 2..5
    const int quad = warp & 3;
    const int nl = quad * 32 + lane;  // weight row inside the tile
    if (p.dependent) pdl_wait();  // C, the partial tiles and the counters may still be in use by the kernels before this one
    OutT* __restrict__ C = reinterpret_cast<OutT*>(p.c);
    auto store_out = [&](int m, int n, float v) {
      if (!WB_CHECK(m >= 0 && m < p.M && n >= 0 && n < p.N, kCheckOutputIndex, (long long)m << 32 | unsigned(n))) return;
      OutT* dst = C + size_t(m) * p.ldc + n;
      if constexpr (sizeof(OutT) == 4) {
        if (p.accumulate) v += *dst;
        *dst = v;
      } else {
        if (p.accumulate) v += __bfloat162float(*dst);
        *dst = __float2bfloat16_rn(v);
      }
    };
    // workspace slot of contributor CTA c for `tile`: slot 0 of a CTA holds its first tile, slot 1 its last
    auto slot_of = [&](int c, int tile) {
      int a0, a1;
      skinny_range(total_units, gridDim.x, c, a0, a1);
      return 2 * c + ((a0 / p.num_kb) == tile ? 0 : 1);
    };
    for (int seg = 0; seg < nseg; ++seg) {
      int tile, kbs, kbe;
      segment(seg, tile, kbs, kbe);
      const int as = seg & 1;
      const int n = tile * 128 + nl;
      const bool whole = (kbs == 0 && kbe == p.num_kb);
      float* part = p.partials + (size_t(2 * blockIdx.x + (tile == first_tile ? 0 : 1)) * p.M) * 128 + nl;
      (void)WB_CHECK(tile >= 0 && tile < p.tiles_n && tile < kSkinnyCounterWords, kCheckCounter, tile);

      // A partial segment: who else contributes to this tile, and have they all published already?
      // If so this CTA is certainly the last one: it keeps its own partial in registers, adds the
      // others' (fetched while the MMAs of this segment still run) and writes C, without the round
      // trip of publishing its own partial first. That is the usual case for the segment a CTA
      // ends with, whose other half was finished early in the neighbour's run.
      int c_lo = 0, ncontrib = 1;
      bool known_last = false;
      // the first two other contributors' first 16 rows are fetched ahead
      float pre0[16], pre1[16];
      int other0 = -1, other1 = -1;
      if (!whole) {
        const int t_lo = tile * p.num_kb;
        c_lo = skinny_owner(total_units, gridDim.x, t_lo);
        ncontrib = skinny_owner(total_units, gridDim.x, t_lo + p.num_kb - 1) - c_lo + 1;
        if (threadIdx.x == 64) {
          unsigned int seen;
          asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.counters + tile) : "memory");
          *known_last_flag = (seen == (unsigned int)(ncontrib - 1)) ? 1u : 0u;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        known_last = (*known_last_flag != 0u);
        if (known_last) {
          __threadfence();
          for (int i = 0; i < ncontrib; ++i) {
            const int c = c_lo + i;
            if (c == int(blockIdx.x)) continue;
            if (other0 < 0) other0 = c;
            else if (other1 < 0) other1 = c;
          }
          if (other0 >= 0) {
            const float* src = p.partials + size_t(slot_of(other0, tile)) * p.M * 128 + nl;
#pragma unroll
            for (int j = 0; j < 16; ++j) pre0[j] = (j < p.M) ? __ldcg(src + size_t(j) * 128) : 0.f;
          }
          if (other1 >= 0) {
            const float* src = p.partials + size_t(slot_of(other1, tile)) * p.M * 128 + nl;
#pragma unroll
            for (int j = 0; j < 16; ++j) pre1[j] = (j < p.M) ? __ldcg(src + size_t(j) * 128) : 0.f;
          }
        }
      }

      mbar_wait(acc_full_bar(as), uint32_t(seg >> 1) & 1u, ctx, WB_DEV_TIMEOUT_EPILOGUE);
      tc_fence_after_sync();
#ifdef WB200_TRACE
      if (threadIdx.x == 64) WB_TRACE_SEG(seg, 2, trace_now());
#endif
      const uint32_t t_acc = tmem_base + (uint32_t(quad * 32) << 16) + (as ? Cfg::ACC_COL1 : 0);
#pragma unroll 1
      for (int c0 = 0; c0 < NP; c0 += 16) {
        uint32_t r[16];
        tmem_ld_32x16(t_acc + c0, r);
        tmem_ld_wait();
        if (c0 + 16 >= NP) {  // accumulator fully read: hand it back to the MMA warp
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_empty_bar(as));
        }
        if (whole) {
          if (n < p.N) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (c0 + j < p.M) store_out(c0 + j, n, __uint_as_float(r[j]));
          }
        } else if (known_last) {
          // contributions are added in CTA order, this CTA's own from registers
          if (n < p.N && c0 < p.M) {
            float acc[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[j] = 0.f;
            for (int i = 0; i < ncontrib; ++i) {
              const int c = c_lo + i;
              if (c == int(blockIdx.x)) {
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[j] += __uint_as_float(r[j]);
              } else if (c0 == 0 && c == other0) {
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[j] += pre0[j];
              } else if (c0 == 0 && c == other1) {
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[j] += pre1[j];
              } else {
                const float* src = p.partials + (size_t(slot_of(c, tile)) * p.M + c0) * 128 + nl;
                float v[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = (c0 + j < p.M) ? __ldcg(src + size_t(j) * 128) : 0.f;
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[j] += v[j];
              }
            }
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (c0 + j < p.M) store_out(c0 + j, n, acc[j]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = c0 + j;
            if (m < p.M) __stcg(part + size_t(m) * 128, __uint_as_float(r[j]));
          }
        }
      }
      if (!whole && known_last) {
        // every other contributor has come and gone: leave the counter clean for the next launch
        if (threadIdx.x == 64) p.counters[tile] = 0u;
        asm volatile("bar.sync 1, 128;" ::: "memory");  // known_last_flag is reused by the next segment
      } else if (!whole) {
        // publish the partial, then find out whether this CTA completes the tile
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64) {
          const unsigned int prev = atomicAdd(p.counters + tile, 1u);
          *last_flag = (prev == (unsigned int)(ncontrib - 1)) ? 1u : 0u;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*last_flag) {
          __threadfence();
          if (n < p.N) {
            // Partials are added in CTA order (fixed, so the sum does not depend on who arrived
            // when), 16 output rows at a time so that the loads of one batch are all in flight.
            int slots[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) slots[i] = (i < ncontrib) ? slot_of(c_lo + i, tile) : 0;
            for (int m0 = 0; m0 < p.M; m0 += 16) {
              float acc[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) acc[j] = 0.f;
              for (int i = 0; i < ncontrib; ++i) {
                const int slot = (i < 4) ? slots[i & 3] : slot_of(c_lo + i, tile);
                const float* src = p.partials + (size_t(slot) * p.M + m0) * 128 + nl;
                float v[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = (m0 + j < p.M) ? __ldcg(src + size_t(j) * 128) : 0.f;
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[j] += v[j];
              }
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (m0 + j < p.M) store_out(m0 + j, n, acc[j]);
            }
          }
          if (threadIdx.x == 64) p.counters[tile] = 0u;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");  // last_flag is reused by the next segment
      }
#ifdef WB200_TRACE
      if (threadIdx.x == 64) WB_TRACE_SEG(seg, 3, trace_now() | (known_last ? (1ull << 62) : 0ull) | (whole ? (1ull << 63) : 0ull));
#endif
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, Cfg::TMEM_COLS);
  }
#ifdef WB200_TRACE
  if (threadIdx.x == 0) WB_TRACE_SET(1, trace_now());
#endif
}

}  // namespace wb
