// MXFP4 x MXFP4 block-scaled GEMM for sm_100a: C[M,N] = dequant(A) * dequant(B)^T.
//
// Replaces, for this one kernel family, what the reference generates from its scaled-GEMM
// templates (wave_lang/kernel/wave/templates/gemm.py:134-205 and
// wave_lang/kernel/wave/templates/tagged_mxfp4_gemm.py:38-145): the K loop of
// read -> bitcast -> scaled_mma and the f32 / bf16 write of C.
//
// Shape of the kernel
//   * persistent: one CTA (or CTA pair) per SM walks a static list of output tiles in an
//     N-grouped order (same intent as tagged_mxfp4_gemm.py:1038-1089: keep the A rows in L2
//     while a group of N tiles is swept down M);
//   * warp-specialised: warp 0 issues TMA loads, warp 1 issues tcgen05.cp / tcgen05.mma,
//     warps 2..5 drain the accumulator (tcgen05.ld -> convert -> 16-byte stores);
//   * A and B tiles arrive as rows of 128 bytes (256 packed E2M1 values) with the 128-byte
//     swizzle; scale factors arrive as 512-byte atoms (128 rows x 4 K-blocks) and are copied to
//     tensor memory with tcgen05.cp before the four K = 64 MMAs of a stage;
//   * two accumulators live in tensor memory so that the epilogue of tile i overlaps the main
//     loop of tile i+1. With BN = 256 the two accumulators overlap by 48 columns (512 columns
//     cannot hold 2 x 256 plus the scale factors); the epilogue drains the shared columns first
//     and releases the next main loop as soon as they are free. With BN = 192 both accumulators
//     and the scale factors fit side by side and no hand-over wait remains;
//   * CG = 2 pairs two CTAs of a cluster on one 256-row tile (cta_group::2): each CTA loads its
//     own 128 rows of A and its half of the B rows with plain TMA loads (no multicast); the loads
//     of both CTAs complete on the leader CTA's barrier, and the leader issues the MMAs.
#pragma once
#include "ptx.cuh"
#include <cuda_bf16.h>

namespace wb {

// EB: bits per operand element, 4 (MXFP4, kind::mxf4) or 8 (MXFP8, kind::mxf8f6f4). Either way a pipeline
// stage is one 128-byte swizzle row of every operand row and four MMAs of 32 bytes of K each; what
// differs is the K extent of a stage (256 or 128 elements) and hence its scale factors (8 or 4 K-blocks
// per row = 2 or 1 atoms per 128 rows).
template <int CG, int BN_, int OUT_BYTES, int EB = 4>
struct GemmCfg {
  static_assert(EB == 4 || EB == 8, "operand elements are 4 or 8 bits");
  static constexpr int BM = 128;  // accumulator rows per CTA (tensor-memory lanes)
  static constexpr int BN = BN_;
  static constexpr int BK = 1024 / EB;  // K elements per pipeline stage = one 128-byte swizzle row
  static constexpr int SF_ATOMS = BK / 128;  // scale-factor atoms (4 K-blocks each) per 128 rows and stage
  static constexpr int B_ROWS = BN / CG;  // B rows this CTA loads
  static constexpr int A_BYTES = BM * 128;
  static constexpr int B_BYTES = B_ROWS * 128;
  static constexpr int SFA_BYTES = SF_ATOMS * 512;        // 128 rows x BK / 32 K-blocks
  // Packed scales come in blocks of 128 rows = 4 tensor-memory columns of 32 rows each. A 192-row
  // tile starts at column 0 or 2 of a block and ends inside the next one: the kernel loads both
  // blocks and points the MMA at the column the tile starts with. (The MMA takes even column
  // offsets only: an odd one, as a 224-row tile would need, raises a misaligned-address fault.)
  // A 224-row tile would start on odd columns too, so it reads a packing of the weight scales made for it: two
  // blocks per tile (rows 0..127 and 128..223 of the tile), the tile always at column 0 (wb200_repack_scales_tiled).
  static constexpr bool TILED_SFB = (BN == 224);
  static constexpr int SFB_BLOCKS = (BN % 128 == 0) ? BN / 128 : TILED_SFB ? 2 : (BN + 64 + 127) / 128;
  static constexpr int SFB_BYTES = SFB_BLOCKS * SF_ATOMS * 512;
  static constexpr int LOAD_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;  // what the loads of a stage deliver
  static constexpr int STAGE_BYTES = (LOAD_BYTES + 1023) / 1024 * 1024;
  // Epilogue staging: each of the 4 epilogue warps owns two buffers of 32 rows x 32 columns of C,
  // written with the TMA store swizzle (64-byte rows for bf16, 128-byte rows for f32).
  // A buffer is 32 rows of 128 bytes: one 32-column chunk of f32, or two neighbouring chunks of bf16
  // (stored together, so that every TMA store writes whole 128-byte lines).
  static constexpr int STORE_BUF_BYTES = 32 * 128;
  static constexpr int STAGING_BYTES = 4 * 2 * STORE_BUF_BYTES;
  static constexpr int SMEM_LIMIT = 232448;  // largest dynamic shared memory a CTA may ask for on sm_100
  static constexpr int STAGES_FIT = (SMEM_LIMIT - 1024 - STAGING_BYTES - 512) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_FIT > 8 ? 8 : STAGES_FIT;
  static constexpr int NUM_BARRIERS = 2 * STAGES + 4;
  static constexpr int SMEM_BYTES = 1024 /*alignment slack*/ + STAGES * STAGE_BYTES + STAGING_BYTES + NUM_BARRIERS * 8 + 64;
  static_assert(STAGES >= 3, "pipeline needs at least 3 stages");
  // tensor-memory columns
  static constexpr int TMEM_COLS = 512;
  static constexpr bool OVERLAP = (BN == 256);
  static constexpr int ACC_COL0 = 0;
  // Scale factors live in a small ring of column sets so that the tcgen05.cp of one K block does
  // not have to wait for the MMAs of the previous block to finish reading theirs.
  // (sized for two atoms per 128 rows also when a stage has one, so that the accumulators sit at the same columns)
  static constexpr int SF_SET_COLS = 8 + SFB_BLOCKS * 8;  // A: 2 atoms x 4 columns, B: blocks x 2 atoms x 4
  static constexpr int SF_SETS = OVERLAP ? 2 : ((512 - 2 * BN) / SF_SET_COLS >= 4 ? 4 : (512 - 2 * BN) / SF_SET_COLS);
  static_assert(SF_SETS >= 2, "the scale-factor ring needs two column sets");
  static constexpr int SF_COL = OVERLAP ? 512 - SF_SETS * SF_SET_COLS : 2 * BN;
  // 32-column chunks shared by the two accumulators: accumulator 1 ends where the scale factors begin
  static constexpr int OVERLAP_CHUNKS = (2 * 256 - SF_COL + 31) / 32;
  static constexpr int ACC_COL1 = OVERLAP ? SF_COL - 256 : BN;
  static_assert(SF_COL + SF_SETS * SF_SET_COLS <= 512, "scale-factor ring does not fit in tensor memory");
  static_assert(!OVERLAP || OVERLAP_CHUNKS % 2 == 0, "bf16 stores pair neighbouring chunks; the shared columns must be whole pairs");
  static constexpr int THREADS = 192;
  static_assert(BN == 128 || BN == 192 || BN == 224 || BN == 256, "BN must be 128, 192, 224 or 256");
  static_assert(BN % 64 == 0 || TILED_SFB, "tiles start on even scale columns unless the scales are packed per tile");
  static_assert(STAGE_BYTES % 1024 == 0, "stages must keep the 1024-byte swizzle alignment");
};

struct GemmParams {
  void* c;
  int M, N, K;
  int ldc;            // elements
  int tiles_m, tiles_n;
  int group_n;        // N tiles per raster group
  int vec_ok;         // C base and row pitch allow 16-byte stores
  int tma_store;      // 1: write C with TMA stores from swizzled shared memory (needs vec_ok, no accumulate);
                      // 2: same staging, then plain 16-byte stores covering whole 128-byte lines (needs vec_ok)
  int accumulate;     // add to the values already in C instead of overwriting them
  int elem_format;    // 8-bit operands only: 0 = E4M3, 1 = E5M2
  int* status;
};

// The tensor maps of one launch, passed by value as a kernel parameter. Index: 0 = a, 1 = b,
// 2 = packed a scales, 3 = packed b scales, 4 = c.
struct PlainMaps {
  static constexpr bool kGrouped = false;
  CUtensorMap m[5];
};
// Grouped (per-expert) launch: five maps per group, each describing only that group's rows, so that
// TMA zero-fills loads and clips stores at the group's end; tile_start is the running count of
// tiles over the groups, rows the row count of each group.
constexpr int kMaxGroups = 32;
struct GroupedMaps {
  static constexpr bool kGrouped = true;
  CUtensorMap m[kMaxGroups * 5];
  void* c_base[kMaxGroups];  // first output row of each group, for the stores that do not go through its tensor map
  int tile_start[kMaxGroups + 1];
  int rows[kMaxGroups];
  int num_groups;
  // interleave != 0: walk the groups round-robin (tile t = tile t / G of group t % G) over tiles_max tiles
  // per group, skipping the ids a shorter group does not have, instead of group after group. Used when the
  // groups differ in WHERE their output goes (another GPU): the remote stores then spread over the whole launch.
  int interleave;
  int tiles_max;
  // aligned != 0: the rows of all groups sit in ONE matrix, every group padded to whole tile_rows-row tiles, and
  // which group a row tile belongs to is read from device memory (expert_ids[M tile], as written by
  // moe_align_block_size with block_size = tile_rows); row tiles at or past *num_rows are skipped. Slots 0, 2, 4
  // of every group's maps describe that one matrix; slots 1, 3 are the group's own weights. The host needs
  // no knowledge of the routing: no read-back, and the launch can be captured in a CUDA graph.
  int aligned;
  int tile_rows;
  int tiles_m_cap;
  const int* expert_ids;
  const int* num_rows;
};

// Tile order: groups of `group_n` N tiles, each group swept down M with N fastest.
__device__ __forceinline__ void raster_tile(int t, int tiles_m, int tiles_n, int group_n, int& mt,
                                            int& nt) {
  const int per_group = group_n * tiles_m;
  const int g = t / per_group;
  const int r = t - g * per_group;
  const int n0 = g * group_n;
  const int gw = min(group_n, tiles_n - n0);
  mt = r / gw;
  nt = n0 + (r - mt * gw);
}

// Tile id -> (group, M tile, N tile, rows of the group) and the group's first tensor map; nullptr for an
// id that names no tile (interleaved walk over groups of unequal size).
template <typename Maps>
__device__ __forceinline__ const CUtensorMap* decode_tile(const Maps& maps, const GemmParams& p, int t, int& mt, int& nt,
                                                          int& rows, void** c_base = nullptr) {
  if constexpr (!Maps::kGrouped) {
    raster_tile(t, p.tiles_m, p.tiles_n, p.group_n, mt, nt);
    rows = p.M;
    if (c_base) *c_base = p.c;
    return &maps.m[0];
  } else {
    if (maps.aligned) {
      raster_tile(t, maps.tiles_m_cap, p.tiles_n, p.group_n, mt, nt);
      const int total = __ldg(maps.num_rows);
      if (mt * maps.tile_rows >= total) return nullptr;
      int e = __ldg(maps.expert_ids + mt);
      if (e < 0 || e >= maps.num_groups) return nullptr;  // never written by a correct router; do not index out of the table
      rows = total;
      if (c_base) *c_base = maps.c_base[0];
      return &maps.m[e * 5];
    }
    int g = 0, local;
    if (maps.interleave) {
      g = t % maps.num_groups;
      local = t / maps.num_groups;
      if (local >= maps.tile_start[g + 1] - maps.tile_start[g]) return nullptr;
    } else {
      while (g + 1 < maps.num_groups && t >= maps.tile_start[g + 1]) ++g;
      local = t - maps.tile_start[g];
    }
    raster_tile(local, (maps.tile_start[g + 1] - maps.tile_start[g]) / p.tiles_n, p.tiles_n, p.group_n, mt, nt);
    rows = maps.rows[g];
    if (c_base) *c_base = maps.c_base[g];
    return &maps.m[g * 5];
  }
}

// Adds the 32 values already in C (row pointer p) to r: the accumulate-into-C form the
// reference's split-K template has (tagged_mxfp4_gemm.py:780-781, caller-initialised C).
template <typename OutT>
__device__ __forceinline__ void add_old_chunk32(const OutT* __restrict__ p, uint32_t (&r)[32], int ncols,
                                                bool vec) {
  if constexpr (sizeof(OutT) == 4) {
    if (vec && ncols == 32) {
      const uint4* q = reinterpret_cast<const uint4*>(p);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint4 v = q[j];
        r[4 * j + 0] = __float_as_uint(__uint_as_float(r[4 * j + 0]) + __uint_as_float(v.x));
        r[4 * j + 1] = __float_as_uint(__uint_as_float(r[4 * j + 1]) + __uint_as_float(v.y));
        r[4 * j + 2] = __float_as_uint(__uint_as_float(r[4 * j + 2]) + __uint_as_float(v.z));
        r[4 * j + 3] = __float_as_uint(__uint_as_float(r[4 * j + 3]) + __uint_as_float(v.w));
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) r[j] = __float_as_uint(__uint_as_float(r[j]) + reinterpret_cast<const float*>(p)[j]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < ncols) r[j] = __float_as_uint(__uint_as_float(r[j]) + __bfloat162float(p[j]));
  }
}

template <typename OutT>
__device__ __forceinline__ void store_chunk32(OutT* __restrict__ p, const uint32_t (&r)[32],
                                              int ncols, bool vec) {
  if constexpr (sizeof(OutT) == 4) {
    if (vec && ncols == 32) {
      uint4* q = reinterpret_cast<uint4*>(p);
#pragma unroll
      for (int j = 0; j < 8; ++j) q[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) reinterpret_cast<uint32_t*>(p)[j] = r[j];
    }
  } else {
    if (vec && ncols == 32) {
      uint4* q = reinterpret_cast<uint4*>(p);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 v;
        v.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
        v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
        v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
        v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
        q[j] = v;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) p[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
    }
  }
}

// One 16-byte load from shared memory.
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}

// One 16-byte store to shared memory.
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// Lane `lane` holds 32 consecutive columns of output row `lane` of a 32 x 32 chunk. Write them to
// the staging buffer in the layout a TMA store with 128-byte rows and the 128-byte swizzle reads:
// an f32 chunk fills a row; a bf16 chunk fills half of it (`half` = 0 / 1 for the left / right
// chunk of a pair). The swizzle also spreads the 32 lanes' 16-byte pieces over all banks.
template <typename OutT>
__device__ __forceinline__ void stage_chunk32(uint32_t buf, int lane, int half, const uint32_t (&r)[32]) {
  const uint32_t row = buf + lane * 128;
  if constexpr (sizeof(OutT) == 4) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      st_shared_v4(row + ((j ^ (lane & 7)) << 4), r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      st_shared_v4(row + (((half * 4 + j) ^ (lane & 7)) << 4),
                   pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1])),
                   pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3])),
                   pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5])),
                   pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7])));
  }
}

template <int CG, int BN, typename OutT, typename Maps, int EB = 4>
__global__ void __launch_bounds__(192, 1)
mxfp4_gemm_kernel(const __grid_constant__ Maps maps, const GemmParams p) {
  using Cfg = GemmCfg<CG, BN, int(sizeof(OutT)), EB>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment for the 128-byte swizzle; identical offset in both CTAs of a pair.
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  pdl_launch_dependents();  // a kernel launched behind this one as a programmatic dependent may take SMs as they free up
  const uint32_t rank = (CG == 2) ? cluster_ctarank() : 0u;
  const bool leader = (rank == 0);

  // barrier block after the stages
  const uint32_t staging_base = smem_base + STAGES * Cfg::STAGE_BYTES;  // 1024-byte aligned
  const uint32_t bar_base = staging_base + Cfg::STAGING_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto acc_full_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
  auto acc_empty_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + 2 + s); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + STAGES * Cfg::STAGE_BYTES + Cfg::STAGING_BYTES +
                                                    Cfg::NUM_BARRIERS * 8);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  WaitCtx ctx{abort_flag, p.status};

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(acc_full_bar(s), 1);
      mbar_init(acc_empty_bar(s), 4 * CG);
    }
    *abort_flag = 0u;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc<CG>(smem_u32(tmem_slot), Cfg::TMEM_COLS);
    tmem_relinquish<CG>();
  }
  if (warp == 0 && lane == 0) {
#pragma unroll
    for (int i = 0; i < 5; ++i) prefetch_tensormap(&maps.m[i]);
  }
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (CG == 2) {  // peer barriers must exist before anyone signals them
    cluster_arrive();
    cluster_wait();
  }
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  int num_tiles = p.tiles_m * p.tiles_n;
  if constexpr (Maps::kGrouped)
    num_tiles = maps.aligned ? maps.tiles_m_cap * p.tiles_n
                             : (maps.interleave ? maps.num_groups * maps.tiles_max : maps.tile_start[maps.num_groups]);
  const int first_tile = (CG == 2) ? (blockIdx.x >> 1) : blockIdx.x;
  const int tile_step = (CG == 2) ? (gridDim.x >> 1) : gridDim.x;
  const int num_kb = (p.K + Cfg::BK - 1) / Cfg::BK;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // The whole warp walks the loop; one elected lane issues the copies.
    uint32_t stage = 0, phase = 0;
#if defined(WB200_MMA_CEILING) && !defined(WB_KEEP_LOADS)
    int stages_loaded = 0;  // measurement build: only the first ring is loaded, the MMAs then re-read it
#endif
    pdl_wait();  // the packed activation scales may be written by the kernel launched just before this one
    for (int t = first_tile; t < num_tiles; t += tile_step) {
      int mt, nt, rows;
      const CUtensorMap* tm = decode_tile(maps, p, t, mt, nt, rows);
      if (Maps::kGrouped && tm == nullptr) continue;
      const int a_row = (mt * CG + int(rank)) * Cfg::BM;
      const int b_row = nt * BN + int(rank) * Cfg::B_ROWS;
      const int sfa_rb = mt * CG + int(rank);
      const int sfb_rb = Cfg::TILED_SFB ? nt * Cfg::SFB_BLOCKS : (nt * BN) / 128;
      for (int kb = 0; kb < num_kb; ++kb) {
        mbar_wait(empty_bar(stage), phase ^ 1u, ctx, WB_DEV_TIMEOUT_PRODUCER);
        const uint32_t sA = smem_base + stage * Cfg::STAGE_BYTES;
        const uint32_t sB = sA + Cfg::A_BYTES;
        const uint32_t sSFA = sB + Cfg::B_BYTES;
        const uint32_t sSFB = sSFA + Cfg::SFA_BYTES;
        // With a CTA pair, every load of both CTAs reports to the leader's barrier, which
        // therefore expects the bytes of two stages; the second CTA only issues its copies.
        const uint32_t fb = (CG == 2) ? mapa_shared(full_bar(stage), 0) : full_bar(stage);
#if defined(WB200_MMA_CEILING) && !defined(WB_KEEP_LOADS)
        if (stages_loaded >= STAGES) {
          if (leader && elect_one()) mbar_arrive(full_bar(stage));
          __syncwarp();
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          continue;
        }
        ++stages_loaded;
#endif
        if (elect_one()) {
          // 4-bit weights expanded by the copy engine (EB == 8 kernels only): the transaction count is the packed size
          if (leader) mbar_expect_tx(full_bar(stage), (Cfg::LOAD_BYTES - ((EB == 8 && (p.elem_format & 0x10)) ? Cfg::B_BYTES / 2 : 0)) * CG);
          tma_load_2d<CG>(sA, tm + 0, kb * 128, a_row, fb);
          tma_load_2d<CG>(sB, tm + 1, kb * 128, b_row, fb);
          // scale factors: SF_ATOMS atoms of 512 bytes (128 32-bit words) per 128-row block and stage
          tma_load_2d<CG>(sSFA, tm + 2, kb * (Cfg::SF_ATOMS * 128), sfa_rb, fb);
          tma_load_2d<CG>(sSFB, tm + 3, kb * (Cfg::SF_ATOMS * 128), sfb_rb, fb);
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (leader) {
      const uint32_t idesc = (EB == 4) ? make_idesc_mxf4(Cfg::BM * CG, BN)
                                       : make_idesc_mxf8(Cfg::BM * CG, BN, act_format_of(p.elem_format), weight_format_of(p.elem_format));
      const uint32_t peer_empty0 = (CG == 2) ? mapa_shared(empty_bar(0), 1) : 0u;
      const uint32_t peer_acc_full0 = (CG == 2) ? mapa_shared(acc_full_bar(0), 1) : 0u;
      uint32_t stage = 0, phase = 0, sf_set = 0;
      int it = 0;
      for (int t = first_tile; t < num_tiles; t += tile_step) {
        // first 32-row group of this tile inside its first 128-row scale block = first scale column (0 or 2)
        uint32_t sfb_group = 0;
        if constexpr ((BN % 128 != 0 && !Cfg::TILED_SFB) || Maps::kGrouped) {
          int mt, nt, rows;
          if (decode_tile(maps, p, t, mt, nt, rows) == nullptr) continue;
          sfb_group = uint32_t((nt * BN) % 128) / 32u;
        }
        const int as = it & 1;
        // accumulator availability
        if constexpr (Cfg::OVERLAP) {
          // Needs the previous tile's epilogue to have drained the 48 shared columns
          // (which also means the tile before that is fully drained).
          if (it > 0) {
            const int ps = (it - 1) & 1;
            mbar_wait<CG == 2>(acc_empty_bar(ps), uint32_t((it - 1) >> 1) & 1u, ctx, WB_DEV_TIMEOUT_MMA_ACC);
          }
        } else {
          if (it >= 2)
            mbar_wait<CG == 2>(acc_empty_bar(as), uint32_t((it - 2) >> 1) & 1u, ctx, WB_DEV_TIMEOUT_MMA_ACC);
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (as ? Cfg::ACC_COL1 : Cfg::ACC_COL0);
        for (int kb = 0; kb < num_kb; ++kb) {
          const uint32_t t_sfa = tmem_base + Cfg::SF_COL + sf_set * Cfg::SF_SET_COLS;
          const uint32_t t_sfb = t_sfa + 8;
          if (++sf_set == Cfg::SF_SETS) sf_set = 0;
          mbar_wait(full_bar(stage), phase, ctx, WB_DEV_TIMEOUT_MMA_FULL);
          tc_fence_after_sync();
          const uint32_t sA = smem_base + stage * Cfg::STAGE_BYTES;
          const uint32_t sB = sA + Cfg::A_BYTES;
          const uint32_t sSFA = sB + Cfg::B_BYTES;
          const uint32_t sSFB = sSFA + Cfg::SFA_BYTES;
          const uint64_t a_desc = make_desc_k_sw128(sA);
          const uint64_t b_desc = make_desc_k_sw128(sB);
          const uint64_t sfa_desc = make_desc_sf_atom(sSFA);
          const uint64_t sfb_desc = make_desc_sf_atom(sSFB);
          if (elect_one()) {
            // scale factors: smem atoms -> tensor memory (4 columns per atom); +32 in the
            // descriptor's address field = +512 bytes = the next atom
            {
#pragma unroll
              for (int a = 0; a < Cfg::SF_ATOMS; ++a) utccp_sf_atom<CG>(t_sfa + a * 4, sfa_desc + uint64_t(a * 32));
#pragma unroll
              for (int j = 0; j < Cfg::SFB_BLOCKS; ++j)
#pragma unroll
                for (int a = 0; a < Cfg::SF_ATOMS; ++a)
                  utccp_sf_atom<CG>(t_sfb + a * (Cfg::SFB_BLOCKS * 4) + j * 4,
                                    sfb_desc + uint64_t((j * Cfg::SF_ATOMS + a) * 32));
            }
            {
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                // one instruction = 32 bytes of K inside the 128-byte swizzle row: 64 E2M1 values with two
                // scales each (bytes 0,1 or 2,3 of the atom's column), or 32 8-bit values with one scale (byte k)
                if constexpr (EB == 4)
                  mma_mxf4<CG>(d_tmem, a_desc + uint64_t(k * 2), b_desc + uint64_t(k * 2),
                               idesc_with_sf_id(idesc, (k & 1) * 2), t_sfa + (k >> 1) * 4,
                               t_sfb + (k >> 1) * (Cfg::SFB_BLOCKS * 4) + sfb_group, (kb > 0 || k > 0) ? 1u : 0u);
                else
                  mma_mxf8<CG>(d_tmem, a_desc + uint64_t(k * 2), b_desc + uint64_t(k * 2), idesc_with_sf_id(idesc, k),
                               t_sfa, t_sfb + sfb_group, (kb > 0 || k > 0) ? 1u : 0u);
              }
            }
            // free the stage in both CTAs once these MMAs have read it
            tc_commit<CG>(empty_bar(stage));
            if constexpr (CG == 2) tc_commit<CG>(peer_empty0 + 8u * stage);
            if (kb == num_kb - 1) {
              tc_commit<CG>(acc_full_bar(as));
              if constexpr (CG == 2) tc_commit<CG>(peer_acc_full0 + 8u * as);
            }
          }
          __syncwarp();
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        ++it;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps 2..5
    const int quad = warp & 3;  // tensor-memory lane quadrant this warp may read
    const uint32_t acc_empty_leader0 = (CG == 2) ? mapa_shared(acc_empty_bar(0), 0) : 0u;
    const uint32_t acc_empty_leader1 = (CG == 2) ? mapa_shared(acc_empty_bar(1), 0) : 0u;
    pdl_wait();  // C may still be read by the kernels before this one
    const uint32_t stg = staging_base + uint32_t(warp - 2) * 2 * Cfg::STORE_BUF_BYTES;
    // C is written once and not read again by this kernel: keep it from pushing A and B out of L2
    const uint64_t store_policy = l2_policy_evict_first();
    int it = 0;
    uint32_t store_count = 0;
    for (int t = first_tile; t < num_tiles; t += tile_step) {
      int mt, nt, rows;
      void* c_group = nullptr;
      const CUtensorMap* tm = decode_tile(maps, p, t, mt, nt, rows, &c_group);
      if (Maps::kGrouped && tm == nullptr) continue;
      const int as = it & 1;
      mbar_wait(acc_full_bar(as), uint32_t(it >> 1) & 1u, ctx, WB_DEV_TIMEOUT_EPILOGUE);
      tc_fence_after_sync();
      const int row0 = (mt * CG + int(rank)) * Cfg::BM + quad * 32;
      const int row = row0 + lane;
      const int col0 = nt * BN;
      const uint32_t t_acc = tmem_base + (uint32_t(quad * 32) << 16) + (as ? Cfg::ACC_COL1 : Cfg::ACC_COL0);
      auto release = [&]() {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          // No data is published here: the tensor-memory reads have completed (wait::ld above).
          if constexpr (CG == 2) mbar_arrive_cluster_relaxed(as ? acc_empty_leader1 : acc_empty_leader0);
          else mbar_arrive(acc_empty_bar(as));
        }
      };
#if defined(WB200_MMA_CEILING) && !defined(WB_KEEP_EPILOGUE)
      release();  // measurement build: the accumulator is neither read nor stored
      ++it;
      continue;
#endif
      constexpr int NCHUNK = BN / 32;
      // Overlapping accumulators: the MMA warp cannot start the next tile before the shared columns are read. Both
      // shared chunks are therefore fetched at once, ahead of any staging, and the accumulator is handed back as soon
      // as they are in registers; `held` keeps the second chunk until its turn.
      [[maybe_unused]] uint32_t held[32];
#pragma unroll 1
      for (int ci = 0; ci < NCHUNK; ++ci) {
        // With overlapping accumulators the columns shared with the other accumulator go first:
        // the last two chunks of accumulator 0, the first two chunks of accumulator 1.
        int chunk = ci;
        if constexpr (Cfg::OVERLAP) {
          if (as == 0)
            chunk = (ci < Cfg::OVERLAP_CHUNKS) ? (NCHUNK - Cfg::OVERLAP_CHUNKS + ci) : (ci - Cfg::OVERLAP_CHUNKS);
        }
        uint32_t r[32];
        if constexpr (Cfg::OVERLAP) {
          static_assert(Cfg::OVERLAP_CHUNKS == 2, "the early hand-back below fetches exactly two shared chunks");
          if (ci == 0) {
            tmem_ld_32x32(t_acc + chunk * 32, r);
            tmem_ld_32x32(t_acc + (chunk + 1) * 32, held);
            tmem_ld_wait();
            release();
          } else if (ci == 1) {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = held[j];
          } else {
            tmem_ld_32x32(t_acc + chunk * 32, r);
            tmem_ld_wait();
          }
        } else {
          tmem_ld_32x32(t_acc + chunk * 32, r);
          tmem_ld_wait();
        }
        const int col = col0 + chunk * 32;
        // bf16 stores go out as pairs of chunks (whole 128-byte lines); with an odd number of chunks (224 columns)
        // the last one has no partner and is written with direct 16-byte stores instead
        constexpr bool kOddChunks = (sizeof(OutT) == 2) && (NCHUNK % 2 == 1);
        const bool lone = kOddChunks && ci == NCHUNK - 1;
        if (p.tma_store && !lone) {
          // Two staging buffers per warp; a store covers one f32 chunk or a pair of bf16 chunks (the
          // chunk order above keeps pairs together). Before a buffer is refilled, the store issued
          // two stores ago must have read it.
          constexpr int PER_STORE = (sizeof(OutT) == 2) ? 2 : 1;
          const int half = ci % PER_STORE;
          const uint32_t buf = stg + (store_count & 1u) * Cfg::STORE_BUF_BYTES;
          if (half == 0) {
            if (p.tma_store == 1 && lane == 0) bulk_wait_group_read<1>();
            __syncwarp();
          }
          stage_chunk32<OutT>(buf, lane, half, r);
          if (Maps::kGrouped && half == PER_STORE - 1 && p.tma_store == 2) {  // compiled for the grouped kernels only
            // Plain stores from the staged rows: each instruction writes four whole 128-byte lines (8 lanes
            // per line). Used where C is another GPU's memory, which is written with ordinary stores.
            __syncwarp();
            constexpr int EPV = 16 / int(sizeof(OutT));  // elements per 16-byte piece
            const int scol = col - (PER_STORE - 1) * 32;
            OutT* cb = reinterpret_cast<OutT*>(c_group);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int rr = i * 4 + (lane >> 3), j = lane & 7;
              const int grow = row0 + rr, gcol = scol + j * EPV;
              if (grow < rows && gcol < p.N && WB_CHECK(grow >= 0 && gcol >= 0, kCheckOutputIndex, (long long)grow << 32 | unsigned(gcol))) {
                const uint4 v = ld_shared_v4(buf + rr * 128 + ((j ^ (rr & 7)) << 4));
                OutT* dst = cb + size_t(grow) * p.ldc + gcol;
                if (gcol + EPV <= p.N) {
                  *reinterpret_cast<uint4*>(dst) = v;
                } else {
                  const OutT* e = reinterpret_cast<const OutT*>(&v);
                  for (int k = 0; k < EPV; ++k)
                    if (gcol + k < p.N) dst[k] = e[k];
                }
              }
            }
            __syncwarp();  // the rows are read before the buffer is staged again
            ++store_count;
          } else if (half == PER_STORE - 1) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              // Rows and columns past M, N are clipped by the store. A store that lies outside C
              // altogether still commits an (empty) group, because the buffer hand-over above counts
              // groups: one group per store, whether or not it wrote anything.
              const int scol = col - (PER_STORE - 1) * 32;
              if (row0 < rows && scol < p.N) tma_store_2d_hint(tm + 4, buf, scol, row0, store_policy);
              bulk_commit_group();
            }
            ++store_count;  // the buffers alternate store by store, across tiles too
          }
        } else if (row < rows && col < p.N && WB_CHECK(row >= 0 && col >= 0, kCheckOutputIndex, (long long)row << 32 | unsigned(col))) {
          OutT* dst = reinterpret_cast<OutT*>(c_group) + size_t(row) * p.ldc + col;
          const int ncols = min(32, p.N - col);
          if (p.accumulate) add_old_chunk32<OutT>(dst, r, ncols, p.vec_ok != 0);
          store_chunk32<OutT>(dst, r, ncols, p.vec_ok != 0);
        }
      }
      if constexpr (!Cfg::OVERLAP) release();
      ++it;
    }
    if (lane == 0) bulk_wait_group<0>();  // all of this warp's stores have left shared memory and landed
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (CG == 2) {  // the pair shares tensor memory traffic and barriers: leave together
    cluster_arrive();
    cluster_wait();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<CG>(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace wb
