// C ABI of the wave_b200 library: argument checks, TMA descriptor set-up, path selection and
// launches. Plays the role of the reference's native launch shim
// (wave_lang/kernel/wave/runtime/runtime.cpp:123-263) for the MXFP4 scaled-GEMM kernels.
#include "../../include/wave_b200.h"
#include "gemm_sm100.cuh"
#include "moe.cuh"
#include "multi_gpu.cuh"
#include "quantize.cuh"
#include "scales.cuh"
#include "skinny_sm100.cuh"
#include "skinny_whole_sm100.cuh"

#include <cudaTypedefs.h>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <cstdlib>
#include <mutex>

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

#define WB_CUDA(expr)                                                                           \
  do {                                                                                          \
    cudaError_t e__ = (expr);                                                                   \
    if (e__ != cudaSuccess)                                                                     \
      return fail(WB200_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), __FILE__, \
                  __LINE__);                                                                    \
  } while (0)

// Device status word written by kernels whose bounded waits give up.
__device__ int g_status_word[4];

constexpr int kMaxDevices = 64;
struct DeviceInfo {
  bool ready = false;
  int sm_count = 0;
  int cc_major = 0;
  int* status_ptr = nullptr;
};
DeviceInfo g_dev[kMaxDevices];
std::mutex g_mu;
PFN_cuTensorMapEncodeTiled g_encode = nullptr;

int get_device(DeviceInfo** out) {
  int dev = 0;
  WB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(WB200_ERR_UNSUPPORTED, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceInfo& d = g_dev[dev];
  if (!d.ready) {
    WB_CUDA(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
    WB_CUDA(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
    if (d.cc_major != 10)
      return fail(WB200_ERR_UNSUPPORTED, "device %d has compute capability %d.x; this library is sm_100a only",
                  dev, d.cc_major);
    void* sp = nullptr;
    WB_CUDA(cudaGetSymbolAddress(&sp, g_status_word));
    d.status_ptr = static_cast<int*>(sp);
    WB_CUDA(cudaMemset(sp, 0, sizeof(int) * 4));
    if (!g_encode) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult qres;
      WB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
      if (qres != cudaDriverEntryPointSuccess || !fn)
        return fail(WB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
      g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled>(fn);
    }
    d.ready = true;
  }
  *out = &d;
  return WB200_OK;
}

// cuTensorMapEncodeTiled behind a small per-thread cache: the same operands come back call after
// call (weights, reused activation and output buffers), and encoding five descriptors per launch is
// a visible part of the host time of a 20-microsecond kernel.
struct MapKey {
  const void* base;
  unsigned long long d0, d1, stride;
  unsigned box0, box1;
  int dtype, swizzle, promo;
  bool operator==(const MapKey& o) const {
    return base == o.base && d0 == o.d0 && d1 == o.d1 && stride == o.stride && box0 == o.box0 && box1 == o.box1 &&
           dtype == o.dtype && swizzle == o.swizzle && promo == o.promo;
  }
};
constexpr int kMapCacheSize = 64;
struct MapCache {
  MapKey keys[kMapCacheSize];
  CUtensorMap maps[kMapCacheSize];
  int used = 0, next = 0;
};
thread_local MapCache g_map_cache;

CUresult encode_2d(CUtensorMap* map, const MapKey& k) {
  MapCache& c = g_map_cache;
  for (int i = 0; i < c.used; ++i)
    if (c.keys[i] == k) {
      *map = c.maps[i];
      return CUDA_SUCCESS;
    }
  cuuint64_t dims[2] = {k.d0, k.d1};
  cuuint64_t strides[1] = {k.stride};
  cuuint32_t box[2] = {k.box0, k.box1};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = g_encode(map, CUtensorMapDataType(k.dtype), 2, const_cast<void*>(k.base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CUtensorMapSwizzle(k.swizzle), CUtensorMapL2promotion(k.promo),
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_SUCCESS) {
    const int slot = (c.used < kMapCacheSize) ? c.used++ : (c.next = (c.next + 1) % kMapCacheSize);
    c.keys[slot] = k;
    c.maps[slot] = *map;
  }
  return r;
}

// True while a launch is to be made a programmatic dependent of the kernel before it in the stream: the GEMM
// behind the repack kernel of wb200_mxfp4_gemm_repack_a, and every launch of a call flagged
// WB200_OVERLAP_PREVIOUS. A dependent kernel starts while its predecessor drains and executes
// griddepcontrol.wait before touching anything but the weights.
static thread_local bool tl_dependent_launch = false;
// N tiles per raster group of the tile kernels, from the WB200_GROUP_N bits of the call in progress
static thread_local int tl_group_n = 16;
static int group_n_from_flags(unsigned flags) {
  const unsigned g = (flags & WB200_GROUP_N_MASK) >> WB200_GROUP_N_SHIFT;
  return g == 0 ? 16 : g == 255 ? (1 << 20) : int(g);
}
// Weight rows per tile of the whole-tile skinny kernel for the call in progress (WB200_B_TILE_ROWS bits): 128, or the
// height the weight scales were packed for with wb200_repack_scales_tiled.
static thread_local int tl_b_tile_rows = 128;
static int b_tile_rows_from_flags(unsigned flags) {
  const unsigned h8 = (flags & WB200_B_TILE_ROWS_MASK) >> WB200_B_TILE_ROWS_SHIFT;
  return h8 == 0 ? 128 : int(h8) * 8;
}
struct GroupNScope {  // restores the previous value on every return path
  int saved;
  explicit GroupNScope(unsigned flags) : saved(tl_group_n) { tl_group_n = group_n_from_flags(flags); }
  ~GroupNScope() { tl_group_n = saved; }
};

// [rows, row_bytes] uint8 matrix (rows pitch_bytes apart; 0 = dense), box = 128 bytes x box_rows, 128-byte swizzle, zero fill.
int make_operand_map(CUtensorMap* map, const void* base, long long rows, long long row_bytes, int box_rows,
                     long long pitch_bytes = 0) {
  const MapKey k{base, (unsigned long long)row_bytes, (unsigned long long)rows,
                 (unsigned long long)(pitch_bytes ? pitch_bytes : row_bytes), 128u,
                 unsigned(box_rows), int(CU_TENSOR_MAP_DATA_TYPE_UINT8), int(CU_TENSOR_MAP_SWIZZLE_128B),
                 int(CU_TENSOR_MAP_L2_PROMOTION_L2_256B)};
  CUresult r = encode_2d(map, k);
  if (r != CUDA_SUCCESS)
    return fail(WB200_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (rows %lld, row bytes %lld)", int(r),
                rows, row_bytes);
  return WB200_OK;
}

// Packed E2M1 weights ([rows, K/2] bytes) for the 8-bit kernels (kind::mxf8f6f4): the copy engine expands every 16
// values (8 bytes) into a 16-byte slot of shared memory, 8 bytes of values and 8 of padding, which is the 8-bit
// container layout the MMA reads 4-bit operands in. One box = 128 values x box_rows = 128 bytes x box_rows of shared
// memory, the footprint of an 8-bit operand tile. K a multiple of 128, base 32-byte aligned (driver rules of this type).
int make_operand_map_u4(CUtensorMap* map, const void* base, long long rows, long long K, int box_rows) {
  if (K % 128 != 0) return fail(WB200_ERR_UNSUPPORTED, "4-bit weights in the 8-bit GEMM need K %% 128 == 0 (K = %lld)", K);
  if (reinterpret_cast<uintptr_t>(base) & 31) return fail(WB200_ERR_ALIGNMENT, "4-bit weights in the 8-bit GEMM must be 32-byte aligned");
  const MapKey k{base, (unsigned long long)K, (unsigned long long)rows, (unsigned long long)(K / 2), 128u, unsigned(box_rows),
                 int(CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B), int(CU_TENSOR_MAP_SWIZZLE_128B), int(CU_TENSOR_MAP_L2_PROMOTION_L2_256B)};
  CUresult r = encode_2d(map, k);
  if (r != CUDA_SUCCESS)
    return fail(WB200_ERR_CUDA, "cuTensorMapEncodeTiled (4-bit weights) failed with CUresult %d (rows %lld, K %lld)", int(r), rows, K);
  return WB200_OK;
}
static bool weights_are_fp4(int EB, int elem_format) { return EB == 8 && (elem_format & 0x10) != 0; }

// Packed scale array ([row_blocks][k_atoms][512 bytes]) as a 2-D tensor of 32-bit words, one
// row per 128-row block; a box is box_atoms atoms of 512 bytes (those of one pipeline stage) x box_rows.
// pitch_atoms: atoms between consecutive row blocks when the map covers a K slice of a wider packed array (0 = k_atoms).
int make_scale_map(CUtensorMap* map, const void* base, int row_blocks, int k_atoms, int box_rows, int box_atoms = 2,
                   int pitch_atoms = 0) {
  const MapKey k{base, (unsigned long long)k_atoms * 128, (unsigned long long)row_blocks,
                 (unsigned long long)(pitch_atoms ? pitch_atoms : k_atoms) * 512,
                 unsigned(box_atoms) * 128u, unsigned(box_rows), int(CU_TENSOR_MAP_DATA_TYPE_UINT32), int(CU_TENSOR_MAP_SWIZZLE_NONE),
                 int(CU_TENSOR_MAP_L2_PROMOTION_L2_256B)};
  CUresult r = encode_2d(map, k);
  if (r != CUDA_SUCCESS)
    return fail(WB200_ERR_CUDA, "cuTensorMapEncodeTiled (scales) failed with CUresult %d (row blocks %d, atoms %d)", int(r),
                row_blocks, k_atoms);
  return WB200_OK;
}

// Raise a kernel's dynamic shared-memory limit once per device (the attribute is per device).
// `done` must be a flag array owned by the caller's template instantiation: this function
// template is instantiated per kernel TYPE, which several kernels share.
template <typename K>
int set_smem(K kernel, int bytes, bool* done) {
  int dev = 0;
  WB_CUDA(cudaGetDevice(&dev));
  if (!done[dev]) {
    WB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    done[dev] = true;
  }
  return WB200_OK;
}


int check_common(int M, int N, int K, const void* a, const void* as, const void* b, const void* bs, const void* c,
                 int c_dtype, long long ldc) {
  if (M <= 0 || N <= 0 || K <= 0) return fail(WB200_ERR_INVALID_ARG, "M, N, K must be positive (got %d, %d, %d)", M, N, K);
  if (K % 32 != 0) return fail(WB200_ERR_INVALID_ARG, "K = %d is not a multiple of the scale group size 32", K);
  if (!a || !as || !b || !bs || !c) return fail(WB200_ERR_INVALID_ARG, "null tensor pointer");
  if (c_dtype != WB200_F32 && c_dtype != WB200_BF16) return fail(WB200_ERR_INVALID_ARG, "unknown output dtype %d", c_dtype);
  if (ldc < N) return fail(WB200_ERR_INVALID_ARG, "ldc = %lld is smaller than N = %d", ldc, N);
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15))
    return fail(WB200_ERR_ALIGNMENT, "a and b must be 16-byte aligned");
  if ((reinterpret_cast<uintptr_t>(as) & 15) || (reinterpret_cast<uintptr_t>(bs) & 15))
    return fail(WB200_ERR_ALIGNMENT, "packed scale arrays must be 16-byte aligned");
  const int esz = (c_dtype == WB200_F32) ? 4 : 2;
  if (reinterpret_cast<uintptr_t>(c) % esz) return fail(WB200_ERR_ALIGNMENT, "c is not aligned to its element size");
  return WB200_OK;
}

// ------------------------------------------------------------------------------------------
// tile paths
// ------------------------------------------------------------------------------------------
// C as a 2-D tensor of output elements for TMA stores: box = 128 bytes (32 f32 or 64 bf16 columns) x 32
// rows with the 128-byte swizzle, the layout of the kernel's staging buffers.
int make_output_map(CUtensorMap* map, void* c, int M, int N, long long ldc, int esz) {
  const MapKey k{c, (unsigned long long)N, (unsigned long long)M, (unsigned long long)ldc * esz, unsigned(128 / esz), 32u,
                 int(esz == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16),
                 int(CU_TENSOR_MAP_SWIZZLE_128B), int(CU_TENSOR_MAP_L2_PROMOTION_NONE)};
  CUresult r = encode_2d(map, k);
  if (r != CUDA_SUCCESS)
    return fail(WB200_ERR_CUDA, "cuTensorMapEncodeTiled (output) failed with CUresult %d (M %d, N %d, ldc %lld)", int(r), M,
                N, ldc);
  return WB200_OK;
}

// C as a 2-D tensor for dense (unswizzled) boxes of box_cols x box_rows elements: the whole-tile decode kernel's stores.
int make_output_map_dense(CUtensorMap* map, void* c, int M, int N, long long ldc, int esz, int box_cols, int box_rows) {
  const MapKey k{c, (unsigned long long)N, (unsigned long long)M, (unsigned long long)ldc * esz, unsigned(box_cols), unsigned(box_rows),
                 int(esz == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16),
                 int(CU_TENSOR_MAP_SWIZZLE_NONE), int(CU_TENSOR_MAP_L2_PROMOTION_NONE)};
  CUresult r = encode_2d(map, k);
  if (r != CUDA_SUCCESS)
    return fail(WB200_ERR_CUDA, "cuTensorMapEncodeTiled (dense output) failed with CUresult %d (M %d, N %d, ldc %lld)", int(r), M, N, ldc);
  return WB200_OK;
}

// EB: bits per operand element (4: MXFP4, 8: MXFP8 with elem_format 0 = E4M3 / 1 = E5M2).
template <int CG, int BN, typename OutT, int EB = 4>
int launch_tile(const DeviceInfo& dev, int M, int N, int K, const void* a, const void* as, const void* b,
                const void* bs, void* c, long long ldc, int sfa_row_blocks, int sfb_row_blocks, int accumulate,
                cudaStream_t stream, int elem_format = 0) {
  using Cfg = wb::GemmCfg<CG, BN, int(sizeof(OutT)), EB>;
  wb::PlainMaps maps;
  CUtensorMap& tmA = maps.m[0];
  CUtensorMap& tmC = maps.m[4];
  const long long row_bytes = (long long)K * EB / 8;
  int rc = make_operand_map(&maps.m[0], a, M, row_bytes, Cfg::BM);
  if (rc) return rc;
  rc = weights_are_fp4(EB, elem_format) ? make_operand_map_u4(&maps.m[1], b, N, K, Cfg::B_ROWS)
                                        : make_operand_map(&maps.m[1], b, N, row_bytes, Cfg::B_ROWS);
  if (rc) return rc;
  rc = make_scale_map(&maps.m[2], as, sfa_row_blocks, wb::sf_k_atoms(K), 1, Cfg::SF_ATOMS);
  if (rc) return rc;
  rc = make_scale_map(&maps.m[3], bs, sfb_row_blocks, wb::sf_k_atoms(K), Cfg::SFB_BLOCKS, Cfg::SF_ATOMS);
  if (rc) return rc;
  wb::GemmParams p;
  p.c = c;
  p.M = M; p.N = N; p.K = K;
  p.ldc = int(ldc);
  p.tiles_m = (M + Cfg::BM * CG - 1) / (Cfg::BM * CG);
  p.tiles_n = (N + BN - 1) / BN;
  p.group_n = std::max(1, std::min(tl_group_n, p.tiles_n));
  const int esz = int(sizeof(OutT));
  p.vec_ok = ((reinterpret_cast<uintptr_t>(c) & 15) == 0 && (ldc * esz) % 16 == 0) ? 1 : 0;
  p.accumulate = accumulate;
  p.elem_format = elem_format;
  p.tma_store = (p.vec_ok && !accumulate) ? 1 : 0;
  if (p.tma_store) {
    rc = make_output_map(&tmC, c, M, N, ldc, esz);
    if (rc) return rc;
  } else {
    tmC = tmA;  // never dereferenced by the kernel on the direct-store path
  }
  p.status = dev.status_ptr;
  auto kernel = wb::mxfp4_gemm_kernel<CG, BN, OutT, wb::PlainMaps, EB>;
  static bool smem_set[kMaxDevices] = {};
  rc = set_smem(kernel, Cfg::SMEM_BYTES, smem_set);
  if (rc) return rc;
  const long long tiles = (long long)p.tiles_m * p.tiles_n;
  const int units = dev.sm_count / CG;  // CTAs or CTA pairs that fit at one per SM
  const int grid = int(tiles < units ? tiles : units) * CG;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(Cfg::THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CG;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = tl_dependent_launch ? 2 : 1;
  WB_CUDA(cudaLaunchKernelEx(&cfg, kernel, maps, p));
  return WB200_OK;
}

template <int CG, int BN>
int launch_tile_dtype(int c_dtype, const DeviceInfo& dev, int M, int N, int K, const void* a, const void* as,
                      const void* b, const void* bs, void* c, long long ldc, int sfa_rb, int sfb_rb,
                      int accumulate, cudaStream_t stream) {
  if (c_dtype == WB200_F32)
    return launch_tile<CG, BN, float>(dev, M, N, K, a, as, b, bs, c, ldc, sfa_rb, sfb_rb, accumulate, stream);
  return launch_tile<CG, BN, __nv_bfloat16>(dev, M, N, K, a, as, b, bs, c, ldc, sfa_rb, sfb_rb, accumulate, stream);
}

int dispatch_tile(unsigned path, int bn, int c_dtype, const DeviceInfo& dev, int M, int N, int K, const void* a,
                  const void* as, const void* b, const void* bs, void* c, long long ldc, int sfa_rb, int sfb_rb,
                  int accumulate, cudaStream_t stream) {
  if (path == WB200_PATH_TILE_2CTA) {
    if (bn == 128) return launch_tile_dtype<2, 128>(c_dtype, dev, M, N, K, a, as, b, bs, c, ldc, sfa_rb, sfb_rb, accumulate, stream);
    if (bn == 192) return launch_tile_dtype<2, 192>(c_dtype, dev, M, N, K, a, as, b, bs, c, ldc, sfa_rb, sfb_rb, accumulate, stream);
    if (bn == 224) return launch_tile_dtype<2, 224>(c_dtype, dev, M, N, K, a, as, b, bs, c, ldc, sfa_rb, (N + 223) / 224 * 2, accumulate, stream);
    return launch_tile_dtype<2, 256>(c_dtype, dev, M, N, K, a, as, b, bs, c, ldc, sfa_rb, sfb_rb, accumulate, stream);
  }
  if (bn == 128) return launch_tile_dtype<1, 128>(c_dtype, dev, M, N, K, a, as, b, bs, c, ldc, sfa_rb, sfb_rb, accumulate, stream);
  if (bn == 192) return launch_tile_dtype<1, 192>(c_dtype, dev, M, N, K, a, as, b, bs, c, ldc, sfa_rb, sfb_rb, accumulate, stream);
  return launch_tile_dtype<1, 256>(c_dtype, dev, M, N, K, a, as, b, bs, c, ldc, sfa_rb, sfb_rb, accumulate, stream);
}

// One persistent launch over the tiles of all groups (CTA pairs, 256 x 256 tiles, TMA-store epilogue).
template <typename OutT>
int launch_grouped(const DeviceInfo& dev, int num_groups, const int* row_offsets, const int* row_block_offsets, int N, int K,
                   const void* a, const void* a_sf, const void* const* b_ptrs, const void* const* b_sf_ptrs, void* c,
                   long long ldc, cudaStream_t stream, void* const* c_ptrs = nullptr, int store_mode = 1) {
  // c_ptrs (optional): group g writes its rows to the matrix that starts at c_ptrs[g] instead of to rows
  // row_offsets[g].. of c; the matrices may live in another GPU's memory mapped into this process.
  constexpr int CG = 2, BN = 256;
  using Cfg = wb::GemmCfg<CG, BN, int(sizeof(OutT))>;
  static wb::GroupedMaps maps;  // ~21 KB: too large for comfort on the stack; guarded by the mutex below
  static std::mutex mu;
  std::lock_guard<std::mutex> lk(mu);
  const int esz = int(sizeof(OutT));
  const int k_atoms = wb::sf_k_atoms(K);
  const size_t atom_row_bytes = size_t(k_atoms) * 512;
  const int tiles_n = (N + BN - 1) / BN;
  maps.num_groups = num_groups;
  maps.interleave = (c_ptrs != nullptr) ? 1 : 0;
  maps.aligned = 0;
  maps.tiles_max = 0;
  maps.tile_start[0] = 0;
  for (int g = 0; g < num_groups; ++g) {
    const int r0 = row_offsets[g], Mg = row_offsets[g + 1] - r0;
    maps.rows[g] = Mg;
    maps.tile_start[g + 1] = maps.tile_start[g] + ((Mg + Cfg::BM * CG - 1) / (Cfg::BM * CG)) * tiles_n;
    if (maps.tile_start[g + 1] - maps.tile_start[g] > maps.tiles_max) maps.tiles_max = maps.tile_start[g + 1] - maps.tile_start[g];
    if (Mg == 0) continue;
    const uint8_t* ag = static_cast<const uint8_t*>(a) + size_t(r0) * (K / 2);
    const uint8_t* asg = static_cast<const uint8_t*>(a_sf) + size_t(row_block_offsets[g]) * atom_row_bytes;
    uint8_t* cg = c_ptrs ? static_cast<uint8_t*>(c_ptrs[g]) : static_cast<uint8_t*>(c) + size_t(r0) * ldc * esz;
    int rc = check_common(Mg, N, K, ag, asg, b_ptrs[g], b_sf_ptrs[g], cg, esz == 4 ? WB200_F32 : WB200_BF16, ldc);
    if (rc) return rc;
    if (reinterpret_cast<uintptr_t>(cg) & 15) return fail(WB200_ERR_ALIGNMENT, "group %d: output must be 16-byte aligned", g);
    CUtensorMap* m = &maps.m[g * 5];
    if ((rc = make_operand_map(m + 0, ag, Mg, K / 2, Cfg::BM))) return rc;
    if ((rc = make_operand_map(m + 1, b_ptrs[g], N, K / 2, Cfg::B_ROWS))) return rc;
    if ((rc = make_scale_map(m + 2, asg, wb::sf_row_blocks(Mg), k_atoms, 1))) return rc;
    if ((rc = make_scale_map(m + 3, b_sf_ptrs[g], wb::sf_row_blocks(N), k_atoms, BN / 128))) return rc;
    if ((rc = make_output_map(m + 4, cg, Mg, N, ldc, esz))) return rc;
    maps.c_base[g] = cg;
  }
  const int tiles = maps.tile_start[num_groups];
  if (tiles == 0) return WB200_OK;
  wb::GemmParams p = {};
  p.c = c;  // not dereferenced: the grouped kernel writes through each group's output map
  p.M = row_offsets[num_groups]; p.N = N; p.K = K;
  p.ldc = int(ldc);
  p.tiles_m = 0;
  p.tiles_n = tiles_n;
  p.group_n = std::max(1, std::min(tl_group_n, p.tiles_n));
  p.vec_ok = 1;
  p.tma_store = store_mode;
  p.accumulate = 0;
  p.status = dev.status_ptr;
  auto kernel = wb::mxfp4_gemm_kernel<CG, BN, OutT, wb::GroupedMaps>;
  static bool smem_set[kMaxDevices] = {};
  int rc = set_smem(kernel, Cfg::SMEM_BYTES, smem_set);
  if (rc) return rc;
  const int units = dev.sm_count / CG;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((tiles < units ? tiles : units) * CG, 1, 1);
  cfg.blockDim = dim3(Cfg::THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CG;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  WB_CUDA(cudaLaunchKernelEx(&cfg, kernel, maps, p));
  return WB200_OK;
}

// Grouped GEMM over a block-aligned row layout described by DEVICE arrays (see GroupedMaps::aligned).
template <typename OutT, int BN = 256>
int launch_aligned(const DeviceInfo& dev, int num_groups, int max_rows, const int* expert_ids, const int* num_rows, int N, int K,
                   const void* a, const void* a_sf, const void* const* b_ptrs, const void* const* b_sf_ptrs, void* c,
                   long long ldc, cudaStream_t stream) {
  constexpr int CG = 2;
  using Cfg = wb::GemmCfg<CG, BN, int(sizeof(OutT))>;
  static wb::GroupedMaps maps;
  static std::mutex mu;
  std::lock_guard<std::mutex> lk(mu);
  const int esz = int(sizeof(OutT));
  const int k_atoms = wb::sf_k_atoms(K);
  maps.num_groups = num_groups;
  maps.interleave = 0;
  maps.aligned = 1;
  maps.tile_rows = Cfg::BM * CG;
  maps.tiles_m_cap = max_rows / (Cfg::BM * CG);
  maps.tiles_max = 0;
  maps.expert_ids = expert_ids;
  maps.num_rows = num_rows;
  maps.c_base[0] = c;
  for (int g = 0; g < num_groups; ++g) {
    int rc = check_common(max_rows, N, K, a, a_sf, b_ptrs[g], b_sf_ptrs[g], c, esz == 4 ? WB200_F32 : WB200_BF16, ldc);
    if (rc) return rc;
    CUtensorMap* m = &maps.m[g * 5];
    if ((rc = make_operand_map(m + 0, a, max_rows, K / 2, Cfg::BM))) return rc;
    if ((rc = make_operand_map(m + 1, b_ptrs[g], N, K / 2, Cfg::B_ROWS))) return rc;
    if ((rc = make_scale_map(m + 2, a_sf, wb::sf_row_blocks(max_rows), k_atoms, 1))) return rc;
    if ((rc = make_scale_map(m + 3, b_sf_ptrs[g], wb::sf_row_blocks(N), k_atoms, Cfg::SFB_BLOCKS))) return rc;
    if ((rc = make_output_map(m + 4, c, max_rows, N, ldc, esz))) return rc;
  }
  wb::GemmParams p = {};
  p.c = c;
  p.M = max_rows; p.N = N; p.K = K;
  p.ldc = int(ldc);
  p.tiles_m = maps.tiles_m_cap;
  p.tiles_n = (N + BN - 1) / BN;
  p.group_n = std::max(1, std::min(tl_group_n, p.tiles_n));
  p.vec_ok = 1;
  p.tma_store = 1;
  p.accumulate = 0;
  p.status = dev.status_ptr;
  auto kernel = wb::mxfp4_gemm_kernel<CG, BN, OutT, wb::GroupedMaps>;
  static bool smem_set[kMaxDevices] = {};
  int rc = set_smem(kernel, Cfg::SMEM_BYTES, smem_set);
  if (rc) return rc;
  const long long tiles = (long long)maps.tiles_m_cap * p.tiles_n;
  if (tiles == 0) return WB200_OK;
  const int units = dev.sm_count / CG;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(int(tiles < units ? tiles : units) * CG, 1, 1);
  cfg.blockDim = dim3(Cfg::THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CG;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  WB_CUDA(cudaLaunchKernelEx(&cfg, kernel, maps, p));
  return WB200_OK;
}

// ------------------------------------------------------------------------------------------
// split-K on the tile path: few output tiles, long K
// ------------------------------------------------------------------------------------------
constexpr size_t kCounterBytes = 16384;  // head of every workspace: the skinny path's tile counters (room for 4096 N tiles)

// How many K slices to cut a problem into so that its 256 x 256 tiles fill one wave of CTA pairs: 0 when the
// tiles alone fill at least half of them, or K is too short for slices of at least 4 pipeline stages.
int splitk_slices(int sm_count, int M, int N, int K) {
  if (M <= 128) return 0;
  const long long tiles = (long long)((M + 255) / 256) * ((N + 255) / 256);
  const int units = sm_count / 2, kb = (K + 255) / 256;
  if (tiles * 2 > units) return 0;
  long long s = units / tiles;
  if (s > kb / 4) s = kb / 4;
  if (s > wb::kMaxGroups) s = wb::kMaxGroups;
  return s >= 2 ? int(s) : 0;
}
size_t splitk_workspace_bytes(int slices, int M, int N) { return kCounterBytes + size_t(slices) * M * N * sizeof(float); }

// One persistent launch over (K slice, tile) pairs, slices walked round-robin, every slice writing its f32
// partial product to its own slot of the workspace; then one pass adds the slots in slice order.
template <typename OutT>
int launch_splitk(const DeviceInfo& dev, int slices, int M, int N, int K, const void* a, const void* as, const void* b,
                  const void* bs, void* c, long long ldc, void* workspace, int accumulate, cudaStream_t stream) {
  constexpr int CG = 2, BN = 256;
  using Cfg = wb::GemmCfg<CG, BN, 4>;
  static wb::GroupedMaps maps;
  static std::mutex mu;
  std::lock_guard<std::mutex> lk(mu);
  const int kb_total = (K + 255) / 256, kb_per = (kb_total + slices - 1) / slices;
  const int atoms_total = wb::sf_k_atoms(K);
  const int tiles_n = (N + BN - 1) / BN, tiles_m = (M + Cfg::BM * CG - 1) / (Cfg::BM * CG);
  float* slots = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + kCounterBytes);
  // The descriptor table depends on the operand addresses and the shape only: a caller that repeats a call
  // (the usual case) reuses the table built last time instead of looking up 5 maps per slice again.
  struct Key { const void *a, *as, *b, *bs, *ws; int M, N, K, slices, dev, zero; };  // 64 bytes, no padding (compared with memcmp)
  static Key last = {};
  static bool last_valid = false;
  static int last_used = 0;
  int cur_dev = 0;
  WB_CUDA(cudaGetDevice(&cur_dev));
  const Key key{a, as, b, bs, workspace, M, N, K, slices, cur_dev, 0};
  const bool reuse = last_valid && memcmp(&last, &key, sizeof(Key)) == 0;
  int used = reuse ? last_used : 0;
  if (!reuse) {
  last_valid = false;
  maps.num_groups = slices;
  maps.interleave = 1;
  maps.aligned = 0;
  maps.tiles_max = tiles_m * tiles_n;
  maps.tile_start[0] = 0;
  for (int g = 0; g < slices; ++g) {
    const int k0 = g * kb_per * 256;
    const int kg = (k0 >= K) ? 0 : ((K - k0 < kb_per * 256) ? K - k0 : kb_per * 256);
    maps.rows[g] = M;
    maps.tile_start[g + 1] = maps.tile_start[g] + (kg > 0 ? tiles_m * tiles_n : 0);
    if (kg == 0) continue;
    used = g + 1;
    const uint8_t* ag = static_cast<const uint8_t*>(a) + k0 / 2;
    const uint8_t* bg = static_cast<const uint8_t*>(b) + k0 / 2;
    const uint8_t* asg = static_cast<const uint8_t*>(as) + size_t(k0 / 128) * 512;
    const uint8_t* bsg = static_cast<const uint8_t*>(bs) + size_t(k0 / 128) * 512;
    float* cg = slots + size_t(g) * M * N;
    CUtensorMap* m = &maps.m[g * 5];
    int rc;
    if ((rc = make_operand_map(m + 0, ag, M, kg / 2, Cfg::BM, K / 2))) return rc;
    if ((rc = make_operand_map(m + 1, bg, N, kg / 2, Cfg::B_ROWS, K / 2))) return rc;
    if ((rc = make_scale_map(m + 2, asg, wb::sf_row_blocks(M), wb::sf_k_atoms(kg), 1, 2, atoms_total))) return rc;
    if ((rc = make_scale_map(m + 3, bsg, wb::sf_row_blocks(N), wb::sf_k_atoms(kg), BN / 128, 2, atoms_total))) return rc;
    if ((rc = make_output_map(m + 4, cg, M, N, N, 4))) return rc;
    maps.c_base[g] = cg;
  }
  last = key;
  last_used = used;
  last_valid = true;
  }
  wb::GemmParams p = {};
  p.c = slots;
  p.M = M; p.N = N; p.K = kb_per * 256;  // every slice runs kb_per stages; a shorter last slice reads zero fill
  p.ldc = N;
  p.tiles_m = tiles_m;
  p.tiles_n = tiles_n;
  p.group_n = std::max(1, std::min(tl_group_n, p.tiles_n));
  p.vec_ok = 1;
  p.tma_store = 1;
  p.accumulate = 0;
  p.status = dev.status_ptr;
  auto kernel = wb::mxfp4_gemm_kernel<CG, BN, float, wb::GroupedMaps>;
  static bool smem_set[kMaxDevices] = {};
  int rc = set_smem(kernel, Cfg::SMEM_BYTES, smem_set);
  if (rc) return rc;
  const long long tiles = (long long)maps.num_groups * maps.tiles_max;
  const int units = dev.sm_count / CG;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(int(tiles < units ? tiles : units) * CG, 1, 1);
  cfg.blockDim = dim3(Cfg::THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CG;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = tl_dependent_launch ? 2 : 1;
  WB_CUDA(cudaLaunchKernelEx(&cfg, kernel, maps, p));
  const long long vecs = (long long)M * ((N + 3) / 4);
  wb::splitk_reduce_kernel<OutT><<<unsigned((vecs + 255) / 256), 256, 0, stream>>>(slots, used, (long long)M * N, M, N,
                                                                                  static_cast<OutT*>(c), ldc, accumulate);
  WB_CUDA(cudaGetLastError());
  return WB200_OK;
}

// ------------------------------------------------------------------------------------------
// skinny path
// ------------------------------------------------------------------------------------------
size_t skinny_workspace_bytes(int sm_count, int M) {
  return kCounterBytes + size_t(2) * sm_count * M * 128 * sizeof(float);
}

template <int NP, int STAGES, typename OutT, int EB = 4>
int launch_skinny(const DeviceInfo& dev, int M, int N, int K, const void* a, const void* as, const void* b,
                  const void* bs, void* c, long long ldc, void* ws, int accumulate, cudaStream_t stream,
                  int elem_format = 0) {
  using Cfg = wb::SkinnyCfg<NP, STAGES, EB>;
  CUtensorMap tmW, tmX, tmSFW, tmSFX;
  const long long row_bytes = (long long)K * EB / 8;
  int rc = weights_are_fp4(EB, elem_format) ? make_operand_map_u4(&tmW, b, N, K, 128) : make_operand_map(&tmW, b, N, row_bytes, 128);
  if (rc) return rc;
  rc = make_operand_map(&tmX, a, M, row_bytes, NP);
  if (rc) return rc;
  rc = make_scale_map(&tmSFW, bs, wb::sf_row_blocks(N), wb::sf_k_atoms(K), 1, Cfg::SF_ATOMS);
  if (rc) return rc;
  rc = make_scale_map(&tmSFX, as, 1, wb::sf_k_atoms(K), 1, Cfg::SF_ATOMS);
  if (rc) return rc;
  wb::SkinnyParams p;
  p.c = c;
  p.counters = static_cast<unsigned int*>(ws);
  p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(ws) + kCounterBytes);
  p.M = M; p.N = N; p.K = K;
  p.ldc = int(ldc);
  p.tiles_n = (N + 127) / 128;
  p.num_kb = (K + Cfg::BK - 1) / Cfg::BK;
  p.accumulate = accumulate;
  p.dependent = tl_dependent_launch ? 1 : 0;
  p.elem_format = elem_format;
  p.status = dev.status_ptr;
  auto kernel = wb::mxfp4_skinny_kernel<NP, STAGES, OutT, EB>;
  static bool smem_set[kMaxDevices] = {};
  rc = set_smem(kernel, Cfg::SMEM_BYTES, smem_set);
  if (rc) return rc;
  const long long units = (long long)p.tiles_n * p.num_kb;
  const int grid = int(units < dev.sm_count ? units : dev.sm_count);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = tl_dependent_launch ? 1 : 0;
  WB_CUDA(cudaLaunchKernelEx(&cfg, kernel, tmW, tmX, tmSFW, tmSFX, p));
  WB_CUDA(cudaGetLastError());
  return WB200_OK;
}

// Whole N tiles taken from an atomic counter instead of a K split (skinny_whole_sm100.cuh), when there is at least one
// tile per SM. For M > 16 always: the K-split kernel's partial tiles (M x 128 f32 each) cost more than any imbalance
// (M = 128: 24.6 us against 29.4 us even at 150 tiles, where only two tiles are left for the second round). For M <= 16
// only when the tiles left over after the full rounds are none, or at least half a round, or a small part of the whole:
// a few stragglers alone run at one SM's bandwidth (150 tiles: 21.9 us whole against 19.2 us K-split; 185 tiles: 22.5
// against 19.9; 224 tiles: 23.3 against 24.9; 148 tiles: 15.7 against 16.4).
bool skinny_takes_whole_tiles(int sm_count, int M, int N, int elem_bits = 4) {
  const int tiles = (N + 127) / 128, rest = tiles % sm_count;
  if (tiles < sm_count) return false;
  if (M > 16) return true;
  // 8-bit operands stream twice the bytes per tile, so a partly empty last round costs twice as much: measured at
  // N = 28672, K = 8192, M = 16: 50.8 us with whole 128-row tiles against 42.5 us with the K split
  if (elem_bits == 8) return rest == 0;
  return rest == 0 || rest * 2 >= sm_count || tiles >= 4 * sm_count;
}

// Tile height that gives every SM the same number of tiles: with 128-row tiles the last round of the whole-tile
// kernel is partly empty (224 tiles on 148 SMs: the second round runs on 76 of them, each bounded by what one SM's
// ring can stream); rounds * SMs tiles of a smaller height, a multiple of 8, keep every SM streaming to the end.
int decode_tile_rows(int sm_count, int N) {
  const int tiles = (N + 127) / 128;
  if (tiles < sm_count || tiles % sm_count == 0) return 128;
  const long long slots = (long long)((tiles + sm_count - 1) / sm_count) * sm_count;
  const int h = int(((N + slots - 1) / slots + 7) / 8 * 8);
  // Low tiles pay when the last round of 128-row tiles is thin, but there the K-split kernel (usual packing) is the
  // better answer for M <= 16, and one packing serves every M: N = 19072 / 20480 (h = 72) 19.0 / 19.4 us against
  // 16.4 / 16.9 us at M = 16, while M = 128 gains under 1 us; from h = 88 up (N = 24576) no M loses.
  return (h >= 88 && h < 128) ? h : 128;
}

template <int NP, int STAGES, typename OutT, int EB = 4, int WR = 128, int SBUFS = 2>
int launch_skinny_whole(const DeviceInfo& dev, int M, int N, int K, const void* a, const void* as, const void* b,
                        const void* bs, void* c, long long ldc, void* ws, int accumulate, cudaStream_t stream,
                        int elem_format = 0) {
  using Base = wb::SkinnyCfg<NP, STAGES, EB, WR>;
  using Cfg = wb::SkinnyWholeCfg<NP, STAGES, EB, WR, SBUFS>;
  CUtensorMap tmW, tmX, tmSFW, tmSFX;
  const long long row_bytes = (long long)K * EB / 8;
  const int tile_rows = tl_b_tile_rows;  // 128 with the usual packing of the weight scales
  const int tiles_n = (N + tile_rows - 1) / tile_rows;
  int rc = weights_are_fp4(EB, elem_format) ? make_operand_map_u4(&tmW, b, N, K, tile_rows) : make_operand_map(&tmW, b, N, row_bytes, tile_rows);
  if (rc) return rc;
  rc = make_operand_map(&tmX, a, M, row_bytes, NP);
  if (rc) return rc;
  rc = make_scale_map(&tmSFW, bs, tiles_n, wb::sf_k_atoms(K), 1, Base::SF_ATOMS);
  if (rc) return rc;
  rc = make_scale_map(&tmSFX, as, 1, wb::sf_k_atoms(K), 1, Base::SF_ATOMS);
  if (rc) return rc;
  wb::SkinnyWholeParams p;
  p.c = c;
  p.counters = static_cast<unsigned int*>(ws);
  p.M = M; p.N = N; p.K = K;
  p.ldc = int(ldc);
  p.tiles_n = tiles_n;
  p.tile_rows = tile_rows;
  p.num_kb = (K + Base::BK - 1) / Base::BK;
  p.accumulate = accumulate;
  p.dependent = tl_dependent_launch ? 1 : 0;
  p.elem_format = elem_format;
  p.c_vec = ((reinterpret_cast<uintptr_t>(c) & 15) == 0 && (ldc * (long long)sizeof(OutT)) % 16 == 0) ? 1 : 0;
  // TMA stores of the staged chunks: 16-byte aligned C, no accumulation, and two staging halves that each hold a chunk
  // in the output type (the single-buffer variant has room for bf16 chunks only)
  p.tma_store = (p.c_vec && !accumulate && (sizeof(OutT) == 2 || SBUFS == 2)) ? 1 : 0;
  CUtensorMap tmC = {};
  if (p.tma_store) {
    rc = make_output_map_dense(&tmC, c, M, N, ldc, int(sizeof(OutT)), tile_rows, 16);
    if (rc) return rc;
  }
  p.status = dev.status_ptr;
  auto kernel = wb::mxfp4_skinny_whole_kernel<NP, STAGES, OutT, EB, WR, SBUFS>;
  static bool smem_set[kMaxDevices] = {};
  rc = set_smem(kernel, Cfg::SMEM_BYTES, smem_set);
  if (rc) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(dev.sm_count, 1, 1);  // one CTA per SM; every CTA's first tile is its own index (tiles >= SMs)
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = tl_dependent_launch ? 1 : 0;
  WB_CUDA(cudaLaunchKernelEx(&cfg, kernel, tmW, tmX, tmSFW, tmSFX, tmC, p));
  WB_CUDA(cudaGetLastError());
  return WB200_OK;
}

template <typename OutT, int EB = 4>
int dispatch_skinny(const DeviceInfo& dev, int M, int N, int K, const void* a, const void* as, const void* b,
                    const void* bs, void* c, long long ldc, void* ws, int accumulate, cudaStream_t stream,
                    int elem_format = 0) {
  if (tl_b_tile_rows != 128) {
    // the weight scales are packed per tile of that height: only the whole-tile kernel reads them that way
    if ((N + tl_b_tile_rows - 1) / tl_b_tile_rows < dev.sm_count)
      return fail(WB200_ERR_UNSUPPORTED, "weight scales packed for %d-row tiles need at least one tile per SM (N = %d, %d SMs); "
                  "pack them with wb200_repack_scales instead", tl_b_tile_rows, N, dev.sm_count);
  }
  if (tl_b_tile_rows <= 104) {
    // tiles of at most 104 rows: stages with room for 104 weight rows, so that the ring holds more of them
    if (M <= 16) return launch_skinny_whole<16, 12, OutT, EB, 104>(dev, M, N, K, a, as, b, bs, c, ldc, ws, accumulate, stream, elem_format);
    if (M <= 32) return launch_skinny_whole<32, 11, OutT, EB, 104>(dev, M, N, K, a, as, b, bs, c, ldc, ws, accumulate, stream, elem_format);
    if (M <= 64) return launch_skinny_whole<64, 9, OutT, EB, 104>(dev, M, N, K, a, as, b, bs, c, ldc, ws, accumulate, stream, elem_format);
    return launch_skinny_whole<128, 7, OutT, EB, 104, 1>(dev, M, N, K, a, as, b, bs, c, ldc, ws, accumulate, stream, elem_format);
  }
  if (tl_b_tile_rows != 128 || skinny_takes_whole_tiles(dev.sm_count, M, N, EB)) {
    if (M <= 16) return launch_skinny_whole<16, 10, OutT, EB>(dev, M, N, K, a, as, b, bs, c, ldc, ws, accumulate, stream, elem_format);
    if (M <= 32) return launch_skinny_whole<32, 9, OutT, EB>(dev, M, N, K, a, as, b, bs, c, ldc, ws, accumulate, stream, elem_format);
    if (M <= 64) return launch_skinny_whole<64, 8, OutT, EB>(dev, M, N, K, a, as, b, bs, c, ldc, ws, accumulate, stream, elem_format);
    return launch_skinny_whole<128, 6, OutT, EB>(dev, M, N, K, a, as, b, bs, c, ldc, ws, accumulate, stream, elem_format);
  }
  if (M <= 16) return launch_skinny<16, 10, OutT, EB>(dev, M, N, K, a, as, b, bs, c, ldc, ws, accumulate, stream, elem_format);
  if (M <= 32) return launch_skinny<32, 9, OutT, EB>(dev, M, N, K, a, as, b, bs, c, ldc, ws, accumulate, stream, elem_format);
  if (M <= 64) return launch_skinny<64, 8, OutT, EB>(dev, M, N, K, a, as, b, bs, c, ldc, ws, accumulate, stream, elem_format);
  return launch_skinny<128, 6, OutT, EB>(dev, M, N, K, a, as, b, bs, c, ldc, ws, accumulate, stream, elem_format);
}

// ------------------------------------------------------------------------------------------
// allocation-free skinny entry point: its scratch lives in the library image
// ------------------------------------------------------------------------------------------
constexpr int kNoAllocMaxM = 16;
constexpr int kNoAllocMaxN = 65536;
constexpr int kNoAllocMaxSMs = 160;
// Same layout as the caller-provided workspace of the skinny path: tile counters, then two f32
// partial tiles (M x 128) per CTA.
constexpr size_t kNoAllocScratchBytes = kCounterBytes + size_t(2) * kNoAllocMaxSMs * kNoAllocMaxM * 128 * sizeof(float);
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];
// In host code the name above is only a handle for the runtime, not a device address; the address
// is asked for once per device, with that device current.
void* g_noalloc_ptr[kMaxDevices] = {};

int noalloc_scratch(void** out) {
  int dev = 0;
  WB_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_noalloc_ptr[dev]) {
    void* ptr = nullptr;
    WB_CUDA(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
    if (!ptr) return fail(WB200_ERR_CUDA, "cudaGetSymbolAddress returned a null address for the scratch array");
    g_noalloc_ptr[dev] = ptr;
  }
  *out = g_noalloc_ptr[dev];
  return WB200_OK;
}

// Self-test of the bounded-wait machinery: one CTA waits on a barrier that nothing will ever signal,
// with a short limit. The wait gives up, records WB_DEV_TIMEOUT_SELFTEST in the status word and the
// kernel ends normally; no fault, trap or endless loop is involved.
__global__ void selftest_wait_timeout_kernel(int* status, long long limit_cycles) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0u;
    wb::mbar_init(wb::smem_u32(&bar), 1);
    wb::fence_mbar_init();
    wb::WaitCtx ctx{&abort_flag, status, limit_cycles};
    wb::mbar_wait(wb::smem_u32(&bar), 0u, ctx, wb::WB_DEV_TIMEOUT_SELFTEST);
  }
}

}  // namespace

extern "C" {

int wb200_version(void) { return 1000; }

const char* wb200_last_error(void) { return g_err; }

int wb200_check_device_status(void* stream, int* detail) {
  DeviceInfo* dev;
  int rc = get_device(&dev);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int word = 0;
  WB_CUDA(cudaMemcpyAsync(&word, dev->status_ptr, sizeof(int), cudaMemcpyDeviceToHost, s));
  WB_CUDA(cudaStreamSynchronize(s));
  if (detail) *detail = word;
  if (word != 0) {
    WB_CUDA(cudaMemsetAsync(dev->status_ptr, 0, sizeof(int), s));
    return fail(WB200_ERR_DEVICE_TIMEOUT, "device-side wait %d gave up in block %d; results of the last launches are invalid",
                word & 0xff, word >> 8);
  }
  return WB200_OK;
}

int wb200_selftest_wait_timeout(long long limit_cycles, void* stream) {
  if (limit_cycles <= 0 || limit_cycles > 200000000LL)
    return fail(WB200_ERR_INVALID_ARG, "selftest: limit of %lld cycles is outside (0, 2e8]", limit_cycles);
  DeviceInfo* dev;
  int rc = get_device(&dev);
  if (rc) return rc;
  selftest_wait_timeout_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(dev->status_ptr, limit_cycles);
  WB_CUDA(cudaGetLastError());
  return WB200_OK;
}

size_t wb200_packed_scale_bytes(int rows, int K) {
  if (rows <= 0 || K <= 0) return 0;
  return wb::sf_packed_bytes(rows, K);
}

int wb200_decode_tile_rows(int N) {
  if (N <= 0) return 128;
  DeviceInfo* dev;
  if (get_device(&dev)) return 128;
  return decode_tile_rows(dev->sm_count, N);
}

static bool tile_rows_ok(int tile_rows) { return (tile_rows >= 8 && tile_rows <= 128 && tile_rows % 8 == 0) || tile_rows == 224; }
static int tiled_row_blocks(int rows, int tile_rows) { return (rows + tile_rows - 1) / tile_rows * ((tile_rows + 127) / 128); }

size_t wb200_packed_scale_bytes_tiled(int rows, int K, int tile_rows) {
  if (rows <= 0 || K <= 0 || !tile_rows_ok(tile_rows)) return 0;
  return size_t(tiled_row_blocks(rows, tile_rows)) * wb::sf_k_atoms(K) * 512;
}

static int repack_scales_impl(const void* src, long long src_row_stride, int rows, int K, void* dst, void* stream,
                              bool broadcast, int block_rows = 128) {
  if (rows <= 0 || K <= 0 || K % 32 != 0)
    return fail(WB200_ERR_INVALID_ARG, "repack_scales: rows = %d, K = %d (K must be a positive multiple of 32)", rows, K);
  if (!src || !dst) return fail(WB200_ERR_INVALID_ARG, "repack_scales: null pointer");
  if (src_row_stride < (broadcast ? 1 : K / 32))
    return fail(WB200_ERR_INVALID_ARG, "repack_scales: row stride %lld < %d", src_row_stride, broadcast ? 1 : K / 32);
  if (reinterpret_cast<uintptr_t>(dst) & 15) return fail(WB200_ERR_ALIGNMENT, "repack_scales: dst must be 16-byte aligned");
  DeviceInfo* dev;
  int rc = get_device(&dev);
  if (rc) return rc;
  const int k_atoms = wb::sf_k_atoms(K);
  dim3 grid((k_atoms + 7) / 8, tiled_row_blocks(rows, block_rows));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(256, 1, 1);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = tl_dependent_launch ? 1 : 0;
  WB_CUDA(cudaLaunchKernelEx(&cfg, wb::repack_scales_kernel, static_cast<const uint8_t*>(src), src_row_stride, rows, K / 32,
                             k_atoms, static_cast<uint8_t*>(dst), broadcast, tl_dependent_launch, block_rows));
  return WB200_OK;
}

int wb200_repack_scales_tiled(const void* src, long long src_row_stride, int rows, int K, int tile_rows, void* dst, void* stream) {
  if (!tile_rows_ok(tile_rows))
    return fail(WB200_ERR_INVALID_ARG, "repack_scales_tiled: %d rows per tile (8 .. 128 in steps of 8, or 224)", tile_rows);
  return repack_scales_impl(src, src_row_stride, rows, K, dst, stream, false, tile_rows);
}

int wb200_repack_scales(const void* src, long long src_row_stride, int rows, int K, void* dst, void* stream) {
  return repack_scales_impl(src, src_row_stride, rows, K, dst, stream, false);
}

int wb200_repack_scales_broadcast(const void* src, long long src_row_stride, int rows, int K, void* dst, void* stream) {
  return repack_scales_impl(src, src_row_stride, rows, K, dst, stream, true);
}

int wb200_repack_scales_grouped(const void* src, long long src_row_stride, int num_groups, const int* row_offsets,
                                const int* row_block_offsets, int K, void* dst, void* stream) {
  if (num_groups <= 0 || num_groups > wb::kMaxRepackGroups || !row_offsets || !row_block_offsets)
    return fail(WB200_ERR_INVALID_ARG, "repack_scales_grouped: 1..%d groups with offset arrays (got %d)", wb::kMaxRepackGroups,
                num_groups);
  if (K <= 0 || K % 32 != 0) return fail(WB200_ERR_INVALID_ARG, "repack_scales_grouped: K = %d must be a positive multiple of 32", K);
  if (!src || !dst) return fail(WB200_ERR_INVALID_ARG, "repack_scales_grouped: null pointer");
  if (src_row_stride < K / 32) return fail(WB200_ERR_INVALID_ARG, "repack_scales_grouped: row stride %lld < K/32", src_row_stride);
  if (reinterpret_cast<uintptr_t>(dst) & 15) return fail(WB200_ERR_ALIGNMENT, "repack_scales_grouped: dst must be 16-byte aligned");
  wb::RepackGroups tab;
  tab.num_groups = num_groups;
  for (int g = 0; g <= num_groups; ++g) {
    tab.row_start[g] = row_offsets[g];
    tab.block_start[g] = row_block_offsets[g];
  }
  for (int g = 0; g < num_groups; ++g) {
    const int rows = row_offsets[g + 1] - row_offsets[g], blocks = row_block_offsets[g + 1] - row_block_offsets[g];
    if (rows < 0 || blocks < (rows + 127) / 128)
      return fail(WB200_ERR_INVALID_ARG, "repack_scales_grouped: group %d has %d rows but %d 128-row blocks", g, rows, blocks);
  }
  const int total_blocks = row_block_offsets[num_groups] - row_block_offsets[0];
  if (total_blocks == 0) return WB200_OK;
  DeviceInfo* dev;
  int rc = get_device(&dev);
  if (rc) return rc;
  const int k_atoms = wb::sf_k_atoms(K);
  dim3 grid((k_atoms + 7) / 8, total_blocks);
  wb::repack_scales_grouped_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(src), src_row_stride, tab, K / 32, k_atoms, static_cast<uint8_t*>(dst));
  WB_CUDA(cudaGetLastError());
  return WB200_OK;
}

int wb200_quantize_mxfp4(const void* x, int x_dtype, long long ldx, int rows, int K, void* q, void* scale_rowmajor,
                         void* scale_packed, void* stream) {
  if (rows <= 0 || K <= 0 || K % 32 != 0)
    return fail(WB200_ERR_INVALID_ARG, "quantize: rows = %d, K = %d (K must be a positive multiple of 32)", rows, K);
  if (!x || !q || (!scale_rowmajor && !scale_packed)) return fail(WB200_ERR_INVALID_ARG, "quantize: null pointer");
  if (x_dtype != WB200_F32 && x_dtype != WB200_BF16) return fail(WB200_ERR_INVALID_ARG, "quantize: unknown input dtype %d", x_dtype);
  if (ldx < K) return fail(WB200_ERR_INVALID_ARG, "quantize: ldx = %lld is smaller than K = %d", ldx, K);
  const int esz = (x_dtype == WB200_F32) ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (ldx * esz) % 16 != 0 || (reinterpret_cast<uintptr_t>(q) & 3))
    return fail(WB200_ERR_ALIGNMENT, "quantize: x rows must be 16-byte aligned and q 4-byte aligned");
  DeviceInfo* dev;
  int rc = get_device(&dev);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int k_atoms = wb::sf_k_atoms(K);
  if (scale_packed && (rows % 128 != 0 || (K / 32) % 8 != 0)) {
    const int rbs = wb::sf_row_blocks(rows);
    const long long total = (long long)rbs * k_atoms * 512;
    wb::fill_scale_padding_kernel<<<unsigned((total + 255) / 256), 256, 0, s>>>(static_cast<uint8_t*>(scale_packed), rows,
                                                                                  K / 32, k_atoms, rbs);
  }
  const dim3 blocks(rows, (K / 32 + 63) / 64);
  if (x_dtype == WB200_F32)
    wb::quantize_mxfp4_kernel<float><<<blocks, 256, 0, s>>>(static_cast<const float*>(x), ldx, rows, K, static_cast<uint8_t*>(q),
                                                            static_cast<uint8_t*>(scale_rowmajor),
                                                            static_cast<uint8_t*>(scale_packed), k_atoms);
  else
    wb::quantize_mxfp4_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(
        static_cast<const __nv_bfloat16*>(x), ldx, rows, K, static_cast<uint8_t*>(q), static_cast<uint8_t*>(scale_rowmajor),
        static_cast<uint8_t*>(scale_packed), k_atoms);
  WB_CUDA(cudaGetLastError());
  return WB200_OK;
}

int wb200_moe_align_block_size(const void* topk_ids, int ids_are_int64, int num_ids, int num_experts, int block_size,
                               int* sorted_ids, int sorted_capacity, int* expert_ids, int expert_ids_capacity,
                               int* num_tokens_post_pad, int* inverse, void* stream) {
  if (num_ids < 0 || num_experts <= 0 || block_size <= 0)
    return fail(WB200_ERR_INVALID_ARG, "moe_align_block_size: num_ids = %d, num_experts = %d, block_size = %d", num_ids,
                num_experts, block_size);
  if (num_experts > wb::kMoeMaxExperts)
    return fail(WB200_ERR_UNSUPPORTED, "moe_align_block_size: at most %d experts (got %d)", wb::kMoeMaxExperts, num_experts);
  if ((!topk_ids && num_ids > 0) || !sorted_ids || !expert_ids || !num_tokens_post_pad)
    return fail(WB200_ERR_INVALID_ARG, "moe_align_block_size: null pointer");
  const long long worst = (long long)num_ids + (long long)num_experts * (block_size - 1);
  if (sorted_capacity < worst || (long long)expert_ids_capacity * block_size < worst)
    return fail(WB200_ERR_INVALID_ARG,
                "moe_align_block_size: sorted_ids needs %lld entries and expert_ids %lld (got %d and %d)", worst,
                (worst + block_size - 1) / block_size, sorted_capacity, expert_ids_capacity);
  DeviceInfo* dev;
  int rc = get_device(&dev);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (ids_are_int64)
    wb::moe_align_block_size_kernel<long long><<<1, 1024, 0, s>>>(static_cast<const long long*>(topk_ids), num_ids, num_experts,
                                                                  block_size, sorted_capacity, sorted_ids, expert_ids,
                                                                  num_tokens_post_pad, inverse);
  else
    wb::moe_align_block_size_kernel<int><<<1, 1024, 0, s>>>(static_cast<const int*>(topk_ids), num_ids, num_experts, block_size,
                                                            sorted_capacity, sorted_ids, expert_ids, num_tokens_post_pad,
                                                            inverse);
  WB_CUDA(cudaGetLastError());
  return WB200_OK;
}

int wb200_moe_gather_rows(const void* src, long long src_pitch, int row_bytes, const int* sorted_ids, int num_rows,
                          int num_ids, int top_k, void* dst, long long dst_pitch, void* stream) {
  if (num_rows < 0 || row_bytes <= 0 || top_k <= 0 || num_ids < 0)
    return fail(WB200_ERR_INVALID_ARG, "moe_gather_rows: num_rows = %d, row_bytes = %d, top_k = %d", num_rows, row_bytes, top_k);
  if (num_rows == 0) return WB200_OK;
  if (!src || !sorted_ids || !dst) return fail(WB200_ERR_INVALID_ARG, "moe_gather_rows: null pointer");
  const int vec = !(row_bytes % 16 || src_pitch % 16 || dst_pitch % 16 || (reinterpret_cast<uintptr_t>(src) & 15) ||
                    (reinterpret_cast<uintptr_t>(dst) & 15));
  if (src_pitch < row_bytes || dst_pitch < row_bytes) return fail(WB200_ERR_INVALID_ARG, "moe_gather_rows: pitch smaller than a row");
  DeviceInfo* dev;
  int rc = get_device(&dev);
  if (rc) return rc;
  wb::moe_gather_rows_kernel<<<(num_rows + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(src), src_pitch, row_bytes, sorted_ids, num_rows, num_ids, top_k,
      static_cast<uint8_t*>(dst), dst_pitch, vec);
  WB_CUDA(cudaGetLastError());
  return WB200_OK;
}

extern "C++" {
template <typename T>
static int launch_silu(const void* x1, const void* x2, long long ld1, long long ld2, int rows, int n, void* out, long long ldo,
                       void* q, void* scale_rm, void* scale_packed, int k_atoms, const int* row_limit, cudaStream_t s) {
  auto ok = [&](const void* p, long long ld) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0 && (ld * sizeof(T)) % 16 == 0; };
  const bool vec = ok(x1, ld1) && ok(x2, ld2) && (!out || ok(out, ldo));
  const dim3 blocks(rows, ((n + 31) / 32 + 64 * wb::kSiluUnroll - 1) / (64 * wb::kSiluUnroll));
  if (vec)
    wb::silu_and_mul_kernel<T, true><<<blocks, 256, 0, s>>>(static_cast<const T*>(x1), static_cast<const T*>(x2), ld1, ld2, rows,
                                                            n, static_cast<T*>(out), ldo, static_cast<uint8_t*>(q),
                                                            static_cast<uint8_t*>(scale_rm),
                                                            static_cast<uint8_t*>(scale_packed), k_atoms, row_limit);
  else
    wb::silu_and_mul_kernel<T, false><<<blocks, 256, 0, s>>>(static_cast<const T*>(x1), static_cast<const T*>(x2), ld1, ld2,
                                                             rows, n, static_cast<T*>(out), ldo, static_cast<uint8_t*>(q),
                                                             static_cast<uint8_t*>(scale_rm),
                                                             static_cast<uint8_t*>(scale_packed), k_atoms, row_limit);
  WB_CUDA(cudaGetLastError());
  return WB200_OK;
}
}  // extern "C++"

int wb200_silu_and_mul(const void* x1, const void* x2, long long ld1, long long ld2, int dtype, int rows, int n, void* out,
                       long long ldo, void* q, void* scale_rowmajor, void* scale_packed, const int* num_rows, void* stream) {
  if (rows <= 0 || n <= 0) return fail(WB200_ERR_INVALID_ARG, "silu_and_mul: rows = %d, n = %d", rows, n);
  if (!x1 || !x2 || (!out && !q)) return fail(WB200_ERR_INVALID_ARG, "silu_and_mul: null pointer");
  if (dtype != WB200_F32 && dtype != WB200_BF16) return fail(WB200_ERR_INVALID_ARG, "silu_and_mul: unknown dtype %d", dtype);
  if (ld1 < n || ld2 < n || (out && ldo < n)) return fail(WB200_ERR_INVALID_ARG, "silu_and_mul: a row pitch is smaller than n = %d", n);
  if (q) {
    if (n % 32 != 0) return fail(WB200_ERR_INVALID_ARG, "silu_and_mul: quantised output needs n %% 32 == 0 (got %d)", n);
    if (!scale_rowmajor && !scale_packed) return fail(WB200_ERR_INVALID_ARG, "silu_and_mul: q given without a scale output");
    if (reinterpret_cast<uintptr_t>(q) & 3) return fail(WB200_ERR_ALIGNMENT, "silu_and_mul: q must be 4-byte aligned");
  }
  DeviceInfo* dev;
  int rc = get_device(&dev);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int k_atoms = q ? wb::sf_k_atoms(n) : 0;
  if (q && scale_packed && (rows % 128 != 0 || (n / 32) % 8 != 0)) {
    const int rbs = wb::sf_row_blocks(rows);
    const long long total = (long long)rbs * k_atoms * 512;
    wb::fill_scale_padding_kernel<<<unsigned((total + 255) / 256), 256, 0, s>>>(static_cast<uint8_t*>(scale_packed), rows,
                                                                                  n / 32, k_atoms, rbs);
  }
  if (dtype == WB200_F32)
    return launch_silu<float>(x1, x2, ld1, ld2, rows, n, out, ldo, q, scale_rowmajor, scale_packed, k_atoms, num_rows, s);
  return launch_silu<__nv_bfloat16>(x1, x2, ld1, ld2, rows, n, out, ldo, q, scale_rowmajor, scale_packed, k_atoms, num_rows, s);
}

int wb200_moe_combine(const void* y, long long ldy, int dtype, const int* row_of, const float* weight, int tokens, int top_k,
                      int cols, void* out, long long ldo, void* stream) {
  if (tokens <= 0 || top_k <= 0 || cols <= 0)
    return fail(WB200_ERR_INVALID_ARG, "moe_combine: tokens = %d, top_k = %d, cols = %d", tokens, top_k, cols);
  if (!y || !row_of || !weight || !out) return fail(WB200_ERR_INVALID_ARG, "moe_combine: null pointer");
  if (dtype != WB200_F32 && dtype != WB200_BF16) return fail(WB200_ERR_INVALID_ARG, "moe_combine: unknown dtype %d", dtype);
  if (ldy < cols || ldo < cols) return fail(WB200_ERR_INVALID_ARG, "moe_combine: a row pitch is smaller than cols = %d", cols);
  DeviceInfo* dev;
  int rc = get_device(&dev);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long threads = (long long)tokens * ((cols + 3) / 4);
  const unsigned blocks = unsigned((threads + 255) / 256);
  if (dtype == WB200_F32)
    wb::moe_combine_kernel<float><<<blocks, 256, 0, s>>>(static_cast<const float*>(y), ldy, row_of, weight, tokens, top_k, cols,
                                                         static_cast<float*>(out), ldo);
  else
    wb::moe_combine_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(y), ldy, row_of, weight,
                                                                 tokens, top_k, cols, static_cast<__nv_bfloat16*>(out), ldo);
  WB_CUDA(cudaGetLastError());
  return WB200_OK;
}

int wb200_quantize_mxfp8(const void* x, int x_dtype, long long ldx, int rows, int K, int elem_format, void* q,
                         void* scale_rowmajor, void* scale_packed, void* stream) {
  if (rows <= 0 || K <= 0 || K % 32 != 0)
    return fail(WB200_ERR_INVALID_ARG, "quantize_mxfp8: rows = %d, K = %d (K must be a positive multiple of 32)", rows, K);
  if (!x || !q || (!scale_rowmajor && !scale_packed)) return fail(WB200_ERR_INVALID_ARG, "quantize_mxfp8: null pointer");
  if (x_dtype != WB200_F32 && x_dtype != WB200_BF16) return fail(WB200_ERR_INVALID_ARG, "quantize_mxfp8: unknown input dtype %d", x_dtype);
  if (elem_format != WB200_E4M3 && elem_format != WB200_E5M2) return fail(WB200_ERR_INVALID_ARG, "quantize_mxfp8: unknown element format %d", elem_format);
  if (ldx < K) return fail(WB200_ERR_INVALID_ARG, "quantize_mxfp8: ldx = %lld is smaller than K = %d", ldx, K);
  const int esz = (x_dtype == WB200_F32) ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (ldx * esz) % 16 != 0 || (reinterpret_cast<uintptr_t>(q) & 7))
    return fail(WB200_ERR_ALIGNMENT, "quantize_mxfp8: x rows must be 16-byte aligned and q 8-byte aligned");
  DeviceInfo* dev;
  int rc = get_device(&dev);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int k_atoms = wb::sf_k_atoms(K);
  if (scale_packed && (rows % 128 != 0 || (K / 32) % 8 != 0)) {
    const int rbs = wb::sf_row_blocks(rows);
    const long long total = (long long)rbs * k_atoms * 512;
    wb::fill_scale_padding_kernel<<<unsigned((total + 255) / 256), 256, 0, s>>>(static_cast<uint8_t*>(scale_packed), rows,
                                                                                  K / 32, k_atoms, rbs);
  }
  const dim3 blocks(rows, (K / 32 + 63) / 64);
  if (x_dtype == WB200_F32)
    wb::quantize_mxfp8_kernel<float><<<blocks, 256, 0, s>>>(static_cast<const float*>(x), ldx, rows, K, elem_format,
                                                            static_cast<uint8_t*>(q), static_cast<uint8_t*>(scale_rowmajor),
                                                            static_cast<uint8_t*>(scale_packed), k_atoms);
  else
    wb::quantize_mxfp8_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), ldx, rows, K, elem_format,
                                                                    static_cast<uint8_t*>(q), static_cast<uint8_t*>(scale_rowmajor),
                                                                    static_cast<uint8_t*>(scale_packed), k_atoms);
  WB_CUDA(cudaGetLastError());
  return WB200_OK;
}

int wb200_moe_quantize_scatter(const void* x, int x_dtype, long long ldx, int tokens, int K, int top_k, const int* dst_rows,
                               void* q, void* scale_rowmajor, void* stream) {
  if (tokens <= 0 || K <= 0 || K % 32 != 0 || top_k <= 0)
    return fail(WB200_ERR_INVALID_ARG, "moe_quantize_scatter: tokens = %d, K = %d, top_k = %d", tokens, K, top_k);
  if (!x || !dst_rows || !q || !scale_rowmajor) return fail(WB200_ERR_INVALID_ARG, "moe_quantize_scatter: null pointer");
  if (x_dtype != WB200_F32 && x_dtype != WB200_BF16) return fail(WB200_ERR_INVALID_ARG, "moe_quantize_scatter: unknown input dtype %d", x_dtype);
  if (ldx < K) return fail(WB200_ERR_INVALID_ARG, "moe_quantize_scatter: ldx = %lld is smaller than K = %d", ldx, K);
  const int esz = (x_dtype == WB200_F32) ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (ldx * esz) % 16 != 0 || (reinterpret_cast<uintptr_t>(q) & 3))
    return fail(WB200_ERR_ALIGNMENT, "moe_quantize_scatter: x rows must be 16-byte aligned and q 4-byte aligned");
  DeviceInfo* dev;
  int rc = get_device(&dev);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 blocks(tokens, (K / 32 + 63) / 64);
  if (x_dtype == WB200_F32)
    wb::quantize_scatter_mxfp4_kernel<float><<<blocks, 256, 0, s>>>(static_cast<const float*>(x), ldx, tokens, K, top_k, dst_rows,
                                                                    static_cast<uint8_t*>(q), static_cast<uint8_t*>(scale_rowmajor));
  else
    wb::quantize_scatter_mxfp4_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), ldx, tokens, K,
                                                                            top_k, dst_rows, static_cast<uint8_t*>(q),
                                                                            static_cast<uint8_t*>(scale_rowmajor));
  WB_CUDA(cudaGetLastError());
  return WB200_OK;
}

int wb200_mxfp4_dequant(const void* q, const void* scale, int rows, int K, float* out, void* stream) {
  if (rows <= 0 || K <= 0 || K % 32 != 0)
    return fail(WB200_ERR_INVALID_ARG, "dequant: rows = %d, K = %d (K must be a positive multiple of 32)", rows, K);
  if (!q || !scale || !out) return fail(WB200_ERR_INVALID_ARG, "dequant: null pointer");
  if (reinterpret_cast<uintptr_t>(out) & 7) return fail(WB200_ERR_ALIGNMENT, "dequant: out must be 8-byte aligned");
  DeviceInfo* dev;
  int rc = get_device(&dev);
  if (rc) return rc;
  const long long total = (long long)rows * (K / 2);
  const unsigned blocks = unsigned((total + 255) / 256);
  wb::dequant_mxfp4_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(q), static_cast<const uint8_t*>(scale), rows, K, out);
  WB_CUDA(cudaGetLastError());
  return WB200_OK;
}

size_t wb200_mxfp4_gemm_workspace_bytes(int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  // The skinny path's buffer is sized for up to 160 SMs so that it fits any sm_100 part. The split-K slice count
  // depends on the SM count: take the largest need over the current device's count, when there is one, and the
  // counts of the sm_100 parts, so that the size serves whichever of them runs the call.
  if (M <= 128) return skinny_workspace_bytes(160, M);
  int counts[4] = {132, 148, 160, 0};
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess)
    counts[3] = sms;
  else
    (void)cudaGetLastError();
  size_t need = 0;
  for (int sm : counts) {
    if (sm <= 0) continue;
    const int slices = splitk_slices(sm, M, N, K);
    const size_t n = slices ? splitk_workspace_bytes(slices, M, N) : 0;
    if (n > need) need = n;
  }
  return need;
}

int wb200_workspace_init(void* workspace, size_t bytes, void* stream) {
  if (!workspace || bytes == 0) return fail(WB200_ERR_INVALID_ARG, "workspace_init: empty workspace");
  const size_t n = bytes < kCounterBytes ? bytes : kCounterBytes;
  WB_CUDA(cudaMemsetAsync(workspace, 0, n, static_cast<cudaStream_t>(stream)));
  return WB200_OK;
}

int wb200_mxfp4_gemm(int M, int N, int K, const void* a, const void* a_scale_packed, const void* b,
                     const void* b_scale_packed, void* c, int c_dtype, long long ldc, void* workspace,
                     size_t workspace_bytes, unsigned flags, void* stream) {
  int rc = check_common(M, N, K, a, a_scale_packed, b, b_scale_packed, c, c_dtype, ldc);
  if (rc) return rc;
  DeviceInfo* dev;
  rc = get_device(&dev);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  unsigned path = flags & WB200_PATH_MASK;
  if ((flags & ~(WB200_PATH_MASK | WB200_TILE_N128 | WB200_TILE_N192 | WB200_ACCUMULATE | WB200_OVERLAP_PREVIOUS | WB200_GROUP_N_MASK |
                 WB200_B_TILE_ROWS_MASK)) != 0)
    return fail(WB200_ERR_INVALID_ARG, "unknown flag bits %#x", flags);
  GroupNScope group_scope(flags);
  struct TileRowsScope {
    int saved;
    explicit TileRowsScope(int h) : saved(tl_b_tile_rows) { tl_b_tile_rows = h; }
    ~TileRowsScope() { tl_b_tile_rows = saved; }
  } tile_rows_scope(b_tile_rows_from_flags(flags));
  const bool wide224 = tl_b_tile_rows == 224;  // weight scales packed for the tile kernel's 224-column tiles
  if (wide224) {
    if (M <= 128 || (path != WB200_PATH_AUTO && path != WB200_PATH_TILE_2CTA) || (flags & (WB200_TILE_N128 | WB200_TILE_N192)))
      return fail(WB200_ERR_UNSUPPORTED, "weight scales packed per 224-row tile are read by the CTA-pair tile kernel only (M > 128, "
                  "WB200_PATH_AUTO or WB200_PATH_TILE_2CTA, no other tile width forced; M = %d, flags %#x)", M, flags);
    path = WB200_PATH_TILE_2CTA;
  } else if (tl_b_tile_rows != 128) {
    if (tl_b_tile_rows > 128) return fail(WB200_ERR_INVALID_ARG, "WB200_B_TILE_ROWS: %d rows per tile (8 .. 128 in steps of 8, or 224)", tl_b_tile_rows);
    if (M > 128 || (path != WB200_PATH_AUTO && path != WB200_PATH_SKINNY))
      return fail(WB200_ERR_UNSUPPORTED, "weight scales packed per %d-row tile are read by the M <= 128 kernel only (M = %d, path %u)",
                  tl_b_tile_rows, M, path);
  }
  // restores the previous value on every return path
  struct DependentScope {
    bool saved;
    explicit DependentScope(bool on) : saved(tl_dependent_launch) { if (on) tl_dependent_launch = true; }
    ~DependentScope() { tl_dependent_launch = saved; }
  } dependent_scope((flags & WB200_OVERLAP_PREVIOUS) != 0);
  if (path > WB200_PATH_TILE_SPLITK) return fail(WB200_ERR_INVALID_ARG, "unknown path flag %u", path);
  if ((flags & WB200_TILE_N128) && (flags & WB200_TILE_N192)) return fail(WB200_ERR_INVALID_ARG, "two tile widths forced at once");
  const int accumulate = (flags & WB200_ACCUMULATE) ? 1 : 0;
  const int slices = splitk_slices(dev->sm_count, M, N, K);
  const bool splitk_ok = slices >= 2 && workspace && workspace_bytes >= splitk_workspace_bytes(slices, M, N) &&
                         (reinterpret_cast<uintptr_t>(workspace) & 15) == 0 && N % 4 == 0;
  if (path == WB200_PATH_AUTO) {
    const bool ws_ok = workspace && workspace_bytes >= skinny_workspace_bytes(dev->sm_count, M);
    if (M <= 128 && ws_ok) path = WB200_PATH_SKINNY;
    // split-K pays from three slices up; with two, 128-wide tiles do better (1024 x 2048 x 16000: 21.7 us
    // with two slices, 18.6 us with 128-wide tiles, 24.3 us with neither)
    else if (splitk_ok && slices >= 3 && !(flags & (WB200_TILE_N128 | WB200_TILE_N192))) path = WB200_PATH_TILE_SPLITK;
    else path = (M > 128) ? WB200_PATH_TILE_2CTA : WB200_PATH_TILE_1CTA;
  }
  if (tl_b_tile_rows != 128 && !wide224 && path != WB200_PATH_SKINNY)
    return fail(WB200_ERR_WORKSPACE, "weight scales packed per %d-row tile need the M <= 128 kernel, which needs a workspace of %zu bytes",
                tl_b_tile_rows, skinny_workspace_bytes(dev->sm_count, M));
  if (path == WB200_PATH_TILE_SPLITK) {
    if (!splitk_ok)
      return fail(slices >= 2 ? WB200_ERR_WORKSPACE : WB200_ERR_UNSUPPORTED,
                  "the split-K tile path needs M > 128, at most %d output tiles of 256 x 256, K >= 2048, N %% 4 == 0 and a 16-byte "
                  "aligned workspace of wb200_mxfp4_gemm_workspace_bytes(M, N, K) bytes", dev->sm_count / 4);
    if (c_dtype == WB200_F32)
      return launch_splitk<float>(*dev, slices, M, N, K, a, a_scale_packed, b, b_scale_packed, c, ldc, workspace, accumulate, s);
    return launch_splitk<__nv_bfloat16>(*dev, slices, M, N, K, a, a_scale_packed, b, b_scale_packed, c, ldc, workspace, accumulate, s);
  }
  if (path == WB200_PATH_SKINNY) {
    if (M > 128) return fail(WB200_ERR_UNSUPPORTED, "the skinny path handles M <= 128 (got %d)", M);
    if (N > 4096 * 128) return fail(WB200_ERR_UNSUPPORTED, "the skinny path handles N <= 524288 (got %d)", N);
    if (!workspace || workspace_bytes < skinny_workspace_bytes(dev->sm_count, M))
      return fail(WB200_ERR_WORKSPACE, "the skinny path needs a workspace of %zu bytes (got %zu)",
                  skinny_workspace_bytes(dev->sm_count, M), workspace ? workspace_bytes : size_t(0));
    if (reinterpret_cast<uintptr_t>(workspace) & 15) return fail(WB200_ERR_ALIGNMENT, "workspace must be 16-byte aligned");
    if (c_dtype == WB200_F32)
      return dispatch_skinny<float>(*dev, M, N, K, a, a_scale_packed, b, b_scale_packed, c, ldc, workspace, accumulate, s);
    return dispatch_skinny<__nv_bfloat16>(*dev, M, N, K, a, a_scale_packed, b, b_scale_packed, c, ldc, workspace, accumulate, s);
  }
  // Narrow problems fill more SMs with 128-wide tiles.
  int bn = (flags & WB200_TILE_N128) ? 128 : (flags & WB200_TILE_N192) ? 192 : 256;
  if (!(flags & (WB200_TILE_N128 | WB200_TILE_N192)) && (flags & WB200_PATH_MASK) == WB200_PATH_AUTO) {
    // 128-wide tiles when the 256-wide ones would leave at least half of the CTAs (or CTA pairs) idle: halving
    // the tile then doubles the parallelism; above that, two waves of half tiles lose to one wave of whole ones
    // (2048 x 2048 x 16000: 31.5 us with 128, 25.8 us with 256).
    const long long tile_rows = (path == WB200_PATH_TILE_2CTA) ? 256 : 128;
    const long long tiles256 = ((M + tile_rows - 1) / tile_rows) * ((N + 255) / 256);
    const long long units_now = (path == WB200_PATH_TILE_2CTA) ? dev->sm_count / 2 : dev->sm_count;
    if (tiles256 * 2 <= units_now) {
      bn = 128;
    } else if (path == WB200_PATH_TILE_2CTA) {
      // 192-wide tiles cost ~4 % more per column (more operand traffic per flop, measured on
      // large shapes) but can fill the last wave of CTA pairs better: compare whole waves.
      const long long units = dev->sm_count / 2, tm = (M + 255) / 256;
      const long long w256 = (tm * ((N + 255) / 256) + units - 1) / units * 256;
      const long long w192 = (tm * ((N + 191) / 192) + units - 1) / units * 192;
      if (w192 * 1045 < w256 * 1000) bn = 192;
    }
  }
  if (wide224) bn = 224;
  return dispatch_tile(path, bn, c_dtype, *dev, M, N, K, a, a_scale_packed, b, b_scale_packed, c, ldc,
                       wb::sf_row_blocks(M), wb::sf_row_blocks(N), accumulate, s);
}

int wb200_mxfp4_gemm_repack_a(int M, int N, int K, const void* a, const void* a_scale, long long a_scale_stride,
                              void* a_scale_scratch, const void* b, const void* b_scale_packed, void* c, int c_dtype,
                              long long ldc, void* workspace, size_t workspace_bytes, unsigned flags, void* stream) {
  if (!a_scale_scratch) return fail(WB200_ERR_INVALID_ARG, "gemm_repack_a: null scratch for the packed activation scales");
  tl_dependent_launch = (flags & WB200_OVERLAP_PREVIOUS) != 0;  // the repack kernel itself overlaps the previous kernel's tail
  int rc = wb200_repack_scales(a_scale, a_scale_stride, M, K, a_scale_scratch, stream);
  tl_dependent_launch = false;
  if (rc) return rc;
  tl_dependent_launch = true;  // the GEMM is the repack kernel's programmatic dependent
  rc = wb200_mxfp4_gemm(M, N, K, a, a_scale_scratch, b, b_scale_packed, c, c_dtype, ldc, workspace, workspace_bytes, flags, stream);
  tl_dependent_launch = false;
  return rc;
}

extern "C++" {
template <int CG, int BN>
static int launch_mxfp8(int c_dtype, const DeviceInfo& dev, int M, int N, int K, const void* a, const void* as, const void* b,
                        const void* bs, void* c, long long ldc, int accumulate, cudaStream_t s, int elem_format) {
  if (c_dtype == WB200_F32)
    return launch_tile<CG, BN, float, 8>(dev, M, N, K, a, as, b, bs, c, ldc, wb::sf_row_blocks(M), wb::sf_row_blocks(N),
                                         accumulate, s, elem_format);
  return launch_tile<CG, BN, __nv_bfloat16, 8>(dev, M, N, K, a, as, b, bs, c, ldc, wb::sf_row_blocks(M), wb::sf_row_blocks(N),
                                               accumulate, s, elem_format);
}
}  // extern "C++"

int wb200_mxfp8_gemm(int M, int N, int K, const void* a, const void* a_scale_packed, const void* b,
                     const void* b_scale_packed, void* c, int c_dtype, long long ldc, int elem_format, void* workspace,
                     size_t workspace_bytes, unsigned flags, void* stream) {
  int rc = check_common(M, N, K, a, a_scale_packed, b, b_scale_packed, c, c_dtype, ldc);
  if (rc) return rc;
  if ((elem_format & ~(1 | WB200_B_FP4)) != 0)
    return fail(WB200_ERR_INVALID_ARG, "mxfp8_gemm: unknown element format %#x (WB200_E4M3 or WB200_E5M2, optionally | WB200_B_FP4)", elem_format);
  if ((elem_format & WB200_B_FP4) && K % 128 != 0)
    return fail(WB200_ERR_UNSUPPORTED, "mxfp8_gemm with 4-bit weights needs K %% 128 == 0 (K = %d)", K);
  if ((flags & ~(WB200_PATH_MASK | WB200_TILE_N128 | WB200_ACCUMULATE | WB200_OVERLAP_PREVIOUS | WB200_GROUP_N_MASK | WB200_B_TILE_ROWS_MASK)) != 0)
    return fail(WB200_ERR_INVALID_ARG, "mxfp8_gemm: unknown flag bits %#x", flags);
  GroupNScope group_scope(flags);
  struct TileRowsScope {
    int saved;
    explicit TileRowsScope(int h) : saved(tl_b_tile_rows) { tl_b_tile_rows = h; }
    ~TileRowsScope() { tl_b_tile_rows = saved; }
  } tile_rows_scope(b_tile_rows_from_flags(flags));
  if (tl_b_tile_rows > 128)
    return fail(WB200_ERR_UNSUPPORTED, "mxfp8_gemm: weight scales packed per %d-row tile (the 8-bit GEMM reads heights of 8 .. 128 on its M <= 128 path)", tl_b_tile_rows);
  struct DependentScope {  // restores the previous value on every return path
    bool saved;
    explicit DependentScope(bool on) : saved(tl_dependent_launch) { if (on) tl_dependent_launch = true; }
    ~DependentScope() { tl_dependent_launch = saved; }
  } dependent_scope((flags & WB200_OVERLAP_PREVIOUS) != 0);
  unsigned path = flags & WB200_PATH_MASK;
  if (path > WB200_PATH_SKINNY)
    return fail(WB200_ERR_UNSUPPORTED, "mxfp8_gemm has the tile paths and the skinny path (path flag %u)", path);
  DeviceInfo* dev;
  rc = get_device(&dev);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int accumulate = (flags & WB200_ACCUMULATE) ? 1 : 0;
  const bool ws_ok = workspace && workspace_bytes >= skinny_workspace_bytes(dev->sm_count, M) &&
                     (reinterpret_cast<uintptr_t>(workspace) & 15) == 0;
  if (path == WB200_PATH_AUTO) path = (M <= 128 && ws_ok) ? WB200_PATH_SKINNY : (M > 128) ? WB200_PATH_TILE_2CTA : WB200_PATH_TILE_1CTA;
  if (tl_b_tile_rows != 128 && path != WB200_PATH_SKINNY)
    return fail(WB200_ERR_UNSUPPORTED, "mxfp8_gemm: weight scales packed per %d-row tile are read by the M <= 128 kernel only, which needs "
                "a workspace (M = %d, path %u)", tl_b_tile_rows, M, path);
  if (path == WB200_PATH_SKINNY) {
    if (M > 128) return fail(WB200_ERR_UNSUPPORTED, "the skinny path handles M <= 128 (got %d)", M);
    if (N > 4096 * 128) return fail(WB200_ERR_UNSUPPORTED, "the skinny path handles N <= 524288 (got %d)", N);
    if (!ws_ok)
      return fail(WB200_ERR_WORKSPACE, "the skinny path needs a 16-byte aligned workspace of %zu bytes (got %zu)",
                  skinny_workspace_bytes(dev->sm_count, M), workspace ? workspace_bytes : size_t(0));
    if (c_dtype == WB200_F32)
      return dispatch_skinny<float, 8>(*dev, M, N, K, a, a_scale_packed, b, b_scale_packed, c, ldc, workspace, accumulate, s, elem_format);
    return dispatch_skinny<__nv_bfloat16, 8>(*dev, M, N, K, a, a_scale_packed, b, b_scale_packed, c, ldc, workspace, accumulate, s, elem_format);
  }
  bool n128 = (flags & WB200_TILE_N128) != 0;
  if (!n128 && (flags & WB200_PATH_MASK) == WB200_PATH_AUTO)
    n128 = (long long)((M + 127) / 128) * ((N + 255) / 256) < dev->sm_count;
  if (path == WB200_PATH_TILE_2CTA)
    return n128 ? launch_mxfp8<2, 128>(c_dtype, *dev, M, N, K, a, a_scale_packed, b, b_scale_packed, c, ldc, accumulate, s, elem_format)
                : launch_mxfp8<2, 256>(c_dtype, *dev, M, N, K, a, a_scale_packed, b, b_scale_packed, c, ldc, accumulate, s, elem_format);
  return n128 ? launch_mxfp8<1, 128>(c_dtype, *dev, M, N, K, a, a_scale_packed, b, b_scale_packed, c, ldc, accumulate, s, elem_format)
              : launch_mxfp8<1, 256>(c_dtype, *dev, M, N, K, a, a_scale_packed, b, b_scale_packed, c, ldc, accumulate, s, elem_format);
}

int wb200_mxfp4_gemm_skinny_noalloc(int M, int N, int K, const void* a, const void* a_scale_packed, const void* b,
                                    const void* b_scale_packed, void* c, int c_dtype, long long ldc, unsigned flags,
                                    void* stream) {
  int rc = check_common(M, N, K, a, a_scale_packed, b, b_scale_packed, c, c_dtype, ldc);
  if (rc) return rc;
  if ((flags & ~WB200_ACCUMULATE) != 0)
    return fail(WB200_ERR_INVALID_ARG, "skinny_noalloc takes no flag other than WB200_ACCUMULATE (got %#x)", flags);
  if (M > kNoAllocMaxM)
    return fail(WB200_ERR_UNSUPPORTED, "skinny_noalloc handles M <= %d (got %d): its built-in scratch array is sized for that; "
                "use wb200_mxfp4_gemm with a workspace", kNoAllocMaxM, M);
  if (N > kNoAllocMaxN)
    return fail(WB200_ERR_UNSUPPORTED, "skinny_noalloc handles N <= %d (got %d): its built-in scratch array is sized for that; "
                "use wb200_mxfp4_gemm with a workspace", kNoAllocMaxN, N);
  DeviceInfo* dev;
  rc = get_device(&dev);
  if (rc) return rc;
  if (dev->sm_count > kNoAllocMaxSMs)
    return fail(WB200_ERR_UNSUPPORTED, "skinny_noalloc is sized for at most %d SMs (device has %d)", kNoAllocMaxSMs, dev->sm_count);
  void* scratch = nullptr;
  rc = noalloc_scratch(&scratch);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call left; the counters at its head must start at zero.
  WB_CUDA(cudaMemsetAsync(scratch, 0, kCounterBytes, s));
  const int accumulate = (flags & WB200_ACCUMULATE) ? 1 : 0;
  if (c_dtype == WB200_F32)
    return dispatch_skinny<float>(*dev, M, N, K, a, a_scale_packed, b, b_scale_packed, c, ldc, scratch, accumulate, s);
  return dispatch_skinny<__nv_bfloat16>(*dev, M, N, K, a, a_scale_packed, b, b_scale_packed, c, ldc, scratch, accumulate, s);
}

int wb200_mxfp4_moe_gemm(int num_experts, int max_rows, const int* expert_ids, const int* num_rows, int N, int K, const void* a,
                         const void* a_scale_packed, const void* const* b_ptrs, const void* const* b_scale_ptrs, void* c,
                         int c_dtype, long long ldc, void* stream) {
  if (num_experts <= 0 || num_experts > wb::kMaxGroups || !expert_ids || !num_rows || !b_ptrs || !b_scale_ptrs)
    return fail(WB200_ERR_INVALID_ARG, "moe_gemm: 1..%d experts with device routing arrays and weight pointers (got %d)",
                wb::kMaxGroups, num_experts);
  if (max_rows <= 0 || max_rows % 256 != 0)
    return fail(WB200_ERR_INVALID_ARG, "moe_gemm: max_rows = %d must be a positive multiple of 256 (the row-block size)", max_rows);
  if (c_dtype != WB200_F32 && c_dtype != WB200_BF16) return fail(WB200_ERR_INVALID_ARG, "unknown output dtype %d", c_dtype);
  const int esz = (c_dtype == WB200_F32) ? 4 : 2;
  if (!c || (reinterpret_cast<uintptr_t>(c) & 15) || (ldc * esz) % 16 != 0 || ldc < N)
    return fail(WB200_ERR_ALIGNMENT, "moe_gemm: c must be 16-byte aligned with a row pitch >= N that is a multiple of 16 bytes");
  DeviceInfo* dev;
  int rc = get_device(&dev);
  if (rc) return rc;
  if (c_dtype == WB200_F32)
    return launch_aligned<float>(*dev, num_experts, max_rows, expert_ids, num_rows, N, K, a, a_scale_packed, b_ptrs, b_scale_ptrs,
                                 c, ldc, static_cast<cudaStream_t>(stream));
  return launch_aligned<__nv_bfloat16>(*dev, num_experts, max_rows, expert_ids, num_rows, N, K, a, a_scale_packed, b_ptrs,
                                       b_scale_ptrs, c, ldc, static_cast<cudaStream_t>(stream));
}

int wb200_mxfp4_gemm_scatter_rows(int num_parts, const int* row_offsets, int N, int K, const void* a,
                                  const void* a_scale_packed, const void* b, const void* b_scale_packed, void* const* c_ptrs,
                                  int c_dtype, long long ldc, unsigned flags, void* stream) {
  if (flags & ~WB200_SCATTER_TMA_STORE) return fail(WB200_ERR_INVALID_ARG, "gemm_scatter_rows: unknown flag bits %#x", flags);
  const int store_mode = (flags & WB200_SCATTER_TMA_STORE) ? 1 : 2;
  if (num_parts <= 0 || num_parts > wb::kMaxGroups || !row_offsets || !c_ptrs)
    return fail(WB200_ERR_INVALID_ARG, "gemm_scatter_rows: 1..%d parts with row offsets and output pointers (got %d)",
                wb::kMaxGroups, num_parts);
  if (K <= 0 || K % 32 != 0) return fail(WB200_ERR_INVALID_ARG, "K = %d is not a positive multiple of 32", K);
  if (c_dtype != WB200_F32 && c_dtype != WB200_BF16) return fail(WB200_ERR_INVALID_ARG, "unknown output dtype %d", c_dtype);
  const int esz = (c_dtype == WB200_F32) ? 4 : 2;
  if (ldc < N || (ldc * esz) % 16 != 0) return fail(WB200_ERR_ALIGNMENT, "gemm_scatter_rows: ldc = %lld must be >= N and a multiple of 16 bytes", ldc);
  int block_offsets[wb::kMaxGroups + 1];
  const void* b_ptrs[wb::kMaxGroups];
  const void* b_sf_ptrs[wb::kMaxGroups];
  for (int g = 0; g <= num_parts; ++g) {
    if (g < num_parts && (row_offsets[g + 1] < row_offsets[g] || (row_offsets[g + 1] > row_offsets[g] && row_offsets[g] % 128 != 0)))
      return fail(WB200_ERR_INVALID_ARG, "gemm_scatter_rows: part %d must start at a multiple of 128 rows and not end before it starts", g);
    block_offsets[g] = (row_offsets[g] + 127) / 128;
    if (g < num_parts) { b_ptrs[g] = b; b_sf_ptrs[g] = b_scale_packed; }
  }
  DeviceInfo* dev;
  int rc = get_device(&dev);
  if (rc) return rc;
  if (c_dtype == WB200_F32)
    return launch_grouped<float>(*dev, num_parts, row_offsets, block_offsets, N, K, a, a_scale_packed, b_ptrs, b_sf_ptrs, nullptr,
                                 ldc, static_cast<cudaStream_t>(stream), c_ptrs, store_mode);
  return launch_grouped<__nv_bfloat16>(*dev, num_parts, row_offsets, block_offsets, N, K, a, a_scale_packed, b_ptrs, b_sf_ptrs,
                                       nullptr, ldc, static_cast<cudaStream_t>(stream), c_ptrs, store_mode);
}

int wb200_peer_buffer_create(size_t bytes, void** ptr, void* handle64) {
  if (!ptr || !handle64 || bytes == 0) return fail(WB200_ERR_INVALID_ARG, "peer_buffer_create: null pointer or empty buffer");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is exchanged as 64 bytes");
  void* p = nullptr;
  WB_CUDA(cudaMalloc(&p, bytes));
  cudaError_t e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle64), p);
  if (e != cudaSuccess) {
    cudaFree(p);
    WB_CUDA(e);
  }
  *ptr = p;
  return WB200_OK;
}

int wb200_peer_buffer_open(const void* handle64, void** ptr) {
  if (!ptr || !handle64) return fail(WB200_ERR_INVALID_ARG, "peer_buffer_open: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  WB_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return WB200_OK;
}

int wb200_peer_buffer_close(void* ptr) {
  if (ptr) WB_CUDA(cudaIpcCloseMemHandle(ptr));
  return WB200_OK;
}

int wb200_peer_buffer_destroy(void* ptr) {
  if (ptr) WB_CUDA(cudaFree(ptr));
  return WB200_OK;
}

#ifdef WB200_TRACE
// Measurement builds only (-DWB200_TRACE): copies the skinny kernel's per-CTA timeline of the last launch on the
// current device into `out` (8-byte words; returns the number of words per CTA, 0 on error). See skinny_sm100.cuh.
int wb200_trace_read(unsigned long long* out, int max_ctas) {
  if (!out || max_ctas <= 0 || max_ctas > 256) return 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return 0;
  if (cudaMemcpyFromSymbol(out, wb::g_skinny_trace, sizeof(unsigned long long) * size_t(max_ctas) * wb::kTraceWords) != cudaSuccess)
    return 0;
  return wb::kTraceWords;
}
#endif

extern "C++" {
// One thread evaluates a predicate that is false by construction and skips the (valid) store behind it: shows that a
// failed check is recorded and nothing else happens.
__global__ void checks_selftest_kernel(int* out, int n) {
  const int i = n;  // one past the end
  if (WB_CHECK(i < n, wb::kCheckSelfTest, i)) out[0] = 1;
}
}

int wb200_debug_checks(unsigned long long* record, int reset) {
#ifdef WB200_CHECKS
  if (!record) return fail(WB200_ERR_INVALID_ARG, "debug_checks: null record");
  WB_CUDA(cudaDeviceSynchronize());
  WB_CUDA(cudaMemcpyFromSymbol(record, wb::g_check_record, 3 * sizeof(unsigned long long)));
  if (reset) {
    const unsigned long long zero[3] = {0, 0, 0};
    WB_CUDA(cudaMemcpyToSymbol(wb::g_check_record, zero, sizeof(zero)));
  }
  return WB200_OK;
#else
  (void)record; (void)reset;
  return fail(WB200_ERR_UNSUPPORTED, "this library was built without -DWB200_CHECKS (python -m wave_b200.build --checks)");
#endif
}

int wb200_debug_checks_selftest(void* stream) {
#ifdef WB200_CHECKS
  DeviceInfo* dev;
  int rc = get_device(&dev);
  if (rc) return rc;
  checks_selftest_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(dev->status_ptr + 1, 1);
  WB_CUDA(cudaGetLastError());
  return WB200_OK;
#else
  (void)stream;
  return fail(WB200_ERR_UNSUPPORTED, "this library was built without -DWB200_CHECKS (python -m wave_b200.build --checks)");
#endif
}

int wb200_copy_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes, size_t rows, void* stream) {
  if (!dst || !src || width_bytes == 0 || rows == 0 || dst_pitch < width_bytes || src_pitch < width_bytes)
    return fail(WB200_ERR_INVALID_ARG, "copy_2d: null pointer, empty copy or a pitch smaller than the row width");
  WB_CUDA(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows, cudaMemcpyDefault, static_cast<cudaStream_t>(stream)));
  return WB200_OK;
}

int wb200_sum_slots(const float* slots, int num_slots, long long slot_stride, long long count, void* out, int out_dtype,
                    void* stream) {
  if (!slots || !out || num_slots <= 0 || count <= 0 || slot_stride < count)
    return fail(WB200_ERR_INVALID_ARG, "sum_slots: num_slots = %d, count = %lld, slot_stride = %lld", num_slots, count, slot_stride);
  if (out_dtype != WB200_F32 && out_dtype != WB200_BF16) return fail(WB200_ERR_INVALID_ARG, "sum_slots: unknown output dtype %d", out_dtype);
  if ((reinterpret_cast<uintptr_t>(slots) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) || slot_stride % 4 != 0)
    return fail(WB200_ERR_ALIGNMENT, "sum_slots: buffers must be 16-byte aligned and the slot stride a multiple of 4 elements");
  DeviceInfo* dev;
  int rc = get_device(&dev);
  if (rc) return rc;
  const long long vecs = (count + 3) / 4;
  const unsigned blocks = unsigned((vecs + 255) / 256);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (out_dtype == WB200_F32)
    wb::sum_slots_kernel<float><<<blocks, 256, 0, s>>>(slots, num_slots, slot_stride, count, static_cast<float*>(out));
  else
    wb::sum_slots_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(slots, num_slots, slot_stride, count,
                                                               static_cast<__nv_bfloat16*>(out));
  WB_CUDA(cudaGetLastError());
  return WB200_OK;
}

int wb200_mxfp4_grouped_gemm(int num_groups, const int* row_offsets, const int* row_block_offsets, int N, int K,
                             const void* a, const void* a_scale_packed, const void* const* b_ptrs,
                             const void* const* b_scale_ptrs, void* c, int c_dtype, long long ldc, void* stream) {
  if (num_groups <= 0 || !row_offsets || !row_block_offsets || !b_ptrs || !b_scale_ptrs)
    return fail(WB200_ERR_INVALID_ARG, "grouped gemm: bad group description");
  if (K <= 0 || K % 32 != 0) return fail(WB200_ERR_INVALID_ARG, "K = %d is not a positive multiple of 32", K);
  DeviceInfo* dev;
  int rc = get_device(&dev);
  if (rc) return rc;
  if (c_dtype != WB200_F32 && c_dtype != WB200_BF16) return fail(WB200_ERR_INVALID_ARG, "unknown output dtype %d", c_dtype);
  const int esz = (c_dtype == WB200_F32) ? 4 : 2;
  for (int g = 0; g < num_groups; ++g)
    if (row_offsets[g + 1] < row_offsets[g]) return fail(WB200_ERR_INVALID_ARG, "grouped gemm: row offsets decrease at group %d", g);
  // One persistent launch when the groups fit the kernel's descriptor table and c can take TMA stores;
  // otherwise one launch per group.
  if (num_groups <= wb::kMaxGroups && c && (reinterpret_cast<uintptr_t>(c) & 15) == 0 && (ldc * esz) % 16 == 0 && ldc >= N) {
    if (c_dtype == WB200_F32)
      return launch_grouped<float>(*dev, num_groups, row_offsets, row_block_offsets, N, K, a, a_scale_packed, b_ptrs,
                                   b_scale_ptrs, c, ldc, static_cast<cudaStream_t>(stream));
    return launch_grouped<__nv_bfloat16>(*dev, num_groups, row_offsets, row_block_offsets, N, K, a, a_scale_packed, b_ptrs,
                                         b_scale_ptrs, c, ldc, static_cast<cudaStream_t>(stream));
  }
  const size_t atom_row_bytes = size_t(wb::sf_k_atoms(K)) * 512;
  for (int g = 0; g < num_groups; ++g) {
    const int r0 = row_offsets[g], r1 = row_offsets[g + 1];
    if (r1 < r0) return fail(WB200_ERR_INVALID_ARG, "grouped gemm: row offsets decrease at group %d", g);
    const int Mg = r1 - r0;
    if (Mg == 0) continue;
    const uint8_t* ag = static_cast<const uint8_t*>(a) + size_t(r0) * (K / 2);
    const uint8_t* asg = static_cast<const uint8_t*>(a_scale_packed) + size_t(row_block_offsets[g]) * atom_row_bytes;
    uint8_t* cg = static_cast<uint8_t*>(c) + size_t(r0) * ldc * esz;
    rc = check_common(Mg, N, K, ag, asg, b_ptrs[g], b_scale_ptrs[g], cg, c_dtype, ldc);
    if (rc) return rc;
    const unsigned path = (Mg > 128) ? WB200_PATH_TILE_2CTA : WB200_PATH_TILE_1CTA;
    rc = dispatch_tile(path, 256, c_dtype, *dev, Mg, N, K, ag, asg, b_ptrs[g], b_scale_ptrs[g], cg, ldc,
                       wb::sf_row_blocks(Mg), wb::sf_row_blocks(N), 0, static_cast<cudaStream_t>(stream));
    if (rc) return rc;
  }
  return WB200_OK;
}

// ------------------------------------------------------------------------------------------
// N-sharded GEMM over several GPUs driven by one process
// ------------------------------------------------------------------------------------------
struct wb200_multi_gpu {
  wb::MultiGpu m;
};

int wb200_multi_gpu_shard_bounds(int N, int num_devices, int index, int granule, int* n0, int* n1) {
  if (N <= 0 || num_devices <= 0 || index < 0 || index >= num_devices || granule <= 0 || !n0 || !n1)
    return fail(WB200_ERR_INVALID_ARG, "shard_bounds: N = %d, num_devices = %d, index = %d, granule = %d", N, num_devices, index, granule);
  wb::shard_bounds(N, num_devices, index, granule, n0, n1);
  return WB200_OK;
}

int wb200_multi_gpu_num_devices(const wb200_multi_gpu_t* h) { return h ? int(h->m.devices.size()) : 0; }

int wb200_multi_gpu_destroy(wb200_multi_gpu_t* h) {
  if (!h) return WB200_OK;
  for (size_t g = 0; g < h->m.devices.size(); ++g) {
    wb::DeviceScope scope(h->m.devices[g]);
    if (g < h->m.streams.size() && h->m.streams[g]) {
      cudaStreamSynchronize(h->m.streams[g]);
      cudaStreamDestroy(h->m.streams[g]);
    }
    if (g < h->m.done.size() && h->m.done[g]) cudaEventDestroy(h->m.done[g]);
    if (g < h->m.t_begin.size() && h->m.t_begin[g]) cudaEventDestroy(h->m.t_begin[g]);
    if (g < h->m.t_end.size() && h->m.t_end[g]) cudaEventDestroy(h->m.t_end[g]);
  }
  delete h;
  return WB200_OK;
}

int wb200_multi_gpu_create(int num_devices, const int* device_ids, wb200_multi_gpu_t** out) {
  if (num_devices <= 0 || num_devices > kMaxDevices || !device_ids || !out)
    return fail(WB200_ERR_INVALID_ARG, "multi_gpu_create: num_devices = %d (1..%d) with a list of device ids", num_devices, kMaxDevices);
  int count = 0;
  WB_CUDA(cudaGetDeviceCount(&count));
  for (int i = 0; i < num_devices; ++i) {
    if (device_ids[i] < 0 || device_ids[i] >= count)
      return fail(WB200_ERR_INVALID_ARG, "multi_gpu_create: device id %d, but this process sees %d device(s)", device_ids[i], count);
    for (int j = 0; j < i; ++j)
      if (device_ids[j] == device_ids[i]) return fail(WB200_ERR_INVALID_ARG, "multi_gpu_create: device %d listed twice", device_ids[i]);
  }
  wb200_multi_gpu_t* h = new wb200_multi_gpu_t;
  h->m.devices.assign(device_ids, device_ids + num_devices);
  h->m.streams.assign(num_devices, nullptr);
  h->m.done.assign(num_devices, nullptr);
  h->m.t_begin.assign(num_devices, nullptr);
  h->m.t_end.assign(num_devices, nullptr);
  auto bail = [&](int rc) { wb200_multi_gpu_destroy(h); return rc; };
  for (int g = 0; g < num_devices; ++g) {
    wb::DeviceScope scope(device_ids[g]);
    if (!scope.ok) return bail(fail(WB200_ERR_CUDA, "multi_gpu_create: cannot make device %d current", device_ids[g]));
    DeviceInfo* info;
    int rc = get_device(&info);  // one-time set-up of the library on this device (and the sm_100 check)
    if (rc) return bail(rc);
    cudaError_t e = cudaStreamCreateWithFlags(&h->m.streams[g], cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->m.done[g], cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreate(&h->m.t_begin[g]);
    if (e == cudaSuccess) e = cudaEventCreate(&h->m.t_end[g]);
    if (e != cudaSuccess) return bail(fail(WB200_ERR_CUDA, "multi_gpu_create: %s on device %d", cudaGetErrorString(e), device_ids[g]));
    for (int j = 0; j < num_devices; ++j) {
      if (j == g) continue;
      int can = 0;
      if (cudaDeviceCanAccessPeer(&can, device_ids[g], device_ids[j]) == cudaSuccess && can) {
        e = cudaDeviceEnablePeerAccess(device_ids[j], 0);
        if (e != cudaSuccess) (void)cudaGetLastError();  // already enabled, or not possible: copies then go through the host
      }
    }
  }
  *out = h;
  return WB200_OK;
}

int wb200_multi_gpu_wait_for(wb200_multi_gpu_t* h, int device, void* stream) {
  if (!h) return fail(WB200_ERR_INVALID_ARG, "multi_gpu_wait_for: null handle");
  cudaEvent_t ev = nullptr;
  {
    wb::DeviceScope scope(device);
    if (!scope.ok) return fail(WB200_ERR_CUDA, "multi_gpu_wait_for: cannot make device %d current", device);
    WB_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    WB_CUDA(cudaEventRecord(ev, static_cast<cudaStream_t>(stream)));
  }
  for (size_t g = 0; g < h->m.devices.size(); ++g) {
    wb::DeviceScope scope(h->m.devices[g]);
    WB_CUDA(cudaStreamWaitEvent(h->m.streams[g], ev, 0));
  }
  WB_CUDA(cudaEventDestroy(ev));  // released once the waits queued above have been satisfied
  return WB200_OK;
}

int wb200_multi_gpu_broadcast_a(wb200_multi_gpu_t* h, int M, int K, const void* a, const void* a_scale, int src_device,
                                const wb200_device_operands* ops) {
  if (!h || !a || !a_scale || !ops || M <= 0 || K <= 0 || K % 32 != 0)
    return fail(WB200_ERR_INVALID_ARG, "multi_gpu_broadcast_a: M = %d, K = %d (a multiple of 32) and non-null arguments", M, K);
  (void)src_device;  // the copies take the direction from the addresses (unified addressing)
  const size_t a_bytes = size_t(M) * (K / 2), s_bytes = size_t(M) * (K / 32);
  for (size_t g = 0; g < h->m.devices.size(); ++g) {
    if (!ops[g].a || !ops[g].a_scale) return fail(WB200_ERR_INVALID_ARG, "multi_gpu_broadcast_a: device %zu has no buffer for a", g);
    wb::DeviceScope scope(h->m.devices[g]);
    if (ops[g].a != a) WB_CUDA(cudaMemcpyAsync(ops[g].a, a, a_bytes, cudaMemcpyDefault, h->m.streams[g]));
    if (ops[g].a_scale != a_scale) WB_CUDA(cudaMemcpyAsync(ops[g].a_scale, a_scale, s_bytes, cudaMemcpyDefault, h->m.streams[g]));
  }
  return WB200_OK;
}

int wb200_multi_gpu_gemm(wb200_multi_gpu_t* h, int M, int K, const int* n_bounds, const wb200_device_operands* ops,
                         int c_dtype, unsigned flags) {
  if (!h || !n_bounds || !ops) return fail(WB200_ERR_INVALID_ARG, "multi_gpu_gemm: null argument");
  const int G = int(h->m.devices.size());
  for (int g = 0; g < G; ++g)
    if (n_bounds[g + 1] < n_bounds[g] || (n_bounds[g + 1] > n_bounds[g] && n_bounds[g] % 128 != 0))
      return fail(WB200_ERR_INVALID_ARG, "multi_gpu_gemm: shard %d must start at a multiple of 128 rows and not end before it starts", g);
  for (int g = 0; g < G; ++g) {
    const int n_g = n_bounds[g + 1] - n_bounds[g];
    if (n_g == 0) continue;
    wb::DeviceScope scope(h->m.devices[g]);
    if (!scope.ok) return fail(WB200_ERR_CUDA, "multi_gpu_gemm: cannot make device %d current", h->m.devices[g]);
    const int rc = wb200_mxfp4_gemm_repack_a(M, n_g, K, ops[g].a, ops[g].a_scale, K / 32, ops[g].a_scale_packed, ops[g].b,
                                             ops[g].b_scale_packed, ops[g].c, c_dtype, ops[g].ldc, ops[g].workspace,
                                             ops[g].workspace_bytes, flags, h->m.streams[g]);
    if (rc) return rc;
  }
  return WB200_OK;
}

int wb200_multi_gpu_gather_c(wb200_multi_gpu_t* h, int M, const int* n_bounds, const wb200_device_operands* ops, int c_dtype,
                             int num_dst, void* const* dst_ptrs, const int* dst_devices, long long dst_ld) {
  if (!h || !n_bounds || !ops || num_dst < 0 || (num_dst > 0 && !dst_ptrs) || M <= 0)
    return fail(WB200_ERR_INVALID_ARG, "multi_gpu_gather_c: null argument");
  if (c_dtype != WB200_F32 && c_dtype != WB200_BF16) return fail(WB200_ERR_INVALID_ARG, "multi_gpu_gather_c: unknown dtype %d", c_dtype);
  (void)dst_devices;  // unified addressing: the copy finds its way from the addresses
  const size_t esz = (c_dtype == WB200_F32) ? 4 : 2;
  const int G = int(h->m.devices.size());
  if (dst_ld < n_bounds[G]) return fail(WB200_ERR_INVALID_ARG, "multi_gpu_gather_c: dst_ld = %lld is smaller than N = %d", dst_ld, n_bounds[G]);
  for (int j = 0; j < num_dst; ++j) {
    if (!dst_ptrs[j]) continue;
    for (int g = 0; g < G; ++g) {
      const int n_g = n_bounds[g + 1] - n_bounds[g];
      if (n_g == 0) continue;
      uint8_t* dst = static_cast<uint8_t*>(dst_ptrs[j]) + size_t(n_bounds[g]) * esz;
      if (dst == ops[g].c && dst_ld == ops[g].ldc) continue;  // the block was computed in place
      wb::DeviceScope scope(h->m.devices[g]);
      WB_CUDA(cudaMemcpy2DAsync(dst, size_t(dst_ld) * esz, ops[g].c, size_t(ops[g].ldc) * esz, size_t(n_g) * esz, size_t(M),
                                cudaMemcpyDefault, h->m.streams[g]));
    }
  }
  return WB200_OK;
}

int wb200_multi_gpu_join(wb200_multi_gpu_t* h, int device, void* stream) {
  if (!h) return fail(WB200_ERR_INVALID_ARG, "multi_gpu_join: null handle");
  for (size_t g = 0; g < h->m.devices.size(); ++g) {
    wb::DeviceScope scope(h->m.devices[g]);
    WB_CUDA(cudaEventRecord(h->m.done[g], h->m.streams[g]));
  }
  wb::DeviceScope scope(device);
  if (!scope.ok) return fail(WB200_ERR_CUDA, "multi_gpu_join: cannot make device %d current", device);
  for (size_t g = 0; g < h->m.devices.size(); ++g) WB_CUDA(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), h->m.done[g], 0));
  return WB200_OK;
}

int wb200_multi_gpu_synchronize(wb200_multi_gpu_t* h) {
  if (!h) return fail(WB200_ERR_INVALID_ARG, "multi_gpu_synchronize: null handle");
  int first = WB200_OK;
  for (size_t g = 0; g < h->m.devices.size(); ++g) {
    wb::DeviceScope scope(h->m.devices[g]);
    const int rc = wb200_check_device_status(h->m.streams[g], nullptr);  // synchronises the stream, reads the device's status word
    if (rc && !first) first = rc;
  }
  return first;
}

int wb200_multi_gpu_time_begin(wb200_multi_gpu_t* h) {
  if (!h) return fail(WB200_ERR_INVALID_ARG, "multi_gpu_time_begin: null handle");
  for (size_t g = 0; g < h->m.devices.size(); ++g) {
    wb::DeviceScope scope(h->m.devices[g]);
    WB_CUDA(cudaEventRecord(h->m.t_begin[g], h->m.streams[g]));
  }
  return WB200_OK;
}

int wb200_multi_gpu_time_end(wb200_multi_gpu_t* h, float* max_ms) {
  if (!h || !max_ms) return fail(WB200_ERR_INVALID_ARG, "multi_gpu_time_end: null argument");
  for (size_t g = 0; g < h->m.devices.size(); ++g) {
    wb::DeviceScope scope(h->m.devices[g]);
    WB_CUDA(cudaEventRecord(h->m.t_end[g], h->m.streams[g]));
  }
  float worst = 0.f;
  for (size_t g = 0; g < h->m.devices.size(); ++g) {
    wb::DeviceScope scope(h->m.devices[g]);
    WB_CUDA(cudaEventSynchronize(h->m.t_end[g]));
    float ms = 0.f;
    WB_CUDA(cudaEventElapsedTime(&ms, h->m.t_begin[g], h->m.t_end[g]));
    if (ms > worst) worst = ms;
  }
  *max_ms = worst;
  return WB200_OK;
}

}  // extern "C"
