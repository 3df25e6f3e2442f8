// Thin inline-PTX wrappers for the sm_100a features the MXFP4 kernels use:
// mbarrier, TMA (tiled and untiled bulk copies, never multicast), tensor memory
// allocation, tcgen05.cp / tcgen05.mma (kind::mxf4 block-scaled) / tcgen05.ld,
// and the smem / instruction descriptor encodings.
//
// Every wait in this file is bounded: when a wait runs out of time it records an
// error code in a device status word, raises a CTA-wide abort flag that makes all
// later waits return at once, and lets the kernel run to its normal end so that
// tensor memory is freed and no copy is left in flight.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "checks.cuh"

namespace wb {

// ---------------------------------------------------------------------------------------------
// status codes written to the device status word (0 = ok)
// ---------------------------------------------------------------------------------------------
enum : int {
  WB_DEV_OK = 0,
  WB_DEV_TIMEOUT_PRODUCER = 1,   // TMA producer waited too long for a free stage
  WB_DEV_TIMEOUT_MMA_FULL = 2,   // MMA issuer waited too long for a filled stage
  WB_DEV_TIMEOUT_MMA_ACC = 3,    // MMA issuer waited too long for a drained accumulator
  WB_DEV_TIMEOUT_EPILOGUE = 4,   // epilogue waited too long for a finished accumulator
  WB_DEV_TIMEOUT_SELFTEST = 7,   // the self-test kernel's wait on a barrier nobody signals
};

// About one second at 1.9 GHz. Generous next to the longest kernel here (a few ms).
static constexpr long long WB_WAIT_LIMIT_CYCLES = 2000000000LL;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// True in exactly one lane of a converged warp. The role loops below are executed by whole warps
// with warp-uniform values, and only the instruction issue is guarded by this predicate: that
// keeps descriptors and addresses in uniform registers, which the TMA and tcgen05 instructions
// take their operands from. Issuing them from a `lane == 0` branch instead costs a
// vector-to-uniform register move per operand and was measured to bound both kernels.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// Map a shared::cta address of this CTA to the same offset in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}

__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Arrive on a barrier that lives in another CTA of the cluster (address from mapa_shared).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar)
               : "memory");
}
// Same, without a release fence: for signals that publish no data written by this thread
// (e.g. "the TMA copies into my shared memory have landed", which the barrier itself observed).
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar)
               : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_try_wait_cluster_acquire(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Per-CTA wait context: a shared abort flag and the global status word.
struct WaitCtx {
  volatile uint32_t* abort_flag;  // shared memory, one per CTA
  int* status;                    // global memory, one per device
  long long limit_cycles = WB_WAIT_LIMIT_CYCLES;
};

// Bounded wait. Returns true when the barrier phase completed, false when the wait was
// abandoned (time limit, or another wait of this CTA already gave up).
template <bool kClusterAcquire = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtx& ctx,
                                          int code) {
  auto poll = [&]() {
    if constexpr (kClusterAcquire) return mbar_try_wait_cluster_acquire(bar, parity);
    else return mbar_try_wait(bar, parity);
  };
  if (poll()) return true;
  const long long t0 = clock64();
  uint32_t it = 0;
  while (!poll()) {
    if ((++it & 15u) == 0u) {
      if (*ctx.abort_flag) return false;
      if (clock64() - t0 > ctx.limit_cycles) {
        *ctx.abort_flag = 1u;
        atomicCAS(ctx.status, 0, code | (int(blockIdx.x) << 8));
        return false;
      }
    }
  }
  return true;
}

// ---------------------------------------------------------------------------------------------
// TMA: tiled 2D load (global -> shared, completes on an mbarrier), untiled bulk load,
// and tiled 2D store (shared -> global). No multicast forms anywhere.
// ---------------------------------------------------------------------------------------------
// CTA_GROUP = 2: the form a CTA pair uses; the mbarrier may then live in the peer CTA
// (a shared::cluster address from mapa_shared) while the data lands in this CTA.
template <int CTA_GROUP = 1>
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap* tmap, int x,
                                            int y, uint32_t bar) {
  if (!WB_CHECK((x & 15) == 0, kCheckTmaLoadCoord, x) || !WB_CHECK((dst_smem & 127u) == 0u, kCheckTmaSmem, dst_smem)) return;
  if constexpr (CTA_GROUP == 1)
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst_smem),
        "l"(tmap), "r"(x), "r"(y), "r"(bar)
        : "memory");
  else
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst_smem),
        "l"(tmap), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst_smem, const CUtensorMap* tmap,
                                                 int x, int y, uint32_t bar, uint64_t policy) {
  if (!WB_CHECK((x & 15) == 0, kCheckTmaLoadCoord, x) || !WB_CHECK((dst_smem & 127u) == 0u, kCheckTmaSmem, dst_smem)) return;
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%2, %3}], [%4], %5;" ::"r"(dst_smem),
      "l"(tmap), "r"(x), "r"(y), "r"(bar), "l"(policy)
      : "memory");
}
// src and dst 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes,
                                          uint32_t bar) {
  if (!WB_CHECK(((reinterpret_cast<uintptr_t>(src) | dst_smem | bytes) & 15u) == 0u, kCheckBulkCopy, bytes)) return;
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst_smem),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tmap, uint32_t src_smem, int x,
                                             int y) {
  if (!WB_CHECK(x >= 0 && y >= 0 && (x & 3) == 0, kCheckTmaStoreCoord, x) || !WB_CHECK((src_smem & 127u) == 0u, kCheckTmaSmem, src_smem)) return;
  asm volatile(
      "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(tmap),
      "r"(src_smem), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d_hint(const CUtensorMap* tmap, uint32_t src_smem, int x, int y,
                                                  uint64_t policy) {
  if (!WB_CHECK(x >= 0 && y >= 0 && (x & 3) == 0, kCheckTmaStoreCoord, x) || !WB_CHECK((src_smem & 127u) == 0u, kCheckTmaSmem, src_smem)) return;
  asm volatile(
      "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%2, %3}], [%1], %4;" ::"l"(tmap),
      "r"(src_smem), "r"(x), "r"(y), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// ---------------------------------------------------------------------------------------------
// tensor memory
// ---------------------------------------------------------------------------------------------
template <int CTA_GROUP>
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  if constexpr (CTA_GROUP == 1)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                 "r"(ncols)
                 : "memory");
  else
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                 "r"(ncols)
                 : "memory");
}
template <int CTA_GROUP>
__device__ __forceinline__ void tmem_relinquish() {
  if constexpr (CTA_GROUP == 1)
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  else
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int CTA_GROUP>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  if constexpr (CTA_GROUP == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
  else
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Shared-memory matrix descriptor, K-major operand tile stored as rows of 128 bytes with the
// 128-byte swizzle (what a TMA box of 128 bytes x rows with SWIZZLE_128B produces).
// Fields: start address >> 4 in [0,14); leading byte offset >> 4 in [16,30) (unused for this
// layout, set to 1); stride byte offset >> 4 in [32,46) = 1024 B between 8-row groups;
// descriptor version 1 in [46,48); layout type 2 (128-byte swizzle) in [61,64).
__device__ __forceinline__ uint64_t make_desc_k_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= uint64_t((smem_addr & 0x3FFFFu) >> 4);
  d |= uint64_t(1) << 16;
  d |= uint64_t(1024 >> 4) << 32;
  d |= uint64_t(1) << 46;
  d |= uint64_t(2) << 61;
  return d;
}
// Descriptor of one 512-byte scale-factor atom for tcgen05.cp 32x128b: 32 rows of 16 bytes,
// no swizzle, 8-row core matrices 128 bytes apart.
__device__ __forceinline__ uint64_t make_desc_sf_atom(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= uint64_t((smem_addr & 0x3FFFFu) >> 4);
  d |= uint64_t(128 >> 4) << 32;
  d |= uint64_t(1) << 46;
  return d;
}

// Instruction descriptor of tcgen05.mma kind::mxf4 block-scaled: E2M1 x E2M1 (format code 1),
// both operands K-major, UE8M0 scales, K = 64 per instruction.
// n >> 3 in [17,23); scale format (1 = E8M0) at 23; m >> 4 in [24,29);
// B scale-factor id in [4,6), A scale-factor id in [29,31): which pair of bytes of the 32-bit
// scale column this K = 64 step reads (0 -> bytes 0,1; 2 -> bytes 2,3).
__host__ __device__ constexpr uint32_t make_idesc_mxf4(int m, int n) {
  return (1u << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (1u << 23) | (uint32_t(m >> 4) << 24);
}
__device__ __forceinline__ uint32_t idesc_with_sf_id(uint32_t idesc, uint32_t sf_id) {
  return idesc | (sf_id << 4) | (sf_id << 29);
}

// Programmatic dependent launch. launch_dependents: kernels launched behind this one with the
// programmatic-serialisation attribute may start now; wait: returns once every kernel this one depends on has
// finished and its writes are visible (a no-op in a kernel launched without the attribute).
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Instruction descriptor of kind::mxf8f6f4 block-scaled: operand formats 0 = E4M3, 1 = E5M2, 5 = E2M1 (4-bit values in
// the 8-bit container layout: 16 values in 8 bytes, then 8 bytes of padding), chosen per operand; K-major, UE8M0
// scales, K = 32 per instruction; the scale-factor id (0..3) picks the byte of the 32-bit scale column that this
// K = 32 step reads.
constexpr uint32_t kFmtE2M1 = 5;
__host__ __device__ constexpr uint32_t make_idesc_mxf8(int m, int n, uint32_t a_fmt, uint32_t b_fmt) {
  return (a_fmt << 7) | (b_fmt << 10) | (uint32_t(n >> 3) << 17) | (1u << 23) | (uint32_t(m >> 4) << 24);
}
// The `elem_format` word of the 8-bit kernels: bit 0 = format of the activations (and of the weights unless bit 4 is
// set), bit 4 = the weights are packed E2M1 ([N, K/2] bytes in global memory, expanded into 8-bit containers by the
// copy engine on their way to shared memory).
__host__ __device__ constexpr uint32_t act_format_of(int elem_format) { return uint32_t(elem_format) & 1u; }
__host__ __device__ constexpr uint32_t weight_format_of(int elem_format) {
  return (elem_format & 0x10) ? kFmtE2M1 : (uint32_t(elem_format) & 1u);
}

template <int CTA_GROUP>
__device__ __forceinline__ void utccp_sf_atom(uint32_t taddr, uint64_t sdesc) {
  if constexpr (CTA_GROUP == 1)
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc)
                 : "memory");
  else
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc)
                 : "memory");
}

// D[tmem] (+)= A[smem] * B[smem] with per-32-element E8M0 scales held in tensor memory.
template <int CTA_GROUP>
__device__ __forceinline__ void mma_mxf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                         uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                                         uint32_t accumulate) {
  if constexpr (CTA_GROUP == 1)
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X "
        "[%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
  else
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.scale_vec::2X "
        "[%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}

// The same with 8-bit operands (MXFP8): one E8M0 scale per 32 elements = per instruction.
template <int CTA_GROUP>
__device__ __forceinline__ void mma_mxf8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                         uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                                         uint32_t accumulate) {
  if constexpr (CTA_GROUP == 1)
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X "
        "[%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
  else
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale.scale_vec::1X "
        "[%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}

// Make an mbarrier (shared::cluster address; a shared::cta address names this CTA's own)
// complete once every tcgen05 operation issued so far by this thread has finished.
template <int CTA_GROUP>
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  if constexpr (CTA_GROUP == 1)
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     bar)
                 : "memory");
  else
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     bar)
                 : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns -> 32 registers per thread (thread t = lane t of the
// warp's lane quadrant, register j = column j).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

}  // namespace wb
