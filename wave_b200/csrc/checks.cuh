// Debug-checked build: compile the library with -DWB200_CHECKS (`python -m wave_b200.build --checks`, which
// writes libwave_b200_checks.so; load it with WAVE_B200_LIB=...). The kernels then test an index predicate in
// front of every copy-engine issue and every global store they make: alignment of the innermost TMA coordinate
// and of the shared-memory side, output row / column inside C, workspace slot and counter inside the workspace.
// A predicate that fails SKIPS the access, counts it, and the first one records (code, CTA, detail) in a
// device word that wb200_debug_checks returns; nothing traps and the context stays usable. This stands in for
// the reference's `use_bound_check` option (wave_lang/kernel/wave/analysis/generate_bound_checks.py:17-63,
// which prints and halts) on a machine where compute-sanitizer is not available. Without the flag WB_CHECK is
// the constant `true` and the shipped kernels are unchanged.
#pragma once

namespace wb {

enum CheckCode : int {
  kCheckTmaLoadCoord = 1,   // innermost coordinate of a tiled load not a multiple of 16 elements
  kCheckTmaSmem = 2,        // shared-memory side of a copy not 128-byte aligned
  kCheckTmaStoreCoord = 3,  // store at a negative coordinate or at a column that is not a multiple of 4
  kCheckBulkCopy = 4,       // untiled bulk copy: address or size not a multiple of 16 bytes
  kCheckOutputIndex = 5,    // output row >= M or column >= N
  kCheckPartialSlot = 6,    // partial-tile slot past the workspace
  kCheckCounter = 7,        // tile counter index past the workspace header
  kCheckSelfTest = 99,      // raised on purpose by wb200_debug_checks_selftest
};

#ifdef WB200_CHECKS
// [0] first failure: code | CTA << 32; [1] its detail word; [2] number of failures
__device__ unsigned long long g_check_record[3];

__device__ __forceinline__ bool check_failed(int code, long long detail) {
  atomicAdd(&g_check_record[2], 1ull);
  const unsigned long long first = (unsigned long long)(unsigned)code | ((unsigned long long)blockIdx.x << 32);
  if (atomicCAS(&g_check_record[0], 0ull, first) == 0ull) g_check_record[1] = (unsigned long long)detail;
  return false;
}
#define WB_CHECK(cond, code, detail) ((cond) ? true : ::wb::check_failed((code), (long long)(detail)))
#else
#define WB_CHECK(cond, code, detail) (true)
#endif

}  // namespace wb
