// One process driving several GPUs: the native counterpart of the reference's multi-device launch
// (wave_lang/runtime/multi_device_launch.py:38-273 creates one HAL device per GPU and invokes once;
// wave_lang/kernel/compiler/host_utils.py:158-376 slices the inputs per device, dispatches one kernel per
// device and merges the output slices). Here: one stream per device, the activations copied to every
// device over NVLink, one GEMM launch per device on its own column block of C, and the column blocks laid
// side by side wherever the caller wants the whole C. No collective library, no kernel that reads another
// GPU's memory: the only traffic between GPUs is copy-engine copies.
#pragma once
#include <cuda_runtime.h>
#include <vector>

namespace wb {

struct MultiGpu {
  std::vector<int> devices;
  std::vector<cudaStream_t> streams;
  std::vector<cudaEvent_t> done;    // recorded on device g's stream by join / timing
  std::vector<cudaEvent_t> t_begin; // timing brackets
  std::vector<cudaEvent_t> t_end;
  cudaEvent_t ready = nullptr;      // recorded on the caller's stream by wait_for
  int ready_device = -1;
};

// RAII: make `dev` current, restore the previous device on scope exit.
struct DeviceScope {
  int saved = -1;
  bool ok = true;
  explicit DeviceScope(int dev) {
    ok = cudaGetDevice(&saved) == cudaSuccess && cudaSetDevice(dev) == cudaSuccess;
  }
  ~DeviceScope() {
    if (saved >= 0) cudaSetDevice(saved);
  }
};

// Rows [n0, n1) of an N-row matrix owned by part `index` of `parts`: N is dealt in multiples of `granule`
// rows as evenly as possible, earlier parts taking the remainder, the last non-empty part the ragged tail.
inline void shard_bounds(int N, int parts, int index, int granule, int* n0, int* n1) {
  const int blocks = (N + granule - 1) / granule;
  const int base = blocks / parts, extra = blocks % parts;
  const long long b0 = (long long)index * base + (index < extra ? index : extra);
  const long long b1 = b0 + base + (index < extra ? 1 : 0);
  const long long r0 = b0 * granule, r1 = b1 * granule;
  *n0 = int(r0 < N ? r0 : N);
  *n1 = int(r1 < N ? r1 : N);
}

}  // namespace wb
