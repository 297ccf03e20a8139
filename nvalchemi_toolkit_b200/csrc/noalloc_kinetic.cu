// SPDX-License-Identifier: Apache-2.0
// Per-system kinetic energy without any allocation: see noalloc_kinetic.h for the contract.  Same arithmetic as
// compute_kinetic_energy in integrators.cu (double accumulation, warp-aggregated atomics), but the accumulator is a
// file-scope device array instead of a tensor obtained from the allocator.
#include "noalloc_kinetic.h"

#include <mutex>
#include <stdio.h>

namespace {

// Device-resident accumulator.  In host code this name is only a handle for cudaGetSymbolAddress: it is NOT a device
// pointer and must never be passed to a kernel directly.
static __device__ __align__(256) double nva_noalloc_ke_scratch[NVA_NOALLOC_MAX_SYSTEMS];

constexpr int kMaxDevices = 64;
double* g_scratch_ptr[kMaxDevices] = {nullptr};
std::mutex g_mutex;                 // guards g_scratch_ptr only
thread_local char g_error[256] = "";  // every thread reads back the text of ITS last failure: no sharing, no lock

__global__ void ke_clear_kernel(double* scratch, int m) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < m) scratch[i] = 0.0;
}

__global__ void ke_accumulate_kernel(const float* __restrict__ v, const float* __restrict__ mass,
                                     const int* __restrict__ seg, int64_t n, int num_systems,
                                     double* __restrict__ scratch) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int s = -1;
  double ke = 0.0;
  if (i < n) {
    s = seg[i];
    // an index outside [0, num_systems) is skipped: it must neither pollute slots that this call did not clear nor
    // reach beyond the fixed array
    if (s < 0 || s >= num_systems) s = -1;
    double x = v[3 * i], y = v[3 * i + 1], z = v[3 * i + 2];
    ke = s >= 0 ? 0.5 * (double)mass[i] * (x * x + y * y + z * z) : 0.0;
  }
  // all 32 lanes take part; a warp whose lanes share one system issues a single atomic
  unsigned peers = __match_any_sync(0xffffffffu, s);
  if (peers == 0xffffffffu) {
    for (int o = 16; o > 0; o >>= 1) ke += __shfl_down_sync(0xffffffffu, ke, o);
    if ((threadIdx.x & 31) == 0 && s >= 0) atomicAdd(scratch + s, ke);
  } else if (s >= 0) {
    atomicAdd(scratch + s, ke);
  }
}

__global__ void ke_store_kernel(const double* scratch, int m, float* out) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < m) out[i] = (float)scratch[i];
}

int fail(int code, const char* what, cudaError_t err) {
  if (err != cudaSuccess) snprintf(g_error, sizeof(g_error), "%s: %s", what, cudaGetErrorString(err));
  else snprintf(g_error, sizeof(g_error), "%s", what);
  return code;
}

}  // namespace

extern "C" const char* nva_noalloc_last_error(void) { return g_error; }

extern "C" int nva_kinetic_energy_noalloc(const float* velocities, const float* masses, const int* batch_idx,
                                          int64_t n_atoms, int num_systems, float* out, cudaStream_t stream) {
  if (num_systems < 0 || n_atoms < 0) return fail(NVA_NOALLOC_E_ARGUMENT, "negative size", cudaSuccess);
  if (num_systems > NVA_NOALLOC_MAX_SYSTEMS) {
    char msg[160];
    snprintf(msg, sizeof(msg), "num_systems = %d exceeds the fixed accumulator size NVA_NOALLOC_MAX_SYSTEMS = %d",
             num_systems, NVA_NOALLOC_MAX_SYSTEMS);
    return fail(NVA_NOALLOC_E_TOO_LARGE, msg, cudaSuccess);
  }
  if (num_systems == 0) return NVA_NOALLOC_OK;
  if (out == nullptr || (n_atoms > 0 && (velocities == nullptr || masses == nullptr || batch_idx == nullptr)))
    return fail(NVA_NOALLOC_E_ARGUMENT, "null pointer argument", cudaSuccess);
  int dev = -1;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return fail(NVA_NOALLOC_E_CUDA, "cudaGetDevice", err);
  if (dev < 0 || dev >= kMaxDevices) return fail(NVA_NOALLOC_E_ARGUMENT, "device index out of range", cudaSuccess);
  double* scratch = nullptr;
  {
    // one-time set-up for this device (with this device current): resolve the device address of the array
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
      void* p = nullptr;
      err = cudaGetSymbolAddress(&p, nva_noalloc_ke_scratch);
      if (err != cudaSuccess || p == nullptr) return fail(NVA_NOALLOC_E_CUDA, "cudaGetSymbolAddress", err);
      g_scratch_ptr[dev] = static_cast<double*>(p);
    }
    scratch = g_scratch_ptr[dev];
  }
  // an error left behind by an earlier, unrelated launch of this thread is not this call's failure: if one is pending,
  // report it as such and launch nothing (cudaPeekAtLastError does not clear it for its owner)
  err = cudaPeekAtLastError();
  if (err != cudaSuccess) return fail(NVA_NOALLOC_E_CUDA, "an earlier CUDA error is pending on this thread", err);
  const int threads = 256;
  int mblocks = (num_systems + threads - 1) / threads;
  ke_clear_kernel<<<mblocks, threads, 0, stream>>>(scratch, num_systems);  // the array keeps the previous call's sums
  if (n_atoms > 0) {
    int64_t blocks = (n_atoms + threads - 1) / threads;
    ke_accumulate_kernel<<<(unsigned)blocks, threads, 0, stream>>>(velocities, masses, batch_idx, n_atoms, num_systems,
                                                                   scratch);
  }
  ke_store_kernel<<<mblocks, threads, 0, stream>>>(scratch, num_systems, out);
  err = cudaGetLastError();
  if (err != cudaSuccess) return fail(NVA_NOALLOC_E_CUDA, "kernel launch", err);
  return NVA_NOALLOC_OK;
}
