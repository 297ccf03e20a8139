// SPDX-License-Identifier: Apache-2.0
// Allocation-free kinetic energy entry point.  This function has no counterpart in the reference toolkit.
//
// Who needs it: code that drives this library from a place where device memory cannot be requested at call time -
// a host loop that must stay free of allocator locks while other threads stream data, an embedding application
// that handed the whole device memory to its own pool, or a plugin ABI that only passes raw pointers.  The regular
// operator (`torch.ops.nvalchemi.compute_kinetic_energy`) asks the tensor allocator for a double-precision
// accumulator and for its result on every call; this variant keeps the accumulator in a fixed device array that is part
// of the loaded library image.
//
// Contract
//   * float32 inputs, contiguous: velocities [n_atoms,3], masses [n_atoms], batch_idx [n_atoms] (int32, values in
//     [0, num_systems); an atom whose index lies outside that range is ignored), output out [num_systems] (float32,
//     written, not accumulated).
//   * The call works on the CURRENT device: all pointers must be device memory of it and `stream` must be a stream of it
//     (or 0).
//   * num_systems <= NVA_NOALLOC_MAX_SYSTEMS, otherwise the call fails with NVA_NOALLOC_E_TOO_LARGE and touches nothing.
//   * The accumulator array (NVA_NOALLOC_MAX_SYSTEMS doubles = 512 KiB) exists once per GPU that loads the library and
//     stays resident until the process exits.  Every call on a device shares it: the part that is used is cleared at
//     the start of each call, and two calls whose kernels overlap on the same GPU (different streams, different threads)
//     race on it - serialise them.
//   * The first call on each device looks up the device address of that array (one `cudaGetSymbolAddress`); make that
//     first call outside any stream capture.
//   * No cudaMalloc / cudaFree / library allocation happens in any call.  Work is enqueued on `stream`; the function
//     returns without synchronising.
#pragma once
#include <cuda_runtime.h>

#include <stdint.h>

#define NVA_NOALLOC_MAX_SYSTEMS 65536
#define NVA_NOALLOC_OK 0
#define NVA_NOALLOC_E_TOO_LARGE 1
#define NVA_NOALLOC_E_CUDA 2
#define NVA_NOALLOC_E_ARGUMENT 3

#ifdef __cplusplus
extern "C" {
#endif

// Returns NVA_NOALLOC_OK or an error code; `nva_noalloc_last_error()` gives the text of the calling thread's last
// failure (the buffer is per thread).
int nva_kinetic_energy_noalloc(const float* velocities, const float* masses, const int* batch_idx, int64_t n_atoms,
                               int num_systems, float* out, cudaStream_t stream);
const char* nva_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
