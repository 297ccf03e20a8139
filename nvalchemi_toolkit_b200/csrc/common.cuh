// SPDX-License-Identifier: Apache-2.0
// Shared helpers for the sm_100a extension: launch wrappers that run the same functor
// as a CUDA kernel or as an OpenMP loop, a counter-based Philox RNG usable on both
// sides, and block/warp reductions for per-system sums.
#pragma once
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime.h>
#include <torch/library.h>

#include <cstdint>

#define NVA_CHECK_CONTIG(x) TORCH_CHECK((x).is_contiguous(), #x " must be contiguous")
#define NVA_HD __host__ __device__ __forceinline__
#define NVA_LAMBDA __host__ __device__

namespace nva {

constexpr int kThreads = 256;

template <typename F>
__global__ void foreach_kernel(int64_t n, F f) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i < n) f(i);
}

// Runs f(i) for i in [0,n): one CUDA thread per index on `cuda`, an OpenMP loop otherwise.
template <typename F>
void for_each(bool cuda, int64_t n, F f) {
  if (n <= 0) return;
  if (cuda) {
    int64_t blocks = (n + kThreads - 1) / kThreads;
    foreach_kernel<<<(unsigned)blocks, kThreads, 0, at::cuda::getCurrentCUDAStream()>>>(n, f);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  } else {
#pragma omp parallel for schedule(static) if (n > 4096)
    for (int64_t i = 0; i < n; ++i) f(i);
  }
}

// ---- Philox4x32-10 (Salmon et al. 2011), counter = (index, stream), key = seed ---------
struct Philox {
  uint32_t c[4];
  uint32_t k[2];
  NVA_HD Philox(uint64_t seed, uint64_t index, uint64_t stream) {
    k[0] = (uint32_t)seed; k[1] = (uint32_t)(seed >> 32);
    c[0] = (uint32_t)index; c[1] = (uint32_t)(index >> 32);
    c[2] = (uint32_t)stream; c[3] = (uint32_t)(stream >> 32);
  }
  static NVA_HD void mulhilo(uint32_t a, uint32_t b, uint32_t& hi, uint32_t& lo) {
    uint64_t p = (uint64_t)a * (uint64_t)b;
    hi = (uint32_t)(p >> 32); lo = (uint32_t)p;
  }
  NVA_HD void round() {
    uint32_t hi0, lo0, hi1, lo1;
    mulhilo(0xD2511F53u, c[0], hi0, lo0);
    mulhilo(0xCD9E8D57u, c[2], hi1, lo1);
    uint32_t n0 = hi1 ^ c[1] ^ k[0], n1 = lo1, n2 = hi0 ^ c[3] ^ k[1], n3 = lo0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
  }
  // Four uniform 32-bit words.
  NVA_HD void generate(uint32_t out[4]) {
    for (int r = 0; r < 10; ++r) {
      round();
      k[0] += 0x9E3779B9u; k[1] += 0xBB67AE85u;
    }
    out[0] = c[0]; out[1] = c[1]; out[2] = c[2]; out[3] = c[3];
  }
};

// Box-Muller: 4 uniform words -> 4 standard normals (double math on host and device for parity).
NVA_HD void philox_normal4(uint64_t seed, uint64_t index, uint64_t stream, double z[4]) {
  Philox p(seed, index, stream);
  uint32_t u[4];
  p.generate(u);
  const double inv = 1.0 / 4294967296.0;
  double u0 = ((double)u[0] + 0.5) * inv, u1 = ((double)u[1] + 0.5) * inv;
  double u2 = ((double)u[2] + 0.5) * inv, u3 = ((double)u[3] + 0.5) * inv;
  double r0 = sqrt(-2.0 * log(u0)), r1 = sqrt(-2.0 * log(u2));
  const double two_pi = 6.283185307179586476925;
  z[0] = r0 * cos(two_pi * u1); z[1] = r0 * sin(two_pi * u1);
  z[2] = r1 * cos(two_pi * u3); z[3] = r1 * sin(two_pi * u3);
}

// ---- per-system accumulation -------------------------------------------------------------
// Adds `v` into out[seg] (double accumulators).  ALL 32 lanes of the warp must call; a lane
// with nothing to add passes seg = -1.  A warp whose lanes share one segment (the common
// case for a batch sorted by system) reduces by shuffles and issues a single atomic.
__device__ __forceinline__ void seg_atomic_add(double* out, int seg, double v) {
  unsigned peers = __match_any_sync(0xffffffffu, seg);
  if (peers == 0xffffffffu) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0 && seg >= 0) atomicAdd(out + seg, v);
  } else if (seg >= 0) {
    atomicAdd(out + seg, v);
  }
}

// Atomic += on a double from device code or from an OpenMP loop.
__host__ __device__ inline void atomic_add_f64(double* p, double v) {
#ifdef __CUDA_ARCH__
  atomicAdd(p, v);
#else
#pragma omp atomic
  *p += v;
#endif
}

inline void check_same_device(const at::Tensor& a, const at::Tensor& b) {
  TORCH_CHECK(a.device() == b.device(), "tensors must be on the same device");
}

}  // namespace nva
