// SPDX-License-Identifier: Apache-2.0
// Per-atom energy readout of the native MACE and its adjoint seed, one kernel each.
//
// Forward (replaces a GEMM + activation + matrix-vector product + add per layer; reference: the readout blocks of
// mace-torch driven by nvalchemi/models/mace.py:872-910):
//   linear readout (R = 1, not the last layer):  e_i += s_i . w1
//   MLP readout (last layer):                     a = s_i W1 [C,R];  e_i += sum_r silu_n(a_r) w2_r;
//                                                 gy_ir = silu_n'(a_r) w2_r   (kept for the adjoint)
// where s_i = the scalar (l = 0) channels of atom i, i.e. the first C floats of its feature row, and silu_n is SiLU
// scaled to unit second moment.  Adjoint:  dh_i[0, c] += coef_i * sum_r gy_ir W1[c, r]   (R = 1: coef_i * w1[c]),
// coef_i = scale * (weight_i if per-atom energy weights are given else 1).
#include "common.cuh"

namespace nva {
using at::Tensor;

constexpr float kSiluNormR = 1.6790176868438721f;

// One warp per atom; W1 ([C, R], R <= 32) staged in shared memory; lane r owns output r.
__global__ void __launch_bounds__(256) readout_fwd_kernel(int64_t n, int C, int R, bool mlp, const float* __restrict__ h,
                                                          int64_t ldh, const float* __restrict__ W1,
                                                          const float* __restrict__ w2, float* __restrict__ node_e,
                                                          float* __restrict__ gy) {
  extern __shared__ float sm[];
  float* sW = sm;                       // [C][R]
  float* sS = sm + C * R;               // [warps][C]
  for (int k = threadIdx.x; k < C * R; k += blockDim.x) sW[k] = W1[k];
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  float* row = sS + warp * C;
  const float w2r = (mlp && lane < R) ? w2[lane] : 0.f;
  for (int64_t i = blockIdx.x * (int64_t)wpb + warp; i < n; i += (int64_t)gridDim.x * wpb) {
    const float* s = h + i * ldh;
    for (int c = lane; c < C; c += 32) row[c] = s[c];
    __syncwarp();
    float e = 0.f;
    if (lane < R) {
      float a = 0.f;
      for (int c = 0; c < C; ++c) a = fmaf(row[c], sW[c * R + lane], a);
      if (mlp) {
        const float sg = __fdividef(1.f, 1.f + __expf(-a));
        e = a * sg * kSiluNormR * w2r;
        gy[i * R + lane] = sg * (1.f + a * (1.f - sg)) * kSiluNormR * w2r;
      } else {
        e = a;
      }
    }
    for (int o = 16; o > 0; o >>= 1) e += __shfl_down_sync(0xffffffffu, e, o);
    if (lane == 0) node_e[i] += e;
    __syncwarp();
  }
}

__global__ void __launch_bounds__(256) readout_bwd_kernel(int64_t n, int C, int R, bool mlp, const float* __restrict__ gy,
                                                          const float* __restrict__ W1, float scale,
                                                          const float* __restrict__ weights, float* __restrict__ dh,
                                                          int64_t ldd) {
  extern __shared__ float sm[];
  for (int k = threadIdx.x; k < C * R; k += blockDim.x) sm[k] = W1[k];
  __syncthreads();
  const int64_t total = n * (int64_t)C;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = t / C;
    const int c = (int)(t - i * C);
    const float coef = scale * (weights != nullptr ? weights[i] : 1.f);
    float v;
    if (mlp) {
      v = 0.f;
      const float* g = gy + i * R;
      for (int r = 0; r < R; ++r) v = fmaf(g[r], sm[c * R + r], v);
    } else {
      v = sm[c];
    }
    dh[i * ldd + c] += coef * v;
  }
}

// h [N, n_lm, C] (rows may be a slice of a wider buffer); w1 [C, R] or [C]; w2 [R] or none; node_e [N] accumulated.
// Returns gy [N, R] for the MLP form (empty tensor for the linear form).
Tensor mace_readout_fwd(const Tensor& h, const Tensor& w1, const c10::optional<Tensor>& w2, Tensor node_e) {
  TORCH_CHECK(h.is_cuda() && h.scalar_type() == at::kFloat && h.dim() == 3 && h.stride(2) == 1 && h.stride(1) == h.size(2),
              "mace_readout_fwd: h must be float32 CUDA [N, n_lm, C] with contiguous rows");
  c10::cuda::CUDAGuard guard(h.device());
  const int64_t n = h.size(0);
  const int C = (int)h.size(2);
  const bool mlp = w2.has_value();
  const int R = mlp ? (int)w1.size(1) : 1;
  TORCH_CHECK(R >= 1 && R <= 32 && w1.numel() == (int64_t)C * R && w1.is_contiguous(), "mace_readout_fwd: W1 must be [C, R <= 32]");
  TORCH_CHECK(node_e.numel() >= n && node_e.is_contiguous(), "mace_readout_fwd: node_e too short");
  Tensor gy = at::empty({mlp ? n : 0, R}, h.options());
  if (n == 0) return gy;
  const int threads = 256, wpb = threads / 32;
  const size_t smem = (size_t)(C * R + wpb * C) * sizeof(float);
  TORCH_CHECK(smem <= 48 * 1024, "mace_readout_fwd: C * R too large for the staging buffer");
  const int64_t blocks = std::min<int64_t>((n + wpb - 1) / wpb, 148 * 8);
  readout_fwd_kernel<<<(unsigned)blocks, threads, smem, at::cuda::getCurrentCUDAStream()>>>(
      n, C, R, mlp, h.data_ptr<float>(), h.stride(0), w1.data_ptr<float>(), mlp ? w2->data_ptr<float>() : nullptr,
      node_e.data_ptr<float>(), mlp ? gy.data_ptr<float>() : nullptr);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return gy;
}

void mace_readout_bwd(const c10::optional<Tensor>& gy, const Tensor& w1, double scale, const c10::optional<Tensor>& weights,
                      Tensor dh) {
  TORCH_CHECK(dh.is_cuda() && dh.scalar_type() == at::kFloat && dh.dim() == 3 && dh.stride(2) == 1,
              "mace_readout_bwd: dh must be float32 CUDA [N, n_lm, C]");
  c10::cuda::CUDAGuard guard(dh.device());
  const int64_t n = dh.size(0);
  const int C = (int)dh.size(2);
  const bool mlp = gy.has_value();
  const int R = mlp ? (int)gy->size(1) : 1;
  TORCH_CHECK(w1.numel() == (int64_t)C * R && w1.is_contiguous(), "mace_readout_bwd: W1 must be [C, R]");
  if (mlp) TORCH_CHECK(gy->is_contiguous() && gy->size(0) == n, "mace_readout_bwd: gy must be [N, R]");
  if (weights.has_value()) TORCH_CHECK(weights->is_contiguous() && weights->numel() >= n, "mace_readout_bwd: weights too short");
  if (n == 0) return;
  const size_t smem = (size_t)C * R * sizeof(float);
  const int64_t blocks = std::min<int64_t>((n * C + 255) / 256, 148 * 16);
  readout_bwd_kernel<<<(unsigned)blocks, 256, smem, at::cuda::getCurrentCUDAStream()>>>(
      n, C, R, mlp, mlp ? gy->data_ptr<float>() : nullptr, w1.data_ptr<float>(), (float)scale,
      weights.has_value() ? weights->data_ptr<float>() : nullptr, dh.data_ptr<float>(), dh.stride(0));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

}  // namespace nva

TORCH_LIBRARY_FRAGMENT(nvalchemi, m) {
  m.def("mace_readout_fwd(Tensor h, Tensor w1, Tensor? w2, Tensor(a!) node_e) -> Tensor", &nva::mace_readout_fwd);
  m.def("mace_readout_bwd(Tensor? gy, Tensor w1, float scale, Tensor? weights, Tensor(a!) dh) -> ()", &nva::mace_readout_bwd);
}
