// SPDX-License-Identifier: Apache-2.0
// First MACE interaction in factorised form.
//
// The input features of the first interaction are a function of the sender's SPECIES only (u_s[c], a table), so the
// channel index can be pulled out of the sum over edges:
//
//   mid[i, lm, c] = sum_{e -> i} R_e[c, l] u_{s(e)}[c] Y_lm(e),   R_e[c, l] = sum_k h3[e, k] W4[k, (l, c)]
//                 = sum_s u_s[c] sum_k W4[k, (l, c)] A[i, s, lm, k],   A[i, s, lm, k] = sum_{e -> i, s(e) = s} Y_lm(e) h3[e, k]
//
// `l0_moments_kernel` accumulates the per-receiver moments A (16 x 64 numbers per receiver and species: 1024
// multiply-adds per edge instead of ~100 per edge AND channel); the channel dimension is then produced by a dense GEMM
// with K = 64 outside this file.  The adjoint runs the other way: a GEMM turns dE/dmsg into
// Q[i, s, lm, k] = dE/dA, and `l0_force_kernel` contracts Q with the value and radial-derivative rows of h3 per edge,
//   dE/dY_lm(e) = sum_k Q[i, s, lm, k] h3[e, k],   dE/dr(e) = sum_lm Y_lm(e) sum_k Q[i, s, lm, k] (dh3/dr)[e, k],
// and converts both into the force along the edge (same per-edge force matrix as the general convolution kernels).
// One warp per receiver; no tensor cores here: the work per edge is 1-2 K multiply-adds and the loops are bound by
// the h3 rows they stream.  Replaces, for the first layer, the cuEquivariance fused tensor product that the
// reference's MACE wrapper calls for every layer (nvalchemi/models/mace.py:205-287).
#include "common.cuh"

#include "mace_device.cuh"

namespace nva {
using at::Tensor;

namespace {

constexpr int L0_WARPS = 8;
constexpr int NLM = 16, NK = 64;
constexpr int L0_MSUB = 16;    // edges per staged sub-batch of the moments kernel (16 x 256 B = 4 KB per warp and slot)
constexpr int L0_SUB = 8;      // edges per staged sub-batch of the force kernel (8 x 512 B = 4 KB per warp and slot)

// 16-byte asynchronous global -> shared copy (Ampere-style cp.async, bypassing L1) and its group fences.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Moments: lane owns hidden units k = lane and lane + 32 for all 16 harmonics.
__global__ void __launch_bounds__(32 * L0_WARPS) l0_moments_kernel(
    const float* __restrict__ h3, int64_t e_chunk0, const float* __restrict__ pos, const float* __restrict__ cell,
    const int* __restrict__ batch_idx, const int* __restrict__ eptr, const int* __restrict__ esend,
    const int* __restrict__ eS, const int* __restrict__ species, int nz, int i0, int ni, float rmax,
    float* __restrict__ A, int hstride) {
  __shared__ __align__(16) float Ys[L0_WARPS][32][NLM];
  extern __shared__ __align__(16) float l0_stage[];  // staged h3 rows, two slots per warp (64 KB: dynamic shared memory)
  float (*Hs)[2][L0_MSUB][NK] = reinterpret_cast<float (*)[2][L0_MSUB][NK]>(l0_stage);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gw = blockIdx.x * L0_WARPS + warp, nw = gridDim.x * L0_WARPS;
  for (int r = gw; r < ni; r += nw) {
    const int i = i0 + r;
    const int e0 = eptr[i], e1 = eptr[i + 1];
    for (int s = 0; s < nz; ++s) {
      float acc0[NLM], acc1[NLM];
#pragma unroll
      for (int b = 0; b < NLM; ++b) { acc0[b] = 0.f; acc1[b] = 0.f; }
      for (int eb = e0; eb < e1; eb += 32) {
        const int e = eb + lane;
        int ok = 0;
        {
          float Y[NLM];
#pragma unroll
          for (int b = 0; b < NLM; ++b) Y[b] = 0.f;
          if (e < e1) {
            const int j = esend[e];
            float v[3];
            edge_vector(pos, cell, batch_idx, i, j, eS + 3 * e, v);
            const float rr = sqrtf(v[0] * v[0] + v[1] * v[1] + v[2] * v[2]);
            if (rr < rmax && rr > 0.f && (nz == 1 || species[j] == s)) {
              const float ri = 1.f / rr;
              sh_l3(v[0] * ri, v[1] * ri, v[2] * ri, Y);
              ok = 1;
            }
          }
          __syncwarp();
          float4* yd = reinterpret_cast<float4*>(Ys[warp][lane]);
          yd[0] = make_float4(Y[0], Y[1], Y[2], Y[3]);
          yd[1] = make_float4(Y[4], Y[5], Y[6], Y[7]);
          yd[2] = make_float4(Y[8], Y[9], Y[10], Y[11]);
          yd[3] = make_float4(Y[12], Y[13], Y[14], Y[15]);
        }
        const unsigned okmask = __ballot_sync(0xffffffffu, ok);
        __syncwarp();
        const int cnt = min(32, e1 - eb);
        if (okmask == 0u) continue;
        // masked edges have Y = 0, so every edge of the batch is processed.  The value rows (256 B each, `hstride` floats
        // apart) are staged in shared memory in sub-batches of L0_MSUB edges with 16-byte asynchronous copies, two
        // sub-batches in flight: the loads of the next edges overlap the multiply-adds of the current ones.
        const float* hbase = h3 + ((int64_t)eb - e_chunk0) * hstride;
        const int nsub = (cnt + L0_MSUB - 1) / L0_MSUB;
        auto stage = [&](int sb) {
          float* dst = &Hs[warp][sb & 1][0][0];
#pragma unroll
          for (int u = 0; u < L0_MSUB / 2; ++u) {
            const int n = 2 * u + (lane >> 4), w = lane & 15;  // edge of the sub-batch, 16-byte piece of its row
            if (sb * L0_MSUB + n < cnt) cp_async16(dst + n * NK + 4 * w, hbase + (int64_t)(sb * L0_MSUB + n) * hstride + 4 * w);
          }
          cp_async_commit();
        };
        stage(0);
        for (int sb = 0; sb < nsub; ++sb) {
          if (sb + 1 < nsub) { stage(sb + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
          __syncwarp();
          const int m = min(L0_MSUB, cnt - sb * L0_MSUB);
#pragma unroll 2
          for (int u = 0; u < m; ++u) {
            const float ha = Hs[warp][sb & 1][u][lane], hb = Hs[warp][sb & 1][u][lane + 32];
            const float4* yp = reinterpret_cast<const float4*>(Ys[warp][sb * L0_MSUB + u]);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float4 y = yp[q];
              acc0[4 * q] = fmaf(y.x, ha, acc0[4 * q]); acc1[4 * q] = fmaf(y.x, hb, acc1[4 * q]);
              acc0[4 * q + 1] = fmaf(y.y, ha, acc0[4 * q + 1]); acc1[4 * q + 1] = fmaf(y.y, hb, acc1[4 * q + 1]);
              acc0[4 * q + 2] = fmaf(y.z, ha, acc0[4 * q + 2]); acc1[4 * q + 2] = fmaf(y.z, hb, acc1[4 * q + 2]);
              acc0[4 * q + 3] = fmaf(y.w, ha, acc0[4 * q + 3]); acc1[4 * q + 3] = fmaf(y.w, hb, acc1[4 * q + 3]);
            }
          }
          __syncwarp();  // the slot is refilled two iterations later
        }
      }
      float* ap = A + (((int64_t)i * nz + s) * NLM) * NK + lane;
#pragma unroll
      for (int b = 0; b < NLM; ++b) { ap[b * NK] = acc0[b]; ap[b * NK + 32] = acc1[b]; }
    }
  }
}

// Forces: lane = (harmonic lm = lane & 15, half = lane >> 4) holds Q[lm, 32 half .. 32 half + 31] in registers; the
// per-edge dot products with the value / derivative rows of h3 are exchanged through shared memory, and the force is
// assembled with lane = edge.  h3 rows alternate value / derivative: row 2e and 2e + 1 of the chunk.
__global__ void __launch_bounds__(32 * L0_WARPS) l0_force_kernel(
    const float* __restrict__ h3, int64_t e_chunk0, const float* __restrict__ Q, const float* __restrict__ pos,
    const float* __restrict__ cell, const int* __restrict__ batch_idx, const int* __restrict__ eptr,
    const int* __restrict__ esend, const int* __restrict__ eS, const int* __restrict__ species, int nz, int i0, int ni,
    float rmax, float* __restrict__ grad_pos, double* __restrict__ virial) {
  __shared__ __align__(16) float P[L0_WARPS][32][32];  // [edge][lm | 16 + lm]: dE/dY and the radial factor per harmonic
  // staged (value | derivative) rows, two slots per warp: 64 KB, above the static limit, hence dynamic shared memory
  extern __shared__ __align__(16) float l0_stage[];
  float (*H)[2][L0_SUB][2 * NK] = reinterpret_cast<float (*)[2][L0_SUB][2 * NK]>(l0_stage);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int lm = lane & 15, half = lane >> 4;
  const int gw = blockIdx.x * L0_WARPS + warp, nw = gridDim.x * L0_WARPS;
  for (int r = gw; r < ni; r += nw) {
    const int i = i0 + r;
    const int e0 = eptr[i], e1 = eptr[i + 1];
    float fi[3] = {0.f, 0.f, 0.f};
    float vir[9];
#pragma unroll
    for (int k = 0; k < 9; ++k) vir[k] = 0.f;
    for (int s = 0; s < nz; ++s) {
      float4 q[8];
      {
        const float4* qp = reinterpret_cast<const float4*>(Q + ((((int64_t)i * nz + s) * NLM + lm) * NK + 32 * half));
#pragma unroll
        for (int k = 0; k < 8; ++k) q[k] = __ldg(qp + k);
      }
      for (int eb = e0; eb < e1; eb += 32) {
        const int e = eb + lane;
        // ---- lane = edge: geometry
        int ok = 0, j = 0;
        float v[3] = {0.f, 0.f, 0.f}, ri = 0.f;
        if (e < e1) {
          j = esend[e];
          edge_vector(pos, cell, batch_idx, i, j, eS + 3 * e, v);
          const float rr = sqrtf(v[0] * v[0] + v[1] * v[1] + v[2] * v[2]);
          if (rr < rmax && rr > 0.f && (nz == 1 || species[j] == s)) { ri = 1.f / rr; ok = 1; }
        }
        const unsigned okmask = __ballot_sync(0xffffffffu, ok);
        // ---- lane = (lm, half): contraction of Q with the two h3 rows of every live edge
        const int cnt = min(32, e1 - eb);
        if (okmask != 0u) {
          // The value and derivative rows of consecutive edges are one contiguous block (512 B per edge).  The warp stages
          // it in shared memory in sub-batches of L0_SUB edges with 16-byte asynchronous copies, two sub-batches in
          // flight, so the loads of the next edges overlap the multiply-adds of the current ones (every edge of the
          // batch is contracted; results of masked edges are not used).
          const float* hblock = h3 + (2 * ((int64_t)eb - e_chunk0)) * NK;
          const int nsub = (cnt + L0_SUB - 1) / L0_SUB;
          auto stage = [&](int sb) {
            float* dst = &H[warp][sb & 1][0][0];
#pragma unroll
            for (int u = 0; u < L0_SUB; ++u)
              if (sb * L0_SUB + u < cnt) cp_async16(dst + u * 2 * NK + 4 * lane, hblock + ((int64_t)(sb * L0_SUB + u)) * 2 * NK + 4 * lane);
            cp_async_commit();
          };
          stage(0);
          for (int sb = 0; sb < nsub; ++sb) {
            if (sb + 1 < nsub) { stage(sb + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
            __syncwarp();
            const int m = min(L0_SUB, cnt - sb * L0_SUB);
            for (int u = 0; u < m; ++u) {
              const float4* hv = reinterpret_cast<const float4*>(&H[warp][sb & 1][u][32 * half]);
              float p0 = 0.f, p1 = 0.f, d0 = 0.f, d1 = 0.f;
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                const float4 a = hv[k], d = hv[NK / 4 + k];
                p0 = fmaf(q[k].x, a.x, p0); p1 = fmaf(q[k].y, a.y, p1); p0 = fmaf(q[k].z, a.z, p0); p1 = fmaf(q[k].w, a.w, p1);
                d0 = fmaf(q[k].x, d.x, d0); d1 = fmaf(q[k].y, d.y, d1); d0 = fmaf(q[k].z, d.z, d0); d1 = fmaf(q[k].w, d.w, d1);
              }
              float p = p0 + p1, pd = d0 + d1;
              p += __shfl_xor_sync(0xffffffffu, p, 16);
              pd += __shfl_xor_sync(0xffffffffu, pd, 16);
              if (half == 0) { P[warp][sb * L0_SUB + u][lm] = p; P[warp][sb * L0_SUB + u][16 + lm] = pd; }
            }
            __syncwarp();  // the slot is refilled two iterations later
          }
        }
        __syncwarp();
        // ---- lane = edge: force along the edge
        if (ok) {
          float Y[NLM], M[48];
          const float n0 = v[0] * ri, n1 = v[1] * ri, n2 = v[2] * ri;
          sh_l3(n0, n1, n2, Y);
          sh_l3_force_matrix(n0, n1, n2, ri, Y, M);
          const float4* pp = reinterpret_cast<const float4*>(P[warp][lane]);
          float dY[NLM], pdv[NLM];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float4 a = pp[k], d = pp[4 + k];
            dY[4 * k] = a.x; dY[4 * k + 1] = a.y; dY[4 * k + 2] = a.z; dY[4 * k + 3] = a.w;
            pdv[4 * k] = d.x; pdv[4 * k + 1] = d.y; pdv[4 * k + 2] = d.z; pdv[4 * k + 3] = d.w;
          }
          float qq = 0.f;
#pragma unroll
          for (int b = 0; b < NLM; ++b) qq = fmaf(Y[b], pdv[b], qq);
          float f[3] = {qq * n0, qq * n1, qq * n2};
#pragma unroll
          for (int b = 0; b < NLM; ++b) {
            f[0] = fmaf(dY[b], M[3 * b], f[0]); f[1] = fmaf(dY[b], M[3 * b + 1], f[1]); f[2] = fmaf(dY[b], M[3 * b + 2], f[2]);
          }
#pragma unroll
          for (int d = 0; d < 3; ++d) {
            atomicAdd(grad_pos + 3 * (int64_t)j + d, -f[d]);
            fi[d] += f[d];
          }
          if (virial != nullptr) {
#pragma unroll
            for (int x = 0; x < 3; ++x)
#pragma unroll
              for (int y = 0; y < 3; ++y) vir[3 * x + y] = fmaf(v[x], f[y], vir[3 * x + y]);
          }
        }
        __syncwarp();
      }
    }
    // receiver side: one reduction over the warp per receiver
#pragma unroll
    for (int d = 0; d < 3; ++d) {
      float t = fi[d];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
      if (lane == 0 && t != 0.f) atomicAdd(grad_pos + 3 * (int64_t)i + d, t);
    }
    if (virial != nullptr) {
      double* vp = virial + 9 * (int64_t)batch_idx[i];
#pragma unroll
      for (int k = 0; k < 9; ++k) {
        float t = vir[k];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) atomicAdd(vp + k, (double)t);
      }
    }
  }
}

int l0_grid(int ni) {
  int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  return std::max(1, std::min((ni + L0_WARPS - 1) / L0_WARPS, sms * 8));
}

}  // namespace

// A [n, nz, 16, 64] (rows i0 .. i0 + ni are overwritten); h3 [E_chunk, 64] value rows of the chunk starting at edge e_chunk0.
void mace_l0_moments(const Tensor& h3, const Tensor& pos, const Tensor& cell, const Tensor& batch_idx, const Tensor& eptr,
                     const Tensor& esend, const Tensor& eS, const Tensor& species, int64_t i0, int64_t ni, int64_t e_chunk0,
                     double rmax, Tensor A) {
  c10::cuda::CUDAGuard guard(pos.device());
  NVA_CHECK_CONTIG(A); NVA_CHECK_CONTIG(pos);
  TORCH_CHECK(h3.dim() == 2 && h3.stride(1) == 1, "mace_l0_moments: h3 is [E, 64] (rows may be strided)");
  TORCH_CHECK(A.dim() == 4 && A.size(2) == NLM && A.size(3) == NK && h3.size(-1) == NK, "mace_l0_moments: bad shapes");
  if (ni == 0) return;
  TORCH_CHECK(h3.stride(0) % 4 == 0 && reinterpret_cast<uintptr_t>(h3.data_ptr<float>()) % 16 == 0,
              "mace_l0_moments: h3 rows must start on 16-byte boundaries");
  constexpr int kStageBytes = L0_WARPS * 2 * L0_MSUB * NK * (int)sizeof(float);
  C10_CUDA_CHECK(cudaFuncSetAttribute(l0_moments_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kStageBytes));
  l0_moments_kernel<<<l0_grid((int)ni), 32 * L0_WARPS, kStageBytes, at::cuda::getCurrentCUDAStream()>>>(
      h3.data_ptr<float>(), e_chunk0, pos.data_ptr<float>(), cell.data_ptr<float>(), batch_idx.data_ptr<int>(),
      eptr.data_ptr<int>(), esend.data_ptr<int>(), eS.data_ptr<int>(), species.data_ptr<int>(), (int)A.size(1), (int)i0,
      (int)ni, (float)rmax, A.data_ptr<float>(), (int)h3.stride(0));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// Q [n, nz, 16, 64] = dE/dA; h3 [E_chunk, 2, 64] (value row, radial-derivative row per edge).
void mace_l0_force(const Tensor& h3, const Tensor& Q, const Tensor& pos, const Tensor& cell, const Tensor& batch_idx,
                   const Tensor& eptr, const Tensor& esend, const Tensor& eS, const Tensor& species, int64_t i0, int64_t ni,
                   int64_t e_chunk0, double rmax, Tensor grad_pos, const c10::optional<Tensor>& virial) {
  c10::cuda::CUDAGuard guard(pos.device());
  NVA_CHECK_CONTIG(h3); NVA_CHECK_CONTIG(Q); NVA_CHECK_CONTIG(pos); NVA_CHECK_CONTIG(grad_pos);
  TORCH_CHECK(Q.dim() == 4 && Q.size(2) == NLM && Q.size(3) == NK && h3.size(-1) == NK, "mace_l0_force: bad shapes");
  if (ni == 0) return;
  constexpr int kStageBytes = L0_WARPS * 2 * L0_SUB * 2 * NK * (int)sizeof(float);
  // above the 48 KB static limit: opt in (per device; a few microseconds per call)
  C10_CUDA_CHECK(cudaFuncSetAttribute(l0_force_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kStageBytes));
  l0_force_kernel<<<l0_grid((int)ni), 32 * L0_WARPS, kStageBytes, at::cuda::getCurrentCUDAStream()>>>(
      h3.data_ptr<float>(), e_chunk0, Q.data_ptr<float>(), pos.data_ptr<float>(), cell.data_ptr<float>(),
      batch_idx.data_ptr<int>(), eptr.data_ptr<int>(), esend.data_ptr<int>(), eS.data_ptr<int>(), species.data_ptr<int>(),
      (int)Q.size(1), (int)i0, (int)ni, (float)rmax, grad_pos.data_ptr<float>(),
      virial.has_value() ? virial->data_ptr<double>() : nullptr);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

}  // namespace nva

TORCH_LIBRARY_FRAGMENT(nvalchemi, m) {
  m.def("mace_l0_moments(Tensor h3, Tensor pos, Tensor cell, Tensor batch_idx, Tensor eptr, Tensor esend, Tensor eS, Tensor species, int i0, int ni, int e_chunk0, float rmax, Tensor(a!) A) -> ()", &nva::mace_l0_moments);
  m.def("mace_l0_force(Tensor h3, Tensor Q, Tensor pos, Tensor cell, Tensor batch_idx, Tensor eptr, Tensor esend, Tensor eS, Tensor species, int i0, int ni, int e_chunk0, float rmax, Tensor(a!) grad_pos, Tensor(b!)? virial) -> ()", &nva::mace_l0_force);
}
