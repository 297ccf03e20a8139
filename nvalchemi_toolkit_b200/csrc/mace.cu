// SPDX-License-Identifier: Apache-2.0
// Native MACE kernels for sm_100a: edge radial features, fused (geometry + channel-wise tensor
// product + neighbour aggregation) convolution forward/backward, symmetric contraction
// forward/backward.  They replace the e3nn / cuEquivariance ops the reference reaches through
// mace-torch (nvalchemi/models/mace.py:205-332,403-411).
//
// Layout: node features [N, n_lm, C] with the channel fastest; one CUDA thread owns one channel of
// one receiver atom, so all global accesses are coalesced over channels and the aggregation over
// neighbours happens in registers (edges are stored CSR by receiver: no atomics in the forward).
// Edge vectors point sender -> receiver: vec = r_i - (r_j + S @ cell).
#include "common.cuh"
#include "mace_tables.h"
#include "mace_device.cuh"

namespace nva {
using at::Tensor;

// ---- radial features: Bessel * polynomial cutoff and their derivative w.r.t. r ----------------
// out [E_chunk, 2, nb]: row 0 = features, row 1 = d/dr (zero features beyond r_max).
__global__ void edge_radial_kernel(int64_t e0, int64_t ne, const float* __restrict__ pos,
                                   const float* __restrict__ cell, const int* __restrict__ batch_idx,
                                   const int* __restrict__ erecv, const int* __restrict__ esend,
                                   const int* __restrict__ eS, float rmax, int nb, int p, bool with_grad,
                                   float* __restrict__ out) {
  int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (t >= ne) return;
  int64_t e = e0 + t;
  float v[3];
  edge_vector(pos, cell, batch_idx, erecv[e], esend[e], eS + 3 * e, v);
  float r = sqrtf(v[0] * v[0] + v[1] * v[1] + v[2] * v[2]);
  int stride = with_grad ? 2 * nb : nb;
  float* o = out + t * stride;
  if (r >= rmax || r <= 0.f) {
    for (int k = 0; k < stride; ++k) o[k] = 0.f;
    return;
  }
  float x = r / rmax, fp = (float)p;
  float xp = powf(x, fp - 1.f);  // x^(p-1)
  float env = 1.f - 0.5f * (fp + 1.f) * (fp + 2.f) * xp * x + fp * (fp + 2.f) * xp * x * x -
              0.5f * fp * (fp + 1.f) * xp * x * x * x;
  float denv = (-0.5f * (fp + 1.f) * (fp + 2.f) * fp * xp + fp * (fp + 2.f) * (fp + 1.f) * xp * x -
                0.5f * fp * (fp + 1.f) * (fp + 2.f) * xp * x * x) / rmax;
  float pref = sqrtf(2.f / rmax), rinv = 1.f / r;
  for (int k = 0; k < nb; ++k) {
    float w = (float)(k + 1) * 3.14159265358979323846f / rmax;
    float sn, cs;
    sincosf(w * r, &sn, &cs);
    float b = pref * sn * rinv;
    o[k] = b * env;
    if (with_grad) o[nb + k] = (pref * w * cs * rinv - b * rinv) * env + b * denv;
  }
}

// ---- convolution forward -------------------------------------------------------------------------
// mid[i, :, c] = sum_{e in edges(i)} TP(u[sender(e), :, c], Y(e), R[e, :, c])      (thread = channel)
template <int NIN, int NPATH, int NMID, bool L1>
__global__ void __launch_bounds__(256) conv_fwd_kernel(
    int i0, const float* __restrict__ u, const float* __restrict__ pos, const float* __restrict__ cell,
    const int* __restrict__ batch_idx, const int* __restrict__ eptr, const int* __restrict__ esend,
    const int* __restrict__ eS, const float* __restrict__ R, int64_t e_chunk0, float rmax, int C,
    float* __restrict__ mid, const int* __restrict__ home_rank, const int* __restrict__ home_row,
    const int64_t* __restrict__ u_ptrs) {
  __shared__ float sY[kEdgeTile][16];
  __shared__ int sj[kEdgeTile];
  __shared__ const float* sup[kEdgeTile];  // sender feature row (local, or a peer GPU's row over NVLink)
  int i = i0 + blockIdx.x;
  int c = threadIdx.x;
  float acc[NMID];
#pragma unroll
  for (int o = 0; o < NMID; ++o) acc[o] = 0.f;
  int eb = eptr[i], ee = eptr[i + 1];
  for (int base = eb; base < ee; base += kEdgeTile) {
    int nt = min(kEdgeTile, ee - base);
    if (threadIdx.x < nt) {
      int e = base + threadIdx.x;
      int j = esend[e];
      float v[3];
      edge_vector(pos, cell, batch_idx, i, j, eS + 3 * e, v);
      float r = sqrtf(v[0] * v[0] + v[1] * v[1] + v[2] * v[2]);
      bool ok = r < rmax && r > 0.f;
      float ri = ok ? 1.f / r : 0.f;
      sh_l3(v[0] * ri, v[1] * ri, v[2] * ri, sY[threadIdx.x]);
      sj[threadIdx.x] = ok ? j : -1;
      const float* ub = u;
      int64_t jr = j;
      if (home_rank != nullptr) { ub = reinterpret_cast<const float*>(u_ptrs[home_rank[j]]); jr = home_row[j]; }
      sup[threadIdx.x] = ub + jr * NIN * C;  // rows of cut-off edges are loaded (prefetch) but never used
    }
    __syncthreads();
    // software pipeline: the loads of edge t+1 are in flight while edge t is being contracted
    float h[NIN], Rv[NPATH], hn[NIN], Rn[NPATH];
    {
      const float* up = sup[0] + c;
      const float* rp = R + ((int64_t)base - e_chunk0) * NPATH * C + c;
#pragma unroll
      for (int a = 0; a < NIN; ++a) hn[a] = __ldg(up + a * C);
#pragma unroll
      for (int p = 0; p < NPATH; ++p) Rn[p] = __ldg(rp + p * C);
    }
    for (int t = 0; t < nt; ++t) {
#pragma unroll
      for (int a = 0; a < NIN; ++a) h[a] = hn[a];
#pragma unroll
      for (int p = 0; p < NPATH; ++p) Rv[p] = Rn[p];
      if (t + 1 < nt) {
        const float* up = sup[t + 1] + c;
        const float* rp = R + ((int64_t)(base + t + 1) - e_chunk0) * NPATH * C + c;
#pragma unroll
        for (int a = 0; a < NIN; ++a) hn[a] = __ldg(up + a * C);
#pragma unroll
        for (int p = 0; p < NPATH; ++p) Rn[p] = __ldg(rp + p * C);
      }
      if (sj[t] < 0) continue;
      const float* Y = sY[t];
      if (L1) { MACE_L1_FWD(h, Y, Rv, acc); } else { MACE_L0_FWD(h, Y, Rv, acc); }
    }
    __syncthreads();
  }
  float* mp = mid + (int64_t)i * NMID * C + c;
#pragma unroll
  for (int o = 0; o < NMID; ++o) mp[o * C] = acc[o];
}

// ---- convolution backward ------------------------------------------------------------------------
// Given G = dE/dmid: du[sender] += ..., dE/dvec per edge -> grad_pos (receiver +, sender -), optional
// per-system virial sum_e vec (x) dE/dvec.  RD holds [R | dR/dr] per edge: [E_chunk, 2, NPATH, C].
template <int NIN, int NPATH, int NMID, int NT, bool L1, bool NEED_DU>
__global__ void __launch_bounds__(256) conv_bwd_kernel(
    int i0, const float* __restrict__ u, const float* __restrict__ G, const float* __restrict__ pos,
    const float* __restrict__ cell, const int* __restrict__ batch_idx, const int* __restrict__ eptr,
    const int* __restrict__ esend, const int* __restrict__ eS, const float* __restrict__ RD, int64_t e_chunk0,
    float rmax, int C, float* __restrict__ du, float* __restrict__ grad_pos, double* __restrict__ virial,
    const int* __restrict__ home_rank, const int* __restrict__ home_row, const int64_t* __restrict__ u_ptrs,
    const int64_t* __restrict__ du_ptrs, const int64_t* __restrict__ gpos_ptrs) {
  __shared__ EdgeGeom sg[kEdgeTile];
  __shared__ const float* sup[kEdgeTile];
  __shared__ float* sdup[kEdgeTile];
  __shared__ float* sgp[kEdgeTile];
  __shared__ float sv[kEdgeTile][3];
  __shared__ int sj[kEdgeTile];
  __shared__ float sred[kEdgeTile][8][3];
  int i = i0 + blockIdx.x;
  int c = threadIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  float T[NT];  // G contracted with the coupling coefficients: constant over the receiver's edges
  {
    float Gr[NMID];
    const float* gp = G + (int64_t)i * NMID * C + c;
#pragma unroll
    for (int o = 0; o < NMID; ++o) Gr[o] = gp[o * C];
    if (L1) { MACE_L1_BWD_PREP(Gr, T); } else { MACE_L0_BWD_PREP(Gr, T); }
  }
  int eb = eptr[i], ee = eptr[i + 1];
  float fi[3] = {0.f, 0.f, 0.f};
  float vir[9] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int base = eb; base < ee; base += kEdgeTile) {
    int nt = min(kEdgeTile, ee - base);
    if (threadIdx.x < nt) {
      int e = base + threadIdx.x;
      int j = esend[e];
      float v[3];
      edge_vector(pos, cell, batch_idx, i, j, eS + 3 * e, v);
      float r = sqrtf(v[0] * v[0] + v[1] * v[1] + v[2] * v[2]);
      bool ok = r < rmax && r > 0.f;
      float ri = ok ? 1.f / r : 0.f;
      EdgeGeom& g = sg[threadIdx.x];
      g.n[0] = v[0] * ri; g.n[1] = v[1] * ri; g.n[2] = v[2] * ri; g.rinv = ri;
      sh_l3(g.n[0], g.n[1], g.n[2], g.Y);
      sv[threadIdx.x][0] = v[0]; sv[threadIdx.x][1] = v[1]; sv[threadIdx.x][2] = v[2];
      sj[threadIdx.x] = ok ? j : -1;
      const float* ub = u;
      float* dub = du;
      float* gpb = grad_pos;
      int64_t jr = j;
      if (home_rank != nullptr) {
        int hr = home_rank[j];
        jr = home_row[j];
        ub = reinterpret_cast<const float*>(u_ptrs[hr]);
        if (NEED_DU) dub = reinterpret_cast<float*>(du_ptrs[hr]);
        gpb = reinterpret_cast<float*>(gpos_ptrs[hr]);
      }
      sup[threadIdx.x] = ub + jr * NIN * C;
      sdup[threadIdx.x] = NEED_DU ? dub + jr * NIN * C : nullptr;
      sgp[threadIdx.x] = gpb + 3 * jr;
    }
    __syncthreads();
    float hn[NIN], Rn[2 * NPATH];
    {
      const float* up = sup[0] + c;
      const float* rp = RD + ((int64_t)base - e_chunk0) * 2 * NPATH * C + c;
#pragma unroll
      for (int a = 0; a < NIN; ++a) hn[a] = __ldg(up + a * C);
#pragma unroll
      for (int p = 0; p < 2 * NPATH; ++p) Rn[p] = __ldg(rp + p * C);
    }
    for (int t = 0; t < nt; ++t) {
      int j = sj[t];
      float f[3] = {0.f, 0.f, 0.f};
      float h[NIN], Rv[NPATH], Rd[NPATH];
#pragma unroll
      for (int a = 0; a < NIN; ++a) h[a] = hn[a];
#pragma unroll
      for (int p = 0; p < NPATH; ++p) { Rv[p] = Rn[p]; Rd[p] = Rn[NPATH + p]; }
      if (t + 1 < nt) {
        const float* up = sup[t + 1] + c;
        const float* rp = RD + ((int64_t)(base + t + 1) - e_chunk0) * 2 * NPATH * C + c;
#pragma unroll
        for (int a = 0; a < NIN; ++a) hn[a] = __ldg(up + a * C);
#pragma unroll
        for (int p = 0; p < 2 * NPATH; ++p) Rn[p] = __ldg(rp + p * C);
      }
      if (j >= 0) {
        float dh[NIN], dY[16], S[NPATH];
#pragma unroll
        for (int a = 0; a < NIN; ++a) dh[a] = 0.f;
#pragma unroll
        for (int b = 0; b < 16; ++b) dY[b] = 0.f;
        const EdgeGeom& g = sg[t];
        const float* Y = g.Y;
        if (L1) { MACE_L1_BWD_EDGE(h, Y, Rv, T, dh, dY, S); } else { MACE_L0_BWD_EDGE(h, Y, Rv, T, dh, dY, S); }
        float q = 0.f;
#pragma unroll
        for (int p = 0; p < NPATH; ++p) q = fmaf(S[p], Rd[p], q);
        float gy[3], s;
        sh_l3_vjp(g.n[0], g.n[1], g.n[2], Y, dY, gy, s);
#pragma unroll
        for (int d = 0; d < 3; ++d) f[d] = (gy[d] - s * g.n[d]) * g.rinv + q * g.n[d];
        if (NEED_DU) {
          float* dp = sdup[t] + c;
#pragma unroll
          for (int a = 0; a < NIN; ++a) atomicAdd(dp + a * C, dh[a]);
        }
      }
#pragma unroll
      for (int d = 0; d < 3; ++d) {
        float x = f[d];
        for (int o = 16; o > 0; o >>= 1) x += __shfl_down_sync(0xffffffffu, x, o);
        if (lane == 0) sred[t][warp][d] = x;
      }
    }
    __syncthreads();
    if (threadIdx.x < nt) {
      int j = sj[threadIdx.x];
      if (j >= 0) {
        float f[3] = {0.f, 0.f, 0.f};
        for (int w = 0; w < nwarp; ++w)
          for (int d = 0; d < 3; ++d) f[d] += sred[threadIdx.x][w][d];
        for (int d = 0; d < 3; ++d) {
          atomicAdd(sgp[threadIdx.x] + d, -f[d]);
          fi[d] += f[d];
        }
        if (virial != nullptr)
          for (int a = 0; a < 3; ++a)
            for (int b = 0; b < 3; ++b) vir[3 * a + b] += sv[threadIdx.x][a] * f[b];
      }
    }
    __syncthreads();
  }
  // threads 0..31 of warp 0 hold per-edge partial sums for the receiver: reduce and commit
  if (warp == 0) {
    for (int d = 0; d < 3; ++d) {
      float x = fi[d];
      for (int o = 16; o > 0; o >>= 1) x += __shfl_down_sync(0xffffffffu, x, o);
      if (lane == 0) atomicAdd(grad_pos + 3 * (int64_t)i + d, x);
    }
    if (virial != nullptr) {
      for (int k = 0; k < 9; ++k) {
        float x = vir[k];
        for (int o = 16; o > 0; o >>= 1) x += __shfl_down_sync(0xffffffffu, x, o);
        if (lane == 0) atomicAdd(virial + 9 * (int64_t)batch_idx[i] + k, (double)x);
      }
    }
  }
}

// ---- symmetric contraction -----------------------------------------------------------------------
// out[n, M, c] = sum_nu sum_eta W_nu[z_n, eta, c] * P_{nu,eta,M}(x[n, :, c]); the polynomials P are emitted as
// straight-line code (mace_tables.h), x and its gradient stay in registers.  Weights are packed per L as
// [Z, nb1 + nb2 + nb3, C] (degree blocks in that order).
#define W(k) __ldg(wp + (k) * C)
template <bool BWD>
__global__ void __launch_bounds__(128) symcon_kernel(int64_t n_nodes, int C, int lmax_out, int correlation,
                                                     const float* __restrict__ xg, const int* __restrict__ species,
                                                     const float* __restrict__ w0, const float* __restrict__ w1,
                                                     int nbtot0, int nbtot1, float* __restrict__ outg,
                                                     const float* __restrict__ gout, float* __restrict__ dxg) {
  int64_t gidx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int64_t n = gidx / C;
  int c = (int)(gidx - n * C);
  if (n >= n_nodes) return;
  float x[16], dx[16];
  const float* xp = xg + n * 16 * C + c;
#pragma unroll
  for (int k = 0; k < 16; ++k) { x[k] = xp[k * C]; dx[k] = 0.f; }
  int z = species[n];
  int nout = (lmax_out + 1) * (lmax_out + 1);
  {
    const float* wp = w0 + (int64_t)z * nbtot0 * C + c;
    float out[1] = {0.f};
    float g[1] = {0.f};
    if (BWD) g[0] = gout[(n * nout) * C + c];
    if (!BWD) { MACE_SYM_FWD_1_0(x, out); } else { MACE_SYM_BWD_1_0(x, g, dx); }
    wp += MACE_SYM_1_0_NBASIS * C;
    if (correlation >= 2) {
      if (!BWD) { MACE_SYM_FWD_2_0(x, out); } else { MACE_SYM_BWD_2_0(x, g, dx); }
      wp += MACE_SYM_2_0_NBASIS * C;
    }
    if (correlation >= 3) {
      if (!BWD) { MACE_SYM_FWD_3_0(x, out); } else { MACE_SYM_BWD_3_0(x, g, dx); }
    }
    if (!BWD) outg[(n * nout) * C + c] = out[0];
  }
  if (lmax_out >= 1) {
    const float* wp = w1 + (int64_t)z * nbtot1 * C + c;
    float out[3] = {0.f, 0.f, 0.f};
    float g[3] = {0.f, 0.f, 0.f};
    if (BWD) {
#pragma unroll
      for (int M = 0; M < 3; ++M) g[M] = gout[(n * nout + 1 + M) * C + c];
    }
    if (!BWD) { MACE_SYM_FWD_1_1(x, out); } else { MACE_SYM_BWD_1_1(x, g, dx); }
    wp += MACE_SYM_1_1_NBASIS * C;
    if (correlation >= 2) {
      if (!BWD) { MACE_SYM_FWD_2_1(x, out); } else { MACE_SYM_BWD_2_1(x, g, dx); }
      wp += MACE_SYM_2_1_NBASIS * C;
    }
    if (correlation >= 3) {
      if (!BWD) { MACE_SYM_FWD_3_1(x, out); } else { MACE_SYM_BWD_3_1(x, g, dx); }
    }
    if (!BWD) {
#pragma unroll
      for (int M = 0; M < 3; ++M) outg[(n * nout + 1 + M) * C + c] = out[M];
    }
  }
  if (BWD) {
    float* dp = dxg + n * 16 * C + c;
#pragma unroll
    for (int k = 0; k < 16; ++k) dp[k * C] = dx[k];
  }
}
#undef W

// ---- radial MLP activation with forward-mode tangent ---------------------------------------------
// a [E, 2, H] in place: row 0 <- silu(a0) * norm, row 1 <- silu'(a0) * norm * a1.
__global__ void silu_tangent_kernel(int64_t total, int H, float* __restrict__ a) {
  int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (t >= total) return;
  int64_t e = t / H;
  int k = (int)(t - e * H);
  float* p = a + e * 2 * H + k;
  float x = p[0], tx = p[H];
  float s = 1.f / (1.f + __expf(-x));
  const float norm = 1.6790176868438721f;
  p[0] = x * s * norm;
  p[H] = s * (1.f + x * (1.f - s)) * norm * tx;
}

void mace_silu_tangent_(Tensor a) {
  c10::cuda::CUDAGuard guard(a.device());
  NVA_CHECK_CONTIG(a);
  TORCH_CHECK(a.dim() == 3 && a.size(1) == 2, "expected [E, 2, H]");
  int64_t total = a.size(0) * a.size(2);
  if (total == 0) return;
  silu_tangent_kernel<<<(unsigned)((total + 255) / 256), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      total, (int)a.size(2), a.data_ptr<float>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// ---- host wrappers -------------------------------------------------------------------------------
Tensor mace_edge_radial(const Tensor& pos, const Tensor& cell, const Tensor& batch_idx, const Tensor& erecv,
                        const Tensor& esend, const Tensor& eS, int64_t e0, int64_t ne, double rmax, int64_t nb,
                        int64_t p, bool with_grad) {
  c10::cuda::CUDAGuard guard(pos.device());
  Tensor out = at::empty({ne, with_grad ? 2 : 1, nb}, pos.options());
  if (ne == 0) return out;
  edge_radial_kernel<<<(unsigned)((ne + 255) / 256), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      e0, ne, pos.data_ptr<float>(), cell.data_ptr<float>(), batch_idx.data_ptr<int>(), erecv.data_ptr<int>(),
      esend.data_ptr<int>(), eS.data_ptr<int>(), (float)rmax, (int)nb, (int)p, with_grad, out.data_ptr<float>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

void mace_conv_fwd(const Tensor& u, const Tensor& pos, const Tensor& cell, const Tensor& batch_idx,
                   const Tensor& eptr, const Tensor& esend, const Tensor& eS, const Tensor& R, int64_t i0,
                   int64_t ni, int64_t e_chunk0, double rmax, Tensor mid, const c10::optional<Tensor>& home_rank,
                   const c10::optional<Tensor>& home_row, const c10::optional<Tensor>& u_ptrs) {
  c10::cuda::CUDAGuard guard(pos.device());
  NVA_CHECK_CONTIG(u); NVA_CHECK_CONTIG(R); NVA_CHECK_CONTIG(mid);
  int C = (int)u.size(2), nin = (int)u.size(1);
  TORCH_CHECK(C % 32 == 0 && C <= 256, "channels must be a multiple of 32 and <= 256");
  if (ni == 0) return;
  auto st = at::cuda::getCurrentCUDAStream();
#define NVA_ARGS (int)i0, u.data_ptr<float>(), pos.data_ptr<float>(), cell.data_ptr<float>(), batch_idx.data_ptr<int>(), \
    eptr.data_ptr<int>(), esend.data_ptr<int>(), eS.data_ptr<int>(), R.data_ptr<float>(), e_chunk0, (float)rmax, C, \
    mid.data_ptr<float>(), home_rank.has_value() ? home_rank->data_ptr<int>() : nullptr, \
    home_row.has_value() ? home_row->data_ptr<int>() : nullptr, u_ptrs.has_value() ? u_ptrs->data_ptr<int64_t>() : nullptr
  if (nin == 1) {
    TORCH_CHECK(mid.size(1) == MACE_L0_NMID && R.size(1) == MACE_L0_NPATH, "layer-0 shapes");
    conv_fwd_kernel<MACE_L0_NIN, MACE_L0_NPATH, MACE_L0_NMID, false><<<(unsigned)ni, C, 0, st>>>(NVA_ARGS);
  } else {
    TORCH_CHECK(nin == 4 && mid.size(1) == MACE_L1_NMID && R.size(1) == MACE_L1_NPATH, "layer-1 shapes");
    conv_fwd_kernel<MACE_L1_NIN, MACE_L1_NPATH, MACE_L1_NMID, true><<<(unsigned)ni, C, 0, st>>>(NVA_ARGS);
  }
#undef NVA_ARGS
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

void mace_conv_bwd(const Tensor& u, const Tensor& G, const Tensor& pos, const Tensor& cell,
                   const Tensor& batch_idx, const Tensor& eptr, const Tensor& esend, const Tensor& eS,
                   const Tensor& RD, int64_t i0, int64_t ni, int64_t e_chunk0, double rmax,
                   const c10::optional<Tensor>& du, Tensor grad_pos, const c10::optional<Tensor>& virial,
                   const c10::optional<Tensor>& home_rank, const c10::optional<Tensor>& home_row,
                   const c10::optional<Tensor>& u_ptrs, const c10::optional<Tensor>& du_ptrs,
                   const c10::optional<Tensor>& gpos_ptrs) {
  c10::cuda::CUDAGuard guard(pos.device());
  NVA_CHECK_CONTIG(u); NVA_CHECK_CONTIG(RD); NVA_CHECK_CONTIG(G);
  int C = (int)u.size(2), nin = (int)u.size(1);
  TORCH_CHECK(C % 32 == 0 && C <= 256, "channels must be a multiple of 32 and <= 256");
  if (ni == 0) return;
  auto st = at::cuda::getCurrentCUDAStream();
  float* dup = du.has_value() ? du->data_ptr<float>() : nullptr;
  double* vp = virial.has_value() ? virial->data_ptr<double>() : nullptr;
#define NVA_ARGS (int)i0, u.data_ptr<float>(), G.data_ptr<float>(), pos.data_ptr<float>(), cell.data_ptr<float>(), \
    batch_idx.data_ptr<int>(), eptr.data_ptr<int>(), esend.data_ptr<int>(), eS.data_ptr<int>(), RD.data_ptr<float>(), \
    e_chunk0, (float)rmax, C, dup, grad_pos.data_ptr<float>(), vp, \
    home_rank.has_value() ? home_rank->data_ptr<int>() : nullptr, home_row.has_value() ? home_row->data_ptr<int>() : nullptr, \
    u_ptrs.has_value() ? u_ptrs->data_ptr<int64_t>() : nullptr, du_ptrs.has_value() ? du_ptrs->data_ptr<int64_t>() : nullptr, \
    gpos_ptrs.has_value() ? gpos_ptrs->data_ptr<int64_t>() : nullptr
  if (nin == 1) {
    if (dup) conv_bwd_kernel<MACE_L0_NIN, MACE_L0_NPATH, MACE_L0_NMID, MACE_L0_NT, false, true><<<(unsigned)ni, C, 0, st>>>(NVA_ARGS);
    else conv_bwd_kernel<MACE_L0_NIN, MACE_L0_NPATH, MACE_L0_NMID, MACE_L0_NT, false, false><<<(unsigned)ni, C, 0, st>>>(NVA_ARGS);
  } else {
    if (dup) conv_bwd_kernel<MACE_L1_NIN, MACE_L1_NPATH, MACE_L1_NMID, MACE_L1_NT, true, true><<<(unsigned)ni, C, 0, st>>>(NVA_ARGS);
    else conv_bwd_kernel<MACE_L1_NIN, MACE_L1_NPATH, MACE_L1_NMID, MACE_L1_NT, true, false><<<(unsigned)ni, C, 0, st>>>(NVA_ARGS);
  }
#undef NVA_ARGS
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

Tensor mace_symcon_fwd(const Tensor& x, const Tensor& species, const Tensor& w0, const c10::optional<Tensor>& w1,
                       int64_t lmax_out, int64_t correlation) {
  c10::cuda::CUDAGuard guard(x.device());
  NVA_CHECK_CONTIG(x); NVA_CHECK_CONTIG(w0);
  int64_t n = x.size(0);
  int C = (int)x.size(2);
  int nout = (int)((lmax_out + 1) * (lmax_out + 1));
  Tensor out = at::empty({n, nout, C}, x.options());
  if (n == 0) return out;
  int threads = 128;
  int64_t total = n * C;
  symcon_kernel<false><<<(unsigned)((total + threads - 1) / threads), threads, 0, at::cuda::getCurrentCUDAStream()>>>(
      n, C, (int)lmax_out, (int)correlation, x.data_ptr<float>(), species.data_ptr<int>(), w0.data_ptr<float>(),
      w1.has_value() ? w1->data_ptr<float>() : nullptr, (int)w0.size(1), w1.has_value() ? (int)w1->size(1) : 0,
      out.data_ptr<float>(), nullptr, nullptr);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

Tensor mace_symcon_bwd(const Tensor& x, const Tensor& species, const Tensor& w0, const c10::optional<Tensor>& w1,
                       int64_t lmax_out, int64_t correlation, const Tensor& gout) {
  c10::cuda::CUDAGuard guard(x.device());
  NVA_CHECK_CONTIG(x); NVA_CHECK_CONTIG(gout);
  int64_t n = x.size(0);
  int C = (int)x.size(2);
  Tensor dx = at::empty_like(x);
  if (n == 0) return dx;
  int threads = 128;
  int64_t total = n * C;
  symcon_kernel<true><<<(unsigned)((total + threads - 1) / threads), threads, 0, at::cuda::getCurrentCUDAStream()>>>(
      n, C, (int)lmax_out, (int)correlation, x.data_ptr<float>(), species.data_ptr<int>(), w0.data_ptr<float>(),
      w1.has_value() ? w1->data_ptr<float>() : nullptr, (int)w0.size(1), w1.has_value() ? (int)w1->size(1) : 0,
      nullptr, gout.data_ptr<float>(), dx.data_ptr<float>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return dx;
}

}  // namespace nva

TORCH_LIBRARY_FRAGMENT(nvalchemi, m) {
  m.def("mace_edge_radial(Tensor pos, Tensor cell, Tensor batch_idx, Tensor erecv, Tensor esend, Tensor eS, int e0, int ne, float rmax, int nb, int p, bool with_grad) -> Tensor", &nva::mace_edge_radial);
  m.def("mace_conv_fwd(Tensor u, Tensor pos, Tensor cell, Tensor batch_idx, Tensor eptr, Tensor esend, Tensor eS, Tensor R, int i0, int ni, int e_chunk0, float rmax, Tensor(a!) mid, Tensor? home_rank=None, Tensor? home_row=None, Tensor? u_ptrs=None) -> ()", &nva::mace_conv_fwd);
  m.def("mace_conv_bwd(Tensor u, Tensor G, Tensor pos, Tensor cell, Tensor batch_idx, Tensor eptr, Tensor esend, Tensor eS, Tensor RD, int i0, int ni, int e_chunk0, float rmax, Tensor(a!)? du, Tensor(b!) grad_pos, Tensor(c!)? virial, Tensor? home_rank=None, Tensor? home_row=None, Tensor? u_ptrs=None, Tensor? du_ptrs=None, Tensor? gpos_ptrs=None) -> ()", &nva::mace_conv_bwd);
  m.def("mace_silu_tangent_(Tensor(a!) a) -> ()", &nva::mace_silu_tangent_);
  m.def("mace_symcon_fwd(Tensor x, Tensor species, Tensor w0, Tensor? w1, int lmax_out, int correlation) -> Tensor", &nva::mace_symcon_fwd);
  m.def("mace_symcon_bwd(Tensor x, Tensor species, Tensor w0, Tensor? w1, int lmax_out, int correlation, Tensor gout) -> Tensor", &nva::mace_symcon_bwd);
}
