// SPDX-License-Identifier: Apache-2.0
// Device helpers shared by the MACE kernels: real spherical harmonics (l <= 3) with their vector-Jacobian
// product, and the sender -> receiver edge vector under periodic images.
#pragma once
#include <cuda_runtime.h>

namespace nva {

constexpr int kEdgeTile = 32;

struct EdgeGeom {  // per-edge quantities shared by the channels of a block
  float Y[16];
  float n[3];
  float rinv;
};

__device__ __forceinline__ void sh_l3(float x, float y, float z, float* Y) {
  const float s3 = 1.7320508075688772f, s5 = 2.23606797749979f, s15 = 3.872983346207417f,
              s70 = 8.366600265340756f, s105 = 10.246950765959598f, s42 = 6.48074069840786f,
              s7 = 2.6457513110645907f;
  float x2 = x * x, y2 = y * y, z2 = z * z;
  Y[0] = 1.f;
  Y[1] = s3 * y; Y[2] = s3 * z; Y[3] = s3 * x;
  Y[4] = s15 * x * y; Y[5] = s15 * y * z; Y[6] = 0.5f * s5 * (2.f * z2 - x2 - y2); Y[7] = s15 * x * z;
  Y[8] = 0.5f * s15 * (x2 - y2);
  Y[9] = 0.25f * s70 * y * (3.f * x2 - y2); Y[10] = s105 * x * y * z;
  Y[11] = 0.25f * s42 * y * (4.f * z2 - x2 - y2); Y[12] = 0.5f * s7 * z * (2.f * z2 - 3.f * x2 - 3.f * y2);
  Y[13] = 0.25f * s42 * x * (4.f * z2 - x2 - y2); Y[14] = 0.5f * s105 * z * (x2 - y2);
  Y[15] = 0.25f * s70 * x * (x2 - 3.f * y2);
}

// g += sum_b dY[b] * dY_b/dn (gradient of the homogeneous polynomials w.r.t. the unit vector),
// s = sum_b l_b dY[b] Y[b]  (Euler term of the projection onto the sphere)
__device__ __forceinline__ void sh_l3_vjp(float x, float y, float z, const float* Y, const float* dY, float* g,
                                          float& s) {
  const float s3 = 1.7320508075688772f, s5 = 2.23606797749979f, s15 = 3.872983346207417f,
              s70 = 8.366600265340756f, s105 = 10.246950765959598f, s42 = 6.48074069840786f,
              s7 = 2.6457513110645907f;
  float x2 = x * x, y2 = y * y, z2 = z * z;
  float gx = 0.f, gy = 0.f, gz = 0.f;
  gy += s3 * dY[1]; gz += s3 * dY[2]; gx += s3 * dY[3];
  gx += s15 * y * dY[4]; gy += s15 * x * dY[4];
  gy += s15 * z * dY[5]; gz += s15 * y * dY[5];
  gx += -s5 * x * dY[6]; gy += -s5 * y * dY[6]; gz += 2.f * s5 * z * dY[6];
  gx += s15 * z * dY[7]; gz += s15 * x * dY[7];
  gx += s15 * x * dY[8]; gy += -s15 * y * dY[8];
  gx += 0.25f * s70 * 6.f * x * y * dY[9]; gy += 0.25f * s70 * (3.f * x2 - 3.f * y2) * dY[9];
  gx += s105 * y * z * dY[10]; gy += s105 * x * z * dY[10]; gz += s105 * x * y * dY[10];
  gx += 0.25f * s42 * (-2.f * x * y) * dY[11]; gy += 0.25f * s42 * (4.f * z2 - x2 - 3.f * y2) * dY[11];
  gz += 0.25f * s42 * 8.f * y * z * dY[11];
  gx += 0.5f * s7 * (-6.f * x * z) * dY[12]; gy += 0.5f * s7 * (-6.f * y * z) * dY[12];
  gz += 0.5f * s7 * (6.f * z2 - 3.f * x2 - 3.f * y2) * dY[12];
  gx += 0.25f * s42 * (4.f * z2 - 3.f * x2 - y2) * dY[13]; gy += 0.25f * s42 * (-2.f * x * y) * dY[13];
  gz += 0.25f * s42 * 8.f * x * z * dY[13];
  gx += 0.5f * s105 * 2.f * x * z * dY[14]; gy += 0.5f * s105 * (-2.f * y * z) * dY[14];
  gz += 0.5f * s105 * (x2 - y2) * dY[14];
  gx += 0.25f * s70 * (3.f * x2 - 3.f * y2) * dY[15]; gy += 0.25f * s70 * (-6.f * x * y) * dY[15];
  g[0] = gx; g[1] = gy; g[2] = gz;
  float s1 = dY[1] * Y[1] + dY[2] * Y[2] + dY[3] * Y[3];
  float s2 = dY[4] * Y[4] + dY[5] * Y[5] + dY[6] * Y[6] + dY[7] * Y[7] + dY[8] * Y[8];
  float s3_ = dY[9] * Y[9] + dY[10] * Y[10] + dY[11] * Y[11] + dY[12] * Y[12] + dY[13] * Y[13] + dY[14] * Y[14] +
              dY[15] * Y[15];
  s = s1 + 2.f * s2 + 3.f * s3_;
}

// M[b][d] (row-major [16][3]) such that the force on the edge direction is  f[d] = sum_b dY[b] * M[b][d]:
// M = (dY_b/dn_d - l_b Y_b n_d) / r, the Jacobian of the harmonics projected onto the sphere and scaled by 1/r.
// Computed once per edge; consumers then need 48 multiply-adds instead of re-deriving the polynomials per channel.
__device__ __forceinline__ void sh_l3_force_matrix(float x, float y, float z, float rinv, const float* Y, float* M) {
  const float s3 = 1.7320508075688772f, s5 = 2.23606797749979f, s15 = 3.872983346207417f,
              s70 = 8.366600265340756f, s105 = 10.246950765959598f, s42 = 6.48074069840786f,
              s7 = 2.6457513110645907f;
  float x2 = x * x, y2 = y * y, z2 = z * z;
  float J[48];
#pragma unroll
  for (int k = 0; k < 48; ++k) J[k] = 0.f;
  J[3 * 1 + 1] = s3; J[3 * 2 + 2] = s3; J[3 * 3 + 0] = s3;
  J[3 * 4 + 0] = s15 * y; J[3 * 4 + 1] = s15 * x;
  J[3 * 5 + 1] = s15 * z; J[3 * 5 + 2] = s15 * y;
  J[3 * 6 + 0] = -s5 * x; J[3 * 6 + 1] = -s5 * y; J[3 * 6 + 2] = 2.f * s5 * z;
  J[3 * 7 + 0] = s15 * z; J[3 * 7 + 2] = s15 * x;
  J[3 * 8 + 0] = s15 * x; J[3 * 8 + 1] = -s15 * y;
  J[3 * 9 + 0] = 0.25f * s70 * 6.f * x * y; J[3 * 9 + 1] = 0.25f * s70 * (3.f * x2 - 3.f * y2);
  J[3 * 10 + 0] = s105 * y * z; J[3 * 10 + 1] = s105 * x * z; J[3 * 10 + 2] = s105 * x * y;
  J[3 * 11 + 0] = 0.25f * s42 * (-2.f * x * y); J[3 * 11 + 1] = 0.25f * s42 * (4.f * z2 - x2 - 3.f * y2);
  J[3 * 11 + 2] = 0.25f * s42 * 8.f * y * z;
  J[3 * 12 + 0] = 0.5f * s7 * (-6.f * x * z); J[3 * 12 + 1] = 0.5f * s7 * (-6.f * y * z);
  J[3 * 12 + 2] = 0.5f * s7 * (6.f * z2 - 3.f * x2 - 3.f * y2);
  J[3 * 13 + 0] = 0.25f * s42 * (4.f * z2 - 3.f * x2 - y2); J[3 * 13 + 1] = 0.25f * s42 * (-2.f * x * y);
  J[3 * 13 + 2] = 0.25f * s42 * 8.f * x * z;
  J[3 * 14 + 0] = 0.5f * s105 * 2.f * x * z; J[3 * 14 + 1] = 0.5f * s105 * (-2.f * y * z);
  J[3 * 14 + 2] = 0.5f * s105 * (x2 - y2);
  J[3 * 15 + 0] = 0.25f * s70 * (3.f * x2 - 3.f * y2); J[3 * 15 + 1] = 0.25f * s70 * (-6.f * x * y);
  const float n[3] = {x, y, z};
#pragma unroll
  for (int b = 0; b < 16; ++b) {
    float l = b == 0 ? 0.f : (b < 4 ? 1.f : (b < 9 ? 2.f : 3.f));
    float ly = l * Y[b];
#pragma unroll
    for (int d = 0; d < 3; ++d) M[3 * b + d] = (J[3 * b + d] - ly * n[d]) * rinv;
  }
}

__device__ __forceinline__ void edge_vector(const float* __restrict__ pos, const float* __restrict__ cell,
                                            const int* __restrict__ batch_idx, int i, int j,
                                            const int* __restrict__ S, float* v) {
  const float* H = cell + 9 * batch_idx[i];
  float s0 = (float)S[0], s1 = (float)S[1], s2 = (float)S[2];
  v[0] = pos[3 * i] - (pos[3 * j] + s0 * H[0] + s1 * H[3] + s2 * H[6]);
  v[1] = pos[3 * i + 1] - (pos[3 * j + 1] + s0 * H[1] + s1 * H[4] + s2 * H[7]);
  v[2] = pos[3 * i + 2] - (pos[3 * j + 2] + s0 * H[2] + s1 * H[5] + s2 * H[8]);
}

}  // namespace nva
