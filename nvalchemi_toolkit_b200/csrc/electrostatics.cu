// SPDX-License-Identifier: Apache-2.0
// Electrostatics kernels: Ewald real space over the dense neighbour matrix, structure factors and their
// back-application (reciprocal forces and potentials), and the three particle-mesh stages (B-spline spread, fused
// reciprocal convolution with energy and virial, gather with forces).  Op surface as in the reference
// (nvalchemi/models/_ops/electrostatics/ewald.py:78-923, pme.py:94-788); every functor runs as a CUDA kernel or an
// OpenMP loop.  Energies are in (charge^2 / length) units; callers multiply by the Coulomb constant.
#include "common.cuh"

namespace nva {
using at::Tensor;

constexpr double kTwoOverSqrtPi = 1.1283791670955125738961589;
constexpr double kPi = 3.14159265358979323846264338;

// ---- Ewald real space -------------------------------------------------------------------------------------------
// Returns per-atom energies [N], forces [N,3], per-system virials [B,9] and potentials dE/dq [N].
std::tuple<Tensor, Tensor, Tensor, Tensor> ewald_real(const Tensor& pos, const Tensor& charges, const Tensor& cell,
                                                      const Tensor& nm, const Tensor& shifts, const Tensor& num,
                                                      const Tensor& batch_idx, const Tensor& alpha, int64_t fill_value,
                                                      double cutoff, bool half_list, int64_t num_systems) {
  c10::cuda::OptionalCUDAGuard guard(pos.is_cuda() ? c10::make_optional(pos.device()) : c10::nullopt);
  NVA_CHECK_CONTIG(pos); NVA_CHECK_CONTIG(nm); NVA_CHECK_CONTIG(shifts); NVA_CHECK_CONTIG(cell); NVA_CHECK_CONTIG(charges);
  TORCH_CHECK(alpha.scalar_type() == at::kDouble && alpha.numel() == num_systems, "alpha: float64 [num_systems]");
  int64_t n = pos.size(0), K = nm.size(1);
  auto dopt = pos.options().dtype(at::kDouble);
  Tensor e = at::zeros({n}, dopt), f = at::zeros({n, 3}, dopt), w = at::zeros({num_systems, 9}, dopt),
         phi = at::zeros({n}, dopt);
  auto st = pos.scalar_type();
  if (n == 0) return {e.to(st), f.to(st), w.to(st), phi.to(st)};
  const int* M = nm.data_ptr<int>();
  const int* S = shifts.data_ptr<int>();
  const int* cnt = num.data_ptr<int>();
  const int* b = batch_idx.data_ptr<int>();
  const double* A = alpha.data_ptr<double>();
  double *E = e.data_ptr<double>(), *F = f.data_ptr<double>(), *W = w.data_ptr<double>(), *P = phi.data_ptr<double>();
  bool cuda = pos.is_cuda();
  AT_DISPATCH_FLOATING_TYPES(st, "ewald_real", [&] {
    const scalar_t* r = pos.data_ptr<scalar_t>();
    const scalar_t* H = cell.data_ptr<scalar_t>();
    const scalar_t* Q = charges.data_ptr<scalar_t>();
    for_each(cuda, n, [=] NVA_LAMBDA(int64_t i) {
      int s = b[i];
      const scalar_t* h = H + 9 * s;
      double a = A[s], qi = Q[i];
      int k_i = cnt[i] < (int)K ? cnt[i] : (int)K;
      double ei = 0, pi_ = 0, fx = 0, fy = 0, fz = 0, vir[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
      double xi = r[3 * i], yi = r[3 * i + 1], zi = r[3 * i + 2];
      double wgt = half_list ? 1.0 : 0.5;
      for (int q = 0; q < k_i; ++q) {
        int j = M[i * K + q];
        if (j >= fill_value || j < 0) continue;
        const int* sh = S + (i * K + q) * 3;
        double dx = (double)r[3 * j] + sh[0] * (double)h[0] + sh[1] * (double)h[3] + sh[2] * (double)h[6] - xi;
        double dy = (double)r[3 * j + 1] + sh[0] * (double)h[1] + sh[1] * (double)h[4] + sh[2] * (double)h[7] - yi;
        double dz = (double)r[3 * j + 2] + sh[0] * (double)h[2] + sh[1] * (double)h[5] + sh[2] * (double)h[8] - zi;
        double r2 = dx * dx + dy * dy + dz * dz;
        if (r2 >= cutoff * cutoff || r2 <= 0.0) continue;
        double rr = sqrt(r2), qj = Q[j];
        double ec = erfc(a * rr) / rr;                                     // erfc(ar)/r
        double dec = -(ec + a * kTwoOverSqrtPi * exp(-a * a * r2)) / rr;   // d/dr of erfc(ar)/r
        ei += wgt * qi * qj * ec;
        pi_ += qj * ec;
        double de = qi * qj * dec;
        double gx = de * dx / rr, gy = de * dy / rr, gz = de * dz / rr;  // dE_pair / d(r_j - r_i)
        fx += gx; fy += gy; fz += gz;
        if (half_list) {
          atomic_add_f64(F + 3 * j, -gx); atomic_add_f64(F + 3 * j + 1, -gy); atomic_add_f64(F + 3 * j + 2, -gz);
          atomic_add_f64(P + j, qi * ec);
        }
        double d[3] = {dx, dy, dz}, g[3] = {gx, gy, gz};
        for (int u = 0; u < 3; ++u)
          for (int v = 0; v < 3; ++v) vir[3 * u + v] -= wgt * d[u] * g[v];
      }
      E[i] = ei;
      atomic_add_f64(P + i, pi_);
      atomic_add_f64(F + 3 * i, fx); atomic_add_f64(F + 3 * i + 1, fy); atomic_add_f64(F + 3 * i + 2, fz);
      for (int u = 0; u < 9; ++u) atomic_add_f64(W + 9 * s + u, vir[u]);
    });
  });
  return {e.to(st), f.to(st), w.to(st), phi.to(st)};
}

// ---- structure factors S(k) = sum_i q_i exp(i k.r_i) over atoms [a0, a1) ----------------------------------------
constexpr int kSkChunk = 128;

Tensor ewald_structure_factors(const Tensor& pos, const Tensor& charges, const Tensor& kvecs, int64_t a0, int64_t a1,
                               const c10::optional<Tensor>& weights) {
  c10::cuda::OptionalCUDAGuard guard(pos.is_cuda() ? c10::make_optional(pos.device()) : c10::nullopt);
  NVA_CHECK_CONTIG(pos); NVA_CHECK_CONTIG(charges); NVA_CHECK_CONTIG(kvecs);
  TORCH_CHECK(kvecs.scalar_type() == at::kDouble, "kvecs must be float64");
  int64_t nk = kvecs.size(0), na = a1 - a0;
  Tensor sk = at::zeros({nk, 2}, pos.options().dtype(at::kDouble));
  if (nk == 0 || na <= 0) return sk;
  int64_t chunks = (na + kSkChunk - 1) / kSkChunk;
  const double* Kv = kvecs.data_ptr<double>();
  double* S = sk.data_ptr<double>();
  bool cuda = pos.is_cuda();
  AT_DISPATCH_FLOATING_TYPES(pos.scalar_type(), "ewald_structure_factors", [&] {
    const scalar_t* r = pos.data_ptr<scalar_t>();
    const scalar_t* Q = charges.data_ptr<scalar_t>();
    const scalar_t* Wt = weights.has_value() ? weights->data_ptr<scalar_t>() : nullptr;
    for_each(cuda, nk * chunks, [=] NVA_LAMBDA(int64_t t) {
      int64_t k = t % nk, c = t / nk;  // consecutive threads share the atom chunk and differ in k
      double kx = Kv[3 * k], ky = Kv[3 * k + 1], kz = Kv[3 * k + 2];
      int64_t lo = a0 + c * kSkChunk, hi = lo + kSkChunk < a1 ? lo + kSkChunk : a1;
      double re = 0, im = 0;
      for (int64_t i = lo; i < hi; ++i) {
        double q = Q[i] * (Wt ? (double)Wt[i] : 1.0);
        double ph = kx * (double)r[3 * i] + ky * (double)r[3 * i + 1] + kz * (double)r[3 * i + 2];
        double sn, cs;
        sincos(ph, &sn, &cs);
        re += q * cs; im += q * sn;
      }
      atomic_add_f64(S + 2 * k, re);
      atomic_add_f64(S + 2 * k + 1, im);
    });
  });
  return sk;
}

// forces F_i = q_i sum_k c_k k Im(exp(i k.r_i) conj S_k) and potentials phi_i = sum_k c_k Re(exp(-i k.r_i) S_k) for atoms
// [a0, a1); `coef` holds c_k (for the half-space sum: (8 pi / V) exp(-k^2/4a^2)/k^2).
std::tuple<Tensor, Tensor> ewald_recip_apply(const Tensor& pos, const Tensor& charges, const Tensor& kvecs,
                                             const Tensor& coef, const Tensor& sk, int64_t a0, int64_t a1) {
  c10::cuda::OptionalCUDAGuard guard(pos.is_cuda() ? c10::make_optional(pos.device()) : c10::nullopt);
  NVA_CHECK_CONTIG(pos); NVA_CHECK_CONTIG(charges); NVA_CHECK_CONTIG(kvecs); NVA_CHECK_CONTIG(coef); NVA_CHECK_CONTIG(sk);
  int64_t nk = kvecs.size(0), na = a1 - a0;
  auto dopt = pos.options().dtype(at::kDouble);
  Tensor f = at::zeros({na > 0 ? na : 0, 3}, dopt), phi = at::zeros({na > 0 ? na : 0}, dopt);
  if (na <= 0 || nk == 0) return {f, phi};
  const double *Kv = kvecs.data_ptr<double>(), *C = coef.data_ptr<double>(), *S = sk.data_ptr<double>();
  double *F = f.data_ptr<double>(), *P = phi.data_ptr<double>();
  bool cuda = pos.is_cuda();
  AT_DISPATCH_FLOATING_TYPES(pos.scalar_type(), "ewald_recip_apply", [&] {
    const scalar_t* r = pos.data_ptr<scalar_t>();
    const scalar_t* Q = charges.data_ptr<scalar_t>();
    for_each(cuda, na, [=] NVA_LAMBDA(int64_t t) {
      int64_t i = a0 + t;
      double x = r[3 * i], y = r[3 * i + 1], z = r[3 * i + 2];
      double fx = 0, fy = 0, fz = 0, p = 0;
      for (int64_t k = 0; k < nk; ++k) {
        double kx = Kv[3 * k], ky = Kv[3 * k + 1], kz = Kv[3 * k + 2];
        double sn, cs;
        sincos(kx * x + ky * y + kz * z, &sn, &cs);
        double sre = S[2 * k], sim = S[2 * k + 1];
        double im = sn * sre - cs * sim;  // Im(e^{ikr} conj S)
        double re = cs * sre + sn * sim;  // Re(e^{-ikr} S)
        double c = C[k];
        fx += c * kx * im; fy += c * ky * im; fz += c * kz * im;
        p += c * re;
      }
      double q = Q[i];
      F[3 * t] = q * fx; F[3 * t + 1] = q * fy; F[3 * t + 2] = q * fz;
      P[t] = p;
    });
  });
  return {f, phi};
}

// ---- particle mesh ----------------------------------------------------------------------------------------------
constexpr int kMaxOrder = 8;

// Cardinal B-spline weights M_p(u - j) on the p grid points touched by fractional offset w in [0,1), and derivatives.
NVA_HD void bspline(double w, int p, double* v, double* dv) {
  v[p - 1] = 0.0; v[1] = w; v[0] = 1.0 - w;
  for (int k = 3; k < p; ++k) {
    double div = 1.0 / (k - 1);
    v[k - 1] = div * w * v[k - 2];
    for (int j = 1; j <= k - 2; ++j) v[k - j - 1] = div * ((w + j) * v[k - j - 2] + (k - j - w) * v[k - j - 1]);
    v[0] = div * (1.0 - w) * v[0];
  }
  dv[0] = -v[0];
  for (int j = 1; j < p; ++j) dv[j] = v[j - 1] - v[j];
  double div = 1.0 / (p - 1);
  v[p - 1] = div * w * v[p - 2];
  for (int j = 1; j <= p - 2; ++j) v[p - j - 1] = div * ((w + j) * v[p - j - 2] + (p - j - w) * v[p - j - 1]);
  v[0] = div * (1.0 - w) * v[0];
}

// Spread charges of atoms [a0,a1) onto a float64 mesh [nx,ny,nz]; `inv` is the inverse cell (3x3, float64).
Tensor pme_spread(const Tensor& pos, const Tensor& charges, const Tensor& inv, int64_t nx, int64_t ny, int64_t nz,
                  int64_t order, int64_t a0, int64_t a1, const c10::optional<Tensor>& weights) {
  c10::cuda::OptionalCUDAGuard guard(pos.is_cuda() ? c10::make_optional(pos.device()) : c10::nullopt);
  NVA_CHECK_CONTIG(pos); NVA_CHECK_CONTIG(charges); NVA_CHECK_CONTIG(inv);
  TORCH_CHECK(order >= 3 && order <= kMaxOrder, "B-spline order must be in [3, 8]");
  TORCH_CHECK(inv.scalar_type() == at::kDouble, "inverse cell must be float64");
  Tensor mesh = at::zeros({nx, ny, nz}, pos.options().dtype(at::kDouble));
  if (a1 <= a0) return mesh;
  const double* I = inv.data_ptr<double>();
  double* G = mesh.data_ptr<double>();
  bool cuda = pos.is_cuda();
  int p = (int)order;
  AT_DISPATCH_FLOATING_TYPES(pos.scalar_type(), "pme_spread", [&] {
    const scalar_t* r = pos.data_ptr<scalar_t>();
    const scalar_t* Q = charges.data_ptr<scalar_t>();
    const scalar_t* Wt = weights.has_value() ? weights->data_ptr<scalar_t>() : nullptr;
    for_each(cuda, a1 - a0, [=] NVA_LAMBDA(int64_t t) {
      int64_t i = a0 + t;
      double q = Q[i] * (Wt ? (double)Wt[i] : 1.0);
      if (q == 0.0) return;
      double x = r[3 * i], y = r[3 * i + 1], z = r[3 * i + 2];
      int64_t dims[3] = {nx, ny, nz};
      int64_t base[3];
      double v[3][kMaxOrder], dv[kMaxOrder];
      for (int d = 0; d < 3; ++d) {
        double fr = x * I[d] + y * I[3 + d] + z * I[6 + d];
        fr -= floor(fr);
        double u = fr * dims[d];
        int64_t fl = (int64_t)floor(u);
        bspline(u - fl, p, v[d], dv);
        base[d] = fl - p + 1;
      }
      for (int a = 0; a < p; ++a) {
        int64_t ia = ((base[0] + a) % nx + nx) % nx;
        for (int b2 = 0; b2 < p; ++b2) {
          int64_t ib = ((base[1] + b2) % ny + ny) % ny;
          double wab = q * v[0][a] * v[1][b2];
          for (int c = 0; c < p; ++c) {
            int64_t ic = ((base[2] + c) % nz + nz) % nz;
            atomic_add_f64(G + (ia * ny + ib) * nz + ic, wab * v[2][c]);
          }
        }
      }
    });
  });
  return mesh;
}

// In place: mesh_k[m] *= G(m) with G = (4 pi / V) exp(-k^2/4a^2)/k^2 * B(m) (zero at m = 0); returns
// [energy, W_xx, W_xy, W_xz, W_yy, W_yz, W_zz] with energy = 1/2 sum |F|^2 G (half-grid weights applied) and
// W = -dE/d(strain).  `mesh_k` is the rfftn output viewed as real [nx, ny, nzh, 2].
Tensor pme_convolve(Tensor mesh_k, const Tensor& inv, const Tensor& bx, const Tensor& by, const Tensor& bz, double alpha,
                    double volume, int64_t nz) {
  c10::cuda::OptionalCUDAGuard guard(mesh_k.is_cuda() ? c10::make_optional(mesh_k.device()) : c10::nullopt);
  NVA_CHECK_CONTIG(mesh_k); NVA_CHECK_CONTIG(inv);
  int64_t nx = mesh_k.size(0), ny = mesh_k.size(1), nzh = mesh_k.size(2);
  Tensor acc = at::zeros({7}, mesh_k.options().dtype(at::kDouble));
  const double *I = inv.data_ptr<double>(), *Bx = bx.data_ptr<double>(), *By = by.data_ptr<double>(),
               *Bz = bz.data_ptr<double>();
  double* A = acc.data_ptr<double>();
  bool cuda = mesh_k.is_cuda();
  AT_DISPATCH_FLOATING_TYPES(mesh_k.scalar_type(), "pme_convolve", [&] {
    scalar_t* Mk = mesh_k.data_ptr<scalar_t>();
    // one thread per (x, y) column keeps the 7 accumulators in registers and issues 7 atomics per column
    for_each(cuda, nx * ny, [=] NVA_LAMBDA(int64_t t) {
      int64_t ix = t / ny, iy = t % ny;
      double mx = ix <= nx / 2 ? (double)ix : (double)(ix - nx);
      double my = iy <= ny / 2 ? (double)iy : (double)(iy - ny);
      double s[7] = {0, 0, 0, 0, 0, 0, 0};
      for (int64_t iz = 0; iz < nzh; ++iz) {
        scalar_t* c = Mk + 2 * ((ix * ny + iy) * nzh + iz);
        if (ix == 0 && iy == 0 && iz == 0) { c[0] = 0; c[1] = 0; continue; }
        double mz = (double)iz;
        // k = 2 pi * inv @ m  (inv columns are reciprocal vectors)
        double kx = 2 * kPi * (I[0] * mx + I[1] * my + I[2] * mz);
        double ky = 2 * kPi * (I[3] * mx + I[4] * my + I[5] * mz);
        double kz = 2 * kPi * (I[6] * mx + I[7] * my + I[8] * mz);
        double k2 = kx * kx + ky * ky + kz * kz;
        double g = (4 * kPi / volume) * exp(-k2 / (4 * alpha * alpha)) / k2 * Bx[ix] * By[iy] * Bz[iz];
        double re = c[0], im = c[1];
        double wt = (iz == 0 || (2 * iz == nz)) ? 1.0 : 2.0;
        double e = 0.5 * wt * g * (re * re + im * im);
        double vf = 2.0 * (1.0 / k2 + 1.0 / (4 * alpha * alpha));
        s[0] += e;
        s[1] += e * (1.0 - vf * kx * kx); s[2] += e * (-vf * kx * ky); s[3] += e * (-vf * kx * kz);
        s[4] += e * (1.0 - vf * ky * ky); s[5] += e * (-vf * ky * kz); s[6] += e * (1.0 - vf * kz * kz);
        c[0] = (scalar_t)(g * re); c[1] = (scalar_t)(g * im);
      }
      for (int q = 0; q < 7; ++q) atomic_add_f64(A + q, s[q]);
    });
  });
  return acc;
}

// Potentials phi_i = sum_x theta_i(x) phi(x) and forces F_i = -q_i sum_x grad theta_i(x) phi(x) for atoms [a0,a1).
std::tuple<Tensor, Tensor> pme_gather(const Tensor& pos, const Tensor& charges, const Tensor& inv, const Tensor& phi_mesh,
                                      int64_t order, int64_t a0, int64_t a1) {
  c10::cuda::OptionalCUDAGuard guard(pos.is_cuda() ? c10::make_optional(pos.device()) : c10::nullopt);
  NVA_CHECK_CONTIG(pos); NVA_CHECK_CONTIG(charges); NVA_CHECK_CONTIG(inv); NVA_CHECK_CONTIG(phi_mesh);
  TORCH_CHECK(order >= 3 && order <= kMaxOrder, "B-spline order must be in [3, 8]");
  int64_t nx = phi_mesh.size(0), ny = phi_mesh.size(1), nz = phi_mesh.size(2), na = a1 - a0;
  auto dopt = pos.options().dtype(at::kDouble);
  Tensor f = at::zeros({na > 0 ? na : 0, 3}, dopt), phi = at::zeros({na > 0 ? na : 0}, dopt);
  if (na <= 0) return {f, phi};
  TORCH_CHECK(phi_mesh.scalar_type() == at::kDouble, "potential mesh must be float64");
  const double* I = inv.data_ptr<double>();
  const double* G = phi_mesh.data_ptr<double>();
  double *F = f.data_ptr<double>(), *P = phi.data_ptr<double>();
  bool cuda = pos.is_cuda();
  int p = (int)order;
  AT_DISPATCH_FLOATING_TYPES(pos.scalar_type(), "pme_gather", [&] {
    const scalar_t* r = pos.data_ptr<scalar_t>();
    const scalar_t* Q = charges.data_ptr<scalar_t>();
    {
      for_each(cuda, na, [=] NVA_LAMBDA(int64_t t) {
        int64_t i = a0 + t;
        double x = r[3 * i], y = r[3 * i + 1], z = r[3 * i + 2];
        int64_t dims[3] = {nx, ny, nz};
        int64_t base[3];
        double v[3][kMaxOrder], dv[3][kMaxOrder];
        for (int d = 0; d < 3; ++d) {
          double fr = x * I[d] + y * I[3 + d] + z * I[6 + d];
          fr -= floor(fr);
          double u = fr * dims[d];
          int64_t fl = (int64_t)floor(u);
          bspline(u - fl, p, v[d], dv[d]);
          base[d] = fl - p + 1;
        }
        double ph = 0, g0 = 0, g1 = 0, g2 = 0;  // gradient w.r.t. the scaled fractional coordinates u_d
        for (int a = 0; a < p; ++a) {
          int64_t ia = ((base[0] + a) % nx + nx) % nx;
          for (int b2 = 0; b2 < p; ++b2) {
            int64_t ib = ((base[1] + b2) % ny + ny) % ny;
            for (int c = 0; c < p; ++c) {
              int64_t ic = ((base[2] + c) % nz + nz) % nz;
              double m = G[(ia * ny + ib) * nz + ic];
              ph += v[0][a] * v[1][b2] * v[2][c] * m;
              g0 += dv[0][a] * v[1][b2] * v[2][c] * m;
              g1 += v[0][a] * dv[1][b2] * v[2][c] * m;
              g2 += v[0][a] * v[1][b2] * dv[2][c] * m;
            }
          }
        }
        g0 *= (double)nx; g1 *= (double)ny; g2 *= (double)nz;
        double q = Q[i];
        // du_d / dr_a = n_d * inv[a][d]
        F[3 * t] = -q * (I[0] * g0 + I[1] * g1 + I[2] * g2);
        F[3 * t + 1] = -q * (I[3] * g0 + I[4] * g1 + I[5] * g2);
        F[3 * t + 2] = -q * (I[6] * g0 + I[7] * g1 + I[8] * g2);
        P[t] = ph;
      });
    }
  });
  return {f, phi};
}

}  // namespace nva

TORCH_LIBRARY_FRAGMENT(nvalchemi, m) {
  m.def("ewald_real(Tensor positions, Tensor charges, Tensor cells, Tensor neighbor_matrix, Tensor neighbor_matrix_shifts, Tensor num_neighbors, Tensor batch_idx, Tensor alpha, int fill_value, float cutoff, bool half_list, int num_systems) -> (Tensor, Tensor, Tensor, Tensor)", &nva::ewald_real);
  m.def("ewald_structure_factors(Tensor positions, Tensor charges, Tensor kvecs, int a0, int a1, Tensor? weights) -> Tensor", &nva::ewald_structure_factors);
  m.def("ewald_recip_apply(Tensor positions, Tensor charges, Tensor kvecs, Tensor coef, Tensor sk, int a0, int a1) -> (Tensor, Tensor)", &nva::ewald_recip_apply);
  m.def("pme_spread(Tensor positions, Tensor charges, Tensor inv_cell, int nx, int ny, int nz, int order, int a0, int a1, Tensor? weights) -> Tensor", &nva::pme_spread);
  m.def("pme_convolve(Tensor(a!) mesh_k, Tensor inv_cell, Tensor bx, Tensor by, Tensor bz, float alpha, float volume, int nz) -> Tensor", &nva::pme_convolve);
  m.def("pme_gather(Tensor positions, Tensor charges, Tensor inv_cell, Tensor phi_mesh, int order, int a0, int a1) -> (Tensor, Tensor)", &nva::pme_gather);
}
