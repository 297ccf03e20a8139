// SPDX-License-Identifier: Apache-2.0
// DFT-D3 with Becke-Johnson damping over the dense neighbour matrix (full lists): coordination numbers, pair energies
// with the CN-interpolated C6 coefficients, and the chain-rule force term through the coordination numbers.  Inputs
// are in atomic units (Bohr, Hartree); the Python wrapper converts.  Behaviour follows the reference's use of
// nvalchemiops' dftd3 (nvalchemi/models/dftd3.py:434-863): per-atom energies, forces and per-system virials, a
// smoothing window at the cutoff, optional per-atom energy weights for domain decomposition.
#include "common.cuh"

namespace nva {
using at::Tensor;

constexpr double kD3K1 = 16.0;
constexpr double kD3K3 = 4.0;
constexpr int kD3Ref = 5;

struct PairGeom {
  double dx, dy, dz, r;
};

template <typename scalar_t>
NVA_HD bool pair_geom(const scalar_t* r, const scalar_t* h, const int* sh, int64_t i, int j, double cutoff, PairGeom& g) {
  g.dx = (double)r[3 * j] + sh[0] * (double)h[0] + sh[1] * (double)h[3] + sh[2] * (double)h[6] - (double)r[3 * i];
  g.dy = (double)r[3 * j + 1] + sh[0] * (double)h[1] + sh[1] * (double)h[4] + sh[2] * (double)h[7] - (double)r[3 * i + 1];
  g.dz = (double)r[3 * j + 2] + sh[0] * (double)h[2] + sh[1] * (double)h[5] + sh[2] * (double)h[8] - (double)r[3 * i + 2];
  double r2 = g.dx * g.dx + g.dy * g.dy + g.dz * g.dz;
  if (r2 >= cutoff * cutoff || r2 <= 1e-20) return false;
  g.r = sqrt(r2);
  return true;
}

NVA_HD void d3_switch(double r, double r_on, double r_c, double& s, double& ds) {
  if (r <= r_on) { s = 1.0; ds = 0.0; return; }
  if (r >= r_c) { s = 0.0; ds = 0.0; return; }
  double x = (r - r_on) / (r_c - r_on);
  s = 1.0 - x * x * x * (10.0 - 15.0 * x + 6.0 * x * x);
  ds = -30.0 * x * x * (1.0 - x) * (1.0 - x) / (r_c - r_on);
}

// CN_i = sum_j 1 / (1 + exp(-k1 ((rc_i + rc_j) / r - 1)))
Tensor d3_coordination(const Tensor& pos, const Tensor& cell, const Tensor& nm, const Tensor& shifts, const Tensor& num,
                       const Tensor& batch_idx, const Tensor& species, const Tensor& rcov, double cutoff) {
  c10::cuda::OptionalCUDAGuard guard(pos.is_cuda() ? c10::make_optional(pos.device()) : c10::nullopt);
  NVA_CHECK_CONTIG(pos); NVA_CHECK_CONTIG(nm); NVA_CHECK_CONTIG(shifts); NVA_CHECK_CONTIG(cell);
  int64_t n = pos.size(0), K = nm.size(1);
  Tensor cn = at::zeros({n}, pos.options().dtype(at::kDouble));
  if (n == 0) return cn;
  const int *M = nm.data_ptr<int>(), *S = shifts.data_ptr<int>(), *cnt = num.data_ptr<int>(), *b = batch_idx.data_ptr<int>();
  const int64_t* Z = species.data_ptr<int64_t>();
  const double* RC = rcov.data_ptr<double>();
  double* CN = cn.data_ptr<double>();
  bool cuda = pos.is_cuda();
  AT_DISPATCH_FLOATING_TYPES(pos.scalar_type(), "d3_coordination", [&] {
    const scalar_t* r = pos.data_ptr<scalar_t>();
    const scalar_t* H = cell.data_ptr<scalar_t>();
    for_each(cuda, n, [=] NVA_LAMBDA(int64_t i) {
      const scalar_t* h = H + 9 * b[i];
      int k_i = cnt[i] < (int)K ? cnt[i] : (int)K;
      double rci = RC[Z[i]], acc = 0;
      for (int q = 0; q < k_i; ++q) {
        int j = M[i * K + q];
        if (j >= n || j < 0) continue;
        PairGeom g;
        if (!pair_geom(r, h, S + (i * K + q) * 3, i, j, cutoff, g)) continue;
        acc += 1.0 / (1.0 + exp(-kD3K1 * ((rci + RC[Z[j]]) / g.r - 1.0)));
      }
      CN[i] = acc;
    });
  });
  return cn;
}

// C6(CN_i, CN_j) and its derivatives with respect to both coordination numbers.
NVA_HD void d3_c6(const double* c6ref, const double* cnref, int64_t nz, int64_t zi, int64_t zj, double cni, double cnj,
                  double& c6, double& dci, double& dcj) {
  const double* tab = c6ref + ((zi * nz + zj) * kD3Ref) * kD3Ref;
  const double *ri = cnref + zi * kD3Ref, *rj = cnref + zj * kD3Ref;
  // shift exponents by the smallest distance so that at least one weight is exp(0): no underflow far from all refs
  double dmin = 1e300;
  for (int a = 0; a < kD3Ref; ++a)
    for (int c = 0; c < kD3Ref; ++c) {
      if (tab[a * kD3Ref + c] <= 0.0) continue;
      double d = (cni - ri[a]) * (cni - ri[a]) + (cnj - rj[c]) * (cnj - rj[c]);
      if (d < dmin) dmin = d;
    }
  double zs = 0, ws = 0, dzi = 0, dwi = 0, dzj = 0, dwj = 0;
  for (int a = 0; a < kD3Ref; ++a)
    for (int c = 0; c < kD3Ref; ++c) {
      double ref = tab[a * kD3Ref + c];
      if (ref <= 0.0) continue;
      double di = cni - ri[a], dj = cnj - rj[c];
      double l = exp(-kD3K3 * (di * di + dj * dj - dmin));
      zs += ref * l; ws += l;
      double li = -2.0 * kD3K3 * di * l, lj = -2.0 * kD3K3 * dj * l;
      dzi += ref * li; dwi += li; dzj += ref * lj; dwj += lj;
    }
  if (ws <= 0.0) { c6 = 0; dci = 0; dcj = 0; return; }
  c6 = zs / ws;
  dci = (dzi - c6 * dwi) / ws;
  dcj = (dzj - c6 * dwj) / ws;
}

// Per-atom energies, direct forces, virials and D_i = dE_w/dCN_i.  params = [s6, s8, a1, a2, r_on, cutoff].
std::tuple<Tensor, Tensor, Tensor, Tensor> d3_pair(const Tensor& pos, const Tensor& cell, const Tensor& nm,
                                                   const Tensor& shifts, const Tensor& num, const Tensor& batch_idx,
                                                   const Tensor& species, const Tensor& cn, const Tensor& c6ref,
                                                   const Tensor& cnref, const Tensor& r4r2, const Tensor& params,
                                                   const c10::optional<Tensor>& weights, int64_t num_systems) {
  c10::cuda::OptionalCUDAGuard guard(pos.is_cuda() ? c10::make_optional(pos.device()) : c10::nullopt);
  NVA_CHECK_CONTIG(pos); NVA_CHECK_CONTIG(nm); NVA_CHECK_CONTIG(shifts); NVA_CHECK_CONTIG(cell); NVA_CHECK_CONTIG(c6ref);
  int64_t n = pos.size(0), K = nm.size(1), nz = c6ref.size(0);
  auto dopt = pos.options().dtype(at::kDouble);
  Tensor e = at::zeros({n}, dopt), f = at::zeros({n, 3}, dopt), w = at::zeros({num_systems, 9}, dopt), dcn = at::zeros({n}, dopt);
  if (n == 0) return {e, f, w, dcn};
  Tensor pc = params.to(at::kCPU, at::kDouble).contiguous();
  const double* pp = pc.data_ptr<double>();
  double s6 = pp[0], s8 = pp[1], a1 = pp[2], a2 = pp[3], r_on = pp[4], cutoff = pp[5];
  const int *M = nm.data_ptr<int>(), *S = shifts.data_ptr<int>(), *cnt = num.data_ptr<int>(), *b = batch_idx.data_ptr<int>();
  const int64_t* Z = species.data_ptr<int64_t>();
  const double *CN = cn.data_ptr<double>(), *C6 = c6ref.data_ptr<double>(), *CR = cnref.data_ptr<double>(),
               *Q = r4r2.data_ptr<double>();
  const double* Wt = weights.has_value() ? weights->data_ptr<double>() : nullptr;
  double *E = e.data_ptr<double>(), *F = f.data_ptr<double>(), *W = w.data_ptr<double>(), *D = dcn.data_ptr<double>();
  bool cuda = pos.is_cuda();
  AT_DISPATCH_FLOATING_TYPES(pos.scalar_type(), "d3_pair", [&] {
    const scalar_t* r = pos.data_ptr<scalar_t>();
    const scalar_t* H = cell.data_ptr<scalar_t>();
    for_each(cuda, n, [=] NVA_LAMBDA(int64_t i) {
      int s = b[i];
      const scalar_t* h = H + 9 * s;
      int k_i = cnt[i] < (int)K ? cnt[i] : (int)K;
      double ei = 0, di = 0, fx = 0, fy = 0, fz = 0, vir[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
      double wi = Wt ? Wt[i] : 1.0;
      for (int q = 0; q < k_i; ++q) {
        int j = M[i * K + q];
        if (j >= n || j < 0) continue;
        PairGeom g;
        if (!pair_geom(r, h, S + (i * K + q) * 3, i, j, cutoff, g)) continue;
        double c6, dci, dcj;
        d3_c6(C6, CR, nz, Z[i], Z[j], CN[i], CN[j], c6, dci, dcj);
        if (c6 <= 0.0) continue;
        double qq = 3.0 * Q[Z[i]] * Q[Z[j]];  // C8 / C6
        double r0 = a1 * sqrt(qq) + a2;
        double r2 = g.r * g.r, r6 = r2 * r2 * r2, r8 = r6 * r2;
        double f2 = r0 * r0, f6 = f2 * f2 * f2, f8 = f6 * f2;
        double t6 = 1.0 / (r6 + f6), t8 = 1.0 / (r8 + f8);
        double per_c6 = -(s6 * t6 + s8 * qq * t8);                               // E_pair / C6
        double dper = s6 * 6.0 * r6 / g.r * t6 * t6 + s8 * qq * 8.0 * r8 / g.r * t8 * t8;  // d(E_pair/C6)/dr
        double sw, dsw;
        d3_switch(g.r, r_on, cutoff, sw, dsw);
        double epair = c6 * per_c6 * sw;
        double depair = c6 * (dper * sw + per_c6 * dsw);
        double pw = 0.5 * (wi + (Wt ? Wt[j] : 1.0));
        ei += 0.5 * epair;
        di += pw * dci * per_c6 * sw;
        double gx = pw * depair * g.dx / g.r, gy = pw * depair * g.dy / g.r, gz = pw * depair * g.dz / g.r;
        fx += gx; fy += gy; fz += gz;  // dE/d(r_j - r_i); the partner row adds the opposite force on j
        double d[3] = {g.dx, g.dy, g.dz}, gg[3] = {gx, gy, gz};
        for (int u = 0; u < 3; ++u)
          for (int v = 0; v < 3; ++v) vir[3 * u + v] -= 0.5 * d[u] * gg[v];
      }
      E[i] = ei; D[i] = di;
      F[3 * i] = fx; F[3 * i + 1] = fy; F[3 * i + 2] = fz;
      for (int u = 0; u < 9; ++u) atomic_add_f64(W + 9 * s + u, vir[u]);
    });
  });
  return {e, f, w, dcn};
}

// Chain term: dE/dr_i += sum_j (D_i + D_j) g'(r_ij) d r_ij / d r_i ; adds into forces and virials in place.
void d3_cn_forces(const Tensor& pos, const Tensor& cell, const Tensor& nm, const Tensor& shifts, const Tensor& num,
                  const Tensor& batch_idx, const Tensor& species, const Tensor& rcov, const Tensor& dcn, double cutoff,
                  Tensor forces, Tensor virial) {
  c10::cuda::OptionalCUDAGuard guard(pos.is_cuda() ? c10::make_optional(pos.device()) : c10::nullopt);
  int64_t n = pos.size(0), K = nm.size(1);
  if (n == 0) return;
  const int *M = nm.data_ptr<int>(), *S = shifts.data_ptr<int>(), *cnt = num.data_ptr<int>(), *b = batch_idx.data_ptr<int>();
  const int64_t* Z = species.data_ptr<int64_t>();
  const double *RC = rcov.data_ptr<double>(), *D = dcn.data_ptr<double>();
  double *F = forces.data_ptr<double>(), *W = virial.data_ptr<double>();
  bool cuda = pos.is_cuda();
  AT_DISPATCH_FLOATING_TYPES(pos.scalar_type(), "d3_cn_forces", [&] {
    const scalar_t* r = pos.data_ptr<scalar_t>();
    const scalar_t* H = cell.data_ptr<scalar_t>();
    for_each(cuda, n, [=] NVA_LAMBDA(int64_t i) {
      int s = b[i];
      const scalar_t* h = H + 9 * s;
      int k_i = cnt[i] < (int)K ? cnt[i] : (int)K;
      double rci = RC[Z[i]], fx = 0, fy = 0, fz = 0, vir[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
      for (int q = 0; q < k_i; ++q) {
        int j = M[i * K + q];
        if (j >= n || j < 0) continue;
        PairGeom g;
        if (!pair_geom(r, h, S + (i * K + q) * 3, i, j, cutoff, g)) continue;
        double rc = rci + RC[Z[j]];
        double ex = exp(-kD3K1 * (rc / g.r - 1.0));
        double dg = -kD3K1 * rc / (g.r * g.r) * ex / ((1.0 + ex) * (1.0 + ex));  // d/dr of the counting function
        double de = (D[i] + D[j]) * dg;
        double gx = de * g.dx / g.r, gy = de * g.dy / g.r, gz = de * g.dz / g.r;
        fx += gx; fy += gy; fz += gz;
        double d[3] = {g.dx, g.dy, g.dz}, gg[3] = {gx, gy, gz};
        for (int u = 0; u < 3; ++u)
          for (int v = 0; v < 3; ++v) vir[3 * u + v] -= 0.5 * d[u] * gg[v];
      }
      F[3 * i] += fx; F[3 * i + 1] += fy; F[3 * i + 2] += fz;
      for (int u = 0; u < 9; ++u) atomic_add_f64(W + 9 * s + u, vir[u]);
    });
  });
}

}  // namespace nva

TORCH_LIBRARY_FRAGMENT(nvalchemi, m) {
  m.def("d3_coordination(Tensor positions, Tensor cells, Tensor neighbor_matrix, Tensor neighbor_matrix_shifts, Tensor num_neighbors, Tensor batch_idx, Tensor species, Tensor rcov, float cutoff) -> Tensor", &nva::d3_coordination);
  m.def("d3_pair(Tensor positions, Tensor cells, Tensor neighbor_matrix, Tensor neighbor_matrix_shifts, Tensor num_neighbors, Tensor batch_idx, Tensor species, Tensor cn, Tensor c6ref, Tensor cnref, Tensor r4r2, Tensor params, Tensor? weights, int num_systems) -> (Tensor, Tensor, Tensor, Tensor)", &nva::d3_pair);
  m.def("d3_cn_forces(Tensor positions, Tensor cells, Tensor neighbor_matrix, Tensor neighbor_matrix_shifts, Tensor num_neighbors, Tensor batch_idx, Tensor species, Tensor rcov, Tensor dcn, float cutoff, Tensor(a!) forces, Tensor(b!) virial) -> ()", &nva::d3_cn_forces);
}
