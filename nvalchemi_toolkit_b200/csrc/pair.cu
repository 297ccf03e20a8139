// SPDX-License-Identifier: Apache-2.0
// Pair-potential kernels over the dense neighbour matrix: Lennard-Jones with a C2 switching function, per-atom
// energies, forces and per-system virials (op surface of the reference: nvalchemi/models/_ops/lj.py:116-345,
// one thread per atom looping over its K neighbours, fp64 pair arithmetic).
#include "common.cuh"

namespace nva {
using at::Tensor;

// Quintic switch on [r_on, r_c]: S(r_on) = 1, S(r_c) = 0 with vanishing first and second derivatives at both ends.
NVA_HD void switch_fn(double r, double r_on, double r_c, double& s, double& ds) {
  if (r <= r_on) { s = 1.0; ds = 0.0; return; }
  if (r >= r_c) { s = 0.0; ds = 0.0; return; }
  double x = (r - r_on) / (r_c - r_on);
  s = 1.0 - x * x * x * (10.0 - 15.0 * x + 6.0 * x * x);
  ds = -30.0 * x * x * (1.0 - x) * (1.0 - x) / (r_c - r_on);
}

std::tuple<Tensor, Tensor, Tensor> lj_energy_forces(const Tensor& pos, const Tensor& cell, const Tensor& nm,
                                                    const Tensor& shifts, const Tensor& num, const Tensor& batch_idx,
                                                    int64_t fill_value, double epsilon, double sigma, double cutoff,
                                                    double switch_width, bool half_list, int64_t num_systems) {
  c10::cuda::OptionalCUDAGuard guard(pos.is_cuda() ? c10::make_optional(pos.device()) : c10::nullopt);
  NVA_CHECK_CONTIG(pos); NVA_CHECK_CONTIG(nm); NVA_CHECK_CONTIG(shifts); NVA_CHECK_CONTIG(cell);
  int64_t n = pos.size(0), K = nm.size(1);
  Tensor e = at::zeros({n}, pos.options().dtype(at::kDouble));
  Tensor f = at::zeros({n, 3}, pos.options().dtype(at::kDouble));
  Tensor w = at::zeros({num_systems, 9}, pos.options().dtype(at::kDouble));
  if (n == 0) return {e.to(pos.scalar_type()), f.to(pos.scalar_type()), w.to(pos.scalar_type())};
  const int* M = nm.data_ptr<int>();
  const int* S = shifts.data_ptr<int>();
  const int* cnt = num.data_ptr<int>();
  const int* b = batch_idx.data_ptr<int>();
  double* E = e.data_ptr<double>();
  double* F = f.data_ptr<double>();
  double* W = w.data_ptr<double>();
  bool cuda = pos.is_cuda();
  double r_on = cutoff - switch_width;
  AT_DISPATCH_FLOATING_TYPES(pos.scalar_type(), "lj_energy_forces", [&] {
    const scalar_t* r = pos.data_ptr<scalar_t>();
    const scalar_t* H = cell.data_ptr<scalar_t>();
    for_each(cuda, n, [=] NVA_LAMBDA(int64_t i) {
      int s = b[i];
      const scalar_t* h = H + 9 * s;
      int k_i = cnt[i] < (int)K ? cnt[i] : (int)K;
      double ei = 0, fx = 0, fy = 0, fz = 0, vir[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
      double xi = r[3 * i], yi = r[3 * i + 1], zi = r[3 * i + 2];
      for (int q = 0; q < k_i; ++q) {
        int j = M[i * K + q];
        if (j >= fill_value || j < 0) continue;
        const int* sh = S + (i * K + q) * 3;
        double dx = (double)r[3 * j] + sh[0] * (double)h[0] + sh[1] * (double)h[3] + sh[2] * (double)h[6] - xi;
        double dy = (double)r[3 * j + 1] + sh[0] * (double)h[1] + sh[1] * (double)h[4] + sh[2] * (double)h[7] - yi;
        double dz = (double)r[3 * j + 2] + sh[0] * (double)h[2] + sh[1] * (double)h[5] + sh[2] * (double)h[8] - zi;
        double r2 = dx * dx + dy * dy + dz * dz;
        if (r2 >= cutoff * cutoff || r2 <= 0.0) continue;
        double rr = sqrt(r2), sr2 = sigma * sigma / r2, sr6 = sr2 * sr2 * sr2;
        double u = 4.0 * epsilon * (sr6 * sr6 - sr6);
        double du = -24.0 * epsilon * (2.0 * sr6 * sr6 - sr6) / rr;  // dU/dr
        double sw = 1.0, dsw = 0.0;
        if (switch_width > 0.0) switch_fn(rr, r_on, cutoff, sw, dsw);
        double de = du * sw + u * dsw;  // d(U S)/dr
        double wgt = half_list ? 1.0 : 0.5;
        ei += wgt * u * sw;
        double gx = de * dx / rr, gy = de * dy / rr, gz = de * dz / rr;  // dE_pair/d(r_j - r_i)
        fx += gx; fy += gy; fz += gz;  // F_i = +grad w.r.t. the displacement
        if (half_list) {
          atomic_add_f64(F + 3 * j, -gx); atomic_add_f64(F + 3 * j + 1, -gy); atomic_add_f64(F + 3 * j + 2, -gz);
        }
        // virial W = -dE/d(strain) = -sum_pairs d (x) dE/dd ; full lists see every pair twice
        double d[3] = {dx, dy, dz}, g[3] = {gx, gy, gz};
        for (int a = 0; a < 3; ++a)
          for (int c = 0; c < 3; ++c) vir[3 * a + c] -= wgt * d[a] * g[c];
      }
      E[i] = ei;
      atomic_add_f64(F + 3 * i, fx); atomic_add_f64(F + 3 * i + 1, fy); atomic_add_f64(F + 3 * i + 2, fz);
      for (int a = 0; a < 9; ++a) atomic_add_f64(W + 9 * s + a, vir[a]);
    });
  });
  return {e.to(pos.scalar_type()), f.to(pos.scalar_type()), w.to(pos.scalar_type())};
}

}  // namespace nva

TORCH_LIBRARY_FRAGMENT(nvalchemi, m) {
  m.def("lj_energy_forces_virial_batch(Tensor positions, Tensor cells, Tensor neighbor_matrix, Tensor neighbor_matrix_shifts, Tensor num_neighbors, Tensor batch_idx, int fill_value, float epsilon, float sigma, float cutoff, float switch_width, bool half_list, int num_systems) -> (Tensor, Tensor, Tensor)", &nva::lj_energy_forces);
}
