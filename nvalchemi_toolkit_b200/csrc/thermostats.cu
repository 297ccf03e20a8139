// SPDX-License-Identifier: Apache-2.0
// Extended-system integrator pieces: Nose-Hoover chains, kinetic tensor, and the per-system affine maps of the
// Martyna-Tobias-Klein barostat (full 3x3 cell coupling), plus cell alignment.  Replaces the reference's Warp-backed ops
// nhc_chain_update / nhc_velocity_half_step / nhc_position_update (nvalchemi/dynamics/_ops/nose_hoover.py:129-325),
// compute_kinetic_tensor, npt_velocity_half_step, npt_position_update, npt_cell_update
// (dynamics/_ops/npt_nph.py:162-207,684-911) and align_cell (dynamics/_ops/cell_align.py:46-125).
// Every kernel has a CPU twin through for_each (same functor in an OpenMP loop).
#include "common.cuh"

namespace nva {
using at::Tensor;

namespace {
// Yoshida-Suzuki weights for orders 1, 3, 5.
NVA_HD int ys_weights(int order, double* w) {
  if (order == 1) { w[0] = 1.0; return 1; }
  if (order == 3) {
    const double a = 1.0 / (2.0 - 1.2599210498948732);  // 2^(1/3)
    w[0] = a; w[1] = 1.0 - 2.0 * a; w[2] = a;
    return 3;
  }
  const double a = 1.0 / (4.0 - 1.5874010519681994);    // 4^(1/3)
  w[0] = a; w[1] = a; w[2] = 1.0 - 4.0 * a; w[3] = a; w[4] = a;
  return 5;
}
}  // namespace

// Half-step propagation of one Nose-Hoover chain per system (thread = system).  ke2 = 2 KE is updated in place, eta and
// eta_dot advance, scale[s] is the factor to apply to the system's velocities.
//   G_0 = (ke2 - ndof kT) / Q_0,  G_k = (Q_{k-1} eta_dot_{k-1}^2 - kT) / Q_k
template <typename T>
void nhc_chain_impl(bool cuda, int64_t M, int C, int order, T* ke2, T* eta, T* eta_dot, const T* Q, const T* kT,
                    const T* ndof, const T* dt, T* scale) {
  for_each(cuda, M, [=] NVA_LAMBDA(int64_t s) {
    double w[5];
    const int nw = ys_weights(order, w);
    T* e = eta + s * C;
    T* ed = eta_dot + s * C;
    const T* q = Q + s * C;
    double k2 = ke2[s], sc = 1.0;
    const double kt = kT[s], nd = ndof[s];
#define NVA_NHC_FORCE(k) (((k) == 0 ? k2 - nd * kt : (double)q[(k) - 1] * (double)ed[(k) - 1] * (double)ed[(k) - 1] - kt) / (double)q[(k)])
    for (int iw = 0; iw < nw; ++iw) {
      const double h = w[iw] * (double)dt[s];
      for (int k = C - 1; k >= 0; --k) {
        const double g = NVA_NHC_FORCE(k);
        if (k == C - 1) {
          ed[k] = (T)((double)ed[k] + 0.25 * h * g);
        } else {
          const double f = exp(-0.125 * h * (double)ed[k + 1]);
          ed[k] = (T)(((double)ed[k] * f + 0.25 * h * g) * f);
        }
      }
      const double sv = exp(-0.5 * h * (double)ed[0]);
      sc *= sv;
      k2 *= sv * sv;
      for (int k = 0; k < C; ++k) e[k] = (T)((double)e[k] + 0.5 * h * (double)ed[k]);
      for (int k = 0; k < C; ++k) {
        const double g = NVA_NHC_FORCE(k);
        if (k == C - 1) {
          ed[k] = (T)((double)ed[k] + 0.25 * h * g);
        } else {
          const double f = exp(-0.125 * h * (double)ed[k + 1]);
          ed[k] = (T)(((double)ed[k] * f + 0.25 * h * g) * f);
        }
      }
    }
#undef NVA_NHC_FORCE
    ke2[s] = (T)k2;
    scale[s] = (T)sc;
  });
}

// Reference argument list (nvalchemi::nhc_chain_update).  With compute_ke the kinetic energies are summed here;
// otherwise ke2 is taken as given (a domain decomposition supplies the cross-rank sum).  total_scale receives the
// velocity factor, which is applied to `velocities`; step_scale and dt_chain are scratch of shape [M] kept for
// signature parity (step_scale receives a copy of the factor, dt_chain the chain time step).
void nhc_chain_update(Tensor velocities, const Tensor& masses, Tensor eta, Tensor eta_dot, const Tensor& Q,
                      const Tensor& temperature, const Tensor& dt, const Tensor& ndof, Tensor ke2, Tensor total_scale,
                      Tensor step_scale, Tensor dt_chain, const Tensor& batch_idx, bool compute_ke, int64_t yoshida_order) {
  c10::cuda::OptionalCUDAGuard guard(velocities.is_cuda() ? c10::make_optional(velocities.device()) : c10::nullopt);
  NVA_CHECK_CONTIG(velocities); NVA_CHECK_CONTIG(eta); NVA_CHECK_CONTIG(eta_dot); NVA_CHECK_CONTIG(Q); NVA_CHECK_CONTIG(ke2);
  TORCH_CHECK(yoshida_order == 1 || yoshida_order == 3 || yoshida_order == 5, "yoshida_order must be 1, 3 or 5");
  const int64_t M = eta.size(0), n = velocities.size(0);
  const int C = (int)eta.size(1);
  const bool cuda = velocities.is_cuda();
  const int* b = batch_idx.data_ptr<int>();
  AT_DISPATCH_FLOATING_TYPES(velocities.scalar_type(), "nhc_chain_update", [&] {
    scalar_t* v = velocities.data_ptr<scalar_t>();
    if (compute_ke) {
      const scalar_t* m = masses.data_ptr<scalar_t>();
      Tensor acc = at::zeros({M}, velocities.options().dtype(at::kDouble));
      double* a = acc.data_ptr<double>();
      for_each(cuda, n, [=] NVA_LAMBDA(int64_t i) {
        const double x = v[3 * i], y = v[3 * i + 1], z = v[3 * i + 2];
        atomic_add_f64(a + b[i], (double)m[i] * (x * x + y * y + z * z));
      });
      ke2.copy_(acc);
    }
    nhc_chain_impl<scalar_t>(cuda, M, C, (int)yoshida_order, ke2.data_ptr<scalar_t>(), eta.data_ptr<scalar_t>(),
                             eta_dot.data_ptr<scalar_t>(), Q.data_ptr<scalar_t>(), temperature.data_ptr<scalar_t>(),
                             ndof.data_ptr<scalar_t>(), dt.data_ptr<scalar_t>(), total_scale.data_ptr<scalar_t>());
    const scalar_t* sc = total_scale.data_ptr<scalar_t>();
    for_each(cuda, n, [=] NVA_LAMBDA(int64_t i) {
      const scalar_t f = sc[b[i]];
      v[3 * i] *= f; v[3 * i + 1] *= f; v[3 * i + 2] *= f;
    });
  });
  if (step_scale.defined() && step_scale.numel() == M) step_scale.copy_(total_scale);
  if (dt_chain.defined() && dt_chain.numel() == M) dt_chain.copy_(dt);
}

// Chain propagation alone (barostat chains have no particles attached): returns the scale factor per system.
Tensor nhc_chain_scalar(Tensor ke2, Tensor eta, Tensor eta_dot, const Tensor& Q, const Tensor& temperature,
                        const Tensor& ndof, const Tensor& dt, int64_t yoshida_order) {
  c10::cuda::OptionalCUDAGuard guard(ke2.is_cuda() ? c10::make_optional(ke2.device()) : c10::nullopt);
  NVA_CHECK_CONTIG(eta); NVA_CHECK_CONTIG(eta_dot); NVA_CHECK_CONTIG(Q); NVA_CHECK_CONTIG(ke2);
  Tensor scale = at::empty_like(ke2);
  AT_DISPATCH_FLOATING_TYPES(ke2.scalar_type(), "nhc_chain_scalar", [&] {
    nhc_chain_impl<scalar_t>(ke2.is_cuda(), eta.size(0), (int)eta.size(1), (int)yoshida_order, ke2.data_ptr<scalar_t>(),
                             eta.data_ptr<scalar_t>(), eta_dot.data_ptr<scalar_t>(), Q.data_ptr<scalar_t>(),
                             temperature.data_ptr<scalar_t>(), ndof.data_ptr<scalar_t>(), dt.data_ptr<scalar_t>(),
                             scale.data_ptr<scalar_t>());
  });
  return scale;
}

// v += (dt / 2) F / m  and  r += dt v  (the particle half-kick and drift of the chain integrator).
void nhc_velocity_half_step(Tensor velocities, const Tensor& forces, const Tensor& masses, const Tensor& dt,
                            const Tensor& batch_idx) {
  c10::cuda::OptionalCUDAGuard guard(velocities.is_cuda() ? c10::make_optional(velocities.device()) : c10::nullopt);
  NVA_CHECK_CONTIG(velocities); NVA_CHECK_CONTIG(forces);
  const int* b = batch_idx.data_ptr<int>();
  AT_DISPATCH_FLOATING_TYPES(velocities.scalar_type(), "nhc_velocity_half_step", [&] {
    scalar_t* v = velocities.data_ptr<scalar_t>();
    const scalar_t *f = forces.data_ptr<scalar_t>(), *m = masses.data_ptr<scalar_t>(), *h = dt.data_ptr<scalar_t>();
    for_each(velocities.is_cuda(), velocities.size(0), [=] NVA_LAMBDA(int64_t i) {
      const scalar_t c = scalar_t(0.5) * h[b[i]] / m[i];
      v[3 * i] += c * f[3 * i]; v[3 * i + 1] += c * f[3 * i + 1]; v[3 * i + 2] += c * f[3 * i + 2];
    });
  });
}

void nhc_position_update(Tensor positions, const Tensor& velocities, const Tensor& dt, const Tensor& batch_idx) {
  c10::cuda::OptionalCUDAGuard guard(positions.is_cuda() ? c10::make_optional(positions.device()) : c10::nullopt);
  NVA_CHECK_CONTIG(positions); NVA_CHECK_CONTIG(velocities);
  const int* b = batch_idx.data_ptr<int>();
  AT_DISPATCH_FLOATING_TYPES(positions.scalar_type(), "nhc_position_update", [&] {
    scalar_t* r = positions.data_ptr<scalar_t>();
    const scalar_t *v = velocities.data_ptr<scalar_t>(), *h = dt.data_ptr<scalar_t>();
    for_each(positions.is_cuda(), positions.size(0), [=] NVA_LAMBDA(int64_t i) {
      const scalar_t c = h[b[i]];
      r[3 * i] += c * v[3 * i]; r[3 * i + 1] += c * v[3 * i + 1]; r[3 * i + 2] += c * v[3 * i + 2];
    });
  });
}

// kinetic_tensors[s, 3a+b] = sum_{i in s} m_i v_ia v_ib  (double accumulation, written in the tensor's dtype).
void compute_kinetic_tensor(const Tensor& velocities, const Tensor& masses, Tensor kinetic_tensors, const Tensor& batch_idx) {
  c10::cuda::OptionalCUDAGuard guard(velocities.is_cuda() ? c10::make_optional(velocities.device()) : c10::nullopt);
  NVA_CHECK_CONTIG(velocities); NVA_CHECK_CONTIG(kinetic_tensors);
  const int64_t M = kinetic_tensors.size(0);
  TORCH_CHECK(kinetic_tensors.numel() == M * 9, "kinetic_tensors must be [M, 9]");
  Tensor acc = at::zeros({M, 9}, velocities.options().dtype(at::kDouble));
  double* a = acc.data_ptr<double>();
  const int* b = batch_idx.data_ptr<int>();
  AT_DISPATCH_FLOATING_TYPES(velocities.scalar_type(), "compute_kinetic_tensor", [&] {
    const scalar_t *v = velocities.data_ptr<scalar_t>(), *m = masses.data_ptr<scalar_t>();
    for_each(velocities.is_cuda(), velocities.size(0), [=] NVA_LAMBDA(int64_t i) {
      const double mi = m[i], x[3] = {(double)v[3 * i], (double)v[3 * i + 1], (double)v[3 * i + 2]};
      double* o = a + 9 * (int64_t)b[i];
      for (int p = 0; p < 3; ++p)
        for (int q = p; q < 3; ++q) {
          const double t = mi * x[p] * x[q];
          atomic_add_f64(o + 3 * p + q, t);
          if (q != p) atomic_add_f64(o + 3 * q + p, t);
        }
    });
  });
  kinetic_tensors.copy_(acc.view_as(kinetic_tensors));
}

// x_i <- x_i A_s + y_i C_s (+ f_i k_s / m_i) with per-system 3x3 matrices (row-vector convention, s = batch_idx[i]):
// the one per-atom primitive behind the barostat's velocity damping (A = exp(-dt/2 (v_g + tr(v_g)/N_f))), the position
// drift (A = exp(dt v_g), C = dt * phi(dt v_g)) and any cell rescaling.  y / C and the kick are optional.
void affine_rows_(Tensor x, const Tensor& A, const c10::optional<Tensor>& y, const c10::optional<Tensor>& C,
                  const c10::optional<Tensor>& forces, const c10::optional<Tensor>& masses, const c10::optional<Tensor>& kick,
                  const Tensor& batch_idx, bool kick_first) {
  c10::cuda::OptionalCUDAGuard guard(x.is_cuda() ? c10::make_optional(x.device()) : c10::nullopt);
  NVA_CHECK_CONTIG(x); NVA_CHECK_CONTIG(A);
  TORCH_CHECK(A.numel() % 9 == 0, "A must be [M, 3, 3]");
  TORCH_CHECK(y.has_value() == C.has_value(), "y and C come together");
  TORCH_CHECK(!forces.has_value() || (masses.has_value() && kick.has_value()), "a kick needs forces, masses and the factor");
  const int* b = batch_idx.data_ptr<int>();
  AT_DISPATCH_FLOATING_TYPES(x.scalar_type(), "affine_rows_", [&] {
    scalar_t* xp = x.data_ptr<scalar_t>();
    const scalar_t* Ap = A.data_ptr<scalar_t>();
    const scalar_t* yp = y.has_value() ? y->contiguous().data_ptr<scalar_t>() : nullptr;
    const scalar_t* Cp = C.has_value() ? C->contiguous().data_ptr<scalar_t>() : nullptr;
    const scalar_t* fp = forces.has_value() ? forces->contiguous().data_ptr<scalar_t>() : nullptr;
    const scalar_t* mp = masses.has_value() ? masses->data_ptr<scalar_t>() : nullptr;
    const scalar_t* kp = kick.has_value() ? kick->data_ptr<scalar_t>() : nullptr;
    for_each(x.is_cuda(), x.size(0), [=] NVA_LAMBDA(int64_t i) {
      const int s = b[i];
      const scalar_t* a = Ap + 9 * s;
      scalar_t v[3] = {xp[3 * i], xp[3 * i + 1], xp[3 * i + 2]};
      scalar_t kf[3] = {0, 0, 0};
      if (fp != nullptr) {
        const scalar_t c = kp[s] / mp[i];
        kf[0] = c * fp[3 * i]; kf[1] = c * fp[3 * i + 1]; kf[2] = c * fp[3 * i + 2];
        if (kick_first) { v[0] += kf[0]; v[1] += kf[1]; v[2] += kf[2]; }
      }
      scalar_t o[3];
      for (int q = 0; q < 3; ++q) o[q] = v[0] * a[q] + v[1] * a[3 + q] + v[2] * a[6 + q];
      if (yp != nullptr) {
        const scalar_t* c = Cp + 9 * s;
        const scalar_t w[3] = {yp[3 * i], yp[3 * i + 1], yp[3 * i + 2]};
        for (int q = 0; q < 3; ++q) o[q] += w[0] * c[q] + w[1] * c[3 + q] + w[2] * c[6 + q];
      }
      if (fp != nullptr && !kick_first) { o[0] += kf[0]; o[1] += kf[1]; o[2] += kf[2]; }
      xp[3 * i] = o[0]; xp[3 * i + 1] = o[1]; xp[3 * i + 2] = o[2];
    });
  });
}

}  // namespace nva

TORCH_LIBRARY_FRAGMENT(nvalchemi, m) {
  m.def("nhc_chain_update(Tensor(a!) velocities, Tensor masses, Tensor(b!) eta, Tensor(c!) eta_dot, Tensor Q, Tensor temperature, Tensor dt, Tensor ndof, Tensor(d!) ke2, Tensor(e!) total_scale, Tensor(f!) step_scale, Tensor(g!) dt_chain, Tensor batch_idx, bool compute_ke, int yoshida_order=3) -> ()", torch::dispatch(c10::DispatchKey::CompositeExplicitAutograd, &nva::nhc_chain_update));
  m.def("nhc_chain_scalar(Tensor(a!) ke2, Tensor(b!) eta, Tensor(c!) eta_dot, Tensor Q, Tensor temperature, Tensor ndof, Tensor dt, int yoshida_order=3) -> Tensor", torch::dispatch(c10::DispatchKey::CompositeExplicitAutograd, &nva::nhc_chain_scalar));
  m.def("nhc_velocity_half_step(Tensor(a!) velocities, Tensor forces, Tensor masses, Tensor dt, Tensor batch_idx) -> ()", torch::dispatch(c10::DispatchKey::CompositeExplicitAutograd, &nva::nhc_velocity_half_step));
  m.def("nhc_position_update(Tensor(a!) positions, Tensor velocities, Tensor dt, Tensor batch_idx) -> ()", torch::dispatch(c10::DispatchKey::CompositeExplicitAutograd, &nva::nhc_position_update));
  m.def("compute_kinetic_tensor(Tensor velocities, Tensor masses, Tensor(a!) kinetic_tensors, Tensor batch_idx) -> ()", torch::dispatch(c10::DispatchKey::CompositeExplicitAutograd, &nva::compute_kinetic_tensor));
  m.def("affine_rows_(Tensor(a!) x, Tensor A, Tensor? y, Tensor? C, Tensor? forces, Tensor? masses, Tensor? kick, Tensor batch_idx, bool kick_first=False) -> ()", torch::dispatch(c10::DispatchKey::CompositeExplicitAutograd, &nva::affine_rows_));
}
