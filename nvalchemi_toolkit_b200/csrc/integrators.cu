// SPDX-License-Identifier: Apache-2.0
// Integrator and thermostat kernels (velocity Verlet, Langevin BAOAB, FIRE, kinetic energy,
// velocity initialisation, COM removal, position wrapping, skin-based rebuild detection).
// Each elementwise kernel is one functor executed either as a CUDA kernel or as an OpenMP
// loop, so CPU and GPU paths share their arithmetic.  Semantics follow the op surface of the
// reference (nvalchemi/dynamics/_ops/velocity_verlet.py:50-143, langevin.py:55-174,
// fire.py:79-363, thermostat_utils.py:177-449, neighbor_list_rebuild.py:37-186).
#include "common.cuh"

namespace nva {

using at::Tensor;

template <typename T>
struct P3 {
  T* p;
  NVA_HD T& operator()(int64_t i, int c) const { return p[3 * i + c]; }
};

// ------------------------------------------------------------------ velocity Verlet
void vv_position_update(Tensor pos, Tensor vel, const Tensor& force, const Tensor& mass, const Tensor& dt,
                        const Tensor& batch_idx) {
  NVA_CHECK_CONTIG(pos); NVA_CHECK_CONTIG(vel); NVA_CHECK_CONTIG(force);
  c10::cuda::OptionalCUDAGuard guard(pos.is_cuda() ? c10::make_optional(pos.device()) : c10::nullopt);
  int64_t n = pos.size(0);
  AT_DISPATCH_FLOATING_TYPES(pos.scalar_type(), "vv_position_update", [&] {
    scalar_t* r = pos.data_ptr<scalar_t>();
    scalar_t* v = vel.data_ptr<scalar_t>();
    const scalar_t* f = force.data_ptr<scalar_t>();
    const scalar_t* m = mass.data_ptr<scalar_t>();
    const scalar_t* d = dt.data_ptr<scalar_t>();
    const int* b = batch_idx.data_ptr<int>();
    for_each(pos.is_cuda(), n, [=] NVA_LAMBDA(int64_t i) {
      scalar_t h = d[b[i]], im = scalar_t(1) / m[i];
      for (int c = 0; c < 3; ++c) {
        scalar_t a = f[3 * i + c] * im;
        r[3 * i + c] += v[3 * i + c] * h + scalar_t(0.5) * a * h * h;
        v[3 * i + c] += scalar_t(0.5) * a * h;
      }
    });
  });
}

void vv_velocity_finalize(Tensor vel, const Tensor& force, const Tensor& mass, const Tensor& dt,
                          const Tensor& batch_idx) {
  NVA_CHECK_CONTIG(vel); NVA_CHECK_CONTIG(force);
  c10::cuda::OptionalCUDAGuard guard(vel.is_cuda() ? c10::make_optional(vel.device()) : c10::nullopt);
  int64_t n = vel.size(0);
  AT_DISPATCH_FLOATING_TYPES(vel.scalar_type(), "vv_velocity_finalize", [&] {
    scalar_t* v = vel.data_ptr<scalar_t>();
    const scalar_t* f = force.data_ptr<scalar_t>();
    const scalar_t* m = mass.data_ptr<scalar_t>();
    const scalar_t* d = dt.data_ptr<scalar_t>();
    const int* b = batch_idx.data_ptr<int>();
    for_each(vel.is_cuda(), n, [=] NVA_LAMBDA(int64_t i) {
      scalar_t s = scalar_t(0.5) * d[b[i]] / m[i];
      for (int c = 0; c < 3; ++c) v[3 * i + c] += s * f[3 * i + c];
    });
  });
}

// ------------------------------------------------------------------ Langevin BAOAB
// half step = B (half kick) A (half drift) O (Ornstein-Uhlenbeck) A (half drift); the closing
// half kick is langevin_finalize (same arithmetic as vv_velocity_finalize).  `kT` is in eV.
// Noise: Philox keyed by `seed`, counter = atom index (+ atom_offset so a domain-decomposed
// run draws the same numbers per global atom).
void langevin_half_step(Tensor pos, Tensor vel, const Tensor& force, const Tensor& mass, const Tensor& dt,
                        const Tensor& kT, const Tensor& friction, int64_t seed, const Tensor& batch_idx,
                        const c10::optional<Tensor>& atom_ids) {
  NVA_CHECK_CONTIG(pos); NVA_CHECK_CONTIG(vel); NVA_CHECK_CONTIG(force);
  c10::cuda::OptionalCUDAGuard guard(pos.is_cuda() ? c10::make_optional(pos.device()) : c10::nullopt);
  int64_t n = pos.size(0);
  const int64_t* ids = atom_ids.has_value() ? atom_ids->data_ptr<int64_t>() : nullptr;
  AT_DISPATCH_FLOATING_TYPES(pos.scalar_type(), "langevin_half_step", [&] {
    scalar_t* r = pos.data_ptr<scalar_t>();
    scalar_t* v = vel.data_ptr<scalar_t>();
    const scalar_t* f = force.data_ptr<scalar_t>();
    const scalar_t* m = mass.data_ptr<scalar_t>();
    const scalar_t* d = dt.data_ptr<scalar_t>();
    const scalar_t* t = kT.data_ptr<scalar_t>();
    const scalar_t* g = friction.data_ptr<scalar_t>();
    const int* b = batch_idx.data_ptr<int>();
    for_each(pos.is_cuda(), n, [=] NVA_LAMBDA(int64_t i) {
      int s = b[i];
      scalar_t h = d[s], im = scalar_t(1) / m[i];
      double c1 = exp(-(double)g[s] * (double)h);
      double c2 = sqrt((1.0 - c1 * c1) * (double)t[s] * (double)im);
      double z[4];
      philox_normal4((uint64_t)seed, (uint64_t)(ids ? ids[i] : i), 0x4c616e67ull, z);
      for (int c = 0; c < 3; ++c) {
        scalar_t vc = v[3 * i + c] + scalar_t(0.5) * h * f[3 * i + c] * im;  // B
        scalar_t rc = r[3 * i + c] + scalar_t(0.5) * h * vc;                  // A
        vc = (scalar_t)(c1 * (double)vc + c2 * z[c]);                         // O
        rc += scalar_t(0.5) * h * vc;                                         // A
        v[3 * i + c] = vc;
        r[3 * i + c] = rc;
      }
    });
  });
}

// ------------------------------------------------------------------ per-system sums
template <typename T, typename F>
__global__ void seg_reduce_kernel(int64_t n, const int* __restrict__ seg, double* __restrict__ out, int nout,
                                  F f) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  bool ok = i < n;
  int s = ok ? seg[i] : -1;
  double vals[4] = {0, 0, 0, 0};
  if (ok) f(i, vals);
  for (int k = 0; k < 4; ++k) {
    if (k < nout) seg_atomic_add(out, s < 0 ? -1 : s * nout + k, vals[k]);
  }
}

// out[M, nout] (double) += per-atom values produced by f(i, vals[4]).
template <typename T, typename F>
void seg_reduce(bool cuda, int64_t n, const int* seg, double* out, int nout, F f) {
  if (n <= 0) return;
  if (cuda) {
    int64_t blocks = (n + kThreads - 1) / kThreads;
    seg_reduce_kernel<T><<<(unsigned)blocks, kThreads, 0, at::cuda::getCurrentCUDAStream()>>>(n, seg, out, nout, f);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  } else {
    for (int64_t i = 0; i < n; ++i) {
      double vals[4] = {0, 0, 0, 0};
      f(i, vals);
      for (int k = 0; k < nout; ++k) out[(int64_t)seg[i] * nout + k] += vals[k];
    }
  }
}

Tensor compute_kinetic_energy(const Tensor& vel, const Tensor& mass, const Tensor& batch_idx, int64_t num_systems) {
  c10::cuda::OptionalCUDAGuard guard(vel.is_cuda() ? c10::make_optional(vel.device()) : c10::nullopt);
  Tensor out = at::zeros({num_systems}, vel.options().dtype(at::kDouble));
  int64_t n = vel.size(0);
  AT_DISPATCH_FLOATING_TYPES(vel.scalar_type(), "compute_kinetic_energy", [&] {
    const scalar_t* v = vel.data_ptr<scalar_t>();
    const scalar_t* m = mass.data_ptr<scalar_t>();
    seg_reduce<scalar_t>(vel.is_cuda(), n, batch_idx.data_ptr<int>(), out.data_ptr<double>(), 1,
                         [=] NVA_LAMBDA(int64_t i, double* o) {
                           double x = v[3 * i], y = v[3 * i + 1], z = v[3 * i + 2];
                           o[0] = 0.5 * (double)m[i] * (x * x + y * y + z * z);
                         });
  });
  return out.to(vel.scalar_type());
}

// ------------------------------------------------------------------ FIRE
// One FIRE iteration on forces evaluated at the current positions (ASE-style ordering):
//   P = F.v per system; P > 0: v <- (1-a) v + a |v| F/|F|, after n_min positive steps
//   dt <- min(dt f_inc, dt_max), a <- a f_alpha; else v <- 0, dt <- max(dt f_dec, dt_min),
//   a <- a_start.  Then v += dt F/m, dr = dt v scaled per system so that no atom moves more
//   than maxstep, r += dr.  vf/vv/ff receive the reductions (they may be supplied already
//   reduced across ranks with compute_reductions = false).
void fire_step(Tensor pos, Tensor vel, const Tensor& force, const Tensor& mass, Tensor alpha, Tensor dt,
               const Tensor& alpha_start, const Tensor& f_alpha, const Tensor& dt_min, const Tensor& dt_max,
               const Tensor& maxstep, Tensor n_pos, const Tensor& n_min, const Tensor& f_dec,
               const Tensor& f_inc, const Tensor& uphill, Tensor vf, Tensor vv, Tensor ff,
               const Tensor& batch_idx, bool compute_reductions, const c10::optional<Tensor>& max_dr,
               int64_t phase) {
  // phase 0: the whole iteration.  phase 1: controller + velocity update only, the per-system largest displacement is
  // left in `max_dr` (float32 [M]); phase 2: position update only, from a `max_dr` the caller has reduced (MAX) over
  // the ranks of a domain decomposition in between, so that every rank applies the same step-length cap.
  NVA_CHECK_CONTIG(pos); NVA_CHECK_CONTIG(vel); NVA_CHECK_CONTIG(force);
  c10::cuda::OptionalCUDAGuard guard(pos.is_cuda() ? c10::make_optional(pos.device()) : c10::nullopt);
  bool cuda = pos.is_cuda();
  int64_t n = pos.size(0), M = alpha.size(0);
  const int* b = batch_idx.data_ptr<int>();
  TORCH_CHECK(phase == 0 || (max_dr.has_value() && max_dr->scalar_type() == at::kFloat && max_dr->numel() == M),
              "fire_step: phases 1 and 2 need a float32 max_dr of one entry per system");
  AT_DISPATCH_FLOATING_TYPES(pos.scalar_type(), "fire_step", [&] {
    scalar_t* r = pos.data_ptr<scalar_t>();
    scalar_t* v = vel.data_ptr<scalar_t>();
    const scalar_t* f = force.data_ptr<scalar_t>();
    const scalar_t* m = mass.data_ptr<scalar_t>();
    Tensor maxdr = max_dr.has_value() ? *max_dr : at::empty({M}, pos.options().dtype(at::kFloat));
    float* md = maxdr.data_ptr<float>();
    const scalar_t* ms = maxstep.data_ptr<scalar_t>();
    scalar_t* d = dt.data_ptr<scalar_t>();
    if (phase == 2) {
      for_each(cuda, n, [=] NVA_LAMBDA(int64_t i) {
        int s = b[i];
        scalar_t h = d[s];
        scalar_t scale = md[s] > (float)ms[s] ? ms[s] / (scalar_t)md[s] : scalar_t(1);
        for (int c = 0; c < 3; ++c) r[3 * i + c] += scale * h * v[3 * i + c];
      });
      return;
    }
    maxdr.zero_();
    if (compute_reductions) {
      Tensor red = at::zeros({M, 3}, pos.options().dtype(at::kDouble));
      seg_reduce<scalar_t>(cuda, n, b, red.data_ptr<double>(), 3, [=] NVA_LAMBDA(int64_t i, double* o) {
        for (int c = 0; c < 3; ++c) {
          double vc = v[3 * i + c], fc = f[3 * i + c];
          o[0] += vc * fc; o[1] += vc * vc; o[2] += fc * fc;
        }
      });
      Tensor redc = red.to(pos.scalar_type());
      vf.copy_(redc.select(1, 0)); vv.copy_(redc.select(1, 1)); ff.copy_(redc.select(1, 2));
    }
    // per-system controller: writes mixing coefficients into scratch [M,3] = (keep, mix, dt)
    Tensor coef = at::empty({M, 3}, pos.options());
    scalar_t* cf = coef.data_ptr<scalar_t>();
    scalar_t* al = alpha.data_ptr<scalar_t>();
    int* np_ = n_pos.data_ptr<int>();
    const scalar_t *as = alpha_start.data_ptr<scalar_t>(), *fa = f_alpha.data_ptr<scalar_t>(),
                   *dmin = dt_min.data_ptr<scalar_t>(), *dmax = dt_max.data_ptr<scalar_t>(),
                   *fd = f_dec.data_ptr<scalar_t>(), *fi = f_inc.data_ptr<scalar_t>();
    const int* nm = n_min.data_ptr<int>();
    const scalar_t *pvf = vf.data_ptr<scalar_t>(), *pvv = vv.data_ptr<scalar_t>(), *pff = ff.data_ptr<scalar_t>();
    for_each(cuda, M, [=] NVA_LAMBDA(int64_t s) {
      scalar_t keep, mix;
      if (pvf[s] > scalar_t(0)) {
        scalar_t a = al[s];
        keep = scalar_t(1) - a;
        mix = pff[s] > scalar_t(0) ? a * sqrt(pvv[s] / pff[s]) : scalar_t(0);
        np_[s] += 1;
        if (np_[s] > nm[s]) {
          d[s] = d[s] * fi[s] < dmax[s] ? d[s] * fi[s] : dmax[s];
          al[s] = a * fa[s];
        }
      } else {
        keep = scalar_t(0); mix = scalar_t(0);
        np_[s] = 0;
        d[s] = d[s] * fd[s] > dmin[s] ? d[s] * fd[s] : dmin[s];
        al[s] = as[s];
      }
      cf[3 * s] = keep; cf[3 * s + 1] = mix; cf[3 * s + 2] = d[s];
    });
    // velocity mixing + kick; per-system max displacement (double accumulators via atomic max on bits)
    for_each(cuda, n, [=] NVA_LAMBDA(int64_t i) {
      int s = b[i];
      scalar_t keep = cf[3 * s], mix = cf[3 * s + 1], h = cf[3 * s + 2], im = scalar_t(1) / m[i];
      scalar_t d2 = 0;
      for (int c = 0; c < 3; ++c) {
        scalar_t vc = keep * v[3 * i + c] + mix * f[3 * i + c] + h * f[3 * i + c] * im;
        v[3 * i + c] = vc;
        d2 += h * vc * h * vc;
      }
      float dn = (float)sqrt((double)d2);
#ifdef __CUDA_ARCH__
      atomicMax((int*)md + s, __float_as_int(dn));  // non-negative floats order like ints
#else
      if (dn > md[s]) md[s] = dn;
#endif
    });
    if (phase == 1) return;
    for_each(cuda, n, [=] NVA_LAMBDA(int64_t i) {
      int s = b[i];
      scalar_t h = cf[3 * s + 2];
      scalar_t scale = md[s] > (float)ms[s] ? ms[s] / (scalar_t)md[s] : scalar_t(1);
      for (int c = 0; c < 3; ++c) r[3 * i + c] += scale * h * v[3 * i + c];
    });
  });
  (void)uphill;
}

// ------------------------------------------------------------------ FIRE2
// One FIRE2 iteration (Guenole et al. 2020; reference op family nvalchemi/dynamics/_ops/fire.py:467-648) on per-system
// state (alpha, dt, nsteps_inc).  The iteration has three per-system reductions, so it is cut into four phases that a
// domain decomposition can interleave with its cross-rank reductions; phase 0 runs all four back to back.
//   1: sums[:,0] = sum v.f
//   2: controller from sums[:,0] (P > 0 for more than `delaystep` steps grows dt and shrinks alpha; P <= 0 shrinks dt,
//      resets alpha); uphill systems step back half a step and stop; v += dt f; sums[:,1] = sum v.v, sums[:,2] = sum f.f
//   3: v <- (1 - alpha) v + alpha sqrt(vv / ff) f; max_dr[s] = max |dt v|
//   4: r += min(1, maxstep / max_dr) dt v
void fire2_step(Tensor pos, Tensor vel, const Tensor& force, const Tensor& batch_idx, Tensor alpha, Tensor dt,
                Tensor nsteps_inc, Tensor sums, Tensor max_dr, int64_t delaystep, double dtgrow, double dtshrink,
                double alphashrink, double alpha0, double tmax, double tmin, double maxstep, int64_t phase) {
  NVA_CHECK_CONTIG(pos); NVA_CHECK_CONTIG(vel); NVA_CHECK_CONTIG(force); NVA_CHECK_CONTIG(sums);
  c10::cuda::OptionalCUDAGuard guard(pos.is_cuda() ? c10::make_optional(pos.device()) : c10::nullopt);
  const bool cuda = pos.is_cuda();
  const int64_t n = pos.size(0), M = alpha.size(0);
  TORCH_CHECK(sums.scalar_type() == at::kDouble && sums.numel() == 3 * M, "fire2_step: sums must be float64 [M, 3]");
  TORCH_CHECK(max_dr.scalar_type() == at::kFloat && max_dr.numel() == M, "fire2_step: max_dr must be float32 [M]");
  TORCH_CHECK(nsteps_inc.scalar_type() == at::kInt && batch_idx.scalar_type() == at::kInt, "fire2_step: int32 counters / batch_idx");
  TORCH_CHECK(phase >= 0 && phase <= 4, "fire2_step: phase must be 0..4");
  const int* b = batch_idx.data_ptr<int>();
  double* sm = sums.data_ptr<double>();
  float* md = max_dr.data_ptr<float>();
  int* nsi = nsteps_inc.data_ptr<int>();
  AT_DISPATCH_FLOATING_TYPES(pos.scalar_type(), "fire2_step", [&] {
    scalar_t* r = pos.data_ptr<scalar_t>();
    scalar_t* v = vel.data_ptr<scalar_t>();
    const scalar_t* f = force.data_ptr<scalar_t>();
    scalar_t* al = alpha.data_ptr<scalar_t>();
    scalar_t* d = dt.data_ptr<scalar_t>();
    if (phase == 0 || phase == 1) {
      sums.zero_();
      seg_reduce<scalar_t>(cuda, n, b, sm, 3, [=] NVA_LAMBDA(int64_t i, double* o) {
        for (int c = 0; c < 3; ++c) o[0] += (double)v[3 * i + c] * (double)f[3 * i + c];
      });
    }
    if (phase == 0 || phase == 2) {
      // controller; the sign of P is kept in max_dr (1 = uphill) until phase 3 overwrites it with the displacements
      for_each(cuda, M, [=] NVA_LAMBDA(int64_t s) {
        const bool neg = !(sm[3 * s] > 0.0);
        const int inc = neg ? 0 : nsi[s] + 1;
        nsi[s] = inc;
        if (neg) {
          const scalar_t nd = d[s] * (scalar_t)dtshrink;
          d[s] = nd > (scalar_t)tmin ? nd : (scalar_t)tmin;
          al[s] = (scalar_t)alpha0;
        } else if (inc > delaystep) {
          const scalar_t nd = d[s] * (scalar_t)dtgrow;
          d[s] = nd < (scalar_t)tmax ? nd : (scalar_t)tmax;
          al[s] = al[s] * (scalar_t)alphashrink;
        }
        md[s] = neg ? 1.0f : 0.0f;
        sm[3 * s + 1] = 0.0; sm[3 * s + 2] = 0.0;
      });
      seg_reduce<scalar_t>(cuda, n, b, sm, 3, [=] NVA_LAMBDA(int64_t i, double* o) {
        const int s = b[i];
        const scalar_t h = d[s];
        const bool neg = md[s] != 0.0f;
        for (int c = 0; c < 3; ++c) {
          scalar_t vc = v[3 * i + c];
          const scalar_t fc = f[3 * i + c];
          if (neg) { r[3 * i + c] -= scalar_t(0.5) * h * vc; vc = scalar_t(0); }
          vc += h * fc;
          v[3 * i + c] = vc;
          o[1] += (double)vc * (double)vc; o[2] += (double)fc * (double)fc;
        }
      });
    }
    if (phase == 0 || phase == 3) {
      max_dr.zero_();
      for_each(cuda, n, [=] NVA_LAMBDA(int64_t i) {
        const int s = b[i];
        const scalar_t a = al[s], h = d[s];
        const double ffs = sm[3 * s + 2];
        const scalar_t mix = a * (scalar_t)sqrt(sm[3 * s + 1] / (ffs > 1e-300 ? ffs : 1e-300));
        scalar_t d2 = 0;
        for (int c = 0; c < 3; ++c) {
          const scalar_t vc = (scalar_t(1) - a) * v[3 * i + c] + mix * f[3 * i + c];
          v[3 * i + c] = vc;
          d2 += h * vc * h * vc;
        }
        const float dn = (float)sqrt((double)d2);
#ifdef __CUDA_ARCH__
        atomicMax((int*)md + s, __float_as_int(dn));  // non-negative floats order like ints
#else
        if (dn > md[s]) md[s] = dn;
#endif
      });
    }
    if (phase == 0 || phase == 4) {
      for_each(cuda, n, [=] NVA_LAMBDA(int64_t i) {
        const int s = b[i];
        const scalar_t h = d[s];
        const scalar_t scale = md[s] > (float)maxstep ? (scalar_t)(maxstep / (double)md[s]) : scalar_t(1);
        for (int c = 0; c < 3; ++c) r[3 * i + c] += scale * h * v[3 * i + c];
      });
    }
  });
}

// ------------------------------------------------------------------ velocities
// Maxwell-Boltzmann draw: v = sqrt(kT/m) * N(0,1), kT in eV per system.
void maxwell_boltzmann(Tensor vel, const Tensor& mass, const Tensor& kT, const Tensor& batch_idx, int64_t seed,
                       const c10::optional<Tensor>& atom_ids) {
  c10::cuda::OptionalCUDAGuard guard(vel.is_cuda() ? c10::make_optional(vel.device()) : c10::nullopt);
  int64_t n = vel.size(0);
  const int64_t* ids = atom_ids.has_value() ? atom_ids->data_ptr<int64_t>() : nullptr;
  AT_DISPATCH_FLOATING_TYPES(vel.scalar_type(), "maxwell_boltzmann", [&] {
    scalar_t* v = vel.data_ptr<scalar_t>();
    const scalar_t* m = mass.data_ptr<scalar_t>();
    const scalar_t* t = kT.data_ptr<scalar_t>();
    const int* b = batch_idx.data_ptr<int>();
    for_each(vel.is_cuda(), n, [=] NVA_LAMBDA(int64_t i) {
      double z[4];
      philox_normal4((uint64_t)seed, (uint64_t)(ids ? ids[i] : i), 0x4d42ull, z);
      double s = sqrt((double)t[b[i]] / (double)m[i]);
      for (int c = 0; c < 3; ++c) v[3 * i + c] = (scalar_t)(s * z[c]);
    });
  });
}

// Per-system mass-weighted sums: out[M,4] = (sum m vx, sum m vy, sum m vz, sum m).
Tensor momentum_sums(const Tensor& vel, const Tensor& mass, const Tensor& batch_idx, int64_t num_systems) {
  c10::cuda::OptionalCUDAGuard guard(vel.is_cuda() ? c10::make_optional(vel.device()) : c10::nullopt);
  Tensor out = at::zeros({num_systems, 4}, vel.options().dtype(at::kDouble));
  AT_DISPATCH_FLOATING_TYPES(vel.scalar_type(), "momentum_sums", [&] {
    const scalar_t* v = vel.data_ptr<scalar_t>();
    const scalar_t* m = mass.data_ptr<scalar_t>();
    seg_reduce<scalar_t>(vel.is_cuda(), vel.size(0), batch_idx.data_ptr<int>(), out.data_ptr<double>(), 4,
                         [=] NVA_LAMBDA(int64_t i, double* o) {
                           double mi = m[i];
                           o[0] = mi * v[3 * i]; o[1] = mi * v[3 * i + 1]; o[2] = mi * v[3 * i + 2]; o[3] = mi;
                         });
  });
  return out;
}

// v[i] = (v[i] - shift[b[i]]) * scale[b[i]]   (COM removal and rescaling in one pass)
void velocity_shift_scale(Tensor vel, const Tensor& shift, const Tensor& scale, const Tensor& batch_idx) {
  c10::cuda::OptionalCUDAGuard guard(vel.is_cuda() ? c10::make_optional(vel.device()) : c10::nullopt);
  AT_DISPATCH_FLOATING_TYPES(vel.scalar_type(), "velocity_shift_scale", [&] {
    scalar_t* v = vel.data_ptr<scalar_t>();
    const scalar_t* sh = shift.data_ptr<scalar_t>();
    const scalar_t* sc = scale.data_ptr<scalar_t>();
    const int* b = batch_idx.data_ptr<int>();
    for_each(vel.is_cuda(), vel.size(0), [=] NVA_LAMBDA(int64_t i) {
      int s = b[i];
      for (int c = 0; c < 3; ++c) v[3 * i + c] = (v[3 * i + c] - sh[3 * s + c]) * sc[s];
    });
  });
}

// ------------------------------------------------------------------ periodic wrapping
// positions -> positions wrapped into the cell along periodic directions (rows of cell are
// lattice vectors; cart = frac @ cell).
Tensor wrap_positions(const Tensor& pos, const Tensor& cell, const Tensor& cell_inv, const Tensor& pbc,
                      const Tensor& batch_idx) {
  c10::cuda::OptionalCUDAGuard guard(pos.is_cuda() ? c10::make_optional(pos.device()) : c10::nullopt);
  Tensor out = at::empty_like(pos);
  AT_DISPATCH_FLOATING_TYPES(pos.scalar_type(), "wrap_positions", [&] {
    const scalar_t* r = pos.data_ptr<scalar_t>();
    scalar_t* o = out.data_ptr<scalar_t>();
    const scalar_t* h = cell.data_ptr<scalar_t>();
    const scalar_t* hi = cell_inv.data_ptr<scalar_t>();
    const bool* pb = pbc.data_ptr<bool>();
    const int* b = batch_idx.data_ptr<int>();
    for_each(pos.is_cuda(), pos.size(0), [=] NVA_LAMBDA(int64_t i) {
      int s = b[i];
      const scalar_t* H = h + 9 * s;
      const scalar_t* Hi = hi + 9 * s;
      scalar_t x = r[3 * i], y = r[3 * i + 1], z = r[3 * i + 2];
      scalar_t fr[3];
      for (int c = 0; c < 3; ++c) {
        scalar_t fc = x * Hi[c] + y * Hi[3 + c] + z * Hi[6 + c];
        fr[c] = pb[3 * s + c] ? fc - floor(fc) : fc;
      }
      for (int c = 0; c < 3; ++c) o[3 * i + c] = fr[0] * H[c] + fr[1] * H[3 + c] + fr[2] * H[6 + c];
    });
  });
  return out;
}

// flags[s] |= any atom of s moved farther than `threshold` (minimum image) from ref; optionally
// refreshes ref for flagged systems in a second pass.
void neighbor_rebuild_check(Tensor ref_pos, const Tensor& pos, const Tensor& batch_idx, Tensor flags,
                            double threshold, bool update_ref, const Tensor& cell, const Tensor& cell_inv,
                            const Tensor& pbc) {
  c10::cuda::OptionalCUDAGuard guard(pos.is_cuda() ? c10::make_optional(pos.device()) : c10::nullopt);
  bool cuda = pos.is_cuda();
  int64_t n = pos.size(0);
  bool* fl = flags.data_ptr<bool>();
  const int* b = batch_idx.data_ptr<int>();
  AT_DISPATCH_FLOATING_TYPES(pos.scalar_type(), "neighbor_rebuild_check", [&] {
    scalar_t* rr = ref_pos.data_ptr<scalar_t>();
    const scalar_t* r = pos.data_ptr<scalar_t>();
    const scalar_t* h = cell.data_ptr<scalar_t>();
    const scalar_t* hi = cell_inv.data_ptr<scalar_t>();
    const bool* pb = pbc.data_ptr<bool>();
    scalar_t t2 = (scalar_t)(threshold * threshold);
    for_each(cuda, n, [=] NVA_LAMBDA(int64_t i) {
      int s = b[i];
      const scalar_t* H = h + 9 * s;
      const scalar_t* Hi = hi + 9 * s;
      scalar_t d[3] = {r[3 * i] - rr[3 * i], r[3 * i + 1] - rr[3 * i + 1], r[3 * i + 2] - rr[3 * i + 2]};
      scalar_t fr[3];
      for (int c = 0; c < 3; ++c) {
        scalar_t fc = d[0] * Hi[c] + d[1] * Hi[3 + c] + d[2] * Hi[6 + c];
        fr[c] = pb[3 * s + c] ? fc - floor(fc + scalar_t(0.5)) : fc;
      }
      scalar_t d2 = 0;
      for (int c = 0; c < 3; ++c) {
        scalar_t x = fr[0] * H[c] + fr[1] * H[3 + c] + fr[2] * H[6 + c];
        d2 += x * x;
      }
      if (d2 > t2) fl[s] = true;  // benign race: every writer stores the same value
    });
    if (update_ref) {
      for_each(cuda, n, [=] NVA_LAMBDA(int64_t i) {
        if (fl[b[i]]) {
          rr[3 * i] = r[3 * i]; rr[3 * i + 1] = r[3 * i + 1]; rr[3 * i + 2] = r[3 * i + 2];
        }
      });
    }
  });
}

}  // namespace nva

TORCH_LIBRARY_FRAGMENT(nvalchemi, m) {
  m.def("vv_position_update(Tensor(a!) positions, Tensor(b!) velocities, Tensor forces, Tensor masses, Tensor dt, Tensor batch_idx) -> ()", torch::dispatch(c10::DispatchKey::CompositeExplicitAutograd, &nva::vv_position_update));
  m.def("vv_velocity_finalize(Tensor(a!) velocities, Tensor forces_new, Tensor masses, Tensor dt, Tensor batch_idx) -> ()", torch::dispatch(c10::DispatchKey::CompositeExplicitAutograd, &nva::vv_velocity_finalize));
  m.def("langevin_half_step(Tensor(a!) positions, Tensor(b!) velocities, Tensor forces, Tensor masses, Tensor dt, Tensor temperature, Tensor friction, int random_seed, Tensor batch_idx, Tensor? atom_ids=None) -> ()", torch::dispatch(c10::DispatchKey::CompositeExplicitAutograd, &nva::langevin_half_step));
  m.def("langevin_finalize(Tensor(a!) velocities, Tensor forces_new, Tensor masses, Tensor dt, Tensor batch_idx) -> ()", torch::dispatch(c10::DispatchKey::CompositeExplicitAutograd, &nva::vv_velocity_finalize));
  m.def("compute_kinetic_energy(Tensor velocities, Tensor masses, Tensor batch_idx, int num_systems) -> Tensor", torch::dispatch(c10::DispatchKey::CompositeExplicitAutograd, &nva::compute_kinetic_energy));
  m.def("fire2_step(Tensor(a!) positions, Tensor(b!) velocities, Tensor forces, Tensor batch_idx, Tensor(c!) alpha, Tensor(d!) dt, Tensor(e!) nsteps_inc, Tensor(f!) sums, Tensor(g!) max_dr, int delaystep, float dtgrow, float dtshrink, float alphashrink, float alpha0, float tmax, float tmin, float maxstep, int phase=0) -> ()", torch::dispatch(c10::DispatchKey::CompositeExplicitAutograd, &nva::fire2_step));
  m.def("_fire_step_op(Tensor(a!) positions, Tensor(b!) velocities, Tensor forces, Tensor masses, Tensor(c!) alpha, Tensor(d!) dt, Tensor alpha_start, Tensor f_alpha, Tensor dt_min, Tensor dt_max, Tensor maxstep, Tensor(e!) n_steps_positive, Tensor n_min, Tensor f_dec, Tensor f_inc, Tensor uphill_flag, Tensor(f!) vf, Tensor(g!) vv, Tensor(h!) ff, Tensor batch_idx, bool compute_reductions, Tensor? max_dr=None, int phase=0) -> ()", torch::dispatch(c10::DispatchKey::CompositeExplicitAutograd, &nva::fire_step));
  m.def("maxwell_boltzmann(Tensor(a!) velocities, Tensor masses, Tensor kT, Tensor batch_idx, int seed, Tensor? atom_ids=None) -> ()", &nva::maxwell_boltzmann);
  m.def("momentum_sums(Tensor velocities, Tensor masses, Tensor batch_idx, int num_systems) -> Tensor", torch::dispatch(c10::DispatchKey::CompositeExplicitAutograd, &nva::momentum_sums));
  m.def("velocity_shift_scale(Tensor(a!) velocities, Tensor shift, Tensor scale, Tensor batch_idx) -> ()", torch::dispatch(c10::DispatchKey::CompositeExplicitAutograd, &nva::velocity_shift_scale));
  m.def("wrap_positions(Tensor positions, Tensor cell, Tensor cell_inv, Tensor pbc, Tensor batch_idx) -> Tensor", torch::dispatch(c10::DispatchKey::CompositeExplicitAutograd, &nva::wrap_positions));
  m.def("neighbor_rebuild_check(Tensor(a!) reference_positions, Tensor current_positions, Tensor batch_idx, Tensor(b!) rebuild_flags, float threshold, bool update_reference_positions, Tensor cell, Tensor cell_inv, Tensor pbc) -> ()", &nva::neighbor_rebuild_check);
}
