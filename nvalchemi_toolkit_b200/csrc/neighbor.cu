// SPDX-License-Identifier: Apache-2.0
// Batched cell-list neighbour search with periodic images for triclinic cells.
// Produces the dense format of the reference's neighbour API (nvalchemi/neighbors.py:55-277,
// hooks/neighbor_list.py:244-394): neighbor_matrix [N,K] int32 (padding = N), num_neighbors [N]
// (true count, so a value > K signals overflow) and integer image shifts [N,K,3] such that the
// neighbour image sits at r_j + shift @ cell.
//
// Pipeline (no host synchronisation): per-system binning frame -> per-atom bin id and wrap
// image -> stable sort by bin (torch) -> CSR bin pointers -> one thread per atom scans the
// (2n+1)^3 neighbouring bins in a fixed order, so rows are deterministic.
#include "common.cuh"

namespace nva {
using at::Tensor;

struct Frame {       // per system, 24 floats/ints packed in two tensors
  // fl: origin[3], inv_width[3] (bins per unit fractional), cutoff2
  // in: nb[3], nsearch[3], bin_offset, pbc mask bits
};

// frames_f [B,8] = (o0,o1,o2, iw0,iw1,iw2, 0, 0); frames_i [B,8] = (nb0,nb1,nb2, ns0,ns1,ns2, bin_off, pbcbits)
template <typename T>
__global__ void bin_atoms_kernel(int64_t n, const T* __restrict__ pos, const T* __restrict__ cell_inv,
                                 const int* __restrict__ batch_idx, const float* __restrict__ ff,
                                 const int* __restrict__ fi, int64_t* __restrict__ bin_id,
                                 int* __restrict__ wrap) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= n) return;
  int s = batch_idx[i];
  const T* Hi = cell_inv + 9 * s;
  const float* F = ff + 8 * s;
  const int* I = fi + 8 * s;
  T x = pos[3 * i], y = pos[3 * i + 1], z = pos[3 * i + 2];
  int64_t lin = 0;
  for (int c = 0; c < 3; ++c) {
    double fc = (double)x * Hi[c] + (double)y * Hi[3 + c] + (double)z * Hi[6 + c];
    int w = 0;
    if (I[7] >> c & 1) {
      w = (int)floor(fc);
      fc -= (double)w;
    }
    wrap[3 * i + c] = w;
    int nb = I[c];
    int b = (int)floor((fc - (double)F[c]) * (double)F[3 + c]);
    b = b < 0 ? 0 : (b >= nb ? nb - 1 : b);
    lin = lin * nb + b;
  }
  bin_id[i] = (int64_t)I[6] + lin;
}

// Per-system bounds of the fractional coordinates (needed for the bin origin / extent of non-periodic directions), in
// one pass over the atoms: block-wide min / max in shared memory when the whole block belongs to one system (atoms are
// sorted by system), thread-level atomics otherwise.  Bounds are kept as order-preserving integer codes of floats.
__device__ __forceinline__ int float_order_code(float f) {
  const int i = __float_as_int(f);
  return i >= 0 ? i : i ^ 0x7fffffff;
}
// Ghost pull folded into the first pass over the atoms (domain decomposition on peer memory): rows >= ghost_row0 of `pos`
// are ghost atoms whose current position lives on another rank; the thread reads it from the owner through the symmetric
// buffer's address table (plain peer load), adds the lattice shift of the image and stores it into the local row, so the
// binning, the search and every later kernel see it without a separate halo kernel.
struct GhostPull {
  int64_t row0;             // first ghost row; < 0: no pull
  const int* home_rank;     // [n - row0]
  const int* home_row;
  const float* shift;       // [n - row0, 3]
  const int64_t* src_ptrs;  // [world] base addresses of the position buffer on every rank
};

template <typename T>
__global__ void frac_bounds_kernel(int64_t n, T* __restrict__ pos, const T* __restrict__ cell_inv,
                                   const int* __restrict__ batch_idx, int* __restrict__ lo, int* __restrict__ hi,
                                   GhostPull gp) {
  __shared__ int s_lo[3], s_hi[3], s_first, s_same;
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const bool live = i < n;
  const int s = live ? batch_idx[i] : -1;
  if (threadIdx.x == 0) {
    s_first = s; s_same = 1;
    for (int c = 0; c < 3; ++c) { s_lo[c] = 0x7fffffff; s_hi[c] = (int)0x80000000; }
  }
  __syncthreads();
  if (live && s != s_first) s_same = 0;  // benign race: every writer stores the same value
  __syncthreads();
  int code[3] = {0, 0, 0};
  if (live) {
    const T* Hi = cell_inv + 9 * s;
    T x, y, z;
    if (gp.row0 >= 0 && i >= gp.row0) {
      const int64_t g = i - gp.row0;
      const float* src = reinterpret_cast<const float*>(gp.src_ptrs[gp.home_rank[g]]) + 3 * (int64_t)gp.home_row[g];
      x = (T)(src[0] + gp.shift[3 * g]); y = (T)(src[1] + gp.shift[3 * g + 1]); z = (T)(src[2] + gp.shift[3 * g + 2]);
      pos[3 * i] = x; pos[3 * i + 1] = y; pos[3 * i + 2] = z;
    } else {
      x = pos[3 * i]; y = pos[3 * i + 1]; z = pos[3 * i + 2];
    }
    for (int c = 0; c < 3; ++c)
      code[c] = float_order_code((float)((double)x * Hi[c] + (double)y * Hi[3 + c] + (double)z * Hi[6 + c]));
  }
  if (s_same) {
    if (live)
      for (int c = 0; c < 3; ++c) { atomicMin(&s_lo[c], code[c]); atomicMax(&s_hi[c], code[c]); }
    __syncthreads();
    if (threadIdx.x < 3 && s_first >= 0) {
      atomicMin(lo + 3 * s_first + threadIdx.x, s_lo[threadIdx.x]);
      atomicMax(hi + 3 * s_first + threadIdx.x, s_hi[threadIdx.x]);
    }
  } else if (live) {
    for (int c = 0; c < 3; ++c) { atomicMin(lo + 3 * s + c, code[c]); atomicMax(hi + 3 * s + c, code[c]); }
  }
}

template <typename T>
__global__ void search_kernel(int64_t n, const T* __restrict__ pos, const T* __restrict__ cell,
                              const int* __restrict__ batch_idx, const int* __restrict__ fi,
                              const int64_t* __restrict__ bin_id, const int* __restrict__ wrap,
                              const int64_t* __restrict__ order, const int64_t* __restrict__ bin_ptr,
                              const bool* __restrict__ rebuild, T cutoff2, int K, bool half_list,
                              int* __restrict__ nm, int* __restrict__ num, int* __restrict__ shifts, int64_t n_rows) {
  int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (t >= n) return;
  // threads walk atoms in bin order so a warp shares its candidate bins
  int64_t i = order[t];
  if (i >= n_rows) return;  // rows beyond n_rows are candidates only (ghost atoms send, they do not receive)
  int s = batch_idx[i];
  if (rebuild != nullptr && !rebuild[s]) return;
  const int* I = fi + 8 * s;
  const T* H = cell + 9 * s;
  int nb0 = I[0], nb1 = I[1], nb2 = I[2];
  int64_t lin = bin_id[i] - I[6];
  int b2 = (int)(lin % nb2); lin /= nb2;
  int b1 = (int)(lin % nb1);
  int b0 = (int)(lin / nb1);
  int pbits = I[7];
  T xi = pos[3 * i], yi = pos[3 * i + 1], zi = pos[3 * i + 2];
  int wi0 = wrap[3 * i], wi1 = wrap[3 * i + 1], wi2 = wrap[3 * i + 2];
  int cnt = 0;
  int* row = nm + i * (int64_t)K;
  int* srow = shifts + i * (int64_t)K * 3;
  for (int d0 = -I[3]; d0 <= I[3]; ++d0) {
    int c0 = b0 + d0, s0 = 0;
    if (pbits & 1) { s0 = (int)floor((double)c0 / nb0); c0 -= s0 * nb0; }
    else if (c0 < 0 || c0 >= nb0) continue;
    for (int d1 = -I[4]; d1 <= I[4]; ++d1) {
      int c1 = b1 + d1, s1 = 0;
      if (pbits & 2) { s1 = (int)floor((double)c1 / nb1); c1 -= s1 * nb1; }
      else if (c1 < 0 || c1 >= nb1) continue;
      for (int d2 = -I[5]; d2 <= I[5]; ++d2) {
        int c2 = b2 + d2, s2 = 0;
        if (pbits & 4) { s2 = (int)floor((double)c2 / nb2); c2 -= s2 * nb2; }
        else if (c2 < 0 || c2 >= nb2) continue;
        int64_t bin = (int64_t)I[6] + ((int64_t)c0 * nb1 + c1) * nb2 + c2;
        for (int64_t q = bin_ptr[bin]; q < bin_ptr[bin + 1]; ++q) {
          int64_t j = order[q];
          int S0 = s0 - wrap[3 * j] + wi0, S1 = s1 - wrap[3 * j + 1] + wi1, S2 = s2 - wrap[3 * j + 2] + wi2;
          bool self_img = (j == i) && S0 == 0 && S1 == 0 && S2 == 0;
          if (self_img) continue;
          if (half_list) {
            if (j < i) continue;
            if (j == i && !(S0 > 0 || (S0 == 0 && (S1 > 0 || (S1 == 0 && S2 > 0))))) continue;
          }
          T dx = pos[3 * j] + S0 * H[0] + S1 * H[3] + S2 * H[6] - xi;
          T dy = pos[3 * j + 1] + S0 * H[1] + S1 * H[4] + S2 * H[7] - yi;
          T dz = pos[3 * j + 2] + S0 * H[2] + S1 * H[5] + S2 * H[8] - zi;
          if (dx * dx + dy * dy + dz * dz < cutoff2) {
            if (cnt < K) {
              row[cnt] = (int)j;
              srow[3 * cnt] = S0; srow[3 * cnt + 1] = S1; srow[3 * cnt + 2] = S2;
            }
            ++cnt;
          }
        }
      }
    }
  }
  int fill = (int)n;
  for (int k = cnt; k < K; ++k) { row[k] = fill; srow[3 * k] = 0; srow[3 * k + 1] = 0; srow[3 * k + 2] = 0; }
  num[i] = cnt;
}

// CPU twin of the two kernels (same arithmetic, serial over atoms inside an OpenMP loop).
template <typename T>
void search_cpu(int64_t n, const T* pos, const T* cell, const int* batch_idx, const int* fi, const int64_t* bin_id,
                const int* wrap, const int64_t* order, const int64_t* bin_ptr, const bool* rebuild, T cutoff2,
                int K, bool half_list, int* nm, int* num, int* shifts, int64_t n_rows) {
#pragma omp parallel for schedule(dynamic, 64)
  for (int64_t t = 0; t < n; ++t) {
    int64_t i = order[t];
    if (i >= n_rows) continue;
    int s = batch_idx[i];
    if (rebuild != nullptr && !rebuild[s]) continue;
    const int* I = fi + 8 * s;
    const T* H = cell + 9 * s;
    int nb0 = I[0], nb1 = I[1], nb2 = I[2];
    int64_t lin = bin_id[i] - I[6];
    int b2 = (int)(lin % nb2); lin /= nb2;
    int b1 = (int)(lin % nb1);
    int b0 = (int)(lin / nb1);
    int pbits = I[7];
    int cnt = 0;
    int* row = nm + i * (int64_t)K;
    int* srow = shifts + i * (int64_t)K * 3;
    for (int d0 = -I[3]; d0 <= I[3]; ++d0) {
      int c0 = b0 + d0, s0 = 0;
      if (pbits & 1) { s0 = (int)std::floor((double)c0 / nb0); c0 -= s0 * nb0; }
      else if (c0 < 0 || c0 >= nb0) continue;
      for (int d1 = -I[4]; d1 <= I[4]; ++d1) {
        int c1 = b1 + d1, s1 = 0;
        if (pbits & 2) { s1 = (int)std::floor((double)c1 / nb1); c1 -= s1 * nb1; }
        else if (c1 < 0 || c1 >= nb1) continue;
        for (int d2 = -I[5]; d2 <= I[5]; ++d2) {
          int c2 = b2 + d2, s2 = 0;
          if (pbits & 4) { s2 = (int)std::floor((double)c2 / nb2); c2 -= s2 * nb2; }
          else if (c2 < 0 || c2 >= nb2) continue;
          int64_t bin = (int64_t)I[6] + ((int64_t)c0 * nb1 + c1) * nb2 + c2;
          for (int64_t q = bin_ptr[bin]; q < bin_ptr[bin + 1]; ++q) {
            int64_t j = order[q];
            int S0 = s0 - wrap[3 * j] + wrap[3 * i], S1 = s1 - wrap[3 * j + 1] + wrap[3 * i + 1],
                S2 = s2 - wrap[3 * j + 2] + wrap[3 * i + 2];
            if (j == i && S0 == 0 && S1 == 0 && S2 == 0) continue;
            if (half_list) {
              if (j < i) continue;
              if (j == i && !(S0 > 0 || (S0 == 0 && (S1 > 0 || (S1 == 0 && S2 > 0))))) continue;
            }
            T dx = pos[3 * j] + S0 * H[0] + S1 * H[3] + S2 * H[6] - pos[3 * i];
            T dy = pos[3 * j + 1] + S0 * H[1] + S1 * H[4] + S2 * H[7] - pos[3 * i + 1];
            T dz = pos[3 * j + 2] + S0 * H[2] + S1 * H[5] + S2 * H[8] - pos[3 * i + 2];
            if (dx * dx + dy * dy + dz * dz < cutoff2) {
              if (cnt < K) {
                row[cnt] = (int)j;
                srow[3 * cnt] = S0; srow[3 * cnt + 1] = S1; srow[3 * cnt + 2] = S2;
              }
              ++cnt;
            }
          }
        }
      }
    }
    for (int k = cnt; k < K; ++k) { row[k] = (int)n; srow[3 * k] = 0; srow[3 * k + 1] = 0; srow[3 * k + 2] = 0; }
    num[i] = cnt;
  }
}

// positions [N,3]; cell [B,3,3]; pbc [B,3] bool; batch_idx [N] int32; batch_ptr [B+1] int32.
// out_* are updated in place (rows of systems whose rebuild flag is false are left untouched).
void neighbor_matrix_build(const Tensor& pos, const Tensor& cell, const Tensor& pbc, const Tensor& batch_idx,
                           const Tensor& batch_ptr, double cutoff, bool half_list, Tensor out_matrix,
                           Tensor out_num, Tensor out_shifts, const c10::optional<Tensor>& rebuild_flags,
                           int64_t num_rows, const c10::optional<Tensor>& ghost_home_rank,
                           const c10::optional<Tensor>& ghost_home_row, const c10::optional<Tensor>& ghost_shift,
                           const c10::optional<Tensor>& ghost_src_ptrs, int64_t ghost_row0) {
  c10::cuda::OptionalCUDAGuard guard(pos.is_cuda() ? c10::make_optional(pos.device()) : c10::nullopt);
  NVA_CHECK_CONTIG(pos); NVA_CHECK_CONTIG(cell); NVA_CHECK_CONTIG(out_matrix); NVA_CHECK_CONTIG(out_shifts);
  int64_t n = pos.size(0), B = cell.size(0), K = out_matrix.size(1);
  if (n == 0) return;
  const int64_t n_rows = num_rows < 0 ? n : std::min<int64_t>(num_rows, n);
  TORCH_CHECK(out_matrix.size(0) >= n_rows && out_num.size(0) >= n_rows && out_shifts.size(0) >= n_rows,
              "neighbor_matrix_build: output has fewer rows than requested");
  auto fopt = pos.options().dtype(at::kDouble);
  Tensor celld = cell.to(at::kDouble);
  Tensor inv = at::linalg_inv(celld);                                    // [B,3,3]
  Tensor face = at::reciprocal(inv.norm(2, {1}));                         // [B,3] distance per unit fractional
  Tensor pbcb = pbc.to(at::kBool);
  Tensor fmin, fmax;
  if (pos.is_cuda()) {
    // one kernel instead of five per-atom library operations (cast, gather of the inverse cells, batched product, two
    // scatter-reductions); the float bounds are widened by a few ulps so that every atom lies inside them
    Tensor lo = at::full({B, 3}, (int64_t)0x7fffffff, pos.options().dtype(at::kInt));
    Tensor hi = at::full({B, 3}, (int64_t)INT32_MIN, pos.options().dtype(at::kInt));
    Tensor inv_p = inv.to(pos.scalar_type()).contiguous();
    const int64_t nb_ = (n + kThreads - 1) / kThreads;
    GhostPull gp{-1, nullptr, nullptr, nullptr, nullptr};
    if (ghost_row0 >= 0 && ghost_home_rank.has_value()) {
      TORCH_CHECK(pos.scalar_type() == at::kFloat && ghost_home_row.has_value() && ghost_shift.has_value() && ghost_src_ptrs.has_value(),
                  "neighbor_matrix_build: the ghost pull needs float32 positions and all four ghost tables");
      TORCH_CHECK(ghost_home_rank->numel() == n - ghost_row0 && ghost_home_row->numel() == n - ghost_row0 &&
                      ghost_shift->numel() == 3 * (n - ghost_row0) && ghost_shift->is_contiguous(),
                  "neighbor_matrix_build: ghost tables must cover rows ghost_row0 .. n");
      gp = GhostPull{ghost_row0, ghost_home_rank->data_ptr<int>(), ghost_home_row->data_ptr<int>(), ghost_shift->data_ptr<float>(),
                     ghost_src_ptrs->data_ptr<int64_t>()};
    }
    AT_DISPATCH_FLOATING_TYPES(pos.scalar_type(), "frac_bounds", [&] {
      frac_bounds_kernel<scalar_t><<<(unsigned)nb_, kThreads, 0, at::cuda::getCurrentCUDAStream()>>>(
          n, pos.data_ptr<scalar_t>(), inv_p.data_ptr<scalar_t>(), batch_idx.data_ptr<int>(), lo.data_ptr<int>(), hi.data_ptr<int>(), gp);
    });
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    auto decode = [](const Tensor& code) {
      return at::where(code >= 0, code, at::bitwise_xor(code, at::full_like(code, (int64_t)0x7fffffff))).view(at::kFloat).to(at::kDouble);
    };
    fmin = at::nan_to_num(decode(lo), 0.0, 0.0, 0.0);  // a system without atoms keeps the initial codes
    fmax = at::nan_to_num(decode(hi), 0.0, 0.0, 0.0);
    fmin = fmin - (fmin.abs() * 4e-7 + 1e-7);
    fmax = fmax + (fmax.abs() * 4e-7 + 1e-7);
  } else {
    Tensor bidx = batch_idx.to(at::kLong);
    Tensor frac = at::bmm(pos.to(at::kDouble).unsqueeze(1), inv.index_select(0, bidx)).squeeze(1);  // [N,3]
    Tensor idx3 = bidx.unsqueeze(1).expand({n, 3});
    fmin = at::full({B, 3}, 1e300, fopt).scatter_reduce(0, idx3, frac, "amin", true);
    fmax = at::full({B, 3}, -1e300, fopt).scatter_reduce(0, idx3, frac, "amax", true);
  }
  Tensor origin = at::where(pbcb, at::zeros_like(fmin), fmin);
  Tensor extent = at::where(pbcb, at::ones_like(fmin), (fmax - fmin) + 1e-6);
  Tensor natoms = (batch_ptr.slice(0, 1) - batch_ptr.slice(0, 0, B)).to(at::kDouble);  // [B]
  Tensor nbf = at::floor(extent * face / cutoff).clamp_min(1.0);         // [B,3]
  Tensor prod = nbf.prod(1);
  Tensor cap = (2.0 * natoms).clamp_min(1.0);
  Tensor shrink = at::pow((cap / prod).clamp_max(1.0), 1.0 / 3.0).unsqueeze(1);
  nbf = at::floor(nbf * shrink).clamp_min(1.0);
  Tensor width = extent * face / nbf;                                    // cartesian bin thickness
  Tensor nsearch = at::ceil(cutoff / width - 1e-9).clamp_min(1.0);
  // non-periodic dims never need to look beyond their own range; cap the search to the bin count
  nsearch = at::where(pbcb, nsearch, at::minimum(nsearch, nbf));
  Tensor nbins = nbf.prod(1).to(at::kLong);
  Tensor bin_off = at::cumsum(nbins, 0) - nbins;
  Tensor bits = (pbcb.to(at::kLong) * at::tensor({1, 2, 4}, pbcb.options().dtype(at::kLong))).sum(1);
  Tensor ff = at::cat({origin, nbf / extent, at::zeros({B, 2}, fopt)}, 1).to(at::kFloat).contiguous();
  Tensor fi = at::cat({nbf.to(at::kLong), nsearch.to(at::kLong), bin_off.unsqueeze(1), bits.unsqueeze(1)}, 1)
                  .to(at::kInt).contiguous();
  int64_t max_bins = 2 * n + B + 1;
  Tensor bin_id = at::empty({n}, pos.options().dtype(at::kLong));
  Tensor wrap = at::empty({n, 3}, pos.options().dtype(at::kInt));
  Tensor inv_t = inv.to(pos.scalar_type()).contiguous();
  Tensor cell_t = cell.contiguous();
  const bool* rb = rebuild_flags.has_value() ? rebuild_flags->data_ptr<bool>() : nullptr;
  int64_t blocks = (n + kThreads - 1) / kThreads;
  AT_DISPATCH_FLOATING_TYPES(pos.scalar_type(), "neighbor_matrix_build", [&] {
    if (pos.is_cuda()) {
      bin_atoms_kernel<scalar_t><<<(unsigned)blocks, kThreads, 0, at::cuda::getCurrentCUDAStream()>>>(
          n, pos.data_ptr<scalar_t>(), inv_t.data_ptr<scalar_t>(), batch_idx.data_ptr<int>(), ff.data_ptr<float>(),
          fi.data_ptr<int>(), bin_id.data_ptr<int64_t>(), wrap.data_ptr<int>());
      C10_CUDA_KERNEL_LAUNCH_CHECK();
    } else {
      const scalar_t* P = pos.data_ptr<scalar_t>();
      const scalar_t* HI = inv_t.data_ptr<scalar_t>();
      const int* b = batch_idx.data_ptr<int>();
      const float* F0 = ff.data_ptr<float>();
      const int* I0 = fi.data_ptr<int>();
      int64_t* bid = bin_id.data_ptr<int64_t>();
      int* wr = wrap.data_ptr<int>();
      for (int64_t i = 0; i < n; ++i) {
        int s = b[i];
        const scalar_t* Hi = HI + 9 * s;
        const float* F = F0 + 8 * s;
        const int* I = I0 + 8 * s;
        int64_t lin = 0;
        for (int c = 0; c < 3; ++c) {
          double fc = (double)P[3 * i] * Hi[c] + (double)P[3 * i + 1] * Hi[3 + c] + (double)P[3 * i + 2] * Hi[6 + c];
          int w = 0;
          if (I[7] >> c & 1) { w = (int)std::floor(fc); fc -= (double)w; }
          wr[3 * i + c] = w;
          int nb = I[c];
          int bb = (int)std::floor((fc - (double)F[c]) * (double)F[3 + c]);
          bb = bb < 0 ? 0 : (bb >= nb ? nb - 1 : bb);
          lin = lin * nb + bb;
        }
        bid[i] = (int64_t)I[6] + lin;
      }
    }
    auto sorted = at::sort(bin_id, /*stable=*/true, 0, false);
    Tensor order = std::get<1>(sorted).contiguous();
    Tensor bounds = at::arange(max_bins + 1, bin_id.options());
    Tensor bin_ptr = at::searchsorted(std::get<0>(sorted).contiguous(), bounds, false, false).contiguous();
    scalar_t c2 = (scalar_t)(cutoff * cutoff);
    if (pos.is_cuda()) {
      search_kernel<scalar_t><<<(unsigned)blocks, kThreads, 0, at::cuda::getCurrentCUDAStream()>>>(
          n, pos.data_ptr<scalar_t>(), cell_t.data_ptr<scalar_t>(), batch_idx.data_ptr<int>(), fi.data_ptr<int>(),
          bin_id.data_ptr<int64_t>(), wrap.data_ptr<int>(), order.data_ptr<int64_t>(), bin_ptr.data_ptr<int64_t>(),
          rb, c2, (int)K, half_list, out_matrix.data_ptr<int>(), out_num.data_ptr<int>(),
          out_shifts.data_ptr<int>(), n_rows);
      C10_CUDA_KERNEL_LAUNCH_CHECK();
    } else {
      search_cpu<scalar_t>(n, pos.data_ptr<scalar_t>(), cell_t.data_ptr<scalar_t>(), batch_idx.data_ptr<int>(),
                           fi.data_ptr<int>(), bin_id.data_ptr<int64_t>(), wrap.data_ptr<int>(),
                           order.data_ptr<int64_t>(), bin_ptr.data_ptr<int64_t>(), rb, c2, (int)K, half_list,
                           out_matrix.data_ptr<int>(), out_num.data_ptr<int>(), out_shifts.data_ptr<int>(), n_rows);
    }
  });
}

// Neighbour matrix -> receiver-major CSR edge arrays in one pass: thread (i, slot) copies its sender and image shift to
// position eptr[i] + slot (eptr = exclusive prefix sum of the clamped counts, computed by the caller).
__global__ void csr_fill_kernel(const int* __restrict__ nm, const int* __restrict__ shifts, const int* __restrict__ eptr,
                                int64_t n, int K, int* __restrict__ esend, int* __restrict__ erecv, int* __restrict__ eS) {
  const int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (idx >= n * K) return;
  const int64_t i = idx / K;
  const int slot = (int)(idx - i * K);
  const int e0 = eptr[i], cnt = eptr[i + 1] - e0;
  if (slot >= cnt) return;
  const int64_t e = (int64_t)e0 + slot;
  esend[e] = nm[idx];
  erecv[e] = (int)i;
  if (shifts != nullptr) {
    eS[3 * e] = shifts[3 * idx]; eS[3 * e + 1] = shifts[3 * idx + 1]; eS[3 * e + 2] = shifts[3 * idx + 2];
  } else {
    eS[3 * e] = 0; eS[3 * e + 1] = 0; eS[3 * e + 2] = 0;
  }
}

void csr_fill(const Tensor& nm, const c10::optional<Tensor>& shifts, const Tensor& eptr, Tensor esend, Tensor erecv, Tensor eS) {
  c10::cuda::CUDAGuard guard(nm.device());
  NVA_CHECK_CONTIG(nm); NVA_CHECK_CONTIG(eptr); NVA_CHECK_CONTIG(esend); NVA_CHECK_CONTIG(erecv); NVA_CHECK_CONTIG(eS);
  TORCH_CHECK(nm.scalar_type() == at::kInt && eptr.scalar_type() == at::kInt, "csr_fill: int32 inputs");
  if (shifts.has_value()) { NVA_CHECK_CONTIG(*shifts); TORCH_CHECK(shifts->scalar_type() == at::kInt, "csr_fill: int32 shifts"); }
  const int64_t n = nm.size(0), K = nm.size(1);
  if (n * K == 0) return;
  const int threads = 256;
  const int64_t blocks = (n * K + threads - 1) / threads;
  csr_fill_kernel<<<(unsigned)blocks, threads, 0, at::cuda::getCurrentCUDAStream()>>>(
      nm.data_ptr<int>(), shifts.has_value() ? shifts->data_ptr<int>() : nullptr, eptr.data_ptr<int>(), n, (int)K,
      esend.data_ptr<int>(), erecv.data_ptr<int>(), eS.data_ptr<int>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

}  // namespace nva

TORCH_LIBRARY_FRAGMENT(nvalchemi, m) {
  m.def("csr_fill(Tensor nm, Tensor? shifts, Tensor eptr, Tensor(a!) esend, Tensor(b!) erecv, Tensor(c!) eS) -> ()", &nva::csr_fill);
  m.def("neighbor_matrix_build(Tensor(d!) positions, Tensor cell, Tensor pbc, Tensor batch_idx, Tensor batch_ptr, float cutoff, bool half_list, Tensor(a!) out_matrix, Tensor(b!) out_num, Tensor(c!) out_shifts, Tensor? rebuild_flags=None, int num_rows=-1, Tensor? ghost_home_rank=None, Tensor? ghost_home_row=None, Tensor? ghost_shift=None, Tensor? ghost_src_ptrs=None, int ghost_row0=-1) -> ()", &nva::neighbor_matrix_build);
}
