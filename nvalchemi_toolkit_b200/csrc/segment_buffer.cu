// SPDX-License-Identifier: Apache-2.0
// Sorted-segment reductions (sum / max / min / mean) and the row-copy primitives behind
// Batch.put / defrag / index_select.  Reference op surface: nvalchemi/dynamics/hooks/_utils.py:58-136
// (segmented_*), nvalchemi/data/buffer_kernels.py and data/level_storage.py:398-424 (expand segments).
#include "common.cuh"

namespace nva {
using at::Tensor;

// values [N, D] with non-decreasing idx [N] -> out [S, D].  One thread per (segment, column)
// walks its rows through a CSR pointer built by searchsorted: deterministic, atomic-free.
// mode: 0 sum, 1 max, 2 min, 3 mean.
Tensor segmented_reduce(const Tensor& values, const Tensor& idx, int64_t num_segments, int64_t mode) {
  c10::cuda::OptionalCUDAGuard guard(values.is_cuda() ? c10::make_optional(values.device()) : c10::nullopt);
  TORCH_CHECK(values.size(0) == idx.size(0), "values and idx disagree on the number of rows");
  Tensor v2 = values.reshape({values.size(0), -1}).contiguous();
  int64_t D = v2.size(1);
  Tensor bounds = at::arange(num_segments + 1, idx.options().dtype(at::kLong));
  Tensor ptr = at::searchsorted(idx.to(at::kLong).contiguous(), bounds, /*out_int32=*/false, /*right=*/false);
  Tensor out = at::zeros({num_segments, D}, v2.options());
  const int64_t* p = ptr.data_ptr<int64_t>();
  AT_DISPATCH_FLOATING_TYPES(v2.scalar_type(), "segmented_reduce", [&] {
    const scalar_t* v = v2.data_ptr<scalar_t>();
    scalar_t* o = out.data_ptr<scalar_t>();
    int m = (int)mode;
    for_each(values.is_cuda(), num_segments * D, [=] NVA_LAMBDA(int64_t t) {
      int64_t s = t / D, d = t % D;
      int64_t a = p[s], b = p[s + 1];
      if (a >= b) { o[t] = 0; return; }
      if (m == 0 || m == 3) {
        double acc = 0;
        for (int64_t r = a; r < b; ++r) acc += (double)v[r * D + d];
        o[t] = (scalar_t)(m == 3 ? acc / (double)(b - a) : acc);
      } else {
        scalar_t acc = v[a * D + d];
        for (int64_t r = a + 1; r < b; ++r) {
          scalar_t x = v[r * D + d];
          acc = m == 1 ? (x > acc ? x : acc) : (x < acc ? x : acc);
        }
        o[t] = acc;
      }
    });
  });
  std::vector<int64_t> shape = values.sizes().vec();
  shape[0] = num_segments;
  return out.reshape(shape);
}

// concat_i arange(starts[i], starts[i] + lens[i]); total = sum(lens) supplied by the caller.
Tensor expand_segments(const Tensor& starts, const Tensor& lens, int64_t total) {
  c10::cuda::OptionalCUDAGuard guard(starts.is_cuda() ? c10::make_optional(starts.device()) : c10::nullopt);
  Tensor out = at::empty({total}, starts.options().dtype(at::kLong));
  if (total == 0) return out;
  Tensor excl = at::cumsum(lens, 0) - lens;
  const int64_t* st = starts.data_ptr<int64_t>();
  const int64_t* ex = excl.data_ptr<int64_t>();
  int64_t nseg = starts.size(0);
  int64_t* o = out.data_ptr<int64_t>();
  for_each(starts.is_cuda(), total, [=] NVA_LAMBDA(int64_t t) {
    int64_t lo = 0, hi = nseg - 1;  // last segment with excl <= t
    while (lo < hi) {
      int64_t mid = (lo + hi + 1) >> 1;
      if (ex[mid] <= t) lo = mid; else hi = mid - 1;
    }
    o[t] = st[lo] + (t - ex[lo]);
  });
  return out;
}

// dst[dst_rows[k], :] = src[src_rows[k], :] as raw bytes; 16-byte vectors when rows allow it.
void copy_rows(const Tensor& src, const Tensor& src_rows, Tensor dst, const Tensor& dst_rows) {
  c10::cuda::OptionalCUDAGuard guard(src.is_cuda() ? c10::make_optional(src.device()) : c10::nullopt);
  TORCH_CHECK(src.scalar_type() == dst.scalar_type(), "copy_rows: dtype mismatch");
  NVA_CHECK_CONTIG(src); NVA_CHECK_CONTIG(dst);
  int64_t k = src_rows.size(0);
  if (k == 0) return;
  int64_t row_bytes = src.size(0) ? (int64_t)src.nbytes() / src.size(0) : 0;
  int64_t dst_row_bytes = dst.size(0) ? (int64_t)dst.nbytes() / dst.size(0) : 0;
  TORCH_CHECK(row_bytes == dst_row_bytes, "copy_rows: row size mismatch");
  if (row_bytes == 0) return;
  const char* s = (const char*)src.data_ptr();
  char* d = (char*)dst.data_ptr();
  const int64_t* sr = src_rows.data_ptr<int64_t>();
  const int64_t* dr = dst_rows.data_ptr<int64_t>();
  bool vec = row_bytes % 16 == 0 && ((uintptr_t)s % 16 == 0) && ((uintptr_t)d % 16 == 0);
  if (vec) {
    int64_t per = row_bytes / 16;
    for_each(src.is_cuda(), k * per, [=] NVA_LAMBDA(int64_t t) {
      int64_t r = t / per, c = t % per;
      ((int4*)(d + dr[r] * row_bytes))[c] = ((const int4*)(s + sr[r] * row_bytes))[c];
    });
  } else if (row_bytes % 4 == 0) {
    int64_t per = row_bytes / 4;
    for_each(src.is_cuda(), k * per, [=] NVA_LAMBDA(int64_t t) {
      int64_t r = t / per, c = t % per;
      ((int*)(d + dr[r] * row_bytes))[c] = ((const int*)(s + sr[r] * row_bytes))[c];
    });
  } else {
    for_each(src.is_cuda(), k * row_bytes, [=] NVA_LAMBDA(int64_t t) {
      int64_t r = t / row_bytes, c = t % row_bytes;
      d[dr[r] * row_bytes + c] = s[sr[r] * row_bytes + c];
    });
  }
}

}  // namespace nva

TORCH_LIBRARY_FRAGMENT(nvalchemi, m) {
  m.def("segmented_reduce(Tensor values, Tensor idx, int num_segments, int mode) -> Tensor", &nva::segmented_reduce);
  m.def("expand_segments(Tensor starts, Tensor lens, int total) -> Tensor", &nva::expand_segments);
  m.def("copy_rows(Tensor src, Tensor src_rows, Tensor(a!) dst, Tensor dst_rows) -> ()", &nva::copy_rows);
}
