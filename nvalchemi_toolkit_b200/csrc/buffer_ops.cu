// SPDX-License-Identifier: Apache-2.0
// Device-resident masked put / defragmentation of fixed-capacity buffers (inflight batching), with all counters kept on
// the device: nothing here reads a count back to the host.  Operator names and argument lists follow the reference's
// custom ops (nvalchemi/data/buffer_kernels.py:496-560, 960-1120, 1215-1741):
//   compute_put_fit_mask_per_system / _segmented, put_masked_per_system / _segmented, defrag_per_system / _segmented.
// Layouts: "per system" = one row per system (uniform level); "segmented" = rows of system s are
// [batch_ptr[s], batch_ptr[s+1]) (atoms, edges).  Rows are copied as raw bytes, so every dtype works.
//
// Each operator is a planning kernel (ONE block: masks -> ranks by a block-wide exclusive scan, slot assignment, counter
// updates) followed by a grid-wide row copy that reads the plan.  The CPU path runs the same plan serially.
#include "common.cuh"

namespace nva {
using at::Tensor;

namespace {
constexpr int kPlanThreads = 1024;

// Exclusive scan of flag(i), i in [0, n), by one block; out[i] = number of set flags before i; returns the total.
// `carry` and `tmp` are shared-memory scratch (tmp: blockDim ints).
template <typename F>
__device__ int block_exclusive_scan(int n, F flag, int* out, int* tmp) {
  __shared__ int carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < n; base += blockDim.x) {
    const int i = base + threadIdx.x;
    const int v = i < n ? flag(i) : 0;
    tmp[threadIdx.x] = v;
    __syncthreads();
    for (int o = 1; o < blockDim.x; o <<= 1) {  // Hillis-Steele inclusive scan
      const int add = threadIdx.x >= o ? tmp[threadIdx.x - o] : 0;
      __syncthreads();
      tmp[threadIdx.x] += add;
      __syncthreads();
    }
    if (i < n) out[i] = carry + tmp[threadIdx.x] - v;
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) carry += tmp[threadIdx.x];
    __syncthreads();
  }
  const int total = carry;
  __syncthreads();  // everyone has read the total before a later call resets it
  return total;
}

// ---- per-system (uniform) -------------------------------------------------------------------------------------
// plan[i] = destination slot of source row i, or -1.  Source rows flagged in src_mask go, in index order, to the empty
// destination slots (dest_mask false) in index order, as many as there are empty slots.
__global__ void plan_put_per_system_kernel(int n_src, int n_dst, const bool* __restrict__ src_mask,
                                           bool* __restrict__ dest_mask, bool* __restrict__ copied, int* __restrict__ plan,
                                           int* __restrict__ rank_src, int* __restrict__ rank_dst, int* __restrict__ slots,
                                           bool commit) {
  __shared__ int tmp[kPlanThreads];
  const int n_masked = block_exclusive_scan(n_src, [&](int i) { return src_mask[i] ? 1 : 0; }, rank_src, tmp);
  const int n_empty = block_exclusive_scan(n_dst, [&](int i) { return dest_mask[i] ? 0 : 1; }, rank_dst, tmp);
  (void)n_masked;
  for (int i = threadIdx.x; i < n_dst; i += blockDim.x)
    if (!dest_mask[i]) slots[rank_dst[i]] = i;  // r-th empty slot
  __syncthreads();
  for (int i = threadIdx.x; i < n_src; i += blockDim.x) {
    const bool go = src_mask[i] && rank_src[i] < n_empty;
    plan[i] = go ? slots[rank_src[i]] : -1;
    if (copied != nullptr) copied[i] = go;
  }
  __syncthreads();
  if (commit)
    for (int i = threadIdx.x; i < n_src; i += blockDim.x)
      if (plan[i] >= 0) dest_mask[plan[i]] = true;
}

__global__ void copy_planned_rows_kernel(int64_t n_src, int64_t row_bytes, int unit, const char* __restrict__ src,
                                         const int* __restrict__ plan, char* __restrict__ dst) {
  const int64_t per = row_bytes / unit;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < n_src * per; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = t / per, c = t - r * per;
    const int d = plan[r];
    if (d < 0) continue;
    const char* s = src + r * row_bytes + c * unit;
    char* o = dst + (int64_t)d * row_bytes + c * unit;
    if (unit == 16) *reinterpret_cast<int4*>(o) = *reinterpret_cast<const int4*>(s);
    else if (unit == 4) *reinterpret_cast<int*>(o) = *reinterpret_cast<const int*>(s);
    else *o = *s;
  }
}

inline int64_t row_bytes_of(const Tensor& t) { return t.size(0) ? (int64_t)t.nbytes() / t.size(0) : 0; }
inline int copy_unit(int64_t row_bytes, const void* a, const void* b) {
  const bool al16 = ((uintptr_t)a % 16 == 0) && ((uintptr_t)b % 16 == 0);
  const bool al4 = ((uintptr_t)a % 4 == 0) && ((uintptr_t)b % 4 == 0);
  return (row_bytes % 16 == 0 && al16) ? 16 : ((row_bytes % 4 == 0 && al4) ? 4 : 1);
}
inline void check_mask(const Tensor& m, const char* name) {
  TORCH_CHECK(m.scalar_type() == at::kBool && m.is_contiguous(), name, " must be a contiguous bool tensor");
}

// Serial statement of the per-system plan (CPU tensors).
void plan_put_per_system_cpu(int n_src, int n_dst, const bool* src_mask, bool* dest_mask, bool* copied, int* plan, bool commit) {
  int d = 0;
  for (int i = 0; i < n_src; ++i) {
    plan[i] = -1;
    if (src_mask[i]) {
      while (d < n_dst && dest_mask[d]) ++d;
      if (d < n_dst) { plan[i] = d; ++d; }
    }
    if (copied != nullptr) copied[i] = plan[i] >= 0;
  }
  if (commit)
    for (int i = 0; i < n_src; ++i)
      if (plan[i] >= 0) dest_mask[plan[i]] = true;
}

Tensor plan_per_system(const Tensor& source_mask, Tensor dest_mask, bool* copied, bool commit) {
  const int n_src = (int)source_mask.numel(), n_dst = (int)dest_mask.numel();
  Tensor plan = at::empty({n_src}, source_mask.options().dtype(at::kInt));
  if (n_src == 0) return plan;
  if (source_mask.is_cuda()) {
    Tensor scratch = at::empty({n_src + 2 * n_dst + 1}, plan.options());
    plan_put_per_system_kernel<<<1, kPlanThreads, 0, at::cuda::getCurrentCUDAStream()>>>(
        n_src, n_dst, source_mask.data_ptr<bool>(), dest_mask.data_ptr<bool>(), copied, plan.data_ptr<int>(),
        scratch.data_ptr<int>(), scratch.data_ptr<int>() + n_src, scratch.data_ptr<int>() + n_src + n_dst, commit);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  } else {
    plan_put_per_system_cpu(n_src, n_dst, source_mask.data_ptr<bool>(), dest_mask.data_ptr<bool>(), copied,
                            plan.data_ptr<int>(), commit);
  }
  return plan;
}

void copy_planned_rows(const Tensor& src, const Tensor& plan, Tensor dst, int64_t n_rows) {
  const int64_t rb = row_bytes_of(src);
  if (rb == 0 || n_rows == 0) return;
  TORCH_CHECK(rb == row_bytes_of(dst), "row sizes of source and destination differ");
  const int unit = copy_unit(rb, src.data_ptr(), dst.data_ptr());
  if (src.is_cuda()) {
    const int64_t work = n_rows * (rb / unit);
    const int64_t blocks = std::min<int64_t>((work + 255) / 256, 148 * 16);
    copy_planned_rows_kernel<<<(unsigned)blocks, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
        n_rows, rb, unit, (const char*)src.data_ptr(), plan.data_ptr<int>(), (char*)dst.data_ptr());
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  } else {
    const char* s = (const char*)src.data_ptr();
    char* d = (char*)dst.data_ptr();
    const int* pl = plan.data_ptr<int>();
    for (int64_t r = 0; r < n_rows; ++r)
      if (pl[r] >= 0) std::memcpy(d + (int64_t)pl[r] * rb, s + r * rb, (size_t)rb);
  }
}
}  // namespace

// fit_mask[i] = source_mask[i] and the i-th masked source row still finds an empty destination slot.
void compute_put_fit_mask_per_system(const Tensor& source_mask, const Tensor& dest_mask, Tensor fit_mask) {
  c10::cuda::OptionalCUDAGuard guard(source_mask.is_cuda() ? c10::make_optional(source_mask.device()) : c10::nullopt);
  check_mask(source_mask, "source_mask"); check_mask(dest_mask, "dest_mask"); check_mask(fit_mask, "fit_mask");
  TORCH_CHECK(fit_mask.numel() >= source_mask.numel(), "fit_mask is shorter than source_mask");
  plan_per_system(source_mask, dest_mask, fit_mask.data_ptr<bool>(), /*commit=*/false);
}

// Copies the rows of `source` flagged in `source_mask` into the first empty rows of `dest` (dest_mask false), marks
// those rows occupied and records in source_data_copied which source rows went.
void put_masked_per_system(const Tensor& source, const Tensor& source_mask, Tensor dest, Tensor dest_mask,
                           Tensor source_data_copied) {
  c10::cuda::OptionalCUDAGuard guard(source.is_cuda() ? c10::make_optional(source.device()) : c10::nullopt);
  check_mask(source_mask, "source_mask"); check_mask(dest_mask, "dest_mask"); check_mask(source_data_copied, "source_data_copied");
  NVA_CHECK_CONTIG(source); NVA_CHECK_CONTIG(dest);
  TORCH_CHECK(source.scalar_type() == dest.scalar_type(), "put_masked_per_system: dtype mismatch");
  TORCH_CHECK(source_mask.numel() <= source.size(0) && dest_mask.numel() <= dest.size(0) &&
                  source_data_copied.numel() >= source_mask.numel(), "put_masked_per_system: masks do not match the buffers");
  Tensor plan = plan_per_system(source_mask, dest_mask, source_data_copied.data_ptr<bool>(), /*commit=*/true);
  copy_planned_rows(source, plan, dest, source_mask.numel());
}

// Keeps the rows not flagged in source_data_copied, moved to the front in their order; the vacated tail is zeroed and the
// flags are cleared.  (The compaction goes through a zero-initialised scratch copy, so no row count is needed on the host.)
void defrag_per_system(Tensor source, Tensor source_data_copied) {
  c10::cuda::OptionalCUDAGuard guard(source.is_cuda() ? c10::make_optional(source.device()) : c10::nullopt);
  check_mask(source_data_copied, "source_data_copied");
  NVA_CHECK_CONTIG(source);
  const int64_t n = source_data_copied.numel();
  TORCH_CHECK(n <= source.size(0), "defrag_per_system: mask longer than the buffer");
  if (n == 0) return;
  Tensor keep = source_data_copied.logical_not();
  Tensor all_empty = at::zeros({n}, keep.options());
  Tensor plan = plan_per_system(keep, all_empty, nullptr, /*commit=*/false);  // kept row i -> slot rank(i)
  Tensor head = source.narrow(0, 0, n);
  Tensor tmp = at::zeros_like(head);
  copy_planned_rows(head, plan, tmp, n);
  head.copy_(tmp);
  source_data_copied.zero_();
}

namespace {
// ---- segmented ------------------------------------------------------------------------------------------------
// One block.  mode 0: fit mask only; mode 1: put (append the flagged segments that fit behind segment n_dst of the
// destination, extend dest_ptr, write the new segment count); mode 2: defrag (keep the segments NOT flagged, rebuild ptr).
// seg_plan[i] = first destination row of source segment i, or -1.
__global__ void plan_segmented_kernel(int mode, int n_src, const int* __restrict__ src_ptr, const bool* __restrict__ flag,
                                      int* __restrict__ dst_ptr, int n_dst_in, const int* __restrict__ n_dst_dev,
                                      int dest_capacity, int max_segments, bool* __restrict__ out_mask,
                                      int* __restrict__ seg_plan, int* __restrict__ new_count, int* __restrict__ s_off,
                                      int* __restrict__ s_rank, int* __restrict__ s_len) {
  __shared__ int tmp[kPlanThreads];
  const int n_dst = mode == 2 ? 0 : (n_dst_dev != nullptr ? n_dst_dev[0] : n_dst_in);
  const int dest_end = mode == 2 ? 0 : dst_ptr[n_dst];
  for (int i = threadIdx.x; i < n_src; i += blockDim.x) {
    const bool take = mode == 2 ? !flag[i] : flag[i];
    s_len[i] = take ? src_ptr[i + 1] - src_ptr[i] : -1;  // -1: not a candidate
  }
  __syncthreads();
  for (int pass = 0; pass < (mode == 2 ? 1 : 2); ++pass) {
    block_exclusive_scan(n_src, [&](int i) { return s_len[i] > 0 ? s_len[i] : 0; }, s_off, tmp);
    block_exclusive_scan(n_src, [&](int i) { return s_len[i] >= 0 ? 1 : 0; }, s_rank, tmp);
    if (mode != 2) {  // candidates that do not fit drop out; the second pass re-packs the survivors without holes
      for (int i = threadIdx.x; i < n_src; i += blockDim.x)
        if (s_len[i] >= 0 && (dest_end + s_off[i] + s_len[i] > dest_capacity || n_dst + s_rank[i] >= max_segments)) s_len[i] = -1;
      __syncthreads();
    }
  }
  const int total_len = block_exclusive_scan(n_src, [&](int i) { return s_len[i] > 0 ? s_len[i] : 0; }, s_off, tmp);
  const int total = block_exclusive_scan(n_src, [&](int i) { return s_len[i] >= 0 ? 1 : 0; }, s_rank, tmp);
  for (int i = threadIdx.x; i < n_src; i += blockDim.x) {
    const bool go = s_len[i] >= 0;
    if (out_mask != nullptr) out_mask[i] = mode == 2 ? false : go;
    if (seg_plan != nullptr) seg_plan[i] = go ? dest_end + s_off[i] : -1;
  }
  if (mode == 0) return;
  __syncthreads();  // every read of the old pointers is done
  if (mode == 1) {
    for (int i = threadIdx.x; i < n_src; i += blockDim.x)
      if (s_len[i] >= 0) dst_ptr[n_dst + s_rank[i] + 1] = dest_end + s_off[i] + s_len[i];
    if (threadIdx.x == 0) new_count[0] = n_dst + total;
  } else {
    for (int i = threadIdx.x; i < n_src; i += blockDim.x) {
      if (s_len[i] >= 0) dst_ptr[s_rank[i] + 1] = s_off[i] + s_len[i];
    }
    __syncthreads();
    for (int k = total + 1 + threadIdx.x; k <= n_src; k += blockDim.x) dst_ptr[k] = total_len;  // empty tail segments
    if (threadIdx.x == 0) { dst_ptr[0] = 0; new_count[0] = total; }
  }
}

// Copies whole segments: block b handles source segments b, b + gridDim.x, ...
__global__ void copy_segments_kernel(int n_src, int64_t row_bytes, int unit, const int* __restrict__ src_ptr,
                                     const int* __restrict__ seg_plan, const char* __restrict__ src, char* __restrict__ dst) {
  for (int s = blockIdx.x; s < n_src; s += gridDim.x) {
    const int d0 = seg_plan[s];
    if (d0 < 0) continue;
    const int r0 = src_ptr[s], r1 = src_ptr[s + 1];
    const int64_t n_units = (int64_t)(r1 - r0) * row_bytes / unit;
    const char* sp = src + (int64_t)r0 * row_bytes;
    char* dp = dst + (int64_t)d0 * row_bytes;
    for (int64_t t = threadIdx.x; t < n_units; t += blockDim.x) {
      if (unit == 16) reinterpret_cast<int4*>(dp)[t] = reinterpret_cast<const int4*>(sp)[t];
      else if (unit == 4) reinterpret_cast<int*>(dp)[t] = reinterpret_cast<const int*>(sp)[t];
      else dp[t] = sp[t];
    }
  }
}
}  // namespace

namespace {
// Serial statement of plan_segmented_kernel (CPU tensors).
void plan_segmented_cpu(int mode, int n_src, const int* src_ptr_in, const bool* flag, int* dst_ptr, int n_dst, int dest_capacity,
                        int max_segments, bool* out_mask, int* seg_plan, int* new_count) {
  std::vector<int> src_ptr(src_ptr_in, src_ptr_in + n_src + 1);  // dst_ptr may alias src_ptr (defrag)
  const int dest_end = mode == 2 ? 0 : dst_ptr[n_dst];
  std::vector<int> len(n_src);
  for (int i = 0; i < n_src; ++i) len[i] = (mode == 2 ? !flag[i] : flag[i]) ? src_ptr[i + 1] - src_ptr[i] : -1;
  if (mode != 2)
    for (int pass = 0; pass < 2; ++pass) {
      int off = 0, rank = 0;
      for (int i = 0; i < n_src; ++i) {
        if (len[i] < 0) continue;
        const int o = off, r = rank;
        off += len[i]; ++rank;  // offsets count every candidate of this pass, like the parallel scan
        if (dest_end + o + len[i] > dest_capacity || n_dst + r >= max_segments) len[i] = -1;
      }
    }
  int off = 0, rank = 0;
  for (int i = 0; i < n_src; ++i) {
    const bool go = len[i] >= 0;
    if (out_mask != nullptr) out_mask[i] = mode == 2 ? false : go;
    if (seg_plan != nullptr) seg_plan[i] = go ? dest_end + off : -1;
    if (go) {
      if (mode == 1) dst_ptr[n_dst + rank + 1] = dest_end + off + len[i];
      if (mode == 2) dst_ptr[rank + 1] = off + len[i];
      off += len[i]; ++rank;
    }
  }
  if (mode == 1) new_count[0] = n_dst + rank;
  if (mode == 2) {
    for (int k = rank + 1; k <= n_src; ++k) dst_ptr[k] = off;
    dst_ptr[0] = 0;
    new_count[0] = rank;
  }
}

void check_ptr(const Tensor& p, const char* name) {
  TORCH_CHECK(p.scalar_type() == at::kInt && p.is_contiguous() && p.dim() == 1, name, " must be a contiguous int32 vector");
}

// Runs the plan; returns seg_plan (first destination row per source segment or -1).
Tensor run_segmented_plan(int mode, const Tensor& src_ptr, const Tensor& flag, Tensor dst_ptr, int64_t n_dst,
                          const Tensor* n_dst_dev, int64_t dest_capacity, bool* out_mask, int* new_count) {
  const int n_src = (int)src_ptr.numel() - 1;
  const int max_segments = (int)dst_ptr.numel() - 1;
  Tensor seg_plan = at::empty({std::max(n_src, 0)}, src_ptr.options());
  if (n_src <= 0) return seg_plan;
  if (src_ptr.is_cuda()) {
    Tensor scratch = at::empty({3 * (int64_t)n_src}, src_ptr.options());
    int* sp = scratch.data_ptr<int>();
    plan_segmented_kernel<<<1, kPlanThreads, 0, at::cuda::getCurrentCUDAStream()>>>(
        mode, n_src, src_ptr.data_ptr<int>(), flag.data_ptr<bool>(), dst_ptr.data_ptr<int>(), (int)n_dst,
        n_dst_dev != nullptr ? n_dst_dev->data_ptr<int>() : nullptr, (int)dest_capacity, max_segments, out_mask,
        seg_plan.data_ptr<int>(), new_count, sp, sp + n_src, sp + 2 * n_src);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  } else {
    const int nd = n_dst_dev != nullptr ? n_dst_dev->data_ptr<int>()[0] : (int)n_dst;
    plan_segmented_cpu(mode, n_src, src_ptr.data_ptr<int>(), flag.data_ptr<bool>(), dst_ptr.data_ptr<int>(), nd,
                       (int)dest_capacity, max_segments, out_mask, seg_plan.data_ptr<int>(), new_count);
  }
  return seg_plan;
}

void copy_segments(const Tensor& src, const Tensor& src_ptr, const Tensor& seg_plan, Tensor dst) {
  const int64_t rb = row_bytes_of(src);
  const int n_src = (int)seg_plan.numel();
  if (rb == 0 || n_src == 0) return;
  TORCH_CHECK(dst.size(0) == 0 || rb == row_bytes_of(dst), "row sizes of source and destination differ");
  const int unit = copy_unit(rb, src.data_ptr(), dst.data_ptr());
  if (src.is_cuda()) {
    copy_segments_kernel<<<std::min(n_src, 148 * 8), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
        n_src, rb, unit, src_ptr.data_ptr<int>(), seg_plan.data_ptr<int>(), (const char*)src.data_ptr(), (char*)dst.data_ptr());
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  } else {
    const int* sp = src_ptr.data_ptr<int>();
    const int* pl = seg_plan.data_ptr<int>();
    for (int s = 0; s < n_src; ++s)
      if (pl[s] >= 0)
        std::memcpy((char*)dst.data_ptr() + (int64_t)pl[s] * rb, (const char*)src.data_ptr() + (int64_t)sp[s] * rb,
                    (size_t)((int64_t)(sp[s + 1] - sp[s]) * rb));
  }
}
}  // namespace

// fit_mask[s] = source segment s is flagged and still fits behind the `num_dest_segments` segments of the destination
// (row capacity `dest_capacity`, segment capacity dest_batch_ptr.numel() - 1), segments considered in index order.
void compute_put_fit_mask_segmented(const Tensor& source_batch_ptr, const Tensor& source_mask, const Tensor& dest_batch_ptr,
                                    int64_t num_dest_segments, int64_t dest_capacity, Tensor fit_mask) {
  c10::cuda::OptionalCUDAGuard guard(source_mask.is_cuda() ? c10::make_optional(source_mask.device()) : c10::nullopt);
  check_ptr(source_batch_ptr, "source_batch_ptr"); check_ptr(dest_batch_ptr, "dest_batch_ptr");
  check_mask(source_mask, "source_mask"); check_mask(fit_mask, "fit_mask");
  TORCH_CHECK(source_mask.numel() >= source_batch_ptr.numel() - 1 && fit_mask.numel() >= source_batch_ptr.numel() - 1,
              "masks are shorter than the number of source segments");
  run_segmented_plan(0, source_batch_ptr, source_mask, dest_batch_ptr, num_dest_segments, nullptr, dest_capacity,
                     fit_mask.data_ptr<bool>(), nullptr);
}

// Appends the flagged source segments that fit to the destination: rows are copied behind row
// dest_batch_ptr[num_dest_segments], dest_batch_ptr is extended, new_num_dest[0] receives the new segment count and
// source_data_copied which segments went.  num_dest_segments < 0 reads the current count from new_num_dest[0] (a counter
// that lives on the device, so consecutive puts need no host round trip).
void put_masked_segmented(const Tensor& source, const Tensor& source_batch_ptr, const Tensor& source_mask, Tensor dest,
                          Tensor dest_batch_ptr, Tensor source_data_copied, Tensor new_num_dest, int64_t num_dest_segments) {
  c10::cuda::OptionalCUDAGuard guard(source.is_cuda() ? c10::make_optional(source.device()) : c10::nullopt);
  check_ptr(source_batch_ptr, "source_batch_ptr"); check_ptr(dest_batch_ptr, "dest_batch_ptr");
  check_mask(source_mask, "source_mask"); check_mask(source_data_copied, "source_data_copied");
  NVA_CHECK_CONTIG(source); NVA_CHECK_CONTIG(dest);
  TORCH_CHECK(source.scalar_type() == dest.scalar_type(), "put_masked_segmented: dtype mismatch");
  TORCH_CHECK(new_num_dest.scalar_type() == at::kInt && new_num_dest.numel() >= 1, "new_num_dest must be an int32 tensor");
  TORCH_CHECK(source_mask.numel() >= source_batch_ptr.numel() - 1 && source_data_copied.numel() >= source_batch_ptr.numel() - 1,
              "masks are shorter than the number of source segments");
  Tensor plan = run_segmented_plan(1, source_batch_ptr, source_mask, dest_batch_ptr, num_dest_segments,
                                   num_dest_segments < 0 ? &new_num_dest : nullptr, dest.size(0),
                                   source_data_copied.data_ptr<bool>(), new_num_dest.data_ptr<int>());
  copy_segments(source, source_batch_ptr, plan, dest);
}

// Removes the segments flagged in source_data_copied: the kept segments move to the front in their order,
// source_batch_ptr is rebuilt (trailing entries = total kept rows), num_kept[0] receives the number of kept segments,
// vacated rows are zeroed and the flags cleared.  `temp` is scratch of the same shape as `source`.
void defrag_segmented(Tensor source, Tensor source_batch_ptr, Tensor source_data_copied, Tensor temp, Tensor num_kept) {
  c10::cuda::OptionalCUDAGuard guard(source.is_cuda() ? c10::make_optional(source.device()) : c10::nullopt);
  check_ptr(source_batch_ptr, "source_batch_ptr"); check_mask(source_data_copied, "source_data_copied");
  NVA_CHECK_CONTIG(source); NVA_CHECK_CONTIG(temp);
  TORCH_CHECK(temp.nbytes() >= source.nbytes() && temp.scalar_type() == source.scalar_type(), "temp must match source");
  TORCH_CHECK(num_kept.scalar_type() == at::kInt && num_kept.numel() >= 1, "num_kept must be an int32 tensor");
  TORCH_CHECK(source_data_copied.numel() >= source_batch_ptr.numel() - 1, "mask shorter than the number of segments");
  Tensor old_ptr = source_batch_ptr.clone();
  Tensor plan = run_segmented_plan(2, old_ptr, source_data_copied, source_batch_ptr, 0, nullptr, source.size(0),
                                   source_data_copied.data_ptr<bool>(), num_kept.data_ptr<int>());
  temp.zero_();
  copy_segments(source, old_ptr, plan, temp);
  source.copy_(temp.view_as(source));
}

// ---- plan once, copy many ---------------------------------------------------------------------------------------
// A buffer holds several arrays per level (positions, velocities, ...) that share one pointer array, so the container
// plans a put / defrag ONCE and then moves every array with the same plan.  `count` is the device-resident number of live
// segments of the destination (read and updated in place); no value returns to the host.
// Returns plan[s] = first destination row of source segment s, or -1; `copied[s]` says whether segment s goes.  With
// commit = false nothing is written but `copied` (the fit mask against the device-resident count).
Tensor segmented_put_plan(const Tensor& source_batch_ptr, const Tensor& source_mask, Tensor dest_batch_ptr, Tensor count,
                          int64_t dest_capacity, Tensor copied, bool commit) {
  c10::cuda::OptionalCUDAGuard guard(source_mask.is_cuda() ? c10::make_optional(source_mask.device()) : c10::nullopt);
  check_ptr(source_batch_ptr, "source_batch_ptr"); check_ptr(dest_batch_ptr, "dest_batch_ptr");
  check_mask(source_mask, "source_mask"); check_mask(copied, "copied");
  TORCH_CHECK(count.scalar_type() == at::kInt && count.numel() >= 1, "count must be an int32 tensor");
  TORCH_CHECK(source_mask.numel() >= source_batch_ptr.numel() - 1 && copied.numel() >= source_batch_ptr.numel() - 1,
              "masks are shorter than the number of source segments");
  return run_segmented_plan(commit ? 1 : 0, source_batch_ptr, source_mask, dest_batch_ptr, -1, &count, dest_capacity,
                            copied.data_ptr<bool>(), count.data_ptr<int>());
}

// Keeps the segments NOT flagged in `removed`; batch_ptr (the live prefix, n + 1 entries) is rebuilt in place and
// count[0] receives the number kept.  Returns (plan, old batch_ptr) for segmented_copy_planned.
std::tuple<Tensor, Tensor> segmented_defrag_plan(Tensor batch_ptr, const Tensor& removed, Tensor count) {
  c10::cuda::OptionalCUDAGuard guard(removed.is_cuda() ? c10::make_optional(removed.device()) : c10::nullopt);
  check_ptr(batch_ptr, "batch_ptr"); check_mask(removed, "removed");
  TORCH_CHECK(count.scalar_type() == at::kInt && count.numel() >= 1, "count must be an int32 tensor");
  TORCH_CHECK(removed.numel() >= batch_ptr.numel() - 1, "mask shorter than the number of segments");
  Tensor old_ptr = batch_ptr.clone();
  Tensor plan = run_segmented_plan(2, old_ptr, removed, batch_ptr, 0, nullptr, 0, nullptr, count.data_ptr<int>());
  return std::make_tuple(plan, old_ptr);
}

// dest rows [plan[s], plan[s] + len(s)) <- source rows of segment s, for every s with plan[s] >= 0.  Source and
// destination must not overlap (a defrag goes through a scratch array).
void segmented_copy_planned(const Tensor& source, const Tensor& source_batch_ptr, const Tensor& plan, Tensor dest) {
  c10::cuda::OptionalCUDAGuard guard(source.is_cuda() ? c10::make_optional(source.device()) : c10::nullopt);
  check_ptr(source_batch_ptr, "source_batch_ptr");
  NVA_CHECK_CONTIG(source); NVA_CHECK_CONTIG(dest);
  TORCH_CHECK(source.scalar_type() == dest.scalar_type(), "segmented_copy_planned: dtype mismatch");
  TORCH_CHECK(plan.scalar_type() == at::kInt && plan.numel() <= source_batch_ptr.numel() - 1, "plan does not match source_batch_ptr");
  copy_segments(source, source_batch_ptr, plan, dest);
}

}  // namespace nva

TORCH_LIBRARY_FRAGMENT(nvalchemi, m) {
  m.def("compute_put_fit_mask_per_system(Tensor source_mask, Tensor dest_mask, Tensor(a!) fit_mask) -> ()", torch::dispatch(c10::DispatchKey::CompositeExplicitAutograd, &nva::compute_put_fit_mask_per_system));
  m.def("put_masked_per_system(Tensor source, Tensor source_mask, Tensor(a!) dest, Tensor(b!) dest_mask, Tensor(c!) source_data_copied) -> ()", torch::dispatch(c10::DispatchKey::CompositeExplicitAutograd, &nva::put_masked_per_system));
  m.def("defrag_per_system(Tensor(a!) source, Tensor(b!) source_data_copied) -> ()", torch::dispatch(c10::DispatchKey::CompositeExplicitAutograd, &nva::defrag_per_system));
  m.def("compute_put_fit_mask_segmented(Tensor source_batch_ptr, Tensor source_mask, Tensor dest_batch_ptr, int num_dest_segments, int dest_capacity, Tensor(a!) fit_mask) -> ()", torch::dispatch(c10::DispatchKey::CompositeExplicitAutograd, &nva::compute_put_fit_mask_segmented));
  m.def("put_masked_segmented(Tensor source, Tensor source_batch_ptr, Tensor source_mask, Tensor(a!) dest, Tensor(b!) dest_batch_ptr, Tensor(c!) source_data_copied, Tensor(d!) new_num_dest, int num_dest_segments) -> ()", torch::dispatch(c10::DispatchKey::CompositeExplicitAutograd, &nva::put_masked_segmented));
  m.def("defrag_segmented(Tensor(a!) source, Tensor(b!) source_batch_ptr, Tensor(c!) source_data_copied, Tensor(d!) temp, Tensor(e!) num_kept) -> ()", torch::dispatch(c10::DispatchKey::CompositeExplicitAutograd, &nva::defrag_segmented));
  m.def("segmented_put_plan(Tensor source_batch_ptr, Tensor source_mask, Tensor(a!) dest_batch_ptr, Tensor(b!) count, int dest_capacity, Tensor(c!) copied, bool commit=True) -> Tensor", torch::dispatch(c10::DispatchKey::CompositeExplicitAutograd, &nva::segmented_put_plan));
  m.def("segmented_defrag_plan(Tensor(a!) batch_ptr, Tensor removed, Tensor(b!) count) -> (Tensor, Tensor)", torch::dispatch(c10::DispatchKey::CompositeExplicitAutograd, &nva::segmented_defrag_plan));
  m.def("segmented_copy_planned(Tensor source, Tensor source_batch_ptr, Tensor plan, Tensor(a!) dest) -> ()", torch::dispatch(c10::DispatchKey::CompositeExplicitAutograd, &nva::segmented_copy_planned));
}
