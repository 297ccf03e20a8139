// SPDX-License-Identifier: Apache-2.0
// Peer-to-peer communication kernels over NVLink (symmetric buffers mapped into every rank):
//   * p2p_barrier      - flag exchange between ranks with a bounded wait (status word on expiry);
//   * halo_push_rows   - packs boundary rows (+ periodic image shift) and stores them straight into the
//                        peers' ghost rows (replaces the count all_gather + all_to_all_v of the reference's
//                        halo build, nvalchemi/distributed/_core/particle_halo.py:279-368);
//   * p2p_allreduce    - one-shot sum over all ranks' symmetric buffers with a fused scale (gradient
//                        all-reduce with the loss-scale division and cast folded in; reference: PyTorch DDP
//                        bucketed NCCL all-reduce, nvalchemi/training/hooks/ddp.py:277-301).
// Peer memory is only ever touched with plain ld/st/red instructions issued by these kernels.
#include "common.cuh"

namespace nva {
using at::Tensor;

// One block, `world` threads.  Thread t publishes `epoch` into rank t's flag row (slot = my rank) and then
// waits until rank t's publication shows up in my own row.  All earlier device-side writes of this rank to
// peer memory are ordered before the flag by the system-scope fence.
__global__ void p2p_barrier_kernel(const int64_t* __restrict__ flag_ptrs, int rank, int world, int epoch,
                                   int* __restrict__ err) {
  int t = threadIdx.x;
  __threadfence_system();
  __syncthreads();
  if (t < world) {
    volatile int* peer = reinterpret_cast<volatile int*>(flag_ptrs[t]);
    peer[rank] = epoch;
    __threadfence_system();
    volatile int* mine = reinterpret_cast<volatile int*>(flag_ptrs[rank]);
    bool ok = false;
    for (int it = 0; it < 4000000; ++it) {  // ~1 s at 250 ns per probe
      if (mine[t] >= epoch) { ok = true; break; }
      __nanosleep(250);
    }
    if (!ok) atomicExch(err, 100 + t);
  }
  __threadfence_system();
}

void p2p_barrier(const Tensor& flag_ptrs, int64_t rank, int64_t world, int64_t epoch, Tensor err) {
  c10::cuda::CUDAGuard guard(flag_ptrs.device());
  TORCH_CHECK(world <= 32, "p2p_barrier supports up to 32 ranks");
  p2p_barrier_kernel<<<1, 32, 0, at::cuda::getCurrentCUDAStream()>>>(flag_ptrs.data_ptr<int64_t>(), (int)rank, (int)world,
                                                                     (int)epoch, err.data_ptr<int>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// dst_r[dst_row[k], :] = src[idx[k], :] (+ shift[k, :]) with dst_r = base pointer of rank peer[k].
__global__ void halo_push_kernel(int64_t n_send, int D, const float* __restrict__ src, const int* __restrict__ idx,
                                 const int* __restrict__ dst_row, const int* __restrict__ peer,
                                 const float* __restrict__ shift, const int64_t* __restrict__ dst_ptrs) {
  int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (t >= n_send * D) return;
  int64_t k = t / D;
  int d = (int)(t - k * D);
  float v = src[(int64_t)idx[k] * D + d];
  if (shift != nullptr) v += shift[k * D + d];
  float* dst = reinterpret_cast<float*>(dst_ptrs[peer[k]]);
  dst[(int64_t)dst_row[k] * D + d] = v;
}

void halo_push_rows(const Tensor& src, const Tensor& idx, const Tensor& dst_row, const Tensor& peer,
                    const c10::optional<Tensor>& shift, const Tensor& dst_ptrs) {
  c10::cuda::CUDAGuard guard(src.device());
  NVA_CHECK_CONTIG(src);
  int64_t n = idx.size(0);
  if (n == 0) return;
  int D = (int)(src.numel() / src.size(0));
  int64_t total = n * D;
  halo_push_kernel<<<(unsigned)((total + 255) / 256), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      n, D, src.data_ptr<float>(), idx.data_ptr<int>(), dst_row.data_ptr<int>(), peer.data_ptr<int>(),
      shift.has_value() ? shift->data_ptr<float>() : nullptr, dst_ptrs.data_ptr<int64_t>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// out[i] = scale * sum_r buf_r[i]; every rank reads all peers in rank order (one-shot all-reduce; sized for the
// latency-bound few-MB gradient buckets of MLIP training and for the float64 structure-factor / charge-mesh sums of the
// Ewald and particle-mesh models: the sum order is fixed, so every rank obtains bitwise the same result).
// 16-byte vector path (V = 4 floats or 2 doubles) when the element range allows.
template <typename T, int V>
__global__ void p2p_allreduce_kernel(int64_t n, const int64_t* __restrict__ buf_ptrs, int world, T scale, T* __restrict__ out) {
  struct alignas(16) Vec { T v[V]; };
  int64_t i = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) * V;
  if (i >= n) return;
  if (i + V <= n) {
    Vec acc;
#pragma unroll
    for (int c = 0; c < V; ++c) acc.v[c] = T(0);
    for (int r = 0; r < world; ++r) {
      Vec x = *reinterpret_cast<const Vec*>(reinterpret_cast<const T*>(buf_ptrs[r]) + i);
#pragma unroll
      for (int c = 0; c < V; ++c) acc.v[c] += x.v[c];
    }
#pragma unroll
    for (int c = 0; c < V; ++c) acc.v[c] *= scale;
    *reinterpret_cast<Vec*>(out + i) = acc;
  } else {
    for (int64_t k = i; k < n; ++k) {
      T acc = T(0);
      for (int r = 0; r < world; ++r) acc += reinterpret_cast<const T*>(buf_ptrs[r])[k];
      out[k] = acc * scale;
    }
  }
}

void p2p_allreduce(const Tensor& buf_ptrs, int64_t world, double scale, Tensor out) {
  c10::cuda::CUDAGuard guard(out.device());
  int64_t n = out.numel();
  if (n == 0) return;
  TORCH_CHECK(out.is_contiguous(), "p2p_allreduce: output must be contiguous");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(out.data_ptr()) & 15) == 0, "p2p_allreduce: output must be 16-byte aligned");
  TORCH_CHECK(buf_ptrs.numel() >= world, "p2p_allreduce: address table shorter than the world size");
  auto stream = at::cuda::getCurrentCUDAStream();
  if (out.scalar_type() == at::kDouble) {
    int64_t threads = (n + 1) / 2;
    p2p_allreduce_kernel<double, 2><<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(
        n, buf_ptrs.data_ptr<int64_t>(), (int)world, scale, out.data_ptr<double>());
  } else {
    TORCH_CHECK(out.scalar_type() == at::kFloat, "p2p_allreduce: float32 or float64 buffers");
    int64_t threads = (n + 3) / 4;
    p2p_allreduce_kernel<float, 4><<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(
        n, buf_ptrs.data_ptr<int64_t>(), (int)world, (float)scale, out.data_ptr<float>());
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// Small all-reduce in ONE launch (push form).  Block b owns elements [b * chunk, (b + 1) * chunk): it stores its chunk
// into slot `rank` of EVERY rank's scratch region (remote stores, nothing waits for them), publishes `epoch` in flag
// (b, rank) of every rank, waits (bounded) until the flags (b, r) of all ranks r have arrived in its own flag row, and
// then adds the `world` slots of its LOCAL scratch region in rank order.  Blocks never wait for other blocks of the same
// GPU, only for the block with the same index on the peers, and every block publishes before it waits, so no launch
// order can deadlock.  Two slot sets alternate with the parity of `epoch`: a rank can start call k + 2 (same parity as
// k) only after every peer has entered call k + 1, i.e. after it finished reading the slots of call k, so no closing
// rendezvous is needed.  Layout of a scratch region: [parity][rank][slot_elems]; of a flag row: [block][rank].
constexpr int kPushBlocks = 16;
constexpr int kPushThreads = 512;

template <typename T>
__global__ void p2p_allreduce_push_kernel(const T* src, T* out, int64_t n, int64_t chunk,  // src may alias out
                                          const int64_t* __restrict__ scratch_ptrs, int64_t slot_elems,
                                          const int64_t* __restrict__ flag_ptrs, int rank, int world, int epoch, T scale,
                                          int* __restrict__ err) {
  __shared__ int s_ok;
  const int b = blockIdx.x, t = threadIdx.x;
  const int64_t lo = (int64_t)b * chunk;
  const int64_t hi = lo + chunk < n ? lo + chunk : n;
  const int64_t set = (int64_t)(epoch & 1) * world;
  if (t == 0) s_ok = 1;
  for (int r = 0; r < world; ++r) {
    T* dst = reinterpret_cast<T*>(scratch_ptrs[r]) + (set + rank) * slot_elems;
    for (int64_t i = lo + t; i < hi; i += kPushThreads) dst[i] = src[i];
  }
  __threadfence_system();
  __syncthreads();
  if (t < world) {
    volatile int* peer = reinterpret_cast<volatile int*>(flag_ptrs[t]);
    peer[b * 32 + rank] = epoch;
    volatile int* mine = reinterpret_cast<volatile int*>(flag_ptrs[rank]);
    bool ok = false;
    for (int it = 0; it < 4000000; ++it) {  // about a second
      if (mine[b * 32 + t] >= epoch) { ok = true; break; }
      __nanosleep(250);
    }
    if (!ok) { atomicExch(err, 100 + t); s_ok = 0; }
    __threadfence_system();
  }
  __syncthreads();
  if (!s_ok) return;  // a peer never arrived: the status word says which; the output is left untouched
  const volatile T* base = reinterpret_cast<const volatile T*>(scratch_ptrs[rank]) + set * slot_elems;
  for (int64_t i = lo + t; i < hi; i += kPushThreads) {
    T acc = T(0);
    for (int r = 0; r < world; ++r) acc += base[r * slot_elems + i];
    out[i] = acc * scale;
  }
}

void p2p_allreduce_push(const Tensor& src, const Tensor& scratch_ptrs, int64_t slot_elems, const Tensor& flag_ptrs, int64_t rank,
                        int64_t world, int64_t epoch, double scale, Tensor err, Tensor out) {
  c10::cuda::CUDAGuard guard(src.device());
  NVA_CHECK_CONTIG(src);
  NVA_CHECK_CONTIG(out);
  const int64_t n = src.numel();
  if (n == 0) return;
  TORCH_CHECK(out.numel() == n && out.scalar_type() == src.scalar_type(), "p2p_allreduce_push: out must match src");
  TORCH_CHECK(n <= slot_elems, "p2p_allreduce_push: ", n, " elements exceed the slot size ", slot_elems);
  TORCH_CHECK(world >= 1 && world <= 32 && rank >= 0 && rank < world, "p2p_allreduce_push: up to 32 ranks");
  TORCH_CHECK(scratch_ptrs.numel() >= world && flag_ptrs.numel() >= world, "p2p_allreduce_push: address tables shorter than the world size");
  int blocks = (int)((n + 511) / 512);  // one element per thread up to 16 blocks: the latency of the remote stores is spread
  blocks = blocks < 1 ? 1 : (blocks > kPushBlocks ? kPushBlocks : blocks);
  const int64_t chunk = (n + blocks - 1) / blocks;
  auto stream = at::cuda::getCurrentCUDAStream();
  if (src.scalar_type() == at::kDouble) {
    p2p_allreduce_push_kernel<double><<<blocks, kPushThreads, 0, stream>>>(
        src.data_ptr<double>(), out.data_ptr<double>(), n, chunk, scratch_ptrs.data_ptr<int64_t>(), slot_elems,
        flag_ptrs.data_ptr<int64_t>(), (int)rank, (int)world, (int)epoch, scale, err.data_ptr<int>());
  } else {
    TORCH_CHECK(src.scalar_type() == at::kFloat, "p2p_allreduce_push: float32 or float64 tensors");
    p2p_allreduce_push_kernel<float><<<blocks, kPushThreads, 0, stream>>>(
        src.data_ptr<float>(), out.data_ptr<float>(), n, chunk, scratch_ptrs.data_ptr<int64_t>(), slot_elems,
        flag_ptrs.data_ptr<int64_t>(), (int)rank, (int)world, (int)epoch, (float)scale, err.data_ptr<int>());
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

}  // namespace nva

TORCH_LIBRARY_FRAGMENT(nvalchemi, m) {
  m.def("p2p_barrier(Tensor flag_ptrs, int rank, int world, int epoch, Tensor(a!) err) -> ()", &nva::p2p_barrier);
  m.def("halo_push_rows(Tensor src, Tensor idx, Tensor dst_row, Tensor peer, Tensor? shift, Tensor dst_ptrs) -> ()", &nva::halo_push_rows);
  m.def("p2p_allreduce(Tensor buf_ptrs, int world, float scale, Tensor(a!) out) -> ()", &nva::p2p_allreduce);
  m.def("p2p_allreduce_push(Tensor src, Tensor scratch_ptrs, int slot_elems, Tensor flag_ptrs, int rank, int world, int epoch, float scale, Tensor(a!) err, Tensor(b!) out) -> ()", &nva::p2p_allreduce_push);
}

namespace nva {
// Ghost refresh by pull: dst[row0 + g, :] = src_{home_rank[g]}[home_row[g], :] (+ shift[g, :]).  The consumer reads
// the owners' rows over NVLink; no send lists or counts have to be negotiated.  Rows whose width is a multiple of four
// floats move as 16-byte vectors, one warp per row with all of a lane's loads issued before its stores (a 512-float
// row keeps 2 KB in flight per warp); narrow rows (positions: three floats) take one thread per row.  `used` (optional,
// one byte per ghost) skips rows that no local edge references.
template <int UNROLL>
__global__ void halo_pull_vec_kernel(int64_t n_ghost, int D4, float4* __restrict__ dst, int64_t row0,
                                     const int* __restrict__ home_rank, const int* __restrict__ home_row,
                                     const int64_t* __restrict__ src_ptrs, const uint8_t* __restrict__ used) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t g = warp; g < n_ghost; g += nwarps) {
    if (used != nullptr && used[g] == 0) continue;
    const float4* src = reinterpret_cast<const float4*>(src_ptrs[home_rank[g]]) + (int64_t)home_row[g] * D4;
    float4* out = dst + (row0 + g) * D4;
    for (int c0 = 0; c0 < D4; c0 += 32 * UNROLL) {
      float4 v[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int c = c0 + u * 32 + lane;
        if (c < D4) v[u] = src[c];
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int c = c0 + u * 32 + lane;
        if (c < D4) out[c] = v[u];
      }
    }
  }
}

__global__ void halo_pull_narrow_kernel(int64_t n_ghost, int D, float* __restrict__ dst, int64_t row0,
                                        const int* __restrict__ home_rank, const int* __restrict__ home_row,
                                        const float* __restrict__ shift, const int64_t* __restrict__ src_ptrs,
                                        const uint8_t* __restrict__ used) {
  const int64_t g = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (g >= n_ghost || (used != nullptr && used[g] == 0)) return;
  const float* src = reinterpret_cast<const float*>(src_ptrs[home_rank[g]]) + (int64_t)home_row[g] * D;
  float* out = dst + (row0 + g) * D;
  for (int d = 0; d < D; ++d) out[d] = src[d] + (shift != nullptr ? shift[g * D + d] : 0.f);
}

void halo_pull_rows(at::Tensor dst, int64_t row0, const at::Tensor& home_rank, const at::Tensor& home_row,
                    const c10::optional<at::Tensor>& shift, const at::Tensor& src_ptrs,
                    const c10::optional<at::Tensor>& used) {
  c10::cuda::CUDAGuard guard(dst.device());
  NVA_CHECK_CONTIG(dst);
  int64_t n = home_rank.size(0);
  if (n == 0) return;
  TORCH_CHECK(row0 + n <= dst.size(0), "halo_pull_rows: ghost rows exceed the destination");
  int D = (int)(dst.numel() / dst.size(0));
  const uint8_t* um = used.has_value() ? used->data_ptr<uint8_t>() : nullptr;
  auto stream = at::cuda::getCurrentCUDAStream();
  if (D % 4 == 0 && !shift.has_value() && (reinterpret_cast<uintptr_t>(dst.data_ptr()) & 15) == 0) {
    int64_t blocks = std::min<int64_t>((n + 7) / 8, 148 * 16);
    halo_pull_vec_kernel<4><<<(unsigned)blocks, 256, 0, stream>>>(
        n, D / 4, reinterpret_cast<float4*>(dst.data_ptr<float>()), row0, home_rank.data_ptr<int>(), home_row.data_ptr<int>(),
        src_ptrs.data_ptr<int64_t>(), um);
  } else {
    halo_pull_narrow_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(
        n, D, dst.data_ptr<float>(), row0, home_rank.data_ptr<int>(), home_row.data_ptr<int>(),
        shift.has_value() ? shift->data_ptr<float>() : nullptr, src_ptrs.data_ptr<int64_t>(), um);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// used[g] = 1 for every ghost row (local row >= n_owned) that appears as a sender in the edge list.
__global__ void mark_used_senders_kernel(int64_t n_edges, const int* __restrict__ esend, int n_owned, int n_local,
                                         uint8_t* __restrict__ used) {
  const int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (e >= n_edges) return;
  const int j = esend[e];
  if (j >= n_owned && j < n_local) used[j - n_owned] = 1;
}

void mark_used_senders(const at::Tensor& esend, int64_t n_edges, int64_t n_owned, at::Tensor used) {
  c10::cuda::CUDAGuard guard(esend.device());
  TORCH_CHECK(esend.scalar_type() == at::kInt && used.scalar_type() == at::kByte, "mark_used_senders: int32 senders, uint8 marks");
  TORCH_CHECK(n_edges <= esend.numel(), "mark_used_senders: edge count exceeds the sender array");
  if (n_edges == 0) return;
  mark_used_senders_kernel<<<(unsigned)((n_edges + 255) / 256), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      n_edges, esend.data_ptr<int>(), (int)n_owned, (int)(n_owned + used.numel()), used.data_ptr<uint8_t>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}
}  // namespace nva

TORCH_LIBRARY_FRAGMENT(nvalchemi, m) {
  m.def("halo_pull_rows(Tensor(a!) dst, int row0, Tensor home_rank, Tensor home_row, Tensor? shift, Tensor src_ptrs, Tensor? used=None) -> ()", &nva::halo_pull_rows);
  m.def("mark_used_senders(Tensor esend, int n_edges, int n_owned, Tensor(a!) used) -> ()", &nva::mark_used_senders);
}

namespace nva {
// Two-shot all-reduce through the NVSwitch: rank r owns slice r of the buffer, reduces it ACROSS ALL RANKS with one
// multimem.ld_reduce per 16 bytes (the switch adds the peers' copies), applies `scale`, and multimem.st writes the
// result back into every rank's buffer.  `mc_ptr` is the multicast address of the symmetric buffer.  The caller puts a
// p2p_barrier before (all inputs written) and after (all slices stored).  n4 = number of float4 elements.
__global__ void multimem_allreduce_kernel(int64_t n4, uint64_t mc_ptr, int rank, int world, float scale) {
  int64_t per = (n4 + world - 1) / world;
  int64_t lo = per * rank, hi = lo + per < n4 ? lo + per : n4;
  for (int64_t i = lo + blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < hi; i += (int64_t)gridDim.x * blockDim.x) {
    uint64_t addr = mc_ptr + (uint64_t)i * 16u;
    float x, y, z, w;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(x), "=f"(y), "=f"(z), "=f"(w)
                 : "l"(addr)
                 : "memory");
    x *= scale; y *= scale; z *= scale; w *= scale;
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(x), "f"(y), "f"(z), "f"(w)
                 : "memory");
  }
}

void multimem_allreduce(int64_t mc_ptr, int64_t byte_offset, int64_t numel, int64_t rank, int64_t world, double scale,
                        const at::Tensor& like) {
  c10::cuda::CUDAGuard guard(like.device());
  TORCH_CHECK(mc_ptr != 0, "multimem_allreduce: no multicast address (NVLS not available for this buffer)");
  TORCH_CHECK(numel % 4 == 0 && byte_offset % 16 == 0, "multimem_allreduce works on 16-byte aligned float4 groups");
  int64_t n4 = numel / 4;
  if (n4 == 0) return;
  int64_t per = (n4 + world - 1) / world;
  int blocks = (int)std::min<int64_t>((per + 255) / 256, 4 * 148);
  multimem_allreduce_kernel<<<blocks > 0 ? blocks : 1, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      n4, (uint64_t)mc_ptr + (uint64_t)byte_offset, (int)rank, (int)world, (float)scale);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}
}  // namespace nva

TORCH_LIBRARY_FRAGMENT(nvalchemi, m) {
  m.def("multimem_allreduce(int mc_ptr, int byte_offset, int numel, int rank, int world, float scale, Tensor like) -> ()", &nva::multimem_allreduce);
}

namespace nva {
// Reverse halo: dst_{home_rank[g]}[home_row[g], :] += src[row0 + g, :].  Gradients that the local kernels accumulated on
// ghost rows travel to the owners once per row (instead of one NVLink reduction per edge from inside the convolution).
// Wide rows leave as 16-byte vector reductions (one warp per row, all-zero vectors skipped), narrow rows as scalar
// reductions from one thread per row.
__global__ void halo_push_add_vec_kernel(int64_t n_ghost, int D4, const float4* __restrict__ src, int64_t row0,
                                         const int* __restrict__ home_rank, const int* __restrict__ home_row,
                                         const int64_t* __restrict__ dst_ptrs, const uint8_t* __restrict__ used) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t g = warp; g < n_ghost; g += nwarps) {
    if (used != nullptr && used[g] == 0) continue;
    float4* dst = reinterpret_cast<float4*>(dst_ptrs[home_rank[g]]) + (int64_t)home_row[g] * D4;
    const float4* in = src + (row0 + g) * D4;
    for (int c = lane; c < D4; c += 32) {
      const float4 v = in[c];
      if (v.x != 0.f || v.y != 0.f || v.z != 0.f || v.w != 0.f) atomicAdd(dst + c, v);
    }
  }
}

__global__ void halo_push_add_narrow_kernel(int64_t n_ghost, int D, const float* __restrict__ src, int64_t row0,
                                            const int* __restrict__ home_rank, const int* __restrict__ home_row,
                                            const int64_t* __restrict__ dst_ptrs, const uint8_t* __restrict__ used) {
  const int64_t g = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (g >= n_ghost || (used != nullptr && used[g] == 0)) return;
  float* dst = reinterpret_cast<float*>(dst_ptrs[home_rank[g]]) + (int64_t)home_row[g] * D;
  const float* in = src + (row0 + g) * D;
  for (int d = 0; d < D; ++d) {
    const float v = in[d];
    if (v != 0.f) atomicAdd(dst + d, v);
  }
}

void halo_push_add_rows(const at::Tensor& src, int64_t row0, const at::Tensor& home_rank, const at::Tensor& home_row,
                        const at::Tensor& dst_ptrs, const c10::optional<at::Tensor>& used) {
  c10::cuda::CUDAGuard guard(src.device());
  NVA_CHECK_CONTIG(src);
  int64_t n = home_rank.size(0);
  if (n == 0) return;
  TORCH_CHECK(row0 + n <= src.size(0), "halo_push_add_rows: ghost rows exceed the source");
  int D = (int)(src.numel() / src.size(0));
  const uint8_t* um = used.has_value() ? used->data_ptr<uint8_t>() : nullptr;
  auto stream = at::cuda::getCurrentCUDAStream();
  if (D % 4 == 0 && (reinterpret_cast<uintptr_t>(src.data_ptr()) & 15) == 0) {
    int64_t blocks = std::min<int64_t>((n + 7) / 8, 148 * 16);
    halo_push_add_vec_kernel<<<(unsigned)blocks, 256, 0, stream>>>(
        n, D / 4, reinterpret_cast<const float4*>(src.data_ptr<float>()), row0, home_rank.data_ptr<int>(),
        home_row.data_ptr<int>(), dst_ptrs.data_ptr<int64_t>(), um);
  } else {
    halo_push_add_narrow_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(
        n, D, src.data_ptr<float>(), row0, home_rank.data_ptr<int>(), home_row.data_ptr<int>(),
        dst_ptrs.data_ptr<int64_t>(), um);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}
}  // namespace nva

TORCH_LIBRARY_FRAGMENT(nvalchemi, m) {
  m.def("halo_push_add_rows(Tensor src, int row0, Tensor home_rank, Tensor home_row, Tensor dst_ptrs, Tensor? used=None) -> ()", &nva::halo_push_add_rows);
}

namespace nva {
// Reverse halo by pull: the OWNER collects what the other ranks accumulated on their ghost copies of its rows,
//   buf[dst_row[k], :] += buf_{peer[k]}[peer_row[k], :]      (same symmetric buffer on both sides),
// with plain 16-byte peer loads (the fast direction of the link) and reductions into local memory; several entries may
// name the same owned row (one per rank / periodic image that holds a copy), hence the local atomics.  `peer_used`
// (optional): table of the peers' per-ghost "some edge used this row" bytes, indexed [peer] -> uint8*, with
// `peer_used_index[k]` the ghost's position in that array; unused copies hold zeros and are skipped without reading them.
__global__ void halo_pull_add_vec_kernel(int64_t n, int D4, float4* __restrict__ buf, const int* __restrict__ dst_row,
                                         const int* __restrict__ peer, const int* __restrict__ peer_row,
                                         const int64_t* __restrict__ ptrs, const int64_t* __restrict__ used_ptrs,
                                         const int* __restrict__ used_index) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t k = warp; k < n; k += nwarps) {
    const int p = peer[k];
    if (used_ptrs != nullptr && reinterpret_cast<const uint8_t*>(used_ptrs[p])[used_index[k]] == 0) continue;
    const float4* src = reinterpret_cast<const float4*>(ptrs[p]) + (int64_t)peer_row[k] * D4;
    float4* out = buf + (int64_t)dst_row[k] * D4;
    for (int c0 = 0; c0 < D4; c0 += 128) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = c0 + u * 32 + lane;
        if (c < D4) v[u] = src[c];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = c0 + u * 32 + lane;
        if (c < D4 && (v[u].x != 0.f || v[u].y != 0.f || v[u].z != 0.f || v[u].w != 0.f)) atomicAdd(out + c, v[u]);
      }
    }
  }
}

__global__ void halo_pull_add_narrow_kernel(int64_t n, int D, float* __restrict__ buf, const int* __restrict__ dst_row,
                                            const int* __restrict__ peer, const int* __restrict__ peer_row,
                                            const int64_t* __restrict__ ptrs, const int64_t* __restrict__ used_ptrs,
                                            const int* __restrict__ used_index) {
  const int64_t k = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (k >= n) return;
  const int p = peer[k];
  if (used_ptrs != nullptr && reinterpret_cast<const uint8_t*>(used_ptrs[p])[used_index[k]] == 0) return;
  const float* src = reinterpret_cast<const float*>(ptrs[p]) + (int64_t)peer_row[k] * D;
  float* out = buf + (int64_t)dst_row[k] * D;
  for (int d = 0; d < D; ++d) {
    const float v = src[d];
    if (v != 0.f) atomicAdd(out + d, v);
  }
}

void halo_pull_add_rows(at::Tensor buf, const at::Tensor& dst_row, const at::Tensor& peer, const at::Tensor& peer_row,
                        const at::Tensor& ptrs, const c10::optional<at::Tensor>& used_ptrs,
                        const c10::optional<at::Tensor>& used_index) {
  c10::cuda::CUDAGuard guard(buf.device());
  NVA_CHECK_CONTIG(buf);
  const int64_t n = dst_row.size(0);
  if (n == 0) return;
  TORCH_CHECK(peer.size(0) == n && peer_row.size(0) == n, "halo_pull_add_rows: tables of different lengths");
  TORCH_CHECK(used_ptrs.has_value() == used_index.has_value(), "halo_pull_add_rows: used_ptrs and used_index come together");
  const int D = (int)(buf.numel() / buf.size(0));
  const int64_t* up = used_ptrs.has_value() ? used_ptrs->data_ptr<int64_t>() : nullptr;
  const int* ui = used_index.has_value() ? used_index->data_ptr<int>() : nullptr;
  auto stream = at::cuda::getCurrentCUDAStream();
  if (D % 4 == 0 && (reinterpret_cast<uintptr_t>(buf.data_ptr()) & 15) == 0) {
    const int64_t blocks = std::min<int64_t>((n + 7) / 8, 148 * 16);
    halo_pull_add_vec_kernel<<<(unsigned)blocks, 256, 0, stream>>>(
        n, D / 4, reinterpret_cast<float4*>(buf.data_ptr<float>()), dst_row.data_ptr<int>(), peer.data_ptr<int>(),
        peer_row.data_ptr<int>(), ptrs.data_ptr<int64_t>(), up, ui);
  } else {
    halo_pull_add_narrow_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(
        n, D, buf.data_ptr<float>(), dst_row.data_ptr<int>(), peer.data_ptr<int>(), peer_row.data_ptr<int>(),
        ptrs.data_ptr<int64_t>(), up, ui);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}
}  // namespace nva

TORCH_LIBRARY_FRAGMENT(nvalchemi, m) {
  m.def("halo_pull_add_rows(Tensor(a!) buf, Tensor dst_row, Tensor peer, Tensor peer_row, Tensor ptrs, Tensor? used_ptrs=None, Tensor? used_index=None) -> ()", &nva::halo_pull_add_rows);
}

namespace nva {
// Reverse halo of the position gradient FUSED with what consumes it: thread i owns atom i, adds the gradients that other
// ranks accumulated on their ghost copies of the atom (plain peer loads through the symmetric buffer's address table,
// copies listed per owned row in CSR form) to its own, writes the force and, when a velocity array is given, applies the
// closing half kick of velocity Verlet / Langevin BAOAB, v += dt/2 F / m, in the same pass: the gradient of a boundary atom
// crosses NVLink once and is never written back to memory as an intermediate.
//   copy_ptr [n_owned + 1], copy_peer / copy_row / copy_used_index [S]: ghost copies of owned row i are entries
//   copy_ptr[i] .. copy_ptr[i + 1]; `used_ptrs` (optional) = the holders' per-ghost "some edge used this row" bytes.
__global__ void halo_force_finalize_kernel(int n_owned, const float* __restrict__ gpos, const int* __restrict__ copy_ptr,
                                           const int* __restrict__ copy_peer, const int* __restrict__ copy_row,
                                           const int* __restrict__ copy_used_index, const int64_t* __restrict__ ptrs,
                                           const int64_t* __restrict__ used_ptrs, float* __restrict__ forces,
                                           float* __restrict__ vel, const float* __restrict__ mass,
                                           const float* __restrict__ dt, const int* __restrict__ batch_idx) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_owned) return;
  float g0 = gpos[3 * i], g1 = gpos[3 * i + 1], g2 = gpos[3 * i + 2];
  for (int k = copy_ptr[i]; k < copy_ptr[i + 1]; ++k) {
    const int p = copy_peer[k];
    if (used_ptrs != nullptr && reinterpret_cast<const uint8_t*>(used_ptrs[p])[copy_used_index[k]] == 0) continue;
    const float* src = reinterpret_cast<const float*>(ptrs[p]) + 3 * (int64_t)copy_row[k];
    g0 += src[0]; g1 += src[1]; g2 += src[2];
  }
  const float f0 = -g0, f1 = -g1, f2 = -g2;
  forces[3 * i] = f0; forces[3 * i + 1] = f1; forces[3 * i + 2] = f2;
  if (vel != nullptr) {
    const float h = 0.5f * dt[batch_idx[i]] / mass[i];
    vel[3 * i] += h * f0; vel[3 * i + 1] += h * f1; vel[3 * i + 2] += h * f2;
  }
}

void halo_force_finalize(const at::Tensor& gpos, const at::Tensor& copy_ptr, const at::Tensor& copy_peer,
                         const at::Tensor& copy_row, const at::Tensor& copy_used_index, const at::Tensor& ptrs,
                         const c10::optional<at::Tensor>& used_ptrs, at::Tensor forces,
                         const c10::optional<at::Tensor>& velocities, const c10::optional<at::Tensor>& masses,
                         const c10::optional<at::Tensor>& dt, const c10::optional<at::Tensor>& batch_idx) {
  c10::cuda::CUDAGuard guard(gpos.device());
  NVA_CHECK_CONTIG(gpos); NVA_CHECK_CONTIG(forces);
  const int64_t n = forces.size(0);
  if (n == 0) return;
  TORCH_CHECK(gpos.scalar_type() == at::kFloat && forces.scalar_type() == at::kFloat && gpos.size(0) >= n &&
                  copy_ptr.numel() == n + 1 && copy_ptr.scalar_type() == at::kInt,
              "halo_force_finalize: float32 gradients / forces and an int32 CSR pointer of n_owned + 1 entries");
  TORCH_CHECK(copy_peer.numel() == copy_row.numel() && copy_peer.numel() == copy_used_index.numel(),
              "halo_force_finalize: copy tables of different lengths");
  const bool kick = velocities.has_value();
  if (kick) {
    TORCH_CHECK(masses.has_value() && dt.has_value() && batch_idx.has_value(), "halo_force_finalize: velocities need masses, dt, batch_idx");
    TORCH_CHECK(velocities->scalar_type() == at::kFloat && velocities->is_contiguous() && velocities->size(0) >= n &&
                    masses->scalar_type() == at::kFloat && dt->scalar_type() == at::kFloat && batch_idx->scalar_type() == at::kInt,
                "halo_force_finalize: float32 velocities / masses / dt and int32 batch_idx");
  }
  halo_force_finalize_kernel<<<(unsigned)((n + 255) / 256), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      (int)n, gpos.data_ptr<float>(), copy_ptr.data_ptr<int>(), copy_peer.data_ptr<int>(), copy_row.data_ptr<int>(),
      copy_used_index.data_ptr<int>(), ptrs.data_ptr<int64_t>(),
      used_ptrs.has_value() ? used_ptrs->data_ptr<int64_t>() : nullptr, forces.data_ptr<float>(),
      kick ? velocities->data_ptr<float>() : nullptr, kick ? masses->data_ptr<float>() : nullptr,
      kick ? dt->data_ptr<float>() : nullptr, kick ? batch_idx->data_ptr<int>() : nullptr);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}
}  // namespace nva

TORCH_LIBRARY_FRAGMENT(nvalchemi, m) {
  m.def("halo_force_finalize(Tensor gpos, Tensor copy_ptr, Tensor copy_peer, Tensor copy_row, Tensor copy_used_index, Tensor ptrs, Tensor? used_ptrs, Tensor(a!) forces, Tensor(b!)? velocities=None, Tensor? masses=None, Tensor? dt=None, Tensor? batch_idx=None) -> ()", &nva::halo_force_finalize);
}
