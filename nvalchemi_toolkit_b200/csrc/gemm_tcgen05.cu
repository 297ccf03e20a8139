// SPDX-License-Identifier: Apache-2.0
// TF32 GEMM on the 5th-generation tensor cores: C[M,N] = act(alpha * A[M,K] @ Bt[N,K]^T).
//
// Used for the dense channel mixes of the native MACE (radial MLP, o3 linear layers, readouts),
// i.e. the ops the reference runs through cuBLAS / cuEquivariance indexed_linear
// (nvalchemi/models/mace.py:408-410).  Structure of one CTA (one 128 x BN output tile):
//   warp 0   : TMA producer  - cp.async.bulk.tensor 2D loads of the A and B k-blocks into a
//              128B-swizzled shared-memory ring, completion on "full" mbarriers;
//   warp 1   : allocates TMEM, then one elected lane issues tcgen05.mma (kind::tf32,
//              cta_group::1, M=128, N=BN, K=8) with the accumulator in TMEM and releases ring
//              slots with tcgen05.commit on "empty" mbarriers;
//   warps 2-5: epilogue - tcgen05.ld (32x32b) of the accumulator rows, scale / activation,
//              vectorised global stores.
// Every mbarrier wait is bounded; on expiry the kernel records an error code in `err`, skips the
// remaining work, releases its TMEM and returns (no trap, no endless spin).
#include "common.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>

#include "tcgen05_utils.cuh"

namespace nva {
using at::Tensor;

constexpr int BM = 128;
constexpr int BK = 32;      // 32 tf32 = 128 bytes = one swizzle row

constexpr float kSiluNorm = 1.6790176868438721f;

// Grouped form: one launch runs G independent products that share M, N and the leading dimensions,
//   C[:, c_col[g] : c_col[g] + N] (+)= act(alpha * A[:, a_col[g] : a_col[g] + k[g]] @ Bt[b_row[g] : b_row[g] + N, : k[g]]^T),
// i.e. column slices of one wide A matrix times row blocks of one packed weight matrix (the per-irrep channel mixes of
// an equivariant layer: one slice per (l, m) component, one weight block per l).  Tiles are scheduled m-tile major so that
// the groups reading the same rows of A run together.
constexpr int kMaxGroups = 64;
struct GemmGroups {
  int n_groups;
  int accumulate;  // 1: add to what C holds
  int a_col[kMaxGroups], k[kMaxGroups], b_row[kMaxGroups], c_col[kMaxGroups];
};

template <int BN, int STAGES, bool GROUPED>
__device__ __forceinline__ void gemm_tf32_body(const CUtensorMap& tmA, const CUtensorMap& tmB, float* __restrict__ C, int M,
                                               int N, int K, int64_t ldc, float alpha, int act, int* __restrict__ err,
                                               const GemmGroups* gt) {
  extern __shared__ uint8_t smem_raw[];
  constexpr uint32_t A_BYTES = BM * BK * 4, B_BYTES = BN * BK * 4, STAGE_BYTES = A_BYTES + B_BYTES;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar0 = base + STAGES * STAGE_BYTES;  // full[STAGES], empty[STAGES], tmem_full
  const uint32_t tmem_slot = bar0 + (2 * STAGES + 1) * 8;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  const uint32_t accum_bar = bar0 + 8u * (2 * STAGES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // 1D grid, N-tiles fastest: the CTAs that share an A row-block run together and hit it in L2
  const int n_tiles = (N + BN - 1) / BN;
  int m0, n0, a_col = 0, b_row = 0;
  bool accumulate = false;
  if constexpr (GROUPED) {
    const int G = gt->n_groups;
    const int g = (int)((blockIdx.x / n_tiles) % G);
    m0 = (int)(blockIdx.x / (n_tiles * G)) * BM;
    n0 = (int)(blockIdx.x % n_tiles) * BN;
    a_col = gt->a_col[g]; b_row = gt->b_row[g]; K = gt->k[g];
    C += gt->c_col[g];
    accumulate = gt->accumulate != 0;
  } else {
    m0 = (int)(blockIdx.x / n_tiles) * BM; n0 = (int)(blockIdx.x % n_tiles) * BN;
  }
  const int num_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    mbar_init(accum_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"((uint32_t)BN)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  uint32_t tmem_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < num_kb; ++kb) {
        int s = kb % STAGES;
        if (!mbar_wait(empty_bar(s), ((kb / STAGES) & 1) ^ 1, err, 1)) break;
        mbar_expect_tx(full_bar(s), STAGE_BYTES);
        uint32_t sa = base + s * STAGE_BYTES;
        tma_load_2d(sa, &tmA, a_col + kb * BK, m0, full_bar(s));
        tma_load_2d(sa + A_BYTES, &tmB, kb * BK, b_row + n0, full_bar(s));
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_tf32(BM, BN);
      bool ok = true;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        int s = kb % STAGES;
        ok = mbar_wait(full_bar(s), (kb / STAGES) & 1, err, 2);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        uint32_t sa = base + s * STAGE_BYTES;
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          uint64_t da = umma_desc_sw128(sa + k * UMMA_K * 4);
          uint64_t db = umma_desc_sw128(sa + A_BYTES + k * UMMA_K * 4);
          umma_tf32(tmem_base, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(empty_bar(s));  // slot reusable once these MMAs have read it
      }
      umma_commit(accum_bar);       // accumulator complete (or abandoned) - releases the epilogue
    }
  } else {
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    if (mbar_wait(accum_bar, 0, err, 3)) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // The ring is idle once the accumulator is complete: reuse it as a per-warp staging tile
      // [32 rows][BN floats] so that global stores are full-row coalesced.  float4 slots are XOR-swizzled
      // by (row & 7): conflict-free for the row-per-lane writes and for the row-wide reads.
      constexpr int SPR = BN / 4;                      // float4 slots per row
      float4* stage = reinterpret_cast<float4*>(smem_raw + (base - smem_u32(smem_raw))) + q * 32 * SPR;
#pragma unroll 1
      for (int cb = 0; cb < BN / 32; ++cb) {
        float v[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(cb * 32), v);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float x = v[j] * alpha;
          // sigmoid by ex2.approx + rcp.approx; an IEEE division would cost about ten more instructions per element
          if (act == 1) {
            x = x * __fdividef(kSiluNorm, 1.f + __expf(-x));
          } else if (act == 2) {
            // rows alternate (value, tangent): even rows get silu(a), odd rows silu'(a_even) * t
            float a = __shfl_sync(0xffffffffu, x, lane & ~1);
            float sg = __fdividef(1.f, 1.f + __expf(-a));
            x = (lane & 1) ? sg * (1.f + a * (1.f - sg)) * kSiluNorm * x : a * sg * kSiluNorm;
          }
          v[j] = x;
        }
#pragma unroll
        for (int g = 0; g < 8; ++g)
          stage[lane * SPR + ((cb * 8 + g) ^ (lane & 7))] = make_float4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
      }
      __syncwarp();
      const bool vec_ok = (ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
      constexpr int RPI = 32 / SPR;                    // rows written per warp instruction
      const int slot = lane % SPR, rsub = lane / SPR;
#pragma unroll 4
      for (int r0 = 0; r0 < 32; r0 += RPI) {
        int r = r0 + rsub;
        int row = m0 + q * 32 + r;
        int col = n0 + 4 * slot;
        if (row < M && col < N) {
          float4 val = stage[r * SPR + (slot ^ (r & 7))];
          float* dst = C + (int64_t)row * ldc + col;
          if (vec_ok && col + 4 <= N) {
            if (accumulate) {
              const float4 old = *reinterpret_cast<const float4*>(dst);
              val.x += old.x; val.y += old.y; val.z += old.z; val.w += old.w;
            }
            *reinterpret_cast<float4*>(dst) = val;
          } else {
            dst[0] = val.x + (accumulate ? dst[0] : 0.f);
            if (col + 1 < N) dst[1] = val.y + (accumulate ? dst[1] : 0.f);
            if (col + 2 < N) dst[2] = val.z + (accumulate ? dst[2] : 0.f);
            if (col + 3 < N) dst[3] = val.w + (accumulate ? dst[3] : 0.f);
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)BN) : "memory");
  }
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(192) gemm_tf32_kernel(const __grid_constant__ CUtensorMap tmA,
                                                        const __grid_constant__ CUtensorMap tmB,
                                                        float* __restrict__ C, int M, int N, int K, int64_t ldc,
                                                        float alpha, int act, int* __restrict__ err) {
  gemm_tf32_body<BN, STAGES, false>(tmA, tmB, C, M, N, K, ldc, alpha, act, err, nullptr);
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(192) gemm_tf32_grouped_kernel(const __grid_constant__ CUtensorMap tmA,
                                                                const __grid_constant__ CUtensorMap tmB,
                                                                const __grid_constant__ GemmGroups groups,
                                                                float* __restrict__ C, int M, int N, int64_t ldc,
                                                                float alpha, int act, int* __restrict__ err) {
  gemm_tf32_body<BN, STAGES, true>(tmA, tmB, C, M, N, 0, ldc, alpha, act, err, &groups);
}

// ---- host side -------------------------------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 get_encode() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    C10_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
    TORCH_CHECK(p != nullptr && q == cudaDriverEntryPointSuccess, "cuTensorMapEncodeTiled is not available");
    fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }
  return fn;
}

// 2D fp32 row-major [rows, cols] with row stride `ld` elements; box = [box_rows, BK], 128B swizzle.
static CUtensorMap make_map(const float* ptr, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
  CUtensorMap m;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = get_encode()(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(ptr), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code ", (int)r);
  return m;
}

static Tensor& error_word(const at::Device& dev) {
  static std::vector<Tensor> words(64);
  Tensor& w = words[dev.index() < 0 ? 0 : dev.index()];
  if (!w.defined()) w = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(dev));
  return w;
}

// a [M,K] (row stride lda, K contiguous), bt [N,K] contiguous -> c [M,N] (new, contiguous) or into `out`.
Tensor gemm_tf32_impl(const Tensor& a, const Tensor& bt, double alpha, int64_t act, const c10::optional<Tensor>& out) {
  TORCH_CHECK(a.is_cuda() && bt.is_cuda() && a.scalar_type() == at::kFloat && bt.scalar_type() == at::kFloat,
              "gemm_tf32 expects float32 CUDA tensors");
  TORCH_CHECK(a.dim() == 2 && bt.dim() == 2 && a.size(1) == bt.size(1), "gemm_tf32: shapes [M,K] x [N,K]");
  TORCH_CHECK(a.stride(1) == 1 && bt.stride(1) == 1, "gemm_tf32: K must be the contiguous axis");
  c10::cuda::CUDAGuard guard(a.device());
  int64_t M = a.size(0), K = a.size(1), N = bt.size(0);
  int64_t lda = a.stride(0), ldb = bt.stride(0);
  TORCH_CHECK(K % 4 == 0 && lda % 4 == 0 && ldb % 4 == 0, "gemm_tf32: K and row strides must be multiples of 4");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(a.data_ptr()) & 15) == 0 && (reinterpret_cast<uintptr_t>(bt.data_ptr()) & 15) == 0,
              "gemm_tf32: operands must be 16-byte aligned");
  Tensor c = out.has_value() ? *out : at::empty({M, N}, a.options());
  TORCH_CHECK(c.size(0) == M && c.size(1) == N && c.stride(1) == 1, "gemm_tf32: bad output");
  if (M == 0 || N == 0) return c;
  if (K == 0) return c.zero_();
  int bn = N <= 64 ? 64 : 128;
  CUtensorMap ma = make_map(a.data_ptr<float>(), M, K, lda, BM);
  CUtensorMap mb = make_map(bt.data_ptr<float>(), N, K, ldb, bn);
  int64_t tiles = ((N + bn - 1) / bn) * ((M + BM - 1) / BM);
  TORCH_CHECK(tiles < (int64_t)2147483647, "gemm_tf32: too many tiles");
  dim3 grid((unsigned)tiles);
  int* err = error_word(a.device()).data_ptr<int>();
  auto st = at::cuda::getCurrentCUDAStream();
  // short-K problems (radial MLP, K <= 64) need only two ring slots: 64 KB of shared memory, three CTAs per SM
  const bool short_k = K <= 2 * BK;
#define NVA_LAUNCH(BN_, ST_)                                                                                        \
  do {                                                                                                              \
    size_t smem = (size_t)ST_ * (BM * BK * 4 + BN_ * BK * 4) + 1024 + 256;                                          \
    static bool configured = false;                                                                                 \
    if (!configured) {                                                                                              \
      C10_CUDA_CHECK(cudaFuncSetAttribute(gemm_tf32_kernel<BN_, ST_>, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                                          (int)smem));                                                              \
      configured = true;                                                                                            \
    }                                                                                                               \
    gemm_tf32_kernel<BN_, ST_><<<grid, 192, smem, st>>>(ma, mb, c.data_ptr<float>(), (int)M, (int)N, (int)K,        \
                                                        c.stride(0), (float)alpha, (int)act, err);                  \
  } while (0)
  if (bn == 64) {
    if (short_k) NVA_LAUNCH(64, 2); else NVA_LAUNCH(64, 4);
  } else {
    if (short_k) NVA_LAUNCH(128, 2); else NVA_LAUNCH(128, 3);
  }
#undef NVA_LAUNCH
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return c;
}

Tensor gemm_tf32(const Tensor& a, const Tensor& bt, double alpha, int64_t act) {
  return gemm_tf32_impl(a, bt, alpha, act, c10::nullopt);
}
void gemm_tf32_out(const Tensor& a, const Tensor& bt, double alpha, int64_t act, Tensor out) {
  gemm_tf32_impl(a, bt, alpha, act, out);
}

// Grouped product (see GemmGroups).  a [M, Wa] (row stride lda), bt [R, Kmax] packed weight blocks (K-major), c [M, Wc]
// (row stride ldc); tables are int lists of one entry per group; every k[g] is a multiple of 32.
void gemm_tf32_grouped(const Tensor& a, const Tensor& bt, Tensor c, int64_t n_cols, std::vector<int64_t> a_col,
                       std::vector<int64_t> k, std::vector<int64_t> b_row, std::vector<int64_t> c_col, double alpha,
                       int64_t act, bool accumulate) {
  TORCH_CHECK(a.is_cuda() && bt.is_cuda() && c.is_cuda() && a.scalar_type() == at::kFloat && bt.scalar_type() == at::kFloat &&
                  c.scalar_type() == at::kFloat, "gemm_tf32_grouped expects float32 CUDA tensors");
  TORCH_CHECK(a.dim() == 2 && bt.dim() == 2 && c.dim() == 2 && a.stride(1) == 1 && bt.stride(1) == 1 && c.stride(1) == 1,
              "gemm_tf32_grouped: 2-D operands with unit inner stride");
  const int64_t G = (int64_t)a_col.size();
  TORCH_CHECK(G >= 1 && G <= kMaxGroups && (int64_t)k.size() == G && (int64_t)b_row.size() == G && (int64_t)c_col.size() == G,
              "gemm_tf32_grouped: 1..", kMaxGroups, " groups with one table entry each");
  c10::cuda::CUDAGuard guard(a.device());
  const int64_t M = a.size(0), N = n_cols;
  TORCH_CHECK(c.size(0) == M, "gemm_tf32_grouped: row counts differ");
  const int64_t lda = a.stride(0), ldb = bt.stride(0);
  TORCH_CHECK(lda % 4 == 0 && ldb % 4 == 0, "gemm_tf32_grouped: row strides must be multiples of 4");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(a.data_ptr()) & 15) == 0 && (reinterpret_cast<uintptr_t>(bt.data_ptr()) & 15) == 0,
              "gemm_tf32_grouped: operands must be 16-byte aligned");
  if (M == 0 || N == 0) return;
  GemmGroups gt;
  gt.n_groups = (int)G;
  gt.accumulate = accumulate ? 1 : 0;
  for (int64_t g = 0; g < G; ++g) {
    TORCH_CHECK(k[g] > 0 && k[g] % BK == 0, "gemm_tf32_grouped: every k must be a positive multiple of ", BK);
    TORCH_CHECK(a_col[g] >= 0 && a_col[g] % 4 == 0 && a_col[g] + k[g] <= a.size(1), "gemm_tf32_grouped: A slice out of range");
    TORCH_CHECK(b_row[g] >= 0 && b_row[g] + N <= bt.size(0) && k[g] <= bt.size(1), "gemm_tf32_grouped: weight block out of range");
    TORCH_CHECK(c_col[g] >= 0 && c_col[g] + N <= c.size(1), "gemm_tf32_grouped: C slice out of range");
    gt.a_col[g] = (int)a_col[g]; gt.k[g] = (int)k[g]; gt.b_row[g] = (int)b_row[g]; gt.c_col[g] = (int)c_col[g];
  }
  const int bn = N <= 64 ? 64 : 128;
  CUtensorMap ma = make_map(a.data_ptr<float>(), M, a.size(1), lda, BM);
  CUtensorMap mb = make_map(bt.data_ptr<float>(), bt.size(0), bt.size(1), ldb, bn);
  const int64_t tiles = ((N + bn - 1) / bn) * ((M + BM - 1) / BM) * G;
  TORCH_CHECK(tiles < (int64_t)2147483647, "gemm_tf32_grouped: too many tiles");
  dim3 grid((unsigned)tiles);
  int* err = error_word(a.device()).data_ptr<int>();
  auto st = at::cuda::getCurrentCUDAStream();
  int64_t kmax = 0;
  for (auto v : k) kmax = std::max(kmax, v);
  const bool short_k = kmax <= 2 * BK;
#define NVA_LAUNCH_G(BN_, ST_)                                                                                      \
  do {                                                                                                              \
    size_t smem = (size_t)ST_ * (BM * BK * 4 + BN_ * BK * 4) + 1024 + 256;                                          \
    static bool configured = false;                                                                                 \
    if (!configured) {                                                                                              \
      C10_CUDA_CHECK(cudaFuncSetAttribute(gemm_tf32_grouped_kernel<BN_, ST_>,                                       \
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));                 \
      configured = true;                                                                                            \
    }                                                                                                               \
    gemm_tf32_grouped_kernel<BN_, ST_><<<grid, 192, smem, st>>>(ma, mb, gt, c.data_ptr<float>(), (int)M, (int)N,    \
                                                                c.stride(0), (float)alpha, (int)act, err);          \
  } while (0)
  if (bn == 64) {
    if (short_k) NVA_LAUNCH_G(64, 2); else NVA_LAUNCH_G(64, 4);
  } else {
    if (short_k) NVA_LAUNCH_G(128, 2); else NVA_LAUNCH_G(128, 3);
  }
#undef NVA_LAUNCH_G
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// Reads (and clears) the error word: 0 = no bounded wait expired since the last call.
int64_t gemm_error_status(const Tensor& like) {
  Tensor& w = error_word(like.device());
  int64_t v = w.item<int>();
  if (v != 0) w.zero_();
  return v;
}

}  // namespace nva

TORCH_LIBRARY_FRAGMENT(nvalchemi, m) {
  m.def("gemm_tf32(Tensor a, Tensor bt, float alpha=1.0, int act=0) -> Tensor", &nva::gemm_tf32);
  m.def("gemm_tf32_out(Tensor a, Tensor bt, float alpha, int act, Tensor(a!) out) -> ()", &nva::gemm_tf32_out);
  m.def("gemm_error_status(Tensor like) -> int", &nva::gemm_error_status);
  m.def("gemm_tf32_grouped(Tensor a, Tensor bt, Tensor(a!) c, int n_cols, int[] a_col, int[] k, int[] b_row, int[] c_col, float alpha=1.0, int act=0, bool accumulate=False) -> ()", &nva::gemm_tf32_grouped);
}
