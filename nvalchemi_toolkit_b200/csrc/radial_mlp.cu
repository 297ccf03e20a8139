// SPDX-License-Identifier: Apache-2.0
// Fused radial MLP for sm_100a: the three hidden layers of MACE's radial network (8 -> 64 -> 64 -> 64, SiLU after
// each) run back to back on the tensor cores without leaving the SM.
//
//   per tile of 128 rows:  A0 (basis, K padded to 32) --MMA--> TMEM --SiLU--> shared (next A operand) --MMA--> ...
//
// The layer weights ([64 x K], K-major, 128-byte swizzle) are loaded once per CTA by TMA and stay resident; the
// epilogue of layer l reads the accumulator row of its thread from TMEM (tcgen05.ld), applies the activation and writes
// the row into shared memory in the K-major swizzled layout that tcgen05.mma expects for the A operand of layer l+1.
// Only the basis functions (32 B per row) are read from and the last hidden layer (256 B per row) is written to HBM;
// the unfused chain moved five 256-byte rows per edge.  With `TANGENT`, global rows alternate (value, d/dr); inside a
// tile the value rows occupy lanes 0-63 and the tangent rows lanes 64-127, and silu'(z_value) travels from the value
// thread to its tangent partner through shared memory.
// Replaces the first three torch.nn.Linear + SiLU layers of the reference's radial network (mace-torch RadialMLP,
// used through nvalchemi/models/mace.py:205-287).  Waits are bounded; failures are reported through `err`.
#include "common.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>

#include "tcgen05_utils.cuh"

namespace nva {
using at::Tensor;

constexpr float kRadialSiluNorm = 1.6790176868438721f;

// byte offset of 16-byte chunk `j` of row `r` inside one [rows x 128 B] k-block with 128-byte swizzle
__device__ __forceinline__ uint32_t sw128_off(int r, int j) {
  return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((j ^ (r & 7)) << 4));
}

template <bool TANGENT>
__global__ void __launch_bounds__(128) radial_mlp_kernel(const __grid_constant__ CUtensorMap tmW1,
                                                         const __grid_constant__ CUtensorMap tmW2,
                                                         const __grid_constant__ CUtensorMap tmW3,
                                                         const float* __restrict__ ef, int64_t rows,
                                                         float* __restrict__ out, int* __restrict__ err) {
  constexpr uint32_t W1_BYTES = 64 * 128, W_BYTES = 2 * 64 * 128, ACT_KB = 128 * 128;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sW1 = base, sW2 = sW1 + W1_BYTES, sW3 = sW2 + W_BYTES, sAct = sW3 + W_BYTES;
  const uint32_t bar_w = sAct + 2 * ACT_KB, bar_mma = bar_w + 8, tmem_slot = bar_w + 16;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  uint8_t* act = gen + W1_BYTES + 2 * W_BYTES;
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;

  if (t == 0) {
    mbar_init(bar_w, 1);
    mbar_init(bar_mma, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(64u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  uint32_t tmem_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

  bool ok = true;
  if (t == 0) {
    mbar_expect_tx(bar_w, W1_BYTES + 2 * W_BYTES);
    tma_load_2d(sW1, &tmW1, 0, 0, bar_w);
    for (int kb = 0; kb < 2; ++kb) {
      tma_load_2d(sW2 + kb * 64 * 128, &tmW2, kb * 32, 0, bar_w);
      tma_load_2d(sW3 + kb * 64 * 128, &tmW3, kb * 32, 0, bar_w);
    }
  }
  ok = mbar_wait(bar_w, 0, err, 31);
  ok = !__syncthreads_or(!ok);

  constexpr uint32_t idesc = umma_idesc_tf32(128, 64);
  const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
  uint32_t phase = 0;
  const int64_t ntiles = (rows + 127) / 128;

  // one layer: MMA over `nkb` k-blocks of the activation tile against weights at `sW`, then this thread's row in v[64]
  auto layer = [&](uint32_t sW, int nkb, float* v) -> bool {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (t == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      for (int kb = 0; kb < nkb; ++kb)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          uint64_t da = umma_desc_sw128(sAct + kb * ACT_KB + k * UMMA_K * 4);
          uint64_t db = umma_desc_sw128(sW + kb * 64 * 128 + k * UMMA_K * 4);
          umma_tf32(tmem_base, da, db, idesc, (kb | k) ? 1u : 0u);
        }
      umma_commit(bar_mma);
    }
    bool good = mbar_wait(bar_mma, phase & 1, err, 32);
    ++phase;
    if (__syncthreads_or(!good)) return false;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    tmem_ld32(lane_addr, v);
    tmem_ld32(lane_addr + 32, v + 32);
    // sigmoid by ex2.approx + rcp.approx (two special-function instructions; an IEEE division costs ~10 more)
    if (!TANGENT) {
#pragma unroll
      for (int j = 0; j < 64; ++j) v[j] = v[j] * __fdividef(kRadialSiluNorm, 1.f + __expf(-v[j]));
    } else {
      // rows 0-63 of the tile are value rows, rows 64-127 the matching tangent rows.  The value thread of an edge
      // computes silu(z) for itself and leaves silu'(z) in the (free) activation row of its tangent partner, which
      // picks it up after a barrier: no shuffles, and the special-function work is done once per edge.
      if (t < 64) {
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float fac[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              float a = v[kb * 32 + 4 * j + q];
              float sg = __fdividef(kRadialSiluNorm, 1.f + __expf(-a));       // norm * sigmoid(a)
              fac[q] = sg * fmaf(a, 1.f - sg * (1.f / kRadialSiluNorm), 1.f);  // norm * silu'(a)
              v[kb * 32 + 4 * j + q] = a * sg;
            }
            *reinterpret_cast<float4*>(act + kb * ACT_KB + sw128_off(t + 64, j)) = make_float4(fac[0], fac[1], fac[2], fac[3]);
          }
      }
      __syncthreads();
      if (t >= 64) {
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float4 fac = *reinterpret_cast<const float4*>(act + kb * ACT_KB + sw128_off(t, j));
            v[kb * 32 + 4 * j] *= fac.x; v[kb * 32 + 4 * j + 1] *= fac.y;
            v[kb * 32 + 4 * j + 2] *= fac.z; v[kb * 32 + 4 * j + 3] *= fac.w;
          }
      }
    }
    return true;
  };
  auto store_act = [&](const float* v) {  // row t of the [128 x 64] activation tile, two k-blocks of 32 columns
#pragma unroll
    for (int kb = 0; kb < 2; ++kb)
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *reinterpret_cast<float4*>(act + kb * ACT_KB + sw128_off(t, j)) =
            make_float4(v[kb * 32 + 4 * j], v[kb * 32 + 4 * j + 1], v[kb * 32 + 4 * j + 2], v[kb * 32 + 4 * j + 3]);
  };

  for (int64_t tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
    // TANGENT: the tile covers 64 edges; thread t < 64 owns the value row of edge t, thread t >= 64 the tangent row of
    // edge t - 64 (global rows interleave value and tangent)
    const int64_t row = TANGENT ? tile * 128 + 2 * (t & 63) + (t >> 6) : tile * 128 + t;
    // basis functions of this thread's row -> A operand (K = 8 padded with zeros to one 32-column k-block)
    float4 b0 = make_float4(0.f, 0.f, 0.f, 0.f), b1 = b0;
    if (row < rows) {
      const float4* p = reinterpret_cast<const float4*>(ef + row * 8);
      b0 = __ldg(p);
      b1 = __ldg(p + 1);
    }
    // The tensor core reads only the upper 19 bits of an fp32 operand (tf32).  The first layer keeps full precision
    // by the split x = hi + lo placed in otherwise unused padding columns: columns 0-7 hold hi, 8-15 lo, 16-23 hi
    // again, and the padded weight rows hold (W_hi, W_hi, W_lo), so the product is x_hi W_hi + x_lo W_hi + x_hi W_lo.
    auto hi4 = [](float4 x) {
      return make_float4(__uint_as_float(__float_as_uint(x.x) & 0xFFFFE000u), __uint_as_float(__float_as_uint(x.y) & 0xFFFFE000u),
                         __uint_as_float(__float_as_uint(x.z) & 0xFFFFE000u), __uint_as_float(__float_as_uint(x.w) & 0xFFFFE000u));
    };
    const float4 h0 = hi4(b0), h1 = hi4(b1);
    const float4 l0 = make_float4(b0.x - h0.x, b0.y - h0.y, b0.z - h0.z, b0.w - h0.w);
    const float4 l1 = make_float4(b1.x - h1.x, b1.y - h1.y, b1.z - h1.z, b1.w - h1.w);
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    *reinterpret_cast<float4*>(act + sw128_off(t, 0)) = h0;
    *reinterpret_cast<float4*>(act + sw128_off(t, 1)) = h1;
    *reinterpret_cast<float4*>(act + sw128_off(t, 2)) = l0;
    *reinterpret_cast<float4*>(act + sw128_off(t, 3)) = l1;
    *reinterpret_cast<float4*>(act + sw128_off(t, 4)) = h0;
    *reinterpret_cast<float4*>(act + sw128_off(t, 5)) = h1;
    *reinterpret_cast<float4*>(act + sw128_off(t, 6)) = zero;
    *reinterpret_cast<float4*>(act + sw128_off(t, 7)) = zero;
    float v[64];
    if (!(ok = layer(sW1, 1, v))) break;
    store_act(v);
    if (!(ok = layer(sW2, 2, v))) break;
    store_act(v);
    if (!(ok = layer(sW3, 2, v))) break;
    // Output through the (now free) activation tile: a thread holds one 256-byte row, so direct stores would touch 32
    // different rows per instruction; staged, a warp writes 512 contiguous bytes per instruction.
    if (TANGENT) __syncthreads();  // partners finished reading the derivative factors left in the tile
    store_act(v);
    __syncthreads();
#pragma unroll 4
    for (int it = 0; it < 16; ++it) {
      const int idx = it * 128 + t;
      const int g = idx >> 4, ch = idx & 15;                       // row of the tile in global order, 16-byte chunk
      const int r = TANGENT ? (g >> 1) + 64 * (g & 1) : g;         // the thread (= tile row) that produced it
      const int64_t grow = tile * 128 + g;
      if (grow < rows)
        *reinterpret_cast<float4*>(out + grow * 64 + ch * 4) =
            *reinterpret_cast<const float4*>(act + (ch >> 3) * ACT_KB + sw128_off(r, ch & 7));
    }
    __syncthreads();  // the next tile's basis functions overwrite the tile
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(64u) : "memory");
  }
}

static PFN_cuTensorMapEncodeTiled_v12000 radial_encode() {
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

static CUtensorMap weight_map(const float* ptr, int64_t k) {  // [64 rows, k] row-major, boxes of 32 columns x 64 rows
  CUtensorMap m;
  cuuint64_t dims[2] = {(cuuint64_t)k, 64};
  cuuint64_t strides[1] = {(cuuint64_t)k * 4};
  cuuint32_t box[2] = {32, 64};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = radial_encode()(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(ptr), dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code ", (int)r);
  return m;
}

template <bool TANGENT>
static void launch_radial(const CUtensorMap& m1, const CUtensorMap& m2, const CUtensorMap& m3, const float* ef, int64_t rows,
                          float* out, int* err, int grid, size_t smem) {
  static bool configured = false;  // one flag per kernel instantiation
  if (!configured) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(radial_mlp_kernel<TANGENT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  radial_mlp_kernel<TANGENT><<<grid, 128, smem, at::cuda::getCurrentCUDAStream()>>>(m1, m2, m3, ef, rows, out, err);
}

// ef: [rows, 8] basis rows (with `tangent`: value and d/dr rows interleaved, rows even); w1t: [64, 32] = first layer
// transposed, columns (W_hi, W_hi, W_lo, 0) with W_hi the tf32-representable part of the weight; w2t, w3t: [64, 64]
// transposed layers.  Returns [rows, 64].
Tensor mace_radial_hidden(const Tensor& ef, const Tensor& w1t, const Tensor& w2t, const Tensor& w3t, bool tangent,
                          Tensor err, const c10::optional<Tensor>& out_buf) {
  c10::cuda::CUDAGuard guard(ef.device());
  NVA_CHECK_CONTIG(ef); NVA_CHECK_CONTIG(w1t); NVA_CHECK_CONTIG(w2t); NVA_CHECK_CONTIG(w3t);
  TORCH_CHECK(ef.scalar_type() == at::kFloat && ef.size(-1) == 8, "basis rows must be float32 [rows, 8]");
  TORCH_CHECK(w1t.size(0) == 64 && w1t.size(1) == 32 && w2t.size(0) == 64 && w2t.size(1) == 64 && w3t.size(0) == 64 &&
                  w3t.size(1) == 64, "fused radial MLP is specialised for 8 -> 64 -> 64 -> 64");
  int64_t rows = ef.numel() / 8;
  TORCH_CHECK(!tangent || rows % 2 == 0, "tangent mode needs interleaved (value, derivative) rows");
  // `out_buf` (optional): caller-owned storage of at least rows * 64 floats, so that a result kept across kernels does
  // not go through the allocator with a slightly different size every step
  Tensor out;
  if (out_buf.has_value()) {
    TORCH_CHECK(out_buf->is_contiguous() && out_buf->scalar_type() == at::kFloat && out_buf->numel() >= rows * 64,
                "mace_radial_hidden: output buffer too small");
    out = out_buf->view({-1}).narrow(0, 0, rows * 64).view({rows, 64});
  } else {
    out = at::empty({rows, 64}, ef.options());
  }
  if (rows == 0) return out;
  CUtensorMap m1 = weight_map(w1t.data_ptr<float>(), 32), m2 = weight_map(w2t.data_ptr<float>(), 64),
              m3 = weight_map(w3t.data_ptr<float>(), 64);
  size_t smem = 64 * 128 + 2 * (2 * 64 * 128) + 2 * 128 * 128 + 64 + 1024;
  int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  int64_t ntiles = (rows + 127) / 128;
  int grid = (int)std::min<int64_t>(ntiles, 3 * (int64_t)sms);
  if (tangent) launch_radial<true>(m1, m2, m3, ef.data_ptr<float>(), rows, out.data_ptr<float>(), err.data_ptr<int>(), grid, smem);
  else launch_radial<false>(m1, m2, m3, ef.data_ptr<float>(), rows, out.data_ptr<float>(), err.data_ptr<int>(), grid, smem);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

}  // namespace nva

TORCH_LIBRARY_FRAGMENT(nvalchemi, m) {
  m.def("mace_radial_hidden(Tensor ef, Tensor w1t, Tensor w2t, Tensor w3t, bool tangent, Tensor(a!) err, Tensor(b!)? out_buf=None) -> Tensor", &nva::mace_radial_hidden);
}
